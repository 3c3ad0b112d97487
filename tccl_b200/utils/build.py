"""In-tree build of ``libtccl_b200.so`` with nvcc for sm_100a.

Every ``csrc/*.cu`` is compiled to an object under ``tccl_b200/_build`` and the
objects are linked into ``tccl_b200/_lib/libtccl_b200.so`` (static cudart, no
libtorch).  A source is recompiled when it, any header beside it, or the flag
set changed.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "csrc"
BUILD = PKG / "_build"
LIBDIR = PKG / "_lib"
LIB = LIBDIR / "libtccl_b200.so"
HOST_LIB = LIBDIR / "libtccl_hostproto.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("TCCL_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set TCCL_NVCC)")


def _digest(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def sources():
    return sorted(CSRC.glob("*.cu"))


def headers():
    return sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False, debug_checks: bool = False) -> Path:
    """Compile what is stale and link; returns the path of the shared library.

    ``debug_checks=True`` builds the second flavour, ``libtccl_b200_dbg.so`` (``-DTCCL_DEBUG_CHECKS``):
    the flat collectives check every vector offset against the extents the host passes along and,
    on a miss, record ``TCCL_BAD_INDEX`` in the status words and skip the access.  The library is
    loaded instead of the regular one when ``TCCL_DEBUG_CHECKS=1`` is set."""
    nvcc = _nvcc()
    BUILD = PKG / ("_build_dbg" if debug_checks else "_build")
    LIB = LIBDIR / ("libtccl_b200_dbg.so" if debug_checks else "libtccl_b200.so")
    BUILD.mkdir(exist_ok=True)
    LIBDIR.mkdir(exist_ok=True)
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else []) + (["-DTCCL_DEBUG_CHECKS=1"] if debug_checks else [])
    hdr = headers()
    jobs = []
    objs = []
    for src in sources():
        obj = BUILD / (src.stem + ".o")
        stamp = BUILD / (src.stem + ".sha")
        dig = _digest([src] + hdr, " ".join(flags))
        objs.append(obj)
        if force or not obj.exists() or not stamp.exists() or stamp.read_text() != dig:
            jobs.append((src, obj, stamp, dig))

    def compile_one(job):
        src, obj, stamp, dig = job
        cmd = [nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        stamp.write_text(dig)
        return src.name, r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for name, err in ex.map(compile_one, jobs):
                if verbose or ptxas_info:
                    print(f"[tccl_b200.build] compiled {name}", file=sys.stderr)
                    if ptxas_info:
                        print(err, file=sys.stderr)
    if jobs or not LIB.exists():
        tmp = LIB.with_suffix(f".tmp{os.getpid()}.so")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB)  # atomic: nobody ever sees a half-written library
        if verbose:
            print(f"[tccl_b200.build] linked {LIB}", file=sys.stderr)
    return LIB


def build_host(verbose: bool = False, force: bool = False) -> Path:
    """Compile the host-side protocol model (csrc/host/*.cpp, plain g++, no CUDA)."""
    LIBDIR.mkdir(exist_ok=True)
    BUILD.mkdir(exist_ok=True)
    srcs = [CSRC / "host" / "host_protocol.cpp"]
    stamp = BUILD / "hostproto.sha"
    dig = _digest(srcs + headers(), "g++ -O2 -std=c++17")
    if force or not HOST_LIB.exists() or not stamp.exists() or stamp.read_text() != dig:
        cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
        tmp = HOST_LIB.with_suffix(f".tmp{os.getpid()}.so")
        cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-pthread", "-I", str(CSRC), "-o", str(tmp),
               *map(str, srcs)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"g++ failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, HOST_LIB)  # atomic: a concurrent loader never sees a half-written file
        stamp.write_text(dig)
        if verbose:
            print(f"[tccl_b200.build] built {HOST_LIB}", file=sys.stderr)
    return HOST_LIB


def build_host_tsan(verbose: bool = False) -> Path:
    """The protocol self-test as a ThreadSanitizer-instrumented executable."""
    BUILD.mkdir(exist_ok=True)
    exe = BUILD / "hostproto_tsan"
    srcs = [CSRC / "host" / "host_protocol.cpp", CSRC / "host" / "selftest_main.cpp"]
    stamp = BUILD / "hostproto_tsan.sha"
    dig = _digest(srcs + headers(), "tsan")
    if not exe.exists() or not stamp.exists() or stamp.read_text() != dig:
        # not every toolchain ships libtsan: try the system compiler first, then $CXX
        errors = []
        for cxx in dict.fromkeys([shutil.which("g++", path="/usr/bin:/bin"), shutil.which("g++"), os.environ.get("CXX")]):
            if not cxx:
                continue
            cmd = [cxx, "-O1", "-g", "-std=c++17", "-fsanitize=thread", "-pthread", "-I", str(CSRC), "-o", str(exe),
                   *map(str, srcs)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode == 0:
                break
            errors.append(f"{cxx}: {r.stderr.strip()[-300:]}")
        else:
            raise RuntimeError("g++ -fsanitize=thread failed:\n" + "\n".join(errors))
        stamp.write_text(dig)
        if verbose:
            print(f"[tccl_b200.build] built {exe}", file=sys.stderr)
    return exe


def ptxas_table() -> str:
    """Registers, spills and static shared memory of every kernel, as ptxas reports them
    (``-Xptxas -v``), one markdown row per kernel template: the instance with the most registers."""
    import re
    import tempfile

    nvcc = _nvcc()
    rows = {}
    with tempfile.TemporaryDirectory() as tmp:
        for src in sources():
            cmd = [nvcc, *NVCC_FLAGS, "-Xptxas", "-v", "-I", str(CSRC), "-c", str(src), "-o", os.path.join(tmp, src.stem + ".o")]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stderr}")
            entry = None
            spill = (0, 0, 0)
            for line in r.stderr.splitlines():
                m = re.search(r"Compiling entry function '(\S+)'", line)
                if m:
                    entry = m.group(1)
                    continue
                m = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", line)
                if m:
                    spill = tuple(int(v) for v in m.groups())
                    continue
                m = re.search(r"Used (\d+) registers(?:, used (\d+) barriers)?(?:, (\d+) bytes cumulative stack size)?(?:, (\d+) bytes smem)?", line)
                if m and entry:
                    name = subprocess.run(["c++filt", entry], capture_output=True, text=True).stdout.strip() or entry
                    name = re.sub(r"\(.*$", "", name)                       # drop the parameter list
                    name = re.sub(r"^void ", "", name)
                    fam = re.sub(r"(?<=<)(.*)(?=>)", lambda mm: re.sub(r"\b\d+\b", "*", mm.group(1)), name)
                    fam = fam.replace("(__nv_bfloat16)", "").replace("tccl::", "")
                    fam = re.sub(r"__nv_bfloat16|__half|float", "T", fam)
                    regs, smem = int(m.group(1)), int(m.group(4) or 0)
                    cur = rows.get((src.name, fam))
                    if cur is None or regs > cur[0]:
                        rows[(src.name, fam)] = (regs, spill, smem, (cur[3] if cur else 0) + 1)
                    else:
                        rows[(src.name, fam)] = (cur[0], cur[1], cur[2], cur[3] + 1)
                    entry = None
    out = ["| source | kernel (template arguments folded) | instances | max registers | stack / spill st / spill ld (B) | static smem (B) |",
           "|---|---|---|---|---|---|"]
    for (src, fam), (regs, spill, smem, cnt) in sorted(rows.items()):
        out.append(f"| `{src}` | `{fam}` | {cnt} | {regs} | {spill[0]} / {spill[1]} / {spill[2]} | {smem} |")
    return "\n".join(out)


if __name__ == "__main__":
    if "--ptxas-table" in sys.argv:
        print(ptxas_table())
        sys.exit(0)
    build_host(verbose=True, force="--force" in sys.argv)
    build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    build(verbose=True, force="--force" in sys.argv, debug_checks=True)
