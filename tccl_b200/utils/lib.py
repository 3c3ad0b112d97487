"""ctypes binding of ``libtccl_b200.so``.

The structs mirror ``csrc/tccl_b200.h``; the numeric constants (flag-region
layout, status words, error codes) are parsed out of that header so that the
Python side cannot drift from the device code.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

PKG = Path(__file__).resolve().parent.parent
# TCCL_DEBUG_CHECKS=1 selects the library flavour whose flat-collective kernels check every vector
# offset against the extents passed by the host (utils/build.py builds both)
DEBUG_CHECKS = os.environ.get("TCCL_DEBUG_CHECKS", "") not in ("", "0")
LIB_PATH = PKG / "_lib" / ("libtccl_b200_dbg.so" if DEBUG_CHECKS else "libtccl_b200.so")


from .consts import K, MAX_WORLD  # noqa: E402,F401  (parsed from csrc/tccl_b200.h)


class Comm(C.Structure):
    _fields_ = [
        ("world", C.c_int32),
        ("rank", C.c_int32),
        ("flags", C.c_uint64 * MAX_WORLD),
        ("mc_flags", C.c_uint64),
        ("local", C.c_uint64),
        ("stage", C.c_uint64 * MAX_WORLD),
        ("mc_stage", C.c_uint64),
        ("stage_bytes", C.c_uint64),
        ("timeout_ns", C.c_uint64),
        ("ll_bytes", C.c_uint64),
        ("tree_bytes", C.c_uint64),
    ]


class CollArgs(C.Structure):
    _fields_ = [
        ("inp", C.c_uint64 * MAX_WORLD),
        ("mc_in", C.c_uint64),
        ("out", C.c_uint64),
        ("out_peer", C.c_uint64 * MAX_WORLD),
        ("mc_out", C.c_uint64),
        ("numel", C.c_uint64),
        ("dtype", C.c_int32),
        ("flags", C.c_int32),
        ("in_bytes", C.c_uint64),
        ("out_bytes", C.c_uint64),
    ]


class BarrierArgs(C.Structure):
    _fields_ = [("rounds", C.c_int32)]


class PadsArgs(C.Structure):
    _fields_ = [("pads", C.c_uint64 * MAX_WORLD)]


class TreeArgs(C.Structure):
    _fields_ = [
        ("inp", C.c_uint64),
        ("buf", C.c_uint64 * MAX_WORLD),
        ("out", C.c_uint64),
        ("numel", C.c_uint64),
        ("chunk_vecs", C.c_uint64),
        ("dtype", C.c_int32),
        ("ctas_per_role", C.c_int32),
        ("parent", C.c_int32 * 2),
        ("left", C.c_int32 * 2),
        ("right", C.c_int32 * 2),
        ("child_slot", C.c_int32 * 2),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_uint64), ("bt", C.c_uint64), ("c", C.c_uint64), ("status", C.c_uint64),
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
        ("lda", C.c_int32), ("ldb", C.c_int32), ("ldc", C.c_int32),
    ]


class GemmRsArgs(C.Structure):
    _fields_ = [
        ("a", C.c_uint64), ("bt", C.c_uint64), ("out", C.c_uint64),
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
        ("lda", C.c_int32), ("ldb", C.c_int32), ("ldo", C.c_int32),
        ("trace", C.c_uint64),
    ]


class AgGemmArgs(C.Structure):
    _fields_ = [
        ("a_shard", C.c_uint64), ("a_full", C.c_uint64 * MAX_WORLD), ("mc_a_full", C.c_uint64),
        ("bt", C.c_uint64), ("out", C.c_uint64),
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
        ("lda_shard", C.c_int32), ("lda_full", C.c_int32), ("ldb", C.c_int32), ("ldo", C.c_int32),
        ("comm_ctas", C.c_int32), ("swiglu", C.c_int32),
        ("trace", C.c_uint64), ("lsu_movers", C.c_int32), ("sched_stride", C.c_int32), ("sched", C.c_uint64),
    ]


class ArnArgs(C.Structure):
    _fields_ = [
        ("x", C.c_uint64 * MAX_WORLD), ("mc_x", C.c_uint64),
        ("out", C.c_uint64 * MAX_WORLD), ("mc_out", C.c_uint64),
        ("res_out", C.c_uint64 * MAX_WORLD), ("mc_res_out", C.c_uint64),
        ("bias", C.c_uint64), ("residual", C.c_uint64), ("weight", C.c_uint64),
        ("eps", C.c_float), ("tokens", C.c_int32), ("hidden", C.c_int32),
        ("dtype", C.c_int32), ("flags", C.c_int32),
    ]


class Launch(C.Structure):
    _fields_ = [
        ("grid", C.c_int32),
        ("block", C.c_int32),
        ("n_emu", C.c_int32),
        ("meta", C.c_int32),
        ("stream", C.c_void_p),
    ]


DTYPES = {torch.bfloat16: K["TCCL_BF16"], torch.float32: K["TCCL_F32"], torch.float16: K["TCCL_F16"]}

_lib = None


class TcclError(RuntimeError):
    """A launcher rejected its arguments or CUDA refused the launch."""


class TcclTimeout(RuntimeError):
    """A device-side wait ran out; carries the decoded status words."""

    def __init__(self, status: dict):
        super().__init__(f"device wait gave up: {status}")
        self.status = status


def lib() -> C.CDLL:
    """Load the shared library (building it first if it is missing and nvcc is
    there).  On a machine with a GPU a missing library is an error, never a
    silent fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists() or os.environ.get("TCCL_REBUILD") == "1":
        from . import build as _build

        _build.build(debug_checks=DEBUG_CHECKS)
    _lib = C.CDLL(str(LIB_PATH))
    _lib.tccl_error_string.restype = C.c_char_p
    _lib.tccl_error_string.argtypes = [C.c_int]
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().tccl_error_string(code).decode()
        raise TcclError(f"{what}: {msg} (code {code})")
