"""Host-side checks that need no GPU: header constants, struct sizes, config."""
import ctypes as C

from tccl_b200.config import Config
from tccl_b200.utils import lib as L


def test_header_constants():
    K = L.K
    assert K["TCCL_MAX_WORLD"] == 8
    assert K["TCCL_FLAG_MCBAR"] == K["TCCL_MAX_BLOCKS"] * K["TCCL_MAX_WORLD"]
    assert K["TCCL_FLAG_WORDS"] > K["TCCL_FLAG_LL"] > K["TCCL_FLAG_TILE"] > K["TCCL_FLAG_TREE_DOWN"]
    assert K["TCCL_TIMEOUT"] == 1 and K["TCCL_ST_ABORT"] == 6


def test_struct_layout_matches_c():
    """Every ctypes mirror has the size the compiler gives the C struct."""
    lib = L.lib()
    lib.tccl_sizeof.argtypes = [C.c_char_p]
    pairs = {"tccl_comm": L.Comm, "tccl_coll_args": L.CollArgs, "tccl_launch": L.Launch,
             "tccl_barrier_args": L.BarrierArgs, "tccl_pads_args": L.PadsArgs, "tccl_tree_args": L.TreeArgs,
             "tccl_arn_args": L.ArnArgs, "tccl_gemm_args": L.GemmArgs, "tccl_gemm_rs_args": L.GemmRsArgs,
             "tccl_ag_gemm_args": L.AgGemmArgs}
    for name, mirror in pairs.items():
        assert lib.tccl_sizeof(name.encode()) == C.sizeof(mirror), name
    assert lib.tccl_sizeof(b"no_such_struct") == -1


def test_config_env(monkeypatch):
    monkeypatch.setenv("TCCL_TIMEOUT_MS", "250")
    monkeypatch.setenv("TCCL_DISABLE_NVLS", "1")
    monkeypatch.setenv("TCCL_MAX_CTAS", "32")
    c = Config.from_env()
    assert c.timeout_ms == 250.0 and c.disable_nvls is True and c.max_ctas == 32
    assert c.timeout_ns == 250_000_000


def test_library_builds_and_loads():
    lib = L.lib()
    assert lib.tccl_version() >= 100
    assert b"invalid" in lib.tccl_error_string(-L.K["TCCL_EINVAL"])
