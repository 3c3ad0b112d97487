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
    # 2 x int32 + 8 ptr + ptr + ptr + 8 ptr + ptr + 2 x u64
    assert C.sizeof(L.Comm) == 8 + 8 * 8 + 8 + 8 + 8 * 8 + 8 + 16
    assert C.sizeof(L.CollArgs) == 8 * 8 + 8 + 8 + 8 * 8 + 8 + 8 + 8
    assert C.sizeof(L.Launch) == 24


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
