import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


def _n_gpus() -> int:
    try:
        import torch

        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def pytest_collection_modifyitems(config, items):
    n = _n_gpus()
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for item in items:
        if "gpu" in item.keywords and n == 0:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and n < 2:
            item.add_marker(skip_multi)


@pytest.fixture(scope="session")
def emu_worlds():
    """Emulated worlds are cached per size for the whole session (their flag
    regions and staging areas are device allocations worth reusing)."""
    from tccl_b200.config import Config
    from tccl_b200.parallel.emu import EmuWorld

    cache = {}

    def get(W: int):
        if W not in cache:
            cfg = Config.from_env()
            cfg.stage_mb = 64
            cfg.timeout_ms = 2000.0
            cache[W] = EmuWorld(W, config=cfg)
        return cache[W]

    return get
