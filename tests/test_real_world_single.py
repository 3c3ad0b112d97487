"""RealWorld code paths and the TP MLP block on a one-rank process group (one GPU)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_one_rank_real_world():
    r = subprocess.run([sys.executable, os.path.join(HERE, "real_world_single.py")], capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0 and "real_world_single: ok" in r.stdout, (r.stdout + r.stderr)[-3000:]
