"""Numeric constants of the C ABI (flag-region layout, status words, error codes),
parsed out of ``csrc/tccl_b200.h`` so that Python cannot drift from the device
code.  Imports nothing heavy: the CPU-only tools use it without torch."""
from __future__ import annotations

import re
from pathlib import Path
from typing import Dict

PKG = Path(__file__).resolve().parent.parent
HEADER = PKG / "csrc" / "tccl_b200.h"


def _parse_header(path: Path) -> Dict[str, int]:
    text = re.sub(r"/\*.*?\*/", "", path.read_text(), flags=re.S)
    consts: Dict[str, int] = {}
    for m in re.finditer(r"^#define\s+(TCCL_\w+)\s+(.+)$", text, flags=re.M):
        name, expr = m.group(1), m.group(2).strip()
        try:
            consts[name] = int(eval(expr, {"__builtins__": {}}, consts))
        except Exception:
            pass
    for m in re.finditer(r"enum\s+\w+\s*\{(.*?)\}", text, flags=re.S):
        nxt = 0
        for item in m.group(1).split(","):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                k, v = (s.strip() for s in item.split("=", 1))
                nxt = int(eval(v, {"__builtins__": {}}, consts))
            else:
                k = item
            consts[k] = nxt
            nxt += 1
    return consts



K = _parse_header(HEADER)
MAX_WORLD = K["TCCL_MAX_WORLD"]
