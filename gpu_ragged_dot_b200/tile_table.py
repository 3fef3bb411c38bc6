"""Committed per-shape tile table: the replacement for the reference's run-time tune-jax
search over block_m/block_k/block_n (tuning.py:49-58).

``tile_table.json`` holds one entry per tuned shape:
    {"op": "gmm" | "gmm_t" | "tgmm", "k": K, "n": N, "g": G, "m_min": a, "m_max": b,
     "tile_n": 64 | 128 | 256, "max_ctas": 0, "cta_group": 0 | 1 | 2, "tile_m": 0 | 128 | 256}
``lookup`` returns the matching ``TileCfg`` or ``None``; with ``None`` the library falls back
to its built-in choice (widest tile that still fills the persistent grid).  Set the
environment variable ``RD_TILE_TABLE`` to use another file.
"""

from __future__ import annotations

import json
import os
from typing import Optional

from . import _lib

_TABLE_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tile_table.json")
_entries = None


def _load():
    global _entries
    if _entries is None:
        path = os.environ.get("RD_TILE_TABLE", _TABLE_PATH)
        with open(path) as f:
            _entries = json.load(f)["entries"]
    return _entries


def lookup(op: str, m: int, k: int, n: int, g: int) -> Optional[_lib.TileCfg]:
    for e in _load():
        if (
            e["op"] == op
            and e["k"] == k
            and e["n"] == n
            and e["g"] == g
            and e.get("m_min", 0) <= m <= e.get("m_max", 1 << 62)
        ):
            return _lib.TileCfg(int(e["tile_n"]), int(e.get("max_ctas", 0)), int(e.get("cta_group", 0)),
                                int(e.get("tile_m", 0)), 0)
    return None
