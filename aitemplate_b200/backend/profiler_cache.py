"""Cache of profiled GEMM launch configurations.

The reference keeps the winners of its compile-time kernel profiling in a database keyed by the op's
configuration and problem size (python/aitemplate/backend/profiler_cache.py:479-560) so that a shape is
profiled once. Here a "configuration" is what the library lets a caller choose per launch: the tile width
(64 / 128 / 256 columns on one CTA, or 512 = 256 x 256 tiles on CTA pairs) and the split-K limit. The cache
is one JSON file: $AIT_B200_CACHE_DIR/gemm_profile_cache.json (default ~/.aitemplate_b200).
"""
from __future__ import annotations

import json
import os
import tempfile
from typing import Dict, Optional, Tuple

CACHE_VERSION = 1


def default_cache_path() -> str:
    root = os.environ.get("AIT_B200_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".aitemplate_b200")
    return os.path.join(root, "gemm_profile_cache.json")


def gemm_key(op_name: str, dtype: str, m: int, n: int, k: int, layout: str = "", device: str = "") -> str:
    return "|".join([op_name, dtype, str(int(m)), str(int(n)), str(int(k)), layout or "-", device or "-"])


class GemmProfileCache:
    """{key: {"tile_n": int, "split_k": int, "us": float}} with atomic saves."""

    def __init__(self, path: Optional[str] = None) -> None:
        self.path = path or default_cache_path()
        self.entries: Dict[str, Dict] = {}
        self.load()

    def load(self) -> None:
        try:
            with open(self.path) as f:
                blob = json.load(f)
            if blob.get("version") == CACHE_VERSION:
                self.entries = dict(blob.get("entries", {}))
        except (OSError, ValueError):
            self.entries = {}

    def save(self) -> None:
        os.makedirs(os.path.dirname(self.path) or ".", exist_ok=True)
        fd, tmp = tempfile.mkstemp(dir=os.path.dirname(self.path) or ".", suffix=".tmp")
        with os.fdopen(fd, "w") as f:
            json.dump({"version": CACHE_VERSION, "entries": self.entries}, f, indent=1, sort_keys=True)
        os.replace(tmp, self.path)

    def lookup(self, key: str) -> Optional[Tuple[int, int]]:
        e = self.entries.get(key)
        return (int(e["tile_n"]), int(e["split_k"])) if e else None

    def insert(self, key: str, tile_n: int, split_k: int, us: float) -> None:
        self.entries[key] = {"tile_n": int(tile_n), "split_k": int(split_k), "us": float(us)}
