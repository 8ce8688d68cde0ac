"""Catalog files <-> the ``[items, levels]`` int32 array the trie builders take.

The reference keeps a catalog as one JSON object whose keys are the items' code paths, ``{"a,b,c": 1, ...}``
(written by ``catalog.py:173-188``; read key by key into Python tuples and dicts by ``search/trie.py``), or, in
RecIF's source files, as packed integers ``a * base^2 + b * base + c`` (``catalog.py:38-48``). Here the keys go
straight into one integer matrix (numpy; sorted, duplicates removed), which ``trie.build_trie_device`` turns into
the CSR / bitmap trie on the GPU without a Python object per item.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import numpy as np

DEFAULT_BASE = 8192


def parse_sid_keys(keys, levels: Optional[int] = None, base: int = DEFAULT_BASE) -> np.ndarray:
    """Item matrix ``[items, levels]`` (int32, rows sorted, unique) from catalog keys: ``"a,b,c"`` paths or
    packed integers (unpacked most significant code first, depth ``levels`` or the smallest depth >= 3 that holds
    the largest key). Keys that do not parse, have another depth, or hold a code outside ``[0, base)`` are dropped
    (the reference counts them as bad keys, ``catalog.py:94-132``)."""
    comma, packed = [], []
    for k in keys:
        text = str(k).strip()
        if "," in text:
            comma.append(text)
        else:
            try:
                packed.append(int(text))
            except ValueError:
                pass
    mats = []
    if packed:
        vals = [p for p in packed if p >= 0]
        depth = 3
        if levels is not None and not comma:
            depth = int(levels)
        else:
            top = max(vals, default=0)
            while top >= base ** depth:
                depth += 1
        rows = [[(v // base ** (depth - 1 - d)) % base for d in range(depth)] for v in vals if v < base ** depth]
        mats.append(np.asarray(rows, dtype=np.int64).reshape(-1, depth))
    if comma:
        rows = []
        for text in comma:
            parts = [p.strip() for p in text.split(",") if p.strip()]
            try:
                codes = [int(p) for p in parts]
            except ValueError:
                continue
            if codes and all(0 <= c < base for c in codes):
                rows.append(codes)
        by_depth = {}
        for r in rows:
            by_depth.setdefault(len(r), []).append(r)
        for d, rs in by_depth.items():
            mats.append(np.asarray(rs, dtype=np.int64))
    if levels is None:
        depths = sorted({m.shape[1] for m in mats if len(m)})
        if not depths:
            raise ValueError("no valid SID keys")
        if len(depths) != 1:
            raise ValueError(f"mixed SID depths {depths}; pass levels")
        levels = depths[0]
    mats = [m for m in mats if m.shape[1] == levels and len(m)]
    if not mats:
        return np.zeros((0, levels), dtype=np.int32)
    items = np.unique(np.concatenate(mats, axis=0), axis=0)  # lexicographic row order
    return items.astype(np.int32)


def read_sid_catalog(path, levels: Optional[int] = None, base: int = DEFAULT_BASE) -> np.ndarray:
    """The catalog file at ``path`` (a JSON object of SID keys) as an item matrix; see ``parse_sid_keys``."""
    data = json.loads(Path(path).read_text(encoding="utf-8"))
    if not isinstance(data, dict):
        raise ValueError("catalog JSON root must be an object of SID keys")
    return parse_sid_keys(data.keys(), levels=levels, base=base)


def write_sid_catalog(items, path) -> None:
    """Write the item matrix as ``{"a,b,c":1,...}``, the form the reference's ``--sid-vocab-file`` reads."""
    items = np.asarray(items)
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with path.open("w", encoding="utf-8") as f:
        f.write("{")
        f.write(",".join('"' + ",".join(str(int(c)) for c in row) + '":1' for row in items))
        f.write("}")
