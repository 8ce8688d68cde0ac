"""Catalog trie in device memory, in the three layouts the beam-step kernels read.

Built from an integer array of items ``[n_items, depth]`` (one code per level).
Node numbering, sentinels and the sorted-key CSR arrays are those of the
reference's ``BeamValidPathTrie`` (search/trie.py:160-343): root = 0, internal
prefixes numbered by (length, prefix) order, ``invalid_node = n_nodes`` (no
legal continuation), ``-1`` = unconstrained (a complete SID was reached); token
of (level l, code c) = ``token_base + sum(sizes[:l]) + c``; CSR key =
``node * vsz + (token - token_base)``.

Two builders give the same arrays: ``build_trie_arrays`` (host-side numpy sort / unique, any
layout afterwards) and ``build_trie_device`` (sort / unique / scan on the GPU, CSR layout only,
for catalogs of tens of millions of items). Neither walks Python dicts.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from flashrec_b200 import _lib
from flashrec_b200._lib import FrTrie


@dataclass
class TrieArrays:
    """Host arrays describing the trie (layout independent)."""

    sizes: list                 # codebook size per level
    token_base: int
    vsz: int                    # sum(sizes)
    n_nodes: int                # internal nodes incl. root; invalid_node == n_nodes
    level_start: np.ndarray     # [depth+1] first node id of each depth (depth L-1 nodes are the last internal ones)
    edge_parent: np.ndarray     # [E] int64 parent node id, ascending
    edge_rel: np.ndarray        # [E] int64 token - token_base
    edge_child: np.ndarray      # [E] int64 child node id, or -1 for leaves
    n_items: int
    max_children: Optional[list] = None  # per level: the largest number of children of a node of that depth

    @property
    def invalid_node(self) -> int:
        return int(self.n_nodes)

    @property
    def csr_keys(self) -> np.ndarray:
        return self.edge_parent * np.int64(self.vsz) + self.edge_rel


def build_trie_arrays(items: np.ndarray, sizes: Sequence[int], token_base: int) -> TrieArrays:
    """Sort-based trie construction. ``items`` is [n, L] with 0 <= items[:, l] < sizes[l]."""
    items = np.asarray(items, dtype=np.int64)
    if items.ndim != 2 or items.shape[1] != len(sizes):
        raise ValueError("items must be [n_items, len(sizes)]")
    L = len(sizes)
    sizes = [int(s) for s in sizes]
    if items.size and ((items < 0).any() or (items >= np.asarray(sizes)[None, :]).any()):
        raise ValueError("item code out of range for its level")
    offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    # lexicographic sort + dedup through one packed key (sizes are small enough for int64)
    packed = np.zeros(items.shape[0], dtype=np.int64)
    for l in range(L):
        packed = packed * np.int64(sizes[l]) + items[:, l]
    packed = np.unique(packed)
    n_items = int(packed.shape[0])
    # suffix radix: prefix key of length d = packed // prod(sizes[d:])
    tail = np.ones(L + 1, dtype=np.int64)
    for l in range(L - 1, -1, -1):
        tail[l] = tail[l + 1] * np.int64(sizes[l])
    prefix_keys = []  # unique prefix keys per length 0..L (sorted)
    for d in range(L + 1):
        pk = packed // tail[d] if d < L else packed
        prefix_keys.append(np.unique(pk) if d > 0 else np.zeros(1 if n_items else 1, dtype=np.int64))
    # node ids: depth d in [0, L-1] are internal nodes
    level_start = np.zeros(L + 1, dtype=np.int64)
    for d in range(L):
        level_start[d + 1] = level_start[d] + prefix_keys[d].shape[0]
    n_nodes = int(level_start[L])
    parents, rels, childs = [], [], []
    for d in range(L):  # edges from depth d to depth d+1
        ck = prefix_keys[d + 1]              # child prefixes (length d+1), sorted
        if n_items == 0:
            continue
        pk = ck // np.int64(sizes[d])        # their parent prefix key (length d)
        code = ck - pk * np.int64(sizes[d])
        pidx = np.searchsorted(prefix_keys[d], pk)
        parents.append(level_start[d] + pidx)
        rels.append(offs[d] + code)
        if d + 1 < L:
            childs.append(level_start[d + 1] + np.arange(ck.shape[0], dtype=np.int64))
        else:
            childs.append(np.full(ck.shape[0], -1, dtype=np.int64))
    cat = lambda xs: np.concatenate(xs) if xs else np.zeros(0, dtype=np.int64)  # noqa: E731
    edge_parent = cat(parents)
    deg = np.bincount(edge_parent, minlength=max(n_nodes, 1))
    max_children = [int(deg[level_start[d]: level_start[d + 1]].max(initial=0)) for d in range(L)]
    return TrieArrays(
        sizes=sizes,
        token_base=int(token_base),
        vsz=int(offs[-1]),
        n_nodes=n_nodes,
        level_start=level_start,
        edge_parent=edge_parent,
        edge_rel=cat(rels),
        edge_child=cat(childs),
        n_items=n_items,
        max_children=max_children,
    )


@dataclass
class DeviceTrie:
    """One device-resident layout of a catalog trie + its ``fr_trie`` descriptor."""

    kind: int
    arrays: TrieArrays
    device: torch.device
    tensors: dict = field(default_factory=dict)

    @property
    def token_base(self) -> int:
        return self.arrays.token_base

    @property
    def vsz(self) -> int:
        return self.arrays.vsz

    @property
    def invalid_node(self) -> int:
        return self.arrays.invalid_node

    @property
    def n_nodes(self) -> int:
        return self.arrays.n_nodes

    def descriptor(self) -> FrTrie:
        t = self.tensors
        tr = FrTrie()
        tr.kind = self.kind
        tr.vsz = self.arrays.vsz
        tr.token_base = self.arrays.token_base
        tr.invalid_node = self.arrays.invalid_node
        if self.kind == _lib.FR_TRIE_DENSE:
            tr.allow = t["allow"].data_ptr()
            tr.next = t["next"].data_ptr()
            tr.next_is_i32 = 1
            tr.n_rows = int(t["allow"].shape[0])
        elif self.kind == _lib.FR_TRIE_CSR:
            tr.csr_keys = t["keys"].data_ptr() if t["keys"].numel() else None
            tr.csr_child = t["child"].data_ptr() if t["child"].numel() else None
            tr.n_edges = int(t["keys"].numel())
        elif self.kind == _lib.FR_TRIE_BITMAP:
            tr.bitmap = t["bitmap"].data_ptr()
            tr.child_base = t["child_base"].data_ptr()
            tr.level_off = t["level_off"].data_ptr()
            tr.words_per_node = int(t["bitmap"].shape[1])
            tr.n_rows = int(t["bitmap"].shape[0])
        return tr

    def nbytes(self) -> int:
        return sum(int(v.numel()) * v.element_size() for v in self.tensors.values())

    def candidate_bound(self, level: int, beam_width: int) -> int:
        """Upper bound on the legal continuations of ``beam_width`` beams at ``level`` (beams of a request sit on
        distinct nodes): beam_width x the largest fan-out of that depth, never more than the nodes (items, at the
        last level) one level down, nor than beam_width x the level's width."""
        a = self.arrays
        L = len(a.sizes)
        below = int(a.level_start[level + 2] - a.level_start[level + 1]) if level + 1 < L else int(a.n_items)
        fan = a.max_children[level] if a.max_children else a.sizes[level]
        return max(1, min(int(beam_width) * int(fan), max(below, int(fan)), int(beam_width) * int(a.sizes[level])))


def trie_to_device(arrays: TrieArrays, layout: str, device) -> DeviceTrie:
    """``layout`` in {"dense", "csr", "bitmap"}.

    dense  : allow u8 / next i32 ``[n_nodes+1, vsz]`` (reference layout; small tries only)
    csr    : sorted keys / child int64 ``[E]`` (reference layout)
    bitmap : per-node bitmap over the node's own level, u32 ``[n_nodes+1, max(sizes)/32]``,
             plus ``level_off`` i32 and ``child_base`` i64 per node
    """
    device = torch.device(device)
    a = arrays
    if layout == "csr":
        keys = torch.from_numpy(a.csr_keys.astype(np.int64)).to(device)
        child = torch.from_numpy(a.edge_child.astype(np.int64)).to(device)
        return DeviceTrie(_lib.FR_TRIE_CSR, a, device, {"keys": keys, "child": child})
    if layout == "dense":
        rows = a.n_nodes + 1
        if rows * a.vsz > (1 << 31):
            raise ValueError("dense trie too large; use 'bitmap' or 'csr'")
        allow = np.zeros((rows, a.vsz), dtype=np.uint8)
        nxt = np.full((rows, a.vsz), a.invalid_node, dtype=np.int32)
        allow[a.edge_parent, a.edge_rel] = 1
        nxt[a.edge_parent, a.edge_rel] = a.edge_child.astype(np.int32)
        return DeviceTrie(
            _lib.FR_TRIE_DENSE, a, device,
            {"allow": torch.from_numpy(allow).to(device), "next": torch.from_numpy(nxt).to(device)},
        )
    if layout == "bitmap":
        rows = a.n_nodes + 1
        words = (max(a.sizes) + 31) // 32
        offs = np.concatenate([[0], np.cumsum(a.sizes)]).astype(np.int64)
        depth_of = np.zeros(rows, dtype=np.int64)
        L = len(a.sizes)
        for d in range(L):
            depth_of[a.level_start[d]: a.level_start[d + 1]] = d
        depth_of[a.n_nodes] = 0
        level_off = offs[depth_of].astype(np.int32)
        code = a.edge_rel - offs[depth_of[a.edge_parent]]
        bitmap = np.zeros((rows, words), dtype=np.uint32)
        np.bitwise_or.at(bitmap, (a.edge_parent, code >> 5), (np.uint32(1) << (code & 31).astype(np.uint32)))
        child_base = np.full(rows, -1, dtype=np.int64)
        if a.edge_parent.size:
            first = np.ones(a.edge_parent.shape[0], dtype=bool)
            first[1:] = a.edge_parent[1:] != a.edge_parent[:-1]
            child_base[a.edge_parent[first]] = a.edge_child[first]
        return DeviceTrie(
            _lib.FR_TRIE_BITMAP, a, device,
            {
                "bitmap": torch.from_numpy(bitmap.view(np.int32)).to(device),
                "child_base": torch.from_numpy(child_base).to(device),
                "level_off": torch.from_numpy(level_off).to(device),
            },
        )
    raise ValueError(f"unknown trie layout {layout!r}")


def build_trie_device(items: torch.Tensor, sizes: Sequence[int], token_base: int, layout: str = "csr") -> DeviceTrie:
    """Trie of the catalog ``items`` (int32 ``[n_items, depth]``, on the GPU) built on the GPU, in the
    ``"csr"`` or the ``"bitmap"`` layout (the latter derived from the CSR arrays on the device):
    the device-side stand-in for ``BeamValidPathTrie._ensure_gpu_cache`` / ``_build_csr_cache``
    (search/trie.py:222-251, 300-327). Same node numbering, keys and children as
    ``build_trie_arrays`` + ``trie_to_device(.., "csr")``. One host read (the counts) at the end."""
    import ctypes

    from flashrec_b200._lib import call, load, ptr, require_cuda, stream_ptr

    require_cuda(items)
    if items.dim() != 2 or items.shape[1] != len(sizes) or items.dtype != torch.int32:
        raise ValueError("items must be an int32 [n_items, len(sizes)] tensor")
    items = items.contiguous()
    dev = items.device
    n, depth = int(items.shape[0]), len(sizes)
    sizes = [int(x) for x in sizes]
    need = int(load().fr_trie_build_workspace_bytes(n))
    if need < 0:
        raise ValueError("catalog too large for one build (n_items must be below 2^31)")
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    cap = max(n * depth, 1)
    keys = torch.empty(cap, dtype=torch.int64, device=dev)
    child = torch.empty(cap, dtype=torch.int64, device=dev)
    counts = torch.zeros(3 + 2 * (depth + 1), dtype=torch.int64, device=dev)
    c_sizes = (ctypes.c_int64 * depth)(*sizes)
    call("fr_trie_build_csr", ptr(items), n, depth, ctypes.cast(c_sizes, ctypes.c_void_p), ptr(keys), ptr(child), cap,
         ptr(counts), ptr(ws), need, stream_ptr(dev))
    c = counts.cpu().numpy()
    if c[0] < 0:
        raise ValueError("item code out of range for its level")
    n_edges = int(c[2])
    level_start = c[3: 3 + depth + 1].copy()
    if n == 0:
        level_start[1:] = 1
    empty = np.zeros(0, dtype=np.int64)
    # the largest fan-out per depth (sizes the candidate lists of the fused head): one more small host read
    max_children = [0] * depth
    if n_edges > 0:
        deg = torch.bincount(keys[:n_edges] // int(sum(sizes)), minlength=max(int(c[1]), 1))
        max_children = [int(deg[int(level_start[d]): int(level_start[d + 1])].max().item())
                        if level_start[d + 1] > level_start[d] else 0 for d in range(depth)]
        del deg
    arrays = TrieArrays(sizes=sizes, token_base=int(token_base), vsz=int(sum(sizes)), n_nodes=int(c[1]),
                        level_start=level_start, edge_parent=empty, edge_rel=empty, edge_child=empty,
                        n_items=int(c[0]), max_children=max_children)
    if layout == "bitmap":
        rows, words = arrays.n_nodes + 1, (max(sizes) + 31) // 32
        bitmap = torch.empty((rows, words), dtype=torch.int32, device=dev)
        child_base = torch.empty(rows, dtype=torch.int64, device=dev)
        level_off = torch.empty(rows, dtype=torch.int32, device=dev)
        c_start = (ctypes.c_int64 * (depth + 1))(*[int(x) for x in level_start])
        call("fr_trie_csr_to_bitmap", ptr(keys), ptr(child), n_edges, depth, ctypes.cast(c_sizes, ctypes.c_void_p),
             ctypes.cast(c_start, ctypes.c_void_p), ptr(bitmap), ptr(child_base), ptr(level_off), words,
             stream_ptr(dev))
        return DeviceTrie(_lib.FR_TRIE_BITMAP, arrays, dev,
                          {"bitmap": bitmap, "child_base": child_base, "level_off": level_off})
    if layout != "csr":
        raise ValueError(f"unknown device-built trie layout {layout!r}")
    # trimmed copies so that the build's capacity-sized buffers are released
    return DeviceTrie(_lib.FR_TRIE_CSR, arrays, dev, {"keys": keys[:n_edges].clone(), "child": child[:n_edges].clone()})
