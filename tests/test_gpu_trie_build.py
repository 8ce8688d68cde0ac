"""Catalog trie built on the GPU (through the C ABI) against the reference's tables (golden fixture),
against the host builder on random catalogs, and at the sizes of the baseline configurations
(1M items x 3 levels of 8192; 10M Zipf-skewed items x 4 levels of 4096) through properties."""

import time

import numpy as np
import pytest
import torch

from conftest import load_golden
from flashrec_b200.trie import build_trie_arrays

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _build(items, sizes, base):
    from flashrec_b200.trie import build_trie_device

    return build_trie_device(torch.from_numpy(np.ascontiguousarray(items, dtype=np.int32)).to(DEV), sizes, base)


def test_device_builder_reproduces_reference_csr_table():
    g = load_golden("trie")
    t = _build(g["items"], g["sizes"].tolist(), int(g["base"]))
    assert t.n_nodes == int(g["n_nodes"]) and t.invalid_node == int(g["invalid"])
    assert np.array_equal(t.tensors["keys"].cpu().numpy(), g["csr_keys"])
    assert np.array_equal(t.tensors["child"].cpu().numpy(), g["csr_child"])


@pytest.mark.parametrize("n,sizes", [(50_000, [256, 256, 256]), (3000, [7, 300]), (1, [5, 5, 5, 5]), (20_000, [4096]),
                                     (100_000, [16, 8, 4, 4, 2, 3])])
def test_device_builder_equals_host_builder(n, sizes):
    rng = np.random.default_rng(n + len(sizes))
    items = np.stack([rng.integers(0, s, n) for s in sizes], 1)  # with duplicates
    a = build_trie_arrays(items, sizes, 151_936)
    t = _build(items, sizes, 151_936)
    assert (t.arrays.n_items, t.n_nodes, t.vsz) == (a.n_items, a.n_nodes, a.vsz)
    assert np.array_equal(t.arrays.level_start, a.level_start)
    assert np.array_equal(t.tensors["keys"].cpu().numpy(), a.csr_keys)
    assert np.array_equal(t.tensors["child"].cpu().numpy(), a.edge_child)


def test_device_builder_empty_and_bad_codes():
    t = _build(np.zeros((0, 3), dtype=np.int32), [8, 8, 8], 100)
    assert t.n_nodes == 1 and t.tensors["keys"].numel() == 0 and t.arrays.level_start.tolist() == [0, 1, 1, 1]
    with pytest.raises(ValueError):
        _build(np.array([[1, 2, 8]]), [8, 8, 8], 100)  # code 8 is outside a level of 8
    with pytest.raises(ValueError):
        _build(np.array([[1, -1, 0]]), [8, 8, 8], 100)


def test_device_trie_drives_the_beam_step_like_the_host_built_one():
    from flashrec_b200.logits import RestrictedLMHead  # noqa: F401  (same import path as the engine)
    from flashrec_b200.sid_decode import sid_beam_step
    from flashrec_b200.trie import trie_to_device

    rng = np.random.default_rng(4)
    sizes, base, bw = [64, 64, 64], 1000, 32
    items = np.stack([rng.integers(0, 64, 3000) for _ in sizes], 1)
    host = trie_to_device(build_trie_arrays(items, sizes, base), "csr", DEV)
    dev = _build(items, sizes, base)
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(2 * bw, 64, generator=g).to(DEV)
    mx, ls = logits.max(dim=1).values, torch.logsumexp(logits - logits.max(dim=1, keepdim=True).values, dim=1)
    cum = torch.full((2, bw), float("-inf"), device=DEV)
    cum[:, 0] = 0
    nodes = torch.zeros((2, bw), dtype=torch.int64, device=DEV)
    a = sid_beam_step(cum, logits, mx, ls, nodes, host, base, bw)
    b = sid_beam_step(cum, logits, mx, ls, nodes, dev, base, bw)
    assert torch.equal(a.vals, b.vals) and torch.equal(a.tokens, b.tokens) and torch.equal(a.child, b.child)


@pytest.mark.parametrize("name,n,sizes,zipf", [("config 3/4", 1_000_000, [8192] * 3, False),
                                               ("config 5", 10_000_000, [4096] * 4, True)])
def test_device_builder_at_baseline_sizes(name, n, sizes, zipf):
    rng = np.random.default_rng(0)
    L = len(sizes)
    if zipf:  # levels 1-2 Zipf(1.1) rank-truncated to the level size, the rest uniform
        cols = [np.minimum(rng.zipf(1.1, n) - 1, sizes[l] - 1) if l < 2 else rng.integers(0, sizes[l], n)
                for l in range(L)]
    else:
        cols = [rng.integers(0, sizes[l], n) for l in range(L)]
    items = np.stack(cols, 1).astype(np.int32)
    d_items = torch.from_numpy(items).to(DEV)
    from flashrec_b200.trie import build_trie_device

    build_trie_device(d_items[:1000], sizes, 151_936)  # warm-up
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    t = build_trie_device(d_items, sizes, 151_936)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    print(f"{name}: {n} items -> {t.n_nodes} nodes, {t.tensors['keys'].numel()} edges in {dt * 1e3:.1f} ms on the GPU")
    keys, child = t.tensors["keys"], t.tensors["child"]
    assert bool((keys[1:] > keys[:-1]).all())  # strictly ascending: searchsorted-ready, no duplicate edge
    # properties that pin the structure at any size: distinct items = leaf edges; walking a sample of
    # items from the root finds every edge and ends in a leaf
    packed = np.zeros(n, dtype=np.int64)
    for l in range(L):
        packed = packed * sizes[l] + items[:, l]
    assert t.arrays.n_items == np.unique(packed).shape[0] == int((child == -1).sum())
    sample = torch.from_numpy(items[rng.integers(0, n, 20_000)].astype(np.int64)).to(DEV)
    offs = np.concatenate([[0], np.cumsum(sizes)])
    node = torch.zeros(sample.shape[0], dtype=torch.int64, device=DEV)
    for l in range(L):
        want = node * t.vsz + int(offs[l]) + sample[:, l]
        pos = torch.searchsorted(keys, want)
        assert bool((keys[pos] == want).all())
        node = child[pos]
        assert bool((node >= 0).all()) if l + 1 < L else bool((node == -1).all())
    assert int(t.arrays.level_start[-1]) == t.n_nodes


@pytest.mark.parametrize("n,sizes", [(50_000, [256, 256, 256]), (3000, [7, 300]), (0, [8, 8]), (200_000, [8192, 8192, 8192])])
def test_device_bitmap_layout_equals_host_built_one(n, sizes):
    from flashrec_b200.trie import build_trie_device, trie_to_device

    rng = np.random.default_rng(n + 7)
    items = np.stack([rng.integers(0, s, n) for s in sizes], 1).astype(np.int32).reshape(n, len(sizes))
    host = trie_to_device(build_trie_arrays(items, sizes, 1000), "bitmap", DEV)
    dev = build_trie_device(torch.from_numpy(items).to(DEV), sizes, 1000, layout="bitmap")
    assert dev.n_nodes == host.n_nodes and dev.kind == host.kind
    for name in ("bitmap", "child_base", "level_off"):
        assert torch.equal(dev.tensors[name], host.tensors[name]), name
