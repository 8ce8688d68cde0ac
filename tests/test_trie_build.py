"""Host-side trie construction against the reference's tables (golden) and its
own invariants."""

import numpy as np

from conftest import load_golden
from flashrec_b200.trie import build_trie_arrays


def test_builder_reproduces_reference_csr_and_dense_tables():
    g = load_golden("trie")
    a = build_trie_arrays(g["items"], g["sizes"].tolist(), int(g["base"]))
    assert a.n_nodes == int(g["n_nodes"]) and a.invalid_node == int(g["invalid"])
    assert np.array_equal(a.csr_keys, g["csr_keys"])
    assert np.array_equal(a.edge_child, g["csr_child"])
    allow = np.zeros_like(g["allow"])
    allow[a.edge_parent, a.edge_rel] = True
    assert np.array_equal(allow, g["allow"])


def test_builder_properties_on_a_larger_catalog():
    rng = np.random.default_rng(0)
    sizes = [256, 256, 256]
    items = rng.integers(0, 256, (50_000, 3))
    a = build_trie_arrays(items, sizes, 151_936)
    uniq = np.unique(items, axis=0)
    assert a.n_items == uniq.shape[0]
    keys = a.csr_keys
    assert (np.diff(keys) > 0).all()  # strictly sorted, no duplicate edges
    # walking every item from the root reaches a leaf (-1)
    node = np.zeros(uniq.shape[0], dtype=np.int64)
    offs = np.concatenate([[0], np.cumsum(sizes)])
    for l in range(3):
        pos = np.searchsorted(keys, node * a.vsz + offs[l] + uniq[:, l])
        assert (keys[pos] == node * a.vsz + offs[l] + uniq[:, l]).all()
        node = a.edge_child[pos]
    assert (node == -1).all()
    # number of edges = distinct prefixes of every length
    n_edges = sum(np.unique(uniq[:, : l + 1], axis=0).shape[0] for l in range(3))
    assert keys.shape[0] == n_edges


def test_empty_and_single_item_catalogs():
    a = build_trie_arrays(np.zeros((0, 2), dtype=np.int64), [4, 4], 10)
    assert a.n_items == 0 and a.csr_keys.shape[0] == 0
    b = build_trie_arrays(np.array([[3, 1]]), [4, 4], 10)
    assert b.n_nodes == 2 and b.csr_keys.tolist() == [3, 1 * 8 + 4 + 1] and b.edge_child.tolist() == [1, -1]
