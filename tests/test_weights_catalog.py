"""Host logic around the path: checkpoint merging / config reading (models/weight.py) and the catalog key
format (catalog.py), against the reference's own functions where the reference is installed under
``oracle/_ref``, and against hand-written expectations everywhere."""

import json
import sys

import numpy as np
import pytest
import torch

import refshim

FP8 = torch.float8_e4m3fn


def _ref(module):
    if not refshim.available():
        return None
    if str(refshim.REF_DIR) not in sys.path:
        sys.path.insert(0, str(refshim.REF_DIR))
    import importlib

    return importlib.import_module(module)


def test_merge_qkv_and_gate_up_keep_rows_and_scales_in_order():
    from flashrec_b200.weights import merge_gate_up_weights, merge_qkv_weights

    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(n, 8, generator=g) for n in (6, 4, 4))
    sq, sk, sv = torch.rand(6, 1, generator=g), torch.rand(4, generator=g), torch.rand(1, generator=g)
    w, s = merge_qkv_weights(q, k, v, sq, sk, sv)
    assert torch.equal(w, torch.cat([q, k, v])) and s.shape == (14,)
    assert torch.equal(s, torch.cat([sq.reshape(-1), sk, sv.expand(4)]))
    assert merge_qkv_weights(q, k, v, sq, None, sv)[1] is None  # a scale only when all three bring one
    with pytest.raises(ValueError):
        merge_qkv_weights(q, k[:, :4], v)
    gate, up = torch.randn(5, 8, generator=g), torch.randn(5, 8, generator=g)
    w, s = merge_gate_up_weights(gate, up, torch.rand(5, generator=g), torch.rand(5, 1, generator=g))
    assert torch.equal(w, torch.cat([gate, up])) and s.shape == (10,)
    with pytest.raises(ValueError):
        merge_gate_up_weights(gate, up[:4])
    # e4m3 matrices are concatenated byte for byte, never requantised
    g8, u8 = gate.to(FP8), up.to(FP8)
    w8, _ = merge_gate_up_weights(g8, u8)
    assert w8.dtype == FP8 and torch.equal(w8.view(torch.uint8), torch.cat([g8.view(torch.uint8), u8.view(torch.uint8)]))
    ref = _ref("flashrec.models.weight")
    if ref is not None:
        rw, rs = ref.merge_qkv_weights(q, k, v, sq, sk, sv)
        mw, ms = merge_qkv_weights(q, k, v, sq, sk, sv)
        assert torch.equal(rw, mw) and torch.equal(rs, ms)
        rw, rs = ref.merge_gate_up_weights(gate, up, sq[:5], sk.new_ones(1))
        mw, ms = merge_gate_up_weights(gate, up, sq[:5], sk.new_ones(1))
        assert torch.equal(rw, mw) and torch.equal(rs, ms)


def test_load_hf_config_reads_the_fields_the_model_needs(tmp_path):
    from flashrec_b200.weights import load_hf_config

    raw = dict(hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
               num_key_value_heads=2, vocab_size=700, rms_norm_eps=1e-5, rope_theta=5e5, max_position_embeddings=1234)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    cfg = load_hf_config(str(tmp_path))
    assert (cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers, cfg.num_attention_heads,
            cfg.num_key_value_heads, cfg.head_dim, cfg.vocab_size) == (512, 1024, 3, 4, 2, 128, 700)
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 5e5 and cfg.max_position_embeddings == 1234
    ref = _ref("flashrec.models.weight")
    if ref is not None:
        r = ref.load_hf_config(str(tmp_path))
        for f in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                  "head_dim", "vocab_size", "rms_norm_eps", "rope_theta", "max_position_embeddings"):
            assert getattr(r, f) == getattr(cfg, f), f


def test_catalog_keys_to_item_matrix_and_back(tmp_path):
    from flashrec_b200.catalog import parse_sid_keys, read_sid_catalog, write_sid_catalog

    rng = np.random.default_rng(3)
    items = np.unique(rng.integers(0, 8192, (500, 3)), axis=0).astype(np.int32)
    path = tmp_path / "cat" / "sid.json"
    write_sid_catalog(items, path)
    back = read_sid_catalog(path)
    assert back.dtype == np.int32 and np.array_equal(back, items)
    # comma keys with blanks, duplicates, junk, a code out of range; packed integers (base 8192, 3 deep)
    keys = ["1,2,3", " 1, 2 ,3 ", "7,0,8191", "x,1,2", "9000,1,1", "4,5", 2 * 8192 ** 2 + 3 * 8192 + 4]
    got = parse_sid_keys(keys, levels=3)
    assert np.array_equal(got, np.array([[1, 2, 3], [2, 3, 4], [7, 0, 8191]], dtype=np.int32))
    with pytest.raises(ValueError):
        parse_sid_keys(["1,2,3", "4,5"])  # mixed depths need an explicit level count
    assert parse_sid_keys(["8192,1"], levels=2).shape == (0, 2)
    ref = _ref("flashrec.catalog")
    if ref is not None:
        mapping = {k: 1 for k in ["1,2,3", "7,0,8191", "9000,1,1", "3,3,3", str(5 * 8192 ** 2 + 6 * 8192 + 7), "zz"]}
        sids, total, bad, packed_only = ref.iter_unique_sids(mapping)
        assert np.array_equal(parse_sid_keys(mapping.keys()), np.asarray(sids, dtype=np.int32))
        assert total == 6 and bad == 2 and not packed_only
        # the file the reference writes is the file this module reads
        out = tmp_path / "ref.json"
        ref.write_sid2vid(sids, out, levels=3)
        assert np.array_equal(read_sid_catalog(out), np.asarray(sids, dtype=np.int32))


def test_item_matrix_from_a_catalog_file_builds_the_same_trie(tmp_path):
    from flashrec_b200.catalog import read_sid_catalog, write_sid_catalog
    from flashrec_b200.trie import build_trie_arrays

    rng = np.random.default_rng(5)
    sizes = [64, 64, 64]
    items = np.unique(np.stack([rng.integers(0, s, 400) for s in sizes], 1), axis=0)
    write_sid_catalog(items, tmp_path / "c.json")
    a = build_trie_arrays(read_sid_catalog(tmp_path / "c.json", base=64), sizes, 1000)
    b = build_trie_arrays(items, sizes, 1000)
    assert np.array_equal(a.csr_keys, b.csr_keys) and np.array_equal(a.edge_child, b.edge_child)


def test_iter_safetensors_reads_shards_through_the_index_and_filters_before_reading(tmp_path):
    from safetensors.torch import save_file

    from flashrec_b200.weights import iter_safetensors

    a = {"model.norm.weight": torch.ones(4), "model.layers.0.mlp.down_proj.weight_scale": torch.rand(3)}
    b = {"model.layers.0.mlp.down_proj.weight": torch.rand(3, 4), "lm_head.weight": torch.rand(5, 4)}
    save_file(a, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file(b, str(tmp_path / "model-00002-of-00002.safetensors"))
    index = {"weight_map": {**{k: "model-00001-of-00002.safetensors" for k in a},
                            **{k: "model-00002-of-00002.safetensors" for k in b}}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    got = dict(iter_safetensors(str(tmp_path)))
    assert set(got) == set(a) | set(b) and all(torch.equal(got[k], {**a, **b}[k]) for k in got)
    scales = dict(iter_safetensors(str(tmp_path), key_filter=lambda k: k.endswith(".weight_scale")))
    assert list(scales) == ["model.layers.0.mlp.down_proj.weight_scale"]
    # a directory without an index falls back to model.safetensors; an empty directory yields nothing
    single = tmp_path / "single"
    single.mkdir()
    save_file(a, str(single / "model.safetensors"))
    assert set(dict(iter_safetensors(str(single)))) == set(a)
    empty = tmp_path / "empty"
    empty.mkdir()
    assert list(iter_safetensors(str(empty))) == []
