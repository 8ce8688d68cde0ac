"""Pins the CPU oracle against outputs of the reference's own torch path
(fixtures written by tests/golden/make_golden.py)."""

import numpy as np
import torch

from conftest import bf16_from_bits, bits8, bits16, fp8_from_bits, load_golden
from oracle import sid_oracle as O


def test_rms_quant_matches_reference_bytes():
    g = load_golden("rms_quant")
    for tag in ("a", "b"):
        x, r, w = (bf16_from_bits(g[f"{tag}_{n}"]) for n in ("x", "r", "w"))
        q, s = O.rmsnorm_quant_fp8(x, w, 1e-6)
        assert np.array_equal(bits16(O.rmsnorm(x, w, 1e-6)), g[f"{tag}_y"])
        assert np.array_equal(bits8(q), g[f"{tag}_q"])
        assert np.array_equal(s.numpy(), g[f"{tag}_s"])
        q2, s2, r2 = O.rmsnorm_quant_fp8(x, w, 1e-6, residual=r.clone())
        assert np.array_equal(bits16(r2), g[f"{tag}_r_out"])
        assert np.array_equal(bits8(q2), g[f"{tag}_q_res"])
        assert np.array_equal(s2.numpy(), g[f"{tag}_s_res"])


def test_token_and_silu_quant_match_reference_bytes():
    g = load_golden("quant_silu")
    q, s = O.per_token_quant_fp8(bf16_from_bits(g["x"]))
    assert np.array_equal(bits8(q), g["q"]) and np.array_equal(s.numpy(), g["s"])
    gu = bf16_from_bits(g["gu"])
    y = O.silu_and_mul(gu)
    # silu is evaluated exactly here and by a float32 polynomial in torch: allow a
    # handful of 1-ulp bf16 differences, and the e4m3 bytes that follow from them
    dy = (bits16(y).astype(np.int32) - g["y_silu"].astype(np.int32))
    assert np.abs(dy).max() <= 1 and (dy != 0).mean() < 1e-3
    qs, ss = O.silu_mul_quant_fp8(gu)
    assert (bits8(qs) != g["q_silu"]).mean() < 1e-3
    assert np.allclose(ss.numpy(), g["s_silu"], rtol=1e-2)


def test_linear_fp8_matches_reference():
    g = load_golden("linear_fp8")
    wq, ws = O.quantize_weight_fp8(torch.from_numpy(g["w"]))
    assert np.array_equal(bits8(wq), g["wq"]) and np.array_equal(ws.numpy(), g["wscale"])
    xq, xs = O.per_token_quant_fp8(bf16_from_bits(g["x"]))
    assert np.array_equal(bits8(xq), g["xq"]) and np.array_equal(xs.numpy(), g["xs"])
    y = O.fp8_scaled_mm(xq, wq, xs, ws)
    assert np.array_equal(bits16(y), g["y"])  # same double rounding as torch._scaled_mm + rescale


def test_rope_cache_and_kv_store_match_reference():
    g = load_golden("rope_kv")
    assert np.array_equal(O.build_cos_sin_cache(128, 64, 1e6).numpy(), g["cos_sin"])
    kc = torch.zeros(40, 2, 128, dtype=torch.uint8).view(torch.float8_e4m3fn)
    vc = torch.zeros(40, 2, 128, dtype=torch.uint8).view(torch.float8_e4m3fn)
    O.store_kv(kc, vc, torch.from_numpy(g["loc"]), bf16_from_bits(g["k"]), bf16_from_bits(g["v"]))
    assert np.array_equal(bits8(kc), g["k_cache"]) and np.array_equal(bits8(vc), g["v_cache"])


def test_norm_rope_building_blocks():
    """The fused arithmetic has no runnable CPU reference; check it against an
    independent float64 evaluation of the same formula."""
    torch.manual_seed(3)
    t, h, d = 5, 3, 128
    q = torch.randn(t, h, d).bfloat16()
    w = (1 + 0.1 * torch.randn(d)).bfloat16()
    cs = O.build_cos_sin_cache(d, 32, 1e6)
    pos = torch.tensor([0, 3, 7, 31, 12])
    c = cs[pos][:, None, : d // 2].double()
    s = cs[pos][:, None, d // 2 :].double()
    x = q.double()
    xn = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6) * w.double()
    ref = torch.cat((xn[..., : d // 2] * c - xn[..., d // 2 :] * s, xn[..., d // 2 :] * c + xn[..., : d // 2] * s), -1)
    got = O._norm_rope(q.float(), w, 1e-6, c.float(), s.float())
    assert torch.allclose(got.double(), ref, rtol=1e-5, atol=1e-5)


def test_gather_and_attention_match_reference():
    g = load_golden("attention")
    kvi = O.gather_kv_indices(torch.from_numpy(g["table"]), torch.from_numpy(g["rows"]), g["seq_lens"].tolist())
    assert np.array_equal(kvi.numpy(), g["kv_indices"])
    out = O.decode_attention(bf16_from_bits(g["q"]), fp8_from_bits(g["k_cache"]), fp8_from_bits(g["v_cache"]),
                             torch.from_numpy(g["indptr"]), kvi, n_rep=2)
    ref = bf16_from_bits(g["out"]).float()
    # the reference evaluates SDPA in bf16; this oracle in fp32
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)


def test_head_logprobs_close_to_reference_bf16_head():
    g = load_golden("head")
    h = bf16_from_bits(g["h"])
    hq, hs = O.per_token_quant_fp8(h)
    logits = O.fp8_logits_f32(hq, fp8_from_bits(g["sid_q"]), hs, torch.from_numpy(g["sid_s"]))
    lp = O.log_softmax_rows(logits)
    # reference head: bf16 activations x bf16 (dequantised) weights, bf16 logits.
    assert torch.allclose(lp, torch.from_numpy(g["lp_all"]), atol=6e-2)
    sizes = g["sizes"].tolist()
    lvl1 = logits[:, sizes[0]: sizes[0] + sizes[1]]
    assert torch.allclose(O.log_softmax_rows(lvl1), torch.from_numpy(g["lp1"]), atol=6e-2)
    mx, ls = O.row_stats(lvl1)
    assert torch.allclose(O.logprobs_from_stats(lvl1, mx, ls), O.log_softmax_rows(lvl1), atol=1e-5)
    assert np.array_equal(g["ids1"], int(g["base"]) + sizes[0] + np.arange(sizes[1]))


def _golden_trie():
    g = load_golden("trie")
    return g, O.OracleTrie(g["csr_keys"], g["csr_child"], int(g["sizes"].sum()), int(g["base"]), int(g["invalid"]))


def test_trie_mask_and_advance_match_reference():
    g, tr = _golden_trie()
    masked = O.trie_mask(torch.from_numpy(g["scores"]), torch.from_numpy(g["toks"]), torch.from_numpy(g["nodes"]), tr)
    assert np.array_equal(masked.numpy(), g["masked"])
    adv = tr.transition(g["nodes"][g["parents"]], g["atoks"])
    assert np.array_equal(adv, g["adv"])
    # dense tables say the same thing as the CSR arrays
    rows, rel = np.nonzero(g["allow"])
    assert np.array_equal(rows * tr.vsz + rel, g["csr_keys"])
    assert np.array_equal(g["next"][rows, rel], g["csr_child"])


def test_mask_topk_expand_matches_reference():
    g, tr = _golden_trie()
    b = load_golden("beam_step")
    res = O.mask_topk_expand(torch.from_numpy(b["cum"]), torch.from_numpy(b["lp"]), torch.from_numpy(b["tok"]),
                             select_k=16, node_ids=torch.from_numpy(b["node_in"]), trie=tr,
                             token_ids=torch.from_numpy(b["token_ids"]), col=1)
    live = np.isfinite(b["vals"])
    assert np.array_equal(res["vals"].numpy()[live], b["vals"][live])
    assert np.array_equal(np.isfinite(res["vals"].numpy()), live)
    for name, key in (("parents", "parents"), ("tokens", "tokens"), ("indices", "indices")):
        assert np.array_equal(res[name].numpy()[live], b[key][live]), name
    rows_live = live  # [n, k] == [n, bw] here
    assert np.array_equal(res["token_ids"].numpy()[rows_live], b["token_ids_out"][rows_live])
    assert np.array_equal(res["node_ids"].numpy()[rows_live], b["node_out"][rows_live])


def _kv_table_replay(g, step_fn, fanout_fn, table):
    """Replay the fixture's three ticks with ``step_fn`` / ``fanout_fn``; yields what each produced."""
    rows, gi = torch.from_numpy(g["rows"]), g["group_indptr"]
    bws, plens = g["bws"].tolist(), g["plens"].tolist()
    for r in range(len(bws)):
        fanout_fn(table, torch.tensor([int(g["srcs"][r])]), rows[gi[r]:gi[r + 1]].view(1, -1), plens[r])
    yield "fanout", table, None
    prefix = torch.tensor(np.repeat(plens, bws), dtype=torch.int32)
    for tick in range(3):
        parents = torch.from_numpy(g[f"parents{tick}"]) if tick else None
        flat = step_fn(table, rows, torch.from_numpy(gi), torch.from_numpy(g[f"seq_lens{tick}"]),
                       torch.from_numpy(g[f"new_slot{tick}"]), parents, prefix)
        yield tick, table, flat


def test_kv_table_ticks_match_reference():
    g = load_golden("kv_table")
    table = torch.from_numpy(g["table0"].copy())
    step = lambda t, rows, gi, sl, ns, par, pre: O.kv_table_step(t, rows, gi, sl, ns, par, pre)[1]
    for tag, tab, flat in _kv_table_replay(g, step, O.copy_prefill_to_beams_many, table):
        if tag == "fanout":
            assert np.array_equal(tab.numpy(), g["table_fanout"])
        else:
            assert np.array_equal(tab.numpy(), g[f"table{tag + 1}"]), tag
            assert np.array_equal(flat.numpy(), g[f"flat{tag}"]), tag


def test_remap_by_parents_known_answer():
    # the reference's own vector (tests/test_kv_remap.py:19-30): a fork gathers columns 2:4 by parent
    table = torch.arange(20).view(4, 5).clone()
    O.remap_by_parents(table, torch.arange(4), torch.tensor([0, 0, 1, 1]), 2, 4)
    assert table[:, 2:4].tolist() == [[2, 3], [2, 3], [7, 8], [7, 8]]
    assert table[:, :2].tolist() == [[0, 1], [5, 6], [10, 11], [15, 16]] and table[:, 4].tolist() == [4, 9, 14, 19]
    before = table.clone()
    O.remap_by_parents(table, torch.arange(4), torch.arange(4), 2, 4)  # identity parents change nothing
    assert torch.equal(table, before)


def _prefill_fixture():
    g = load_golden("prefill_attention")
    ext, pre = g["ext"].tolist(), g["pre"].tolist()
    qo = np.concatenate(([0], np.cumsum(ext))).astype(np.int32)
    kv = np.concatenate(([0], np.cumsum([e + p for e, p in zip(ext, pre)]))).astype(np.int32)
    return g, torch.from_numpy(qo), torch.from_numpy(kv)


def test_prefill_attention_matches_reference():
    g, qo, kv = _prefill_fixture()
    out = O.prefill_attention(bf16_from_bits(g["q"]), fp8_from_bits(g["k_cache"]), fp8_from_bits(g["v_cache"]), qo, kv,
                              torch.from_numpy(g["kv_indices"]), n_rep=2)
    ref = bf16_from_bits(g["out"]).float()
    # the reference evaluates SDPA in bf16; this oracle in fp32
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)


def test_fused_qk_norm_rope_float32_arithmetic_matches_reference_triton_kernel():
    """The reference's fused QK-norm + RoPE Triton kernel, executed by Triton's CPU interpreter, writes Q as
    the TRUNCATED float32 result (the interpreter's float32 -> bfloat16 cast truncates; the hardware cast is
    round-to-nearest). Truncating this oracle's float32 result gives the same bits: the float32 arithmetic
    (norm, weight, NeoX pairing, cos/sin row) is the kernel's, bit for bit; the rounded result is within one
    bfloat16 ulp of the fixture everywhere."""
    g = load_golden("rope_triton_interp")
    q = bf16_from_bits(g["q"])
    cs = torch.from_numpy(g["cos_sin"]).float()
    cos, sin = cs[:, None, :64], cs[:, None, 64:]
    y = O._norm_rope(q.float(), bf16_from_bits(g["qw"]), 1e-6, cos, sin)
    truncated = (y.contiguous().view(torch.int32) >> 16).to(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(truncated, g["q_out_truncated"])
    rounded = bits16(y.to(torch.bfloat16)).astype(np.int32)
    assert np.abs(rounded - g["q_out_truncated"].astype(np.int32)).max() <= 1


def test_selection_with_stop_tokens_and_rank_noise_matches_reference():
    """joint_select / select_final_topk / apply_temperature (search/select.py:72-179, search/expand.py:61-70):
    the oracle's plain walk against the reference's cumsum / scatter formulation, every output slot."""
    g = load_golden("select")
    for i in range(int(g["n_cases"])):
        cum, lp, tok, pert = (torch.from_numpy(g[f"c{i}_{n}"]) for n in ("cum", "lp", "tok", "pert"))
        st, k = torch.from_numpy(g[f"c{i}_stop"]), int(g[f"c{i}_k"])
        for tag, pt in (("plain", None), ("noise", pert)):
            r = O.joint_select(cum, lp, tok, st, k, pt)
            for f, v in r.items():
                assert np.array_equal(np.asarray(v), g[f"c{i}_{tag}_{f}"]), (i, tag, f)
            if f"c{i}_{tag}_final_tokens" in g.files:
                kk = g[f"c{i}_{tag}_final_tokens"].shape[0]
                fr = O.select_final_topk(cum, lp, tok, kk, pt)
                assert np.array_equal(fr["tokens"].numpy(), g[f"c{i}_{tag}_final_tokens"])
                assert np.array_equal(fr["parent_idx"].numpy(), g[f"c{i}_{tag}_final_parent"])
                assert np.array_equal(fr["cum_logprobs"].numpy(), g[f"c{i}_{tag}_final_cum"])
        assert np.allclose(O.apply_temperature(lp, 0.7).numpy(), g[f"c{i}_temp"], atol=1e-6)
