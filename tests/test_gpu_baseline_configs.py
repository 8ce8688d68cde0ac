"""GPU parity at the sizes the baseline configurations name (through the C ABI).

Config 1: RMSNorm -> FP8 then one W8A8 linear, 512 rows x 2048 -> 6144, seed-0 inputs.
Config 3: trie-constrained SID head, 512 beams, 3 levels x 8192 codes, a catalog of uniform random
3-tuples (200k items, and the configuration's own 1M), CSR and bitmap tries, three
decode steps: every step against the CPU oracle bit for bit, and the properties the step must have
at any size (legal SIDs only, sorted scores, distinct beams, layouts agree).
Config 2 at full size is the last case of tests/test_gpu_engine.py::test_decoder_layer_vs_oracle.
"""

import ctypes

import numpy as np
import pytest
import torch

from oracle import sid_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FP8 = torch.float8_e4m3fn


def _bytes(t):
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def test_config1_rmsnorm_fp8_linear_512x2048x6144():
    from flashrec_b200.kernel.rms_fp8 import rmsnorm_per_token_quant_fp8
    from flashrec_b200.kernel.sglops import fp8_scaled_mm
    from flashrec_b200.layers import quantize_weight_fp8

    g = torch.Generator().manual_seed(0)
    x = torch.randn(512, 2048, generator=g).bfloat16()
    gamma = (1 + 0.1 * torch.randn(2048, generator=g)).bfloat16()
    w = 0.02 * torch.randn(6144, 2048, generator=g)
    q_ref, s_ref = O.rmsnorm_quant_fp8(x, gamma, 1e-6)
    wq_ref, ws_ref = O.quantize_weight_fp8(w)
    out_ref = O.fp8_scaled_mm(q_ref, wq_ref, s_ref, ws_ref).float()

    q, s = rmsnorm_per_token_quant_fp8(x.to(DEV), gamma.to(DEV), 1e-6)
    assert np.array_equal(_bytes(q), _bytes(q_ref)) and torch.equal(s.cpu(), s_ref)  # FP8 bytes and scales: bit-exact
    wq, ws = quantize_weight_fp8(w.to(DEV))
    assert np.array_equal(_bytes(wq), _bytes(wq_ref)) and torch.equal(ws.cpu().reshape(-1), ws_ref.reshape(-1))
    out = fp8_scaled_mm(q, wq.t(), s, ws, torch.bfloat16)
    assert out.shape == (512, 6144) and out.dtype == torch.bfloat16
    err = (out.float().cpu() - out_ref).abs().max() / out_ref.abs().max()
    assert err < 2e-2, err  # bf16 GEMM output: 2e-2 relative
    # every kernel that can take this shape stays within the same bound
    for hint in (64, 128, 256, 512, 1024):
        o2 = fp8_scaled_mm(q, wq.t(), s, ws, torch.bfloat16, block_n=hint)
        assert (o2.float().cpu() - out_ref).abs().max() / out_ref.abs().max() < 2e-2, hint


@pytest.mark.parametrize("catalog", [200_000, 1_000_000])
def test_config3_trie_constrained_head_three_steps(catalog):
    from flashrec_b200.logits import RestrictedLMHead
    from flashrec_b200.sid_decode import sid_beam_step
    from flashrec_b200.trie import build_trie_arrays, trie_to_device

    bw, kl, hidden, base = 512, 8192, 2048, 151_936
    sizes = [kl, kl, kl]
    items = np.unique(np.random.default_rng(0).integers(0, kl, (catalog, 3)), axis=0)
    arrays = build_trie_arrays(items, sizes, base)
    otr = O.OracleTrie(arrays.csr_keys, arrays.edge_child, arrays.vsz, base, arrays.invalid_node)
    legal = {tuple(r) for r in items.tolist()}

    g = torch.Generator().manual_seed(3)
    w = 0.02 * torch.randn(3 * kl, hidden, generator=g)
    wq, ws = O.quantize_weight_fp8(w)
    head = RestrictedLMHead(list(range(base, base + 3 * kl)))
    head.bind_quantized(wq.to(DEV), ws.reshape(-1).to(DEV))
    head.bind_codebook(sizes)
    hs = [torch.randn(bw, hidden, generator=torch.Generator().manual_seed(lv)).bfloat16() for lv in range(3)]

    results = {}
    for layout in ("csr", "bitmap"):
        trie = trie_to_device(arrays, layout, DEV)
        cum = torch.full((1, bw), float("-inf"))
        cum[0, 0] = 0.0  # step 0: one live beam at the root
        nodes = torch.zeros((1, bw), dtype=torch.int64)
        toks = torch.zeros((1, bw, 3), dtype=torch.int64)
        cum_d, nodes_d, toks_d = cum.to(DEV), nodes.to(DEV), toks.to(DEV)
        for lv in range(3):
            lg, mx, ls, _ = head.logits_level(hs[lv].to(DEV), lv)
            tok_out = torch.zeros_like(toks_d)
            node_out = torch.zeros_like(nodes_d)
            col = torch.full((1,), lv, dtype=torch.int32, device=DEV)
            out = sid_beam_step(cum_d, lg, mx, ls, nodes_d, trie, base + kl * lv, bw, token_ids_in=toks_d,
                                token_ids_out=tok_out, node_ids_out=node_out, col=col)
            # the CPU oracle on the device's own logits and statistics (the head GEMM has its own test)
            ref = O.sid_beam_step(cum_d.cpu(), lg.cpu(), nodes_d.cpu(), otr, base + kl * lv, bw,
                                  token_ids=toks_d.cpu(), col=lv, stats=(mx.cpu(), ls.cpu()))
            assert torch.equal(out.vals.cpu(), ref["vals"]), (layout, lv)
            assert torch.equal(out.parents.cpu(), ref["parents"]) and torch.equal(out.tokens.cpu(), ref["tokens"])
            assert torch.equal(tok_out.cpu(), ref["token_ids"]) and torch.equal(node_out.cpu(), ref["node_ids"])
            v = out.vals[0]
            assert (v[:-1] >= v[1:]).all()  # sorted scores
            cum_d, nodes_d, toks_d = out.vals.clone(), node_out, tok_out
        live = torch.isfinite(cum_d[0]).cpu().numpy()
        assert live.sum() == bw  # catalogs of this size keep all 512 beams alive after three levels
        codes = (toks_d[0].cpu() - torch.tensor([base, base + kl, base + 2 * kl])).numpy()
        rows = [tuple(c) for c in codes[live]]
        assert all(r in legal for r in rows)  # illegal-SID rate 0
        assert len(set(rows)) == len(rows)  # beams are distinct items
        assert (nodes_d[0].cpu().numpy()[live] == -1).all()  # complete SIDs: leaves reached
        results[layout] = (cum_d.cpu(), toks_d.cpu())
    assert torch.equal(results["csr"][0], results["bitmap"][0]) and torch.equal(results["csr"][1], results["bitmap"][1])


def test_config5_wide_beam_sharded_head_2048_beams_4x4096():
    """Config 5 on one GPU: 2048 beams, 4 levels x 4096 codes, a Zipf-skewed catalog (2M items here; the
    10M build has its own test) built on the device, head sharded by token range over 8 emulated ranks.
    Every level: the unsharded step against the CPU oracle bit for bit, and statistics + per-shard steps +
    merge against the unsharded step bit for bit; the final beams are distinct legal items."""
    from flashrec_b200._lib import call, ptr, stream_ptr
    from flashrec_b200.sid_decode import BeamStepOut, sid_beam_step
    from flashrec_b200.trie import build_trie_arrays, build_trie_device

    n, bw, L, kl, S, base, items_n = 2, 2048, 4, 4096, 8, 151_936, 2_000_000
    sizes = [kl] * L
    rng = np.random.default_rng(0)
    cols = [np.minimum(rng.zipf(1.1, items_n) - 1, kl - 1) if l < 2 else rng.integers(0, kl, items_n)
            for l in range(L)]
    items = np.stack(cols, 1)
    trie = build_trie_device(torch.from_numpy(items.astype(np.int32)).to(DEV), sizes, base)
    host = build_trie_arrays(items, sizes, base)
    otr = O.OracleTrie(host.csr_keys, host.edge_child, host.vsz, base, host.invalid_node)
    assert np.array_equal(trie.tensors["keys"].cpu().numpy(), host.csr_keys)

    cum = torch.full((n, bw), float("-inf"), device=DEV)
    cum[:, 0] = 0.0
    nodes = torch.zeros((n, bw), dtype=torch.int64, device=DEV)
    toks = torch.zeros((n, bw, L), dtype=torch.int64, device=DEV)
    w = kl // S
    for lv in range(L):
        g = torch.Generator().manual_seed(50 + lv)
        logits = (3.0 * torch.randn(n * bw, kl, generator=g)).to(DEV)
        mx, ls = torch.empty(n * bw, device=DEV), torch.empty(n * bw, device=DEV)
        call("fr_logsumexp_rows", ptr(logits), logits.stride(0), ptr(mx), ptr(ls), None, 0, n * bw, kl, stream_ptr(DEV))
        col = torch.full((n,), lv, dtype=torch.int32, device=DEV)
        tok_ref, node_ref = torch.zeros_like(toks), torch.zeros_like(nodes)
        full = sid_beam_step(cum, logits, mx, ls, nodes, trie, base + lv * kl, bw, token_ids_in=toks,
                             token_ids_out=tok_ref, node_ids_out=node_ref, col=col)
        ref = O.sid_beam_step(cum.cpu(), logits.cpu(), nodes.cpu(), otr, base + lv * kl, bw, token_ids=toks.cpu(),
                              col=lv, stats=(mx.cpu(), ls.cpu()))
        assert torch.equal(full.vals.cpu(), ref["vals"]) and torch.equal(full.tokens.cpu(), ref["tokens"]), lv
        assert torch.equal(full.parents.cpu(), ref["parents"]) and torch.equal(tok_ref.cpu(), ref["token_ids"]), lv
        assert torch.equal(node_ref.cpu(), ref["node_ids"]), lv
        # the same step through 8 token-range shards
        smx, sls = torch.empty((S, n * bw), device=DEV), torch.empty((S, n * bw), device=DEV)
        for s in range(S):
            part = logits[:, s * w:(s + 1) * w]
            call("fr_logsumexp_rows", ptr(part), part.stride(0), ptr(smx[s]), ptr(sls[s]), None, 0, n * bw, w,
                 stream_ptr(DEV))
        gmx, gls = torch.empty_like(mx), torch.empty_like(ls)
        call("fr_lse_combine_shards", ptr(smx), ptr(sls), ptr(gmx), ptr(gls), S, n * bw, 0, stream_ptr(DEV))
        vals = torch.empty((S, n, bw), device=DEV)
        idx = torch.empty((S, n, bw), dtype=torch.int64, device=DEV)
        child = torch.empty((S, n, bw), dtype=torch.int64, device=DEV)
        for s in range(S):
            o = sid_beam_step(cum, logits[:, s * w:(s + 1) * w], mx, ls, nodes, trie, base + lv * kl, bw,
                              idx_base=s * w, idx_width=kl)
            vals[s], idx[s], child[s] = o.vals, o.indices, o.child
        m = BeamStepOut(*(torch.empty((n, bw), dtype=dt, device=DEV)
                          for dt in (torch.float32, torch.int64, torch.int64, torch.int64, torch.int64)))
        tok_out, node_out = torch.zeros_like(toks), torch.zeros_like(nodes)
        trie_desc = trie.descriptor()
        call("fr_topk_merge_shards", ptr(m.vals), ptr(m.parents), ptr(m.tokens), ptr(m.indices), ptr(m.child),
             ptr(vals), ptr(idx), ptr(child), None, ptr(nodes), ptr(toks), ptr(tok_out), ptr(node_out), None, ptr(col),
             ctypes.byref(trie_desc), base + lv * kl, kl, S, n, bw, bw, L, 1, 1, stream_ptr(DEV))
        for a, b in ((m.vals, full.vals), (m.parents, full.parents), (m.tokens, full.tokens),
                     (m.indices, full.indices), (m.child, full.child), (tok_out, tok_ref), (node_out, node_ref)):
            assert torch.equal(a, b), lv
        cum, nodes, toks = full.vals.clone(), node_ref, tok_ref
    live = torch.isfinite(cum).cpu().numpy()
    assert live.all()
    codes = (toks.cpu() - torch.tensor([base + l * kl for l in range(L)])).numpy()
    legal = {tuple(r) for r in np.unique(items, axis=0).tolist()}
    for r in range(n):
        rows = [tuple(c) for c in codes[r]]
        assert all(x in legal for x in rows) and len(set(rows)) == len(rows)
    assert (nodes == -1).all()


def test_config4_full_size_wave_slot_lists_kv_bytes_and_legality():
    """Config 4 at its stated size on one GPU: 28 layers, 32 requests x 512 beams = 16384 rows, prompts
    U[128, 1024] sharing a 64-token prefix, 3 levels x 8192 codes, the 1M-item catalog (CSR), one wave from
    CUDA graphs. Checked against the oracle: the slot table and the last flat slot list of all 16384 rows
    (bit-exact integer bookkeeping, replayed with the parents the wave chose), the e4m3 K / V bytes the first
    layer wrote at step 0 for a sample of rows (at most 4 % of the bytes differ, K by one e4m3 step at most:
    they are conversions of the qkv GEMM's bf16 output, which itself is compared at 2e-2), and for
    every request: only catalog items, distinct, scores sorted, complete SIDs."""
    from flashrec_b200.decoder import Qwen3Config
    from flashrec_b200.sid_decode import SidDecodeEngine
    from flashrec_b200.trie import build_trie_device

    n, bw, kl, base = 32, 512, 8192, 151_936
    sizes = [kl] * 3
    rng = np.random.default_rng(0)
    items = np.stack([rng.integers(0, s, 1_000_000) for s in sizes], axis=1)
    trie = build_trie_device(torch.from_numpy(items.astype(np.int32)).to(DEV), sizes, base, layout="csr")
    prompts = [int(x) for x in np.random.default_rng(1000).integers(128, 1025, n)]
    cfg = Qwen3Config(num_hidden_layers=28)
    eng = SidDecodeEngine(cfg, n, bw, prompts, sizes, base, trie, DEV, shared_prefix=64, page_size=16, seed=0)
    table0 = eng.req_to_token.cpu().clone()
    eng.capture()
    eng.run(host_io=True)
    torch.cuda.synchronize()

    # (1) slot table and last flat list: the reference's bookkeeping replayed on the host
    exp = table0.clone()
    O.copy_prefill_to_beams_many(exp, eng.prefill_rows.cpu(), eng.rows_idx.cpu().view(n, bw), max(prompts))
    pre = eng.prefix_len_rows.cpu()
    for s in range(eng.steps):
        par = eng.outs[s - 1].parents.cpu().view(-1) if s else None
        indptr, flat = O.kv_table_step(exp, eng.rows_idx.cpu(), eng.group_indptr.cpu(), pre + s + 1, eng.h_loc[s], par,
                                       pre)
    n_flat = int(indptr[-1])
    assert torch.equal(eng.kv_indptr.cpu(), indptr) and torch.equal(eng.kv_indices.cpu()[:n_flat], flat)
    tab = eng.req_to_token.cpu()
    cols = torch.arange(tab.shape[1])[None, :]
    reach = cols < (pre[:, None] + eng.steps)  # columns a reader can reach: [:seq_len]
    assert torch.equal(torch.where(reach, tab[: eng.rows], 0), torch.where(reach, exp[: eng.rows], 0))

    # (2) first layer's K / V bytes of step 0 for a sample of rows
    layer = eng.model.layers[0]
    a = layer.self_attn
    sample = torch.tensor([0, 1, 511, 512, 7000, 16383])
    x = eng.model.embed_tokens[base].cpu()[None, :].repeat(len(sample), 1)
    q8, s8 = O.rmsnorm_quant_fp8(x, layer.input_layernorm.weight.cpu(), cfg.rms_norm_eps)
    qkv = O.fp8_scaled_mm(q8, a.qkv_proj._fp8_weight.t().cpu().contiguous(), s8, a.qkv_proj._fp8_scale.cpu())
    heads = qkv.view(len(sample), 32, 128)
    kc = torch.zeros(len(sample) + 1, 8, 128, dtype=torch.uint8).view(FP8)
    vc = torch.zeros(len(sample) + 1, 8, 128, dtype=torch.uint8).view(FP8)
    pos = torch.tensor([prompts[int(r) // bw] for r in sample])
    O.qk_norm_rope_store_fp8(heads[:, :16], heads[:, 16:24], heads[:, 24:], pos, torch.arange(1, len(sample) + 1),
                             a.q_norm.weight.cpu(), a.k_norm.weight.cpu(), cfg.rms_norm_eps,
                             eng.model.rotary.cos_sin_cache.cpu(), kc, vc)
    slots = eng.h_loc[0][sample]
    got_k, got_v = _bytes(eng.pool.k[0][slots.to(DEV)]), _bytes(eng.pool.v[0][slots.to(DEV)])
    ref_k, ref_v = _bytes(kc[1:]), _bytes(vc[1:])
    assert (got_v != ref_v).mean() <= 0.04 and (got_k != ref_k).mean() <= 0.04, ((got_v != ref_v).mean(),
                                                                                  (got_k != ref_k).mean())
    ref_kf, got_kf = kc[1:].float().numpy(), eng.pool.k[0][slots.to(DEV)].float().cpu().numpy()
    # one e4m3 step at most (a step is up to 1/7 of the smaller neighbour); where the rotation cancels two
    # large terms into a small value, one bf16 ulp of either term (0.03 in absolute terms) is the bound instead
    assert (np.abs(ref_kf - got_kf) <= np.maximum(0.15 * np.maximum(np.abs(ref_kf), np.abs(got_kf)), 0.03)).all()

    # (3) every request: catalog items only, distinct, sorted, complete
    legal_keys = np.unique(items[:, 0].astype(np.int64) * kl * kl + items[:, 1] * kl + items[:, 2])
    codes = (eng.h_tokens - torch.tensor([base, base + kl, base + 2 * kl])).numpy().astype(np.int64)
    keys = codes[..., 0] * kl * kl + codes[..., 1] * kl + codes[..., 2]
    assert np.isfinite(eng.h_vals.numpy()).all()
    assert np.isin(keys, legal_keys).all()  # illegal-SID rate 0
    assert all(len(np.unique(keys[r])) == bw for r in range(n))
    assert (eng.h_vals[:, :-1] >= eng.h_vals[:, 1:]).all()
    assert (eng.final_nodes == -1).all()
