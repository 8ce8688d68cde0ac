"""Generate the golden fixtures in this directory by running the reference itself.

Usage (only where the reference checkout is available):

    python tests/golden/make_golden.py <reference>/python [--only kv_table | prefill_attention | select | rope_triton_interp]

(``--only NAME`` writes just ``NAME.npz``, leaving the other files as they are; ``rope_triton_interp`` is only
written that way, in a process of its own.)

Every fixture holds seeded inputs and the outputs of the reference's own torch
CPU code path (its ``sgl_kernel`` branch is absent, so each wrapper takes its
torch branch). bf16 tensors are stored as their uint16 bit patterns, e4m3
tensors as uint8. The tests never import the reference; they read these files.
"""

from __future__ import annotations

import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def bits8(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).numpy().copy()


def select_fixture() -> None:
    """joint_select / select_final_topk / apply_temperature of the reference (search/select.py, search/expand.py)
    on seeded inputs: with and without stop tokens, with rank noise, with more survivors than candidates allow."""
    from flashrec.search.expand import apply_temperature
    from flashrec.search.select import joint_select, select_final_topk

    g = torch.Generator().manual_seed(11)
    out = {}
    cases = [(6, 8, 4, [3, 5]), (16, 32, 8, []), (5, 64, 40, [1, 2, 3, 4, 5, 6, 7, 8, 9, 10]), (3, 4, 16, [7])]
    for i, (r, c, k, stops) in enumerate(cases):
        cum = torch.randn(r, generator=g)
        lp = torch.log_softmax(torch.randn(r, c, generator=g), dim=-1)
        tok = torch.randint(0, 20 if stops else 1000, (r, c), generator=g)
        pert = -torch.log(-torch.log(torch.rand(r, c, generator=g).clamp_min(1e-30)))
        st = torch.tensor(stops, dtype=torch.int64)
        for tag, pt in (("plain", None), ("noise", pert)):
            res = joint_select(cum, lp, tok, st, k, perturb=pt)
            for f in ("next_tokens", "parent_idx", "new_cum_logprobs", "num_survivors", "fin_tokens", "fin_parent_idx",
                      "fin_cum_logprobs", "num_finished"):
                out[f"c{i}_{tag}_{f}"] = getattr(res, f).numpy()
            if k <= r * c:
                fin = select_final_topk(cum, lp, tok, min(k, c), perturb=pt)
                out[f"c{i}_{tag}_final_tokens"] = fin.tokens.numpy()
                out[f"c{i}_{tag}_final_parent"] = fin.parent_idx.numpy()
                out[f"c{i}_{tag}_final_cum"] = fin.cum_logprobs.numpy()
        out[f"c{i}_cum"], out[f"c{i}_lp"], out[f"c{i}_tok"], out[f"c{i}_pert"] = cum.numpy(), lp.numpy(), tok.numpy(), pert.numpy()
        out[f"c{i}_stop"], out[f"c{i}_k"] = st.numpy(), np.array(k)
        out[f"c{i}_temp"] = apply_temperature(lp, 0.7).numpy()
    out["n_cases"] = np.array(len(cases))
    np.savez_compressed(HERE / "select.npz", **out)


def kv_table_fixture() -> None:
    """Three decode ticks on a small slot table with the reference's own functions:
    copy_prefill_to_beams_many, then per tick the deferred remap_by_parents of every
    request, the batched write_decode statement of the scheduler and gather_kv_indices."""
    from flashrec.attention.kv_indices import gather_kv_indices
    from flashrec.engine.engine import ModelEngine
    from flashrec.scheduler.kv_remap import remap_by_parents

    g = torch.Generator().manual_seed(7)
    bws, plens, max_seq = [4, 6, 1, 5], [5, 9, 3, 7], 16
    n_req, n_rows = len(bws), sum(bws)
    table = torch.randint(1, 1000, (n_req + n_rows + 2, max_seq), generator=g, dtype=torch.int32)
    out = {"table0": table.numpy().copy(), "bws": np.array(bws), "plens": np.array(plens)}
    srcs = [1, 0, 3, 2]  # prefill rows
    # beam rows of the requests: shuffled table rows above the prefill rows
    perm = (torch.randperm(n_rows + 2, generator=g)[:n_rows] + n_req).to(torch.int64)
    gi = np.concatenate(([0], np.cumsum(bws)))
    out["rows"], out["group_indptr"], out["srcs"] = perm.numpy(), gi.astype(np.int32), np.array(srcs)
    # fan-out: the batched call needs one beam width, so run it per width class as the engine does
    fake = types.SimpleNamespace(req_pool=types.SimpleNamespace(req_to_token=table), _stage=None)
    for r in range(n_req):
        ModelEngine.copy_prefill_to_beams_many(fake, [srcs[r]], perm[gi[r]:gi[r + 1]].view(1, -1), [plens[r]])
    out["table_fanout"] = table.numpy().copy()
    next_slot = 2000
    parents = None
    for tick in range(3):
        if parents is not None:  # remaps deferred from the previous tick (scheduler.py:1590-1610)
            for r in range(n_req):
                remap_by_parents(table, perm[gi[r]:gi[r + 1]], parents[gi[r]:gi[r + 1]], plens[r], plens[r] + tick)
        out_cache = torch.arange(next_slot, next_slot + n_rows, dtype=torch.int64)
        next_slot += n_rows
        col_idx = torch.tensor(np.repeat(plens, bws)) + tick
        table[perm, col_idx] = out_cache.to(dtype=table.dtype).view(-1)  # scheduler.py:1305-1310
        seq_lens = (col_idx + 1).to(torch.int32)
        flat = gather_kv_indices(table, perm, seq_lens.tolist())
        out[f"new_slot{tick}"], out[f"seq_lens{tick}"] = out_cache.numpy(), seq_lens.numpy()
        out[f"flat{tick}"], out[f"table{tick + 1}"] = flat.numpy(), table.numpy().copy()
        if parents is not None:
            out[f"parents{tick}"] = parents.numpy()
        # parents chosen by this tick's expand: forks, permutations and out-of-range values (clamped)
        parents = torch.cat([torch.randint(-1, bw + 1, (bw,), generator=g) for bw in bws]).to(torch.int64)
    np.savez_compressed(HERE / "kv_table.npz", **out)
    print("wrote kv_table.npz")


def prefill_attention_fixture() -> None:
    """The reference's SDPA attention in its prefill branch (causal with and without a cached prefix)."""
    from flashrec.attention.flashinfer import AttentionBackend
    from flashrec.kvcache.pool import TokenToKVPool

    g = torch.Generator().manual_seed(11)
    hq, hkv, d, slots = 2, 1, 128, 200
    pool = TokenToKVPool(1, slots, hkv, d, torch.float8_e4m3fn, torch.device("cpu"))
    pool.k[0].copy_(torch.randn(slots, hkv, d, generator=g).bfloat16().to(torch.float8_e4m3fn))
    pool.v[0].copy_(torch.randn(slots, hkv, d, generator=g).bfloat16().to(torch.float8_e4m3fn))
    ext, pre = [70, 1, 33, 66], [0, 5, 64, 17]
    seq = [e + p for e, p in zip(ext, pre)]
    kvi = torch.cat([torch.randperm(slots - 1, generator=g)[:s] + 1 for s in seq]).to(torch.int32)
    q = torch.randn(sum(ext), hq, d, generator=g).bfloat16()
    fake = types.SimpleNamespace(kv_pool=pool, n_rep=hq // hkv, head_dim=d)
    batch = types.SimpleNamespace(n_rows=len(ext), seq_lens_cpu=torch.tensor(seq), extend_prefix_lens=pre,
                                  extend_seq_lens=ext, is_prefill=True, kv_indices=kvi)
    o = AttentionBackend._sdpa(fake, q, 0, batch)
    np.savez_compressed(HERE / "prefill_attention.npz", ext=np.array(ext), pre=np.array(pre), kv_indices=kvi.numpy(),
                        q=bits16(q), k_cache=bits8(pool.k[0]), v_cache=bits8(pool.v[0]), out=bits16(o))
    print("wrote prefill_attention.npz")


def rope_triton_interp_fixture() -> None:
    """The reference's fused QK-norm + RoPE + KV-store Triton kernel (kernel/qk_rope_kv.py:28-155) run on
    CPU tensors by Triton's interpreter (TRITON_INTERPRET=1, which must be set before triton is imported:
    run this in a process of its own, ``--only rope_triton_interp``). The interpreter evaluates the
    kernel's float32 arithmetic faithfully but its narrowing casts are not the hardware's (float32 ->
    bfloat16 truncates, float32 -> e4m3 mis-rounds across exponent boundaries), so the fixture keeps the
    in-place Q output, whose bits are the TRUNCATED float32 results, and drops the cache bytes."""
    os.environ["TRITON_INTERPRET"] = "1"
    import flashrec.kernel.qk_rope_kv as qk
    from flashrec.layers.rotary import RotaryEmbedding

    kernel = qk._try_triton()
    assert type(kernel).__name__ == "InterpretedFunction", "triton was imported before TRITON_INTERPRET was set"
    g = torch.Generator().manual_seed(21)
    t, n_q, n_kv, d = 6, 4, 2, 128
    qkv = torch.randn(t, n_q + 2 * n_kv, d, generator=g).bfloat16()  # strided views of one buffer, as the model has
    q, k, v = qkv[:, :n_q], qkv[:, n_q:n_q + n_kv], qkv[:, n_q + n_kv:]
    qw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16()
    kw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16()
    pos = torch.tensor([0, 1, 17, 100, 255, 4095])
    loc = torch.tensor([4, 1, 7, 2, 9, 3])
    rot = RotaryEmbedding(d, 4096, 1_000_000.0)
    cs = rot.cos_sin_cache.float().contiguous()
    kc = torch.zeros(12, n_kv, d, dtype=torch.uint8).view(torch.float8_e4m3fn)
    vc = torch.zeros(12, n_kv, d, dtype=torch.uint8).view(torch.float8_e4m3fn)
    q_in = q.clone()
    kernel[(t,)](q, k, v, qw, kw, pos, loc, cs, kc, vc, q.stride(0), q.stride(1), k.stride(0), k.stride(1),
                 v.stride(0), v.stride(1), kc.stride(0), kc.stride(1), vc.stride(0), vc.stride(1), n_q, n_kv, d, 1e-6,
                 BLOCK=128, HALF=64, num_warps=4)
    np.savez_compressed(HERE / "rope_triton_interp.npz", q=bits16(q_in), k=bits16(k.contiguous()), qw=bits16(qw),
                        kw=bits16(kw), pos=pos.numpy(), cos_sin=cs.numpy()[pos.numpy()], q_out_truncated=bits16(q.contiguous()))
    print("wrote rope_triton_interp.npz")


def main() -> None:
    torch.set_num_threads(1)
    os.environ.setdefault("FLASHREC_TRIE_DENSE_MAX_CELLS", str(1 << 29))
    from flashrec.kernel import sglops
    from flashrec.kernel.beam_trie import genrec_mask_topk_expand
    from flashrec.kernel.rms_fp8 import (
        fused_add_rmsnorm_per_token_quant_fp8,
        rmsnorm_per_token_quant_fp8,
    )
    from flashrec.kernel.silu_fp8 import silu_and_mul_per_token_quant_fp8
    from flashrec.layers.linear import Linear, quantize_weight_fp8
    from flashrec.layers.rotary import RotaryEmbedding
    from flashrec.attention.kv_indices import gather_kv_indices
    from flashrec.kvcache.pool import TokenToKVPool
    from flashrec.logits import RestrictedLMHead
    import flashrec.search.trie as trie_mod
    from flashrec.search.trie import BeamValidPathTrie

    assert sglops.SGL is None, "fixtures must come from the torch CPU path"
    g = torch.Generator().manual_seed(0)

    # ---- 1. RMSNorm -> FP8 (with / without residual), two widths --------------
    out = {}
    for tag, rows, hidden in (("a", 8, 2048), ("b", 5, 384)):
        x = torch.randn(rows, hidden, generator=g).bfloat16()
        r = torch.randn(rows, hidden, generator=g).bfloat16()
        w = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16()
        q, s = rmsnorm_per_token_quant_fp8(x, w, 1e-6)
        q2, s2, r2 = fused_add_rmsnorm_per_token_quant_fp8(x, r.clone(), w, 1e-6)
        y = sglops.rmsnorm(x, w, 1e-6)
        out.update({
            f"{tag}_x": bits16(x), f"{tag}_r": bits16(r), f"{tag}_w": bits16(w),
            f"{tag}_q": bits8(q), f"{tag}_s": s.numpy(), f"{tag}_y": bits16(y),
            f"{tag}_q_res": bits8(q2), f"{tag}_s_res": s2.numpy(), f"{tag}_r_out": bits16(r2),
        })
    np.savez_compressed(HERE / "rms_quant.npz", **out)

    # ---- 2. per-token quant + SwiGLU quant --------------------------------------
    x = (3 * torch.randn(6, 2048, generator=g)).bfloat16()
    q, s = sglops.per_token_quant_fp8(x)
    gu = (2 * torch.randn(4, 2 * 6144, generator=g)).bfloat16()
    qs, ss = silu_and_mul_per_token_quant_fp8(gu)
    ys = sglops.silu_and_mul(gu)
    np.savez_compressed(HERE / "quant_silu.npz", x=bits16(x), q=bits8(q), s=s.numpy(), gu=bits16(gu),
                        q_silu=bits8(qs), s_silu=ss.numpy(), y_silu=bits16(ys))

    # ---- 3. FP8 linear ---------------------------------------------------------
    m, k, n = 24, 256, 96
    x = torch.randn(m, k, generator=g).bfloat16()
    w = 0.02 * torch.randn(n, k, generator=g)
    wq, wscale = quantize_weight_fp8(w)
    lin = Linear(k, n)
    lin.load(w, quantize_fp8=True)
    xq, xs = sglops.per_token_quant_fp8(x)
    y = lin.forward_fp8(xq, xs, (m, k), torch.bfloat16)
    np.savez_compressed(HERE / "linear_fp8.npz", x=bits16(x), w=w.numpy(), wq=bits8(wq), wscale=wscale.numpy(),
                        xq=bits8(xq), xs=xs.numpy(), y=bits16(y))

    # ---- 4. RoPE cache + KV store ------------------------------------------------
    rot = RotaryEmbedding(128, 64, 1e6)
    pool = TokenToKVPool(1, 40, 2, 128, torch.float8_e4m3fn, torch.device("cpu"))
    kk = torch.randn(7, 2, 128, generator=g).bfloat16()
    vv = torch.randn(7, 2, 128, generator=g).bfloat16()
    loc = torch.tensor([3, 9, 1, 22, 39, 17, 5])
    pool.store(0, kk, vv, loc)
    np.savez_compressed(HERE / "rope_kv.npz", cos_sin=rot.cos_sin_cache.numpy(), k=bits16(kk), v=bits16(vv),
                        loc=loc.numpy(), k_cache=bits8(pool.k[0]), v_cache=bits8(pool.v[0]))

    # ---- 5. kv index gather + SDPA decode attention -----------------------------------
    table = torch.randint(1, 200, (6, 32), generator=g, dtype=torch.int32)
    rows = torch.tensor([4, 0, 5, 2])
    seq_lens = [7, 1, 32, 12]
    kvi = gather_kv_indices(table, rows, seq_lens)
    from flashrec.attention.flashinfer import AttentionBackend
    hq, hkv, d, slots = 4, 2, 128, 200
    pool2 = TokenToKVPool(1, slots, hkv, d, torch.float8_e4m3fn, torch.device("cpu"))
    pool2.k[0].copy_(torch.randn(slots, hkv, d, generator=g).bfloat16().to(torch.float8_e4m3fn))
    pool2.v[0].copy_(torch.randn(slots, hkv, d, generator=g).bfloat16().to(torch.float8_e4m3fn))
    q = torch.randn(4, hq, d, generator=g).bfloat16()
    fake = types.SimpleNamespace(kv_pool=pool2, n_rep=hq // hkv, head_dim=d)
    indptr = torch.tensor([0] + list(np.cumsum(seq_lens)), dtype=torch.int32)
    batch = types.SimpleNamespace(n_rows=4, seq_lens_cpu=torch.tensor(seq_lens), extend_prefix_lens=None,
                                  extend_seq_lens=None, is_prefill=False, kv_indices=kvi)
    o = AttentionBackend._sdpa(fake, q, 0, batch)
    np.savez_compressed(HERE / "attention.npz", table=table.numpy(), rows=rows.numpy(), seq_lens=np.array(seq_lens),
                        kv_indices=kvi.numpy(), indptr=indptr.numpy(), q=bits16(q), k_cache=bits8(pool2.k[0]),
                        v_cache=bits8(pool2.v[0]), out=bits16(o))

    # ---- 6. restricted head (bf16 reference head on dequantised FP8 weights) -------------
    sizes, base, hidden = [32, 32, 32], 1000, 256
    vocab = base + sum(sizes) + 8
    lm_w = 0.02 * torch.randn(vocab, hidden, generator=g)
    sid_q, sid_s = quantize_weight_fp8(lm_w[base: base + sum(sizes)])
    lm_deq = lm_w.clone()
    lm_deq[base: base + sum(sizes)] = sid_q.float() * sid_s[:, None]
    head = RestrictedLMHead(list(range(base, base + sum(sizes))))
    head.bind(lm_deq.bfloat16())
    head.bind_codebook(sizes)
    h = torch.randn(12, hidden, generator=g).bfloat16()
    lp_all, ids_all = head.compute(h, lm_deq.bfloat16())
    lp1, ids1 = head.compute_level(h, 1)
    np.savez_compressed(HERE / "head.npz", sizes=np.array(sizes), base=base, h=bits16(h), sid_q=bits8(sid_q),
                        sid_s=sid_s.numpy(), lp_all=lp_all.numpy(), ids_all=ids_all.numpy(), lp1=lp1.numpy(),
                        ids1=ids1.numpy())

    # ---- 7. trie: dense vs CSR tables, mask / advance ----------------------------------
    rng = np.random.default_rng(7)
    sizes, base = [8, 8, 8], 100
    offs = np.concatenate([[0], np.cumsum(sizes)])
    items = rng.integers(0, 8, (60, 3))

    def build(dense: bool):
        tr = BeamValidPathTrie(mode="trie")
        tr.max_depth = 3
        alltok = set()
        for it in items:
            toks = [int(base + offs[l] + it[l]) for l in range(3)]
            for dd in range(3):
                tr.children.setdefault(tuple(toks[:dd]), set()).add(toks[dd])
                alltok.add(toks[dd])
        tr.all_tokens = alltok
        tr.finalize_index(token_base=base, vocab_size=int(offs[-1]))
        trie_mod._DENSE_MAX_CELLS = (1 << 29) if dense else 0
        tr._ensure_gpu_cache(torch.device("cpu"))
        return tr

    dense, csr = build(True), build(False)
    n_nodes = len(dense._prefix_to_node)
    nodes = torch.tensor(rng.integers(-1, n_nodes + 1, 16))
    toks = torch.tensor(rng.integers(base - 3, base + offs[-1] + 3, (16, 24)))
    scores = torch.randn(16, 24, generator=g)
    masked_d = dense.mask_candidates(None, toks, scores.clone(), cur_len=1, node_ids=nodes)
    masked_c = csr.mask_candidates(None, toks, scores.clone(), cur_len=1, node_ids=nodes)
    assert torch.equal(masked_d, masked_c)
    parents = torch.tensor(rng.integers(0, 16, 16))
    atoks = torch.tensor(rng.integers(base - 3, base + offs[-1] + 3, 16))
    adv = dense.advance_node_ids(nodes, parents, atoks)
    assert torch.equal(adv, csr.advance_node_ids(nodes, parents, atoks))
    np.savez_compressed(HERE / "trie.npz", items=items, sizes=np.array(sizes), base=base, n_nodes=n_nodes,
                        invalid=dense._invalid_node, allow=dense._allow_table.numpy(),
                        next=dense._next_node.numpy(), csr_keys=csr._csr_keys.numpy(),
                        csr_child=csr._csr_child.numpy(), nodes=nodes.numpy(), toks=toks.numpy(),
                        scores=scores.numpy(), masked=masked_d.numpy(), parents=parents.numpy(),
                        atoks=atoks.numpy(), adv=adv.numpy())

    # ---- 8. fused mask + top-k + expand + advance (torch restatement) -----------------------
    n, bw, c, kk_, L = 3, 16, 12, 16, 4
    cum = torch.randn(n, bw, generator=g)
    lp = torch.sort(torch.randn(n, bw, c, generator=g), dim=-1, descending=True).values
    # tokens: legal continuations mixed with illegal ones, level-1 range
    tt = torch.tensor(rng.integers(base + offs[1], base + offs[2], (n, bw, c)))
    node_in = torch.tensor(rng.integers(1, 1 + len(set(items[:, 0])), (n, bw)))
    token_ids = torch.tensor(rng.integers(base, base + 8, (n, bw, L)))
    res = genrec_mask_topk_expand(cum, lp, tt, select_k=kk_, node_ids=node_in, allow_table=dense._allow_table,
                                  token_base=base, token_ids=token_ids.clone(), col=1,
                                  next_node=dense._next_node, invalid_node=dense._invalid_node)
    np.savez_compressed(HERE / "beam_step.npz", cum=cum.numpy(), lp=lp.numpy(), tok=tt.numpy(),
                        node_in=node_in.numpy(), token_ids=token_ids.numpy(), vals=res.vals.numpy(),
                        parents=res.parents.numpy(), tokens=res.tokens.numpy(), indices=res.indices.numpy(),
                        token_ids_out=res.token_ids.numpy(), node_out=res.node_ids.numpy())
    kv_table_fixture()
    prefill_attention_fixture()
    select_fixture()
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    # the reference checkout's `python/` directory: argument 1 or $FLASHREC_REFERENCE
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FLASHREC_REFERENCE")
    if not ref:
        sys.exit("usage: make_golden.py <reference checkout>/python   (or set FLASHREC_REFERENCE)")
    if ref not in sys.path:
        sys.path.insert(0, ref)
    if sys.argv[2:4] == ["--only", "kv_table"]:
        kv_table_fixture()
    elif sys.argv[2:4] == ["--only", "prefill_attention"]:
        prefill_attention_fixture()
    elif sys.argv[2:4] == ["--only", "select"]:
        select_fixture()
    elif sys.argv[2:4] == ["--only", "rope_triton_interp"]:
        rope_triton_interp_fixture()
    else:
        main()
