"""CPU oracle for the quantized SID decode-step hot path.

TEST INFRASTRUCTURE ONLY. This module restates, in plain torch-CPU / numpy, the
arithmetic of the reference engine's decode path so that the CUDA kernels can
be checked against it. Nothing in the product package imports it; only
``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs do.

Each function names the reference code it follows (paths inside the
reference's ``python/flashrec`` tree). Pinning: ``tests/golden/*.npz`` holds
inputs and outputs produced by importing the reference itself
(``tests/golden/make_golden.py``); ``tests/test_oracle_golden.py`` checks this
module against them. The fused QK-norm+RoPE arithmetic has no torch path in the
reference (its fallback multiplies 64-wide cos/sin into 128-wide heads, which raises);
it is pinned by the reference's Triton kernel run under Triton's CPU interpreter,
whose Q output equals this module's float32 result truncated to bfloat16, bit for
bit (``rope_triton_interp.npz``). One piece stays "parity unpinned" beyond its
building blocks: the FP8 lm_head (the reference's head is bf16).

Deliberate, documented deviations from the literal torch path:
  * sums of squares are accumulated in float64 and rounded once to float32
    (torch reduces in float32 in an order that depends on build and thread
    count); everything after that follows torch's float32 / bfloat16 roundings;
  * silu is evaluated in float64 and rounded to float32 then bfloat16 (torch
    evaluates exp in float32 with a vectorised polynomial).
Both make the result independent of reduction order so that a GPU can match it
bit for bit; the golden tests report how many bytes differ from the literal
reference (none on the committed fixtures except where stated).
"""

from __future__ import annotations

from typing import Optional

import numpy as np
import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


# ---------------------------------------------------------------------------
# quantisers
# ---------------------------------------------------------------------------
def per_token_quant_fp8(x: torch.Tensor):
    """kernel/sglops.py:84-96 (torch branch)."""
    x2 = x.reshape(-1, x.shape[-1])
    x_f = x2.float()
    amax = x_f.abs().amax(dim=-1, keepdim=True).clamp(min=1e-12)
    scale = (amax / FP8_MAX).to(torch.float32)
    q = (x_f / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q, scale


def quantize_weight_fp8(w: torch.Tensor):
    """layers/linear.py:26-32."""
    wf = w.float()
    amax = wf.abs().amax(dim=-1).clamp(min=1e-12)
    scale = (amax / FP8_MAX).to(torch.float32)
    q = (wf / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q, scale


def _rstd(x_f: torch.Tensor, eps: float) -> torch.Tensor:
    """rsqrt(mean(x^2)+eps): float64 sum rounded once to float32, then the float32 add and
    ``torch.rsqrt`` of kernel/sglops.py:36-38. On a CPU torch.rsqrt is 1/sqrt with both steps
    correctly rounded (checked against numpy on 10^7 inputs), which is what the CUDA kernels
    compute; ``1.0 / torch.sqrt(x)`` is NOT the same thing: torch's vectorised float sqrt is one ulp
    off on 0.6 % of inputs."""
    ss = (x_f.double() * x_f.double()).sum(dim=-1, keepdim=True)
    var = (ss / x_f.shape[-1]).float()
    return torch.rsqrt(var + torch.tensor(eps, dtype=torch.float32))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """kernel/sglops.py:34-39: (x_f * rstd) * w -> x.dtype."""
    x_f = x.float()
    y = x_f * _rstd(x_f, eps)
    return (y * weight.float()).to(x.dtype)


def fused_add_rmsnorm(x, residual, weight, eps):
    """kernel/sglops.py:48-55: residual = residual + x (in bf16), then rmsnorm."""
    residual = residual + x
    return rmsnorm(residual, weight, eps), residual


def rmsnorm_quant_fp8(x, weight, eps, residual: Optional[torch.Tensor] = None):
    """RMSNorm.quant_fp8 on the torch path (kernel/rms_fp8.py:120-145 fallbacks):
    rmsnorm -> bf16 -> per_token_quant_fp8. Returns (q, scale[, residual])."""
    if residual is None:
        q, s = per_token_quant_fp8(rmsnorm(x, weight.to(x.dtype), eps))
        return q, s
    h, residual = fused_add_rmsnorm(x, residual, weight.to(x.dtype), eps)
    q, s = per_token_quant_fp8(h)
    return q, s, residual


def silu_bf16(g: torch.Tensor) -> torch.Tensor:
    """F.silu on a bf16 tensor: x / (1 + exp(-x)) rounded to fp32 then bf16."""
    gd = g.double()
    return (gd / (1.0 + torch.exp(-gd))).float().to(torch.bfloat16)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    """kernel/sglops.py:143-151 on bf16: silu (-> bf16) times up (-> bf16)."""
    d = x.shape[-1] // 2
    return silu_bf16(x[..., :d]) * x[..., d:]


def silu_mul_quant_fp8(x: torch.Tensor):
    """kernel/silu_fp8.py:79-83 (fallback): per_token_quant_fp8(silu_and_mul(x))."""
    return per_token_quant_fp8(silu_and_mul(x))


# ---------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------
def fp8_gemm_acc(a_q: torch.Tensor, b_q_nk: torch.Tensor) -> torch.Tensor:
    """Exact-ish fp32 accumulator sum_k a*b from the e4m3 bytes (products of two
    e4m3 values are exact in fp32; the float64 matmul makes the sum order-free)."""
    return (a_q.float().double() @ b_q_nk.float().double().t()).float()


# How fp8_scaled_mm rounds. "two_step" is the reference's torch branch, the one that runs on a CPU:
# torch._scaled_mm with unit scales rounds the accumulator to the output dtype, the scales are applied in
# fp32 and the result is rounded again (kernel/sglops.py:111-135). "one_step" is what the reference's GPU
# branch asks of sgl-kernel's fp8_scaled_mm (kernel/sglops.py:109-110; third-party, sgl-kernel>=0.3.21,<0.4):
# the scales are applied to the fp32 accumulator in the GEMM epilogue and the result is rounded once. The
# CUDA kernels of this repository round once; the two differ by one bf16 ulp on about a third of the outputs.
GEMM_ROUNDING = "two_step"


class gemm_rounding:
    """``with gemm_rounding("one_step"): ...`` switches fp8_scaled_mm for the duration of the block."""

    def __init__(self, mode: str):
        assert mode in ("two_step", "one_step")
        self.mode = mode

    def __enter__(self):
        global GEMM_ROUNDING
        self.prev, GEMM_ROUNDING = GEMM_ROUNDING, self.mode

    def __exit__(self, *a):
        global GEMM_ROUNDING
        GEMM_ROUNDING = self.prev


def fp8_scaled_mm(a_q, b_q_nk, scale_a, scale_b, out_dtype=torch.bfloat16, bias=None):
    """kernel/sglops.py:99-140. Default ("two_step", the torch branch): _scaled_mm with unit scales -> out
    dtype, then * scale_a * scale_b in fp32 -> out dtype (two roundings). See GEMM_ROUNDING."""
    acc = fp8_gemm_acc(a_q, b_q_nk)
    if GEMM_ROUNDING == "two_step":
        acc = acc.to(out_dtype).float()
    out = (acc * scale_a.reshape(-1, 1).float() * scale_b.reshape(1, -1).float()).to(out_dtype)
    if bias is not None:
        out = out + bias.to(out_dtype)
    return out


def fp8_logits_f32(a_q, b_q_nk, scale_a, scale_b) -> torch.Tensor:
    """fp32 logits of the FP8 lm_head: (acc * scale_a) * scale_b, no bf16 rounding."""
    acc = fp8_gemm_acc(a_q, b_q_nk)
    return (acc * scale_a.reshape(-1, 1).float()) * scale_b.reshape(1, -1).float()


# ---------------------------------------------------------------------------
# QK-norm + RoPE + KV write
# ---------------------------------------------------------------------------
def build_cos_sin_cache(head_dim: int, max_position: int, base: float) -> torch.Tensor:
    """layers/rotary.py:21-34."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    t = torch.arange(max_position, dtype=torch.float32)
    freqs = torch.einsum("i,j->ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1)


def _norm_rope(x: torch.Tensor, w: torch.Tensor, eps: float, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """kernel/qk_rope_kv.py:64-98: fp32 x*rstd*w, NeoX halves, separate roundings.
    x: [T, H, D] float32; cos/sin: [T, 1, D/2]. Returns float32 [T, H, D]."""
    half = x.shape[-1] // 2
    rstd = _rstd(x, eps)
    xn = (x * rstd) * w.float()
    x1, x2 = xn[..., :half], xn[..., half:]
    y1 = x1 * cos - x2 * sin
    y2 = x2 * cos + x1 * sin
    return torch.cat((y1, y2), dim=-1)


def qk_norm_rope_store_fp8(q, k, v, positions, loc, q_weight, k_weight, eps, cos_sin_cache, k_cache, v_cache):
    """kernel/qk_rope_kv.py:28-155. q/k/v: bf16 [T, H, D]; returns the new q (bf16)
    and writes k_cache[loc] / v_cache[loc] (e4m3 [slots, Hkv, D]) in place."""
    d = q.shape[-1]
    cs = cos_sin_cache[positions.long()].float()
    cos, sin = cs[:, None, : d // 2], cs[:, None, d // 2 :]
    q_new = _norm_rope(q.float(), q_weight.to(q.dtype), eps, cos, sin).to(q.dtype)
    k_new = _norm_rope(k.float(), k_weight.to(k.dtype), eps, cos, sin).to(torch.bfloat16).to(FP8)
    k_cache[loc.long()] = k_new
    v_cache[loc.long()] = v.to(FP8)
    return q_new


def rope_neox(positions, query, key, head_size: int, cos_sin_cache):
    """Rotation only (no norm) of ``query`` [T, Hq * D] and ``key`` [T, Hkv * D]: what
    ``apply_rope_inplace`` asks of sgl-kernel's ``apply_rope_with_cos_sin_cache_inplace``
    (kernel/sglops.py:65-82; third-party, ``sgl-kernel>=0.3.21,<0.4`` in the reference's
    pyproject.toml:49) and what ``RotaryEmbedding.forward`` intends with its torch formula
    ``q * cos + rotate_half(q) * sin`` (layers/rotary.py:55-71, which raises as written because it
    multiplies 64-wide cos / sin into 128-wide heads): NeoX halves, float32 products and sums, one
    rounding to the input dtype. The rotation arithmetic is the one of ``_norm_rope`` above (pinned by
    the reference's Triton kernel under the interpreter) with the norm step left out. Returns new (q, k)."""
    d = int(head_size)
    cs = cos_sin_cache[positions.long()].float()
    cos, sin = cs[:, None, : d // 2], cs[:, None, d // 2:]

    def rot(x):
        x3 = x.float().view(x.shape[0], x.shape[1] // d, d)
        x1, x2 = x3[..., : d // 2], x3[..., d // 2:]
        return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(x.dtype).view(x.shape)

    return rot(query), rot(key)


def store_kv(k_cache, v_cache, loc, k, v):
    """kvcache/pool.py:121-139 + kernel/sglops.py:207-222 (index_put of converted rows)."""
    k_cache[loc.long()] = k.to(FP8)
    v_cache[loc.long()] = v.to(FP8)


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------
def gather_kv_indices(req_to_token: torch.Tensor, rows: torch.Tensor, seq_lens) -> torch.Tensor:
    """attention/kv_indices.py:122-131 (torch branch)."""
    out = [req_to_token[int(r), : int(s)].to(torch.int32) for r, s in zip(rows.tolist(), list(seq_lens))]
    return torch.cat(out) if out else torch.empty(0, dtype=torch.int32)


def remap_by_parents(table: torch.Tensor, beam_rows: torch.Tensor, parents_rel: torch.Tensor, prefix_len: int,
                     seq_len: int) -> None:
    """scheduler/kv_remap.py:30-66: columns [prefix_len, seq_len) of a request's rows, gathered in
    place by (clamped) parent."""
    seq_len = min(int(seq_len), int(table.shape[1]))
    prefix_len = max(int(prefix_len), 0)
    k = int(beam_rows.numel())
    if prefix_len >= seq_len or k == 0 or int(parents_rel.numel()) != k:
        return
    rows = beam_rows.to(torch.int64)
    parents = parents_rel.to(torch.int64).view(-1).clamp(0, k - 1)
    window = table[rows, prefix_len:seq_len]
    table[rows, prefix_len:seq_len] = window[parents]


def kv_table_step(table, rows, group_indptr, seq_lens, new_slot=None, parents_rel=None, prefix_len=None):
    """One tick on the slot table, the reference's three steps in its order: per-request
    remap_by_parents of the window [prefix, seq_len - 1) (scheduler/scheduler.py:1598-1610), the
    batched write_decode ``table[rows, col] = new_slot`` (scheduler/scheduler.py:1305-1310),
    gather_kv_indices of ``[:seq_len]``. ``table`` is updated in place; returns (indptr, flat list)."""
    n_new = 0 if new_slot is None else 1
    if parents_rel is not None:
        gi = [int(x) for x in group_indptr]
        for g in range(len(gi) - 1):
            a, b = gi[g], gi[g + 1]
            if b > a:
                remap_by_parents(table, rows[a:b], parents_rel[a:b], int(prefix_len[a]), int(seq_lens[a]) - n_new)
    if new_slot is not None:
        table[rows.to(torch.int64), seq_lens.to(torch.int64) - 1] = new_slot.to(table.dtype)
    flat = gather_kv_indices(table, rows, seq_lens.tolist())
    indptr = torch.zeros(len(seq_lens) + 1, dtype=torch.int32)
    indptr[1:] = torch.cumsum(seq_lens.to(torch.int64), 0).to(torch.int32)
    return indptr, flat


def copy_prefill_to_beams_many(table, srcs, beam_rows, m: int) -> None:
    """engine/engine.py:252-274: ``table[beam_rows, :m] = table[srcs, :m].unsqueeze(1)``."""
    table[beam_rows.to(torch.int64), :m] = table[srcs.to(torch.int64), :m].unsqueeze(1)


def decode_attention(q, k_cache, v_cache, kv_indptr, kv_indices, n_rep: int) -> torch.Tensor:
    """attention/flashinfer.py:380-431 (_sdpa, decode branch), evaluated in fp32:
    per row softmax(q K^T / sqrt(D)) V over the row's slot list, GQA by repeat."""
    t, hq, d = q.shape
    out = torch.zeros((t, hq, d), dtype=torch.float32)
    scale = d ** -0.5
    kf, vf = k_cache.float(), v_cache.float()
    for i in range(t):
        idx = kv_indices[int(kv_indptr[i]) : int(kv_indptr[i + 1])].long()
        if idx.numel() == 0:
            continue
        k = kf[idx].repeat_interleave(n_rep, dim=1)  # [L, Hq, D]
        v = vf[idx].repeat_interleave(n_rep, dim=1)
        s = torch.einsum("hd,lhd->hl", q[i].float(), k) * scale
        p = torch.softmax(s, dim=-1)
        out[i] = torch.einsum("hl,lhd->hd", p, v)
    return out.to(q.dtype)


def prefill_attention(q, k_cache, v_cache, qo_indptr, kv_indptr, kv_indices, n_rep: int) -> torch.Tensor:
    """attention/flashinfer.py:380-431 (_sdpa, prefill branch), evaluated in fp32: extend token e of a
    request attends to the keys s <= prefix + e of the request's slot list, prefix = keys - extend
    tokens (the mask ``s_idx <= pfx + e_idx``; ``is_causal`` when the prefix is empty)."""
    t, hq, d = q.shape
    out = torch.zeros((t, hq, d), dtype=torch.float32)
    scale = d ** -0.5
    kf, vf = k_cache.float(), v_cache.float()
    for g in range(len(qo_indptr) - 1):
        q0, q1 = int(qo_indptr[g]), int(qo_indptr[g + 1])
        idx = kv_indices[int(kv_indptr[g]) : int(kv_indptr[g + 1])].long()
        e, sl = q1 - q0, int(idx.numel())
        if e == 0 or sl == 0:
            continue
        pfx = sl - e
        k = kf[idx].repeat_interleave(n_rep, dim=1)  # [L, Hq, D]
        v = vf[idx].repeat_interleave(n_rep, dim=1)
        sc = torch.einsum("ehd,lhd->hel", q[q0:q1].float(), k) * scale
        mask = torch.arange(sl)[None, :] <= (pfx + torch.arange(e)[:, None])
        sc = sc.masked_fill(~mask[None], float("-inf"))
        out[q0:q1] = torch.einsum("hel,lhd->ehd", torch.softmax(sc, dim=-1), v)
    return out.to(q.dtype)


def decoder_layer(x, residual, w, norms, positions, loc, cos_sin_cache, k_cache, v_cache, kv_indptr, kv_indices,
                  hq: int, hkv: int, d: int, eps: float = 1e-6, trace: Optional[dict] = None, attn_out=None):
    """FP8 branch of Qwen3DecoderLayer.forward (models/qwen3.py:198-215) with
    Qwen3Attention.forward (:62-134) and Qwen3MLP.forward (:144-172) inlined.
    ``w`` maps qkv / o / gate_up / down to (e4m3 [N,K], scale [N]); ``norms`` maps
    input / post / q / k to bf16 weights. residual None = first layer. If ``trace``
    is a dict, every intermediate tensor is stored in it. ``attn_out`` (bf16 [rows, hq * d]), when given,
    stands in for this module's attention result: attention is the one stage whose device arithmetic (fp16
    probabilities, approximate exponentials) is only comparable within a tolerance, and a test that wants to
    follow the rest of the chain exactly feeds the device's attention output in here."""
    t = trace if trace is not None else {}
    rows = x.shape[0]
    if residual is None:
        residual = x
        q, s = rmsnorm_quant_fp8(x, norms["input"], eps)
    else:
        q, s, residual = rmsnorm_quant_fp8(x, norms["input"], eps, residual=residual)
    t.update(q1=q, s1=s, res1=residual)
    qkv = fp8_scaled_mm(q, w["qkv"][0], s, w["qkv"][1])
    t["qkv"] = qkv.clone()
    qkv = qkv.view(rows, hq + 2 * hkv, d)
    qn = qk_norm_rope_store_fp8(qkv[:, :hq], qkv[:, hq:hq + hkv], qkv[:, hq + hkv:], positions, loc, norms["q"],
                                norms["k"], eps, cos_sin_cache, k_cache, v_cache)
    t["qn"] = qn
    if attn_out is None:
        a = decode_attention(qn, k_cache, v_cache, kv_indptr, kv_indices, hq // hkv).reshape(rows, -1)
    else:
        a = attn_out.reshape(rows, -1).to(qn.dtype)
    t["attn"] = a
    aq, asc = per_token_quant_fp8(a)
    t.update(aq=aq, asc=asc)
    h = fp8_scaled_mm(aq, w["o"][0], asc, w["o"][1])
    t["o"] = h
    q, s, residual = rmsnorm_quant_fp8(h, norms["post"], eps, residual=residual)
    t.update(q2=q, s2=s, res2=residual)
    gu = fp8_scaled_mm(q, w["gate_up"][0], s, w["gate_up"][1])
    t["gu"] = gu
    yq, ys = silu_mul_quant_fp8(gu)
    t.update(yq=yq, ys=ys)
    out = fp8_scaled_mm(yq, w["down"][0], ys, w["down"][1])
    t["out"] = out
    return out, residual


def model_forward(input_ids, embed, layers, final_norm, positions, loc, cos_sin_cache, k_caches, v_caches, kv_indptr,
                  kv_indices, hq: int, hkv: int, d: int, eps: float = 1e-6, attn_outs=None) -> torch.Tensor:
    """Qwen3ForCausalLM.forward on the FP8 branch (models/qwen3.py:262-273): embedding lookup, the
    decoder layers chained through (hidden, residual), final fused add + RMSNorm. ``layers`` is a list of
    (weights, norms) as ``decoder_layer`` takes them; ``k_caches`` / ``v_caches`` one e4m3 pool per layer
    (written in place at ``loc``); ``attn_outs``: optional per-layer attention results to use instead of
    this module's (see ``decoder_layer``). Returns the normalised hidden states, bf16 [rows, hidden]."""
    x = embed[input_ids.long()]
    residual = None
    for li, (w, norms) in enumerate(layers):
        x, residual = decoder_layer(x, residual, w, norms, positions, loc, cos_sin_cache, k_caches[li], v_caches[li],
                                    kv_indptr, kv_indices, hq, hkv, d, eps,
                                    attn_out=None if attn_outs is None else attn_outs[li])
    if residual is None:
        return rmsnorm(x, final_norm, eps)
    return fused_add_rmsnorm(x, residual, final_norm, eps)[0]


def decode_wave(embed, layers, final_norm, head_w, head_s, sizes, token_base: int, trie, table, k_caches, v_caches,
                prompt_lens, beam_width: int, slot_of_step, cos_sin_cache, hq: int, hkv: int, d: int,
                first_token: int, eps: float = 1e-6, trace: Optional[list] = None, attn_outs=None):
    """A whole wave of trie-constrained SID beam search, every stage from this module: the device
    work of the reference's decode ticks (``BeamRecEngine._forward_decode`` / ``_expand_decode_body``,
    scheduler/scheduler.py:1261-1456) for ``len(prompt_lens)`` requests x ``beam_width`` beams over
    ``len(sizes)`` levels, with the whole level as candidate set. Per level: slot-table tick (window
    remap by last level's parents, new slot, flat lists), model body, FP8 head of the level's rows
    (``head_w`` e4m3 [sum(sizes), hidden], ``head_s`` f32) with the unmasked fp32 log-softmax, beam step.

    ``table``: int32 [n * bw + n, max_seq] slot table whose last n rows are the requests' prompt rows;
    ``slot_of_step[s]``: int64 [n * bw] KV slots the rows write at level s; step 0 starts from one live
    beam per request at the trie root with input token ``first_token``; ``attn_outs[s][layer]``: optional
    attention results to use instead of this module's (see ``decoder_layer``). Returns dict(vals [n, bw] f32
    sorted descending, tokens [n, bw, L] int64, nodes [n, bw]) — the ranking the scheduler returns for
    length_penalty 0 (scheduler/scheduler.py:805-807: stable argsort of the cumulative score)."""
    n, bw, L = len(prompt_lens), int(beam_width), len(sizes)
    rows = n * bw
    table = table.clone()
    rows_idx = torch.arange(rows)
    beam_rows = rows_idx.view(n, bw)
    copy_prefill_to_beams_many(table, torch.arange(rows, rows + n), beam_rows, max(prompt_lens))
    plen_rows = torch.tensor(prompt_lens, dtype=torch.int64).repeat_interleave(bw)
    group_indptr = torch.arange(n + 1) * bw
    cum = torch.full((n, bw), float("-inf"))
    cum[:, 0] = 0.0
    nodes = torch.zeros((n, bw), dtype=torch.int64)
    toks = torch.zeros((n, bw, L), dtype=torch.int64)
    input_ids = torch.full((rows,), int(first_token), dtype=torch.int64)
    positions = plen_rows.clone()
    seq_lens = (plen_rows + 1).to(torch.int32)
    parents = None
    off = 0
    for s in range(L):
        loc = slot_of_step[s].to(torch.int64)
        indptr, flat = kv_table_step(table, rows_idx, group_indptr, seq_lens, new_slot=loc, parents_rel=parents,
                                     prefix_len=plen_rows.to(torch.int32))
        hidden = model_forward(input_ids, embed, layers, final_norm, positions, loc, cos_sin_cache, k_caches, v_caches,
                               indptr, flat, hq, hkv, d, eps, attn_outs=None if attn_outs is None else attn_outs[s])
        hq8, hs = per_token_quant_fp8(hidden)
        logits = fp8_logits_f32(hq8, head_w[off: off + sizes[s]], hs, head_s[off: off + sizes[s]])
        out = sid_beam_step(cum, logits, nodes, trie, token_base + off, bw, token_ids=toks, col=s)
        if trace is not None:
            trace.append(dict(hidden=hidden, logits=logits, vals=out["vals"].clone(), tokens=out["tokens"].clone(),
                              parents=out["parents"].clone()))
        cum = out["vals"]
        toks = out["token_ids"][:, :bw]
        nodes = out["node_ids"][:, :bw] if out["node_ids"] is not None else nodes
        parents = out["parents"].reshape(-1)
        input_ids = out["tokens"].reshape(-1)
        positions = positions + 1
        seq_lens = seq_lens + 1
        off += sizes[s]
    return dict(vals=cum, tokens=toks, nodes=nodes)


# ---------------------------------------------------------------------------
# SID head + beam step
# ---------------------------------------------------------------------------
def log_softmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """logits.py:119-120: F.log_softmax(logits.float(), dim=-1)."""
    return torch.log_softmax(logits.float(), dim=-1)


def row_stats(logits: torch.Tensor):
    mx = logits.float().amax(dim=-1)
    ls = torch.log(torch.exp(logits.float() - mx[:, None]).sum(dim=-1))
    return mx, ls


def logprobs_from_stats(logits, mx, ls):
    return (logits.float() - mx[:, None]) - ls[:, None]


def topk_rows(x: torch.Tensor, k: int):
    """Sorted top-k with the deterministic tie rule (value desc, index asc)."""
    xs = x.float()
    order = np.lexsort((np.arange(xs.shape[-1])[None, :].repeat(xs.shape[0], 0), -xs.numpy().astype(np.float64)), axis=-1)
    idx = torch.from_numpy(order[:, :k].copy())
    return torch.gather(xs, 1, idx), idx


class OracleTrie:
    """Dense tables / sorted-key CSR with the reference's sentinels
    (search/trie.py:160-343): node -1 unconstrained, invalid_node all-false."""

    def __init__(self, keys: np.ndarray, child: np.ndarray, vsz: int, token_base: int, invalid_node: int):
        self.keys = np.asarray(keys, dtype=np.int64)
        self.child = np.asarray(child, dtype=np.int64)
        self.vsz = int(vsz)
        self.token_base = int(token_base)
        self.invalid_node = int(invalid_node)

    def lookup(self, nodes: np.ndarray, toks: np.ndarray):
        """search/trie.py:345-368 (_csr_lookup) + range / sentinel handling of
        mask_candidates (:491-500) and advance_node_ids (:541-558)."""
        nodes = np.asarray(nodes, dtype=np.int64)
        rel = np.asarray(toks, dtype=np.int64) - self.token_base
        in_range = (rel >= 0) & (rel < self.vsz)
        key = np.clip(nodes, 0, None) * self.vsz + np.clip(rel, 0, self.vsz - 1)
        e = self.keys.shape[0]
        if e == 0:
            found = np.zeros(key.shape, dtype=bool)
            child = np.full(key.shape, self.invalid_node, dtype=np.int64)
        else:
            pos = np.searchsorted(self.keys, key)
            posc = np.clip(pos, 0, e - 1)
            found = (pos < e) & (self.keys[posc] == key)
            child = np.where(found, self.child[posc], self.invalid_node)
        found = found & in_range
        child = np.where(found, child, self.invalid_node)
        return found, child

    def allowed(self, nodes, toks):
        found, _ = self.lookup(nodes, toks)
        return found | (np.asarray(nodes) < 0)

    def transition(self, old, toks):
        _, child = self.lookup(old, toks)
        old = np.asarray(old, dtype=np.int64)
        return np.where(old < 0, old, child)


def trie_mask(scores, cand_tokens, node_ids, trie: OracleTrie):
    """kernel/beam_trie.py:104-117."""
    ok = trie.allowed(node_ids.numpy()[:, None].repeat(cand_tokens.shape[1], 1), cand_tokens.numpy())
    return scores.masked_fill(~torch.from_numpy(ok), float("-inf"))


def select_topk_flat(scores: np.ndarray, k: int, masked: bool):
    """Deterministic sorted top-k over a flat score vector: score desc, index asc.
    With ``masked`` a -inf score is not a candidate; missing winners are filled
    with (-inf, index 0) (kernel/csrc/beam_trie.cuh:640-683)."""
    s = scores.astype(np.float32)
    idx_all = np.arange(s.shape[0])
    live = s != -np.inf if masked else np.ones_like(s, dtype=bool)
    cand = idx_all[live]
    order = cand[np.lexsort((cand, -s[cand].astype(np.float64)))]
    take = order[:k]
    vals = np.full(k, -np.inf, dtype=np.float32)
    idx = np.zeros(k, dtype=np.int64)
    vals[: take.shape[0]] = s[take]
    idx[: take.shape[0]] = take
    return vals, idx, int(take.shape[0])


def mask_topk_expand(cum, top_logprobs, top_tokens, select_k, node_ids=None, trie: Optional[OracleTrie] = None,
                     token_ids=None, col=0, do_expand=None, apply_mask=True, apply_expand=True, apply_advance=True):
    """genrec_mask_topk_expand (kernel/beam_trie.py:536-630, csrc/beam_trie.cuh:548-755)
    with the CUDA kernel's deterministic ordering. All tensors on CPU.
    Returns dict(vals, parents, tokens, indices, token_ids, node_ids, child)."""
    n, bw, c = top_logprobs.shape
    k = int(select_k)
    masked = bool(apply_mask and node_ids is not None and trie is not None)
    out = dict(
        vals=torch.empty((n, k)), parents=torch.empty((n, k), dtype=torch.int64),
        tokens=torch.empty((n, k), dtype=torch.int64), indices=torch.empty((n, k), dtype=torch.int64),
        token_ids=None, node_ids=None, child=None,
    )
    do_exp = bool(apply_expand and token_ids is not None)
    do_adv = bool(apply_advance and masked and do_exp)
    # output planes hold max(bw, k) beams: k > bw when a request fans out from fewer input beams than it
    # selects (level 0 from one prefill row, search/expand.py:168-237); rows past k keep their input
    if do_exp:
        out["token_ids"] = torch.zeros((n, max(bw, k), token_ids.shape[2]), dtype=token_ids.dtype)
        out["token_ids"][:, :bw] = token_ids
    if do_adv:
        out["node_ids"] = torch.zeros((n, max(bw, k)), dtype=node_ids.dtype)
        out["node_ids"][:, :bw] = node_ids
    if node_ids is not None and trie is not None:
        out["child"] = torch.zeros((n, k), dtype=torch.int64)
    cols = col if isinstance(col, torch.Tensor) else torch.full((n,), int(col))
    for i in range(n):
        scores = (cum[i].float()[:, None] + top_logprobs[i].float())
        if masked:
            ok = trie.allowed(node_ids[i].numpy()[:, None].repeat(c, 1), top_tokens[i].numpy())
            scores = scores.masked_fill(~torch.from_numpy(ok), float("-inf"))
        vals, idx, _ = select_topk_flat(scores.reshape(-1).numpy(), k, masked)
        parents = idx // c
        toks = top_tokens[i].reshape(-1).numpy()[idx]
        out["vals"][i] = torch.from_numpy(vals)
        out["indices"][i] = torch.from_numpy(idx)
        out["parents"][i] = torch.from_numpy(parents)
        out["tokens"][i] = torch.from_numpy(toks)
        child = None
        if node_ids is not None and trie is not None:
            child = trie.transition(node_ids[i].numpy()[np.clip(parents, 0, bw - 1)], toks)
            out["child"][i] = torch.from_numpy(child)
        if do_exp and (do_expand is None or bool(do_expand[i])):
            rows = token_ids[i][torch.from_numpy(np.clip(parents, 0, bw - 1))].clone()
            cc = int(cols[i])
            if 0 <= cc < rows.shape[1]:
                rows[:, cc] = torch.from_numpy(toks)
            out["token_ids"][i, :k] = rows
            if do_adv:
                out["node_ids"][i, :k] = torch.from_numpy(child)
    return out


def sid_beam_step(cum, logits, node_ids, trie: Optional[OracleTrie], level_tok_base: int, select_k: int,
                  token_ids=None, col=0, stats=None):
    """Full-width step: every code of the level is a candidate of every beam;
    score = cum + ((logit - max) - logsum); -inf scores are not candidates.
    cum [N,BW], logits [N*BW, K_l] fp32, node_ids [N,BW]."""
    n, bw = cum.shape
    kl = logits.shape[1]
    mx, ls = row_stats(logits) if stats is None else stats
    lp = logprobs_from_stats(logits, mx, ls).view(n, bw, kl)
    if trie is None:  # unconstrained: every node id behaves like -1, -inf scores are still dropped
        trie = OracleTrie(np.zeros(0, np.int64), np.zeros(0, np.int64), 1, 0, 0)
        node_ids = torch.full((n, bw), -1, dtype=torch.int64)
    toks = (level_tok_base + torch.arange(kl, dtype=torch.int64))[None, None, :].expand(n, bw, kl)
    return mask_topk_expand(cum, lp, toks, select_k, node_ids=node_ids, trie=trie, token_ids=token_ids, col=col,
                            apply_mask=True)


# ---------------------------------------------------------------------------
# Selection with stop tokens and rank noise (search/select.py, search/expand.py)
# ---------------------------------------------------------------------------
def ranked_candidates(cum, top_logprobs, top_tokens, num_out, perturb=None):
    """_ranked_candidates (search/select.py:72-95): the ``num_out`` best of the rows x C extensions by
    cum + log-prob (+ perturb for the ranking only), in order; ties by lower flat index.
    Returns (scores without noise, parent rows, tokens)."""
    c = int(top_logprobs.shape[1])
    scores = (cum.float()[:, None] + top_logprobs.float()).reshape(-1).numpy()
    key = scores if perturb is None else (torch.from_numpy(scores) + perturb.float().reshape(-1)).numpy()
    order = np.lexsort((np.arange(key.shape[0]), -key.astype(np.float64)))[: int(num_out)]
    idx = torch.from_numpy(order.copy())
    return torch.from_numpy(scores)[idx], idx // c, top_tokens.reshape(-1)[idx]


def joint_select(cum, top_logprobs, top_tokens, stop_token_ids, beam_width, perturb=None):
    """joint_select (search/select.py:98-161) as a plain walk over the C best candidates: a stop-token
    candidate is finished, any other survives, while fewer than ``beam_width`` survivors precede it.
    Returns a dict with the reference's SelectResult field names (unused slots zero)."""
    c, k = int(top_logprobs.shape[1]), int(beam_width)
    scores, parent, tokens = ranked_candidates(cum, top_logprobs, top_tokens, c, perturb)
    stops = set(int(t) for t in stop_token_ids.reshape(-1).tolist())
    out = dict(next_tokens=torch.zeros(k, dtype=torch.int64), parent_idx=torch.zeros(k, dtype=torch.int64),
               new_cum_logprobs=torch.zeros(k), fin_tokens=torch.zeros(c, dtype=torch.int64),
               fin_parent_idx=torch.zeros(c, dtype=torch.int64), fin_cum_logprobs=torch.zeros(c))
    surv = fin = 0
    for i in range(c):
        if surv >= k:
            break  # nothing after the k-th survivor is examined
        if int(tokens[i]) in stops:
            out["fin_tokens"][fin], out["fin_parent_idx"][fin], out["fin_cum_logprobs"][fin] = tokens[i], parent[i], scores[i]
            fin += 1
        else:
            out["next_tokens"][surv], out["parent_idx"][surv], out["new_cum_logprobs"][surv] = tokens[i], parent[i], scores[i]
            surv += 1
    out["num_survivors"], out["num_finished"] = torch.tensor(surv), torch.tensor(fin)
    return out


def select_final_topk(cum, top_logprobs, top_tokens, beam_width, perturb=None):
    """select_final_topk (search/select.py:164-179)."""
    scores, parent, tokens = ranked_candidates(cum, top_logprobs, top_tokens, beam_width, perturb)
    return dict(tokens=tokens, parent_idx=parent, cum_logprobs=scores)


def apply_temperature(logprobs, temperature):
    """apply_temperature (search/expand.py:61-70)."""
    if temperature is None or temperature <= 0.0 or abs(temperature - 1.0) < 1e-6:
        return logprobs
    return log_softmax_rows(logprobs.float() / float(temperature))
