"""Fused Q/K RMSNorm + NeoX RoPE + e4m3 KV scatter, reference signature of
``flashrec.kernel.qk_rope_kv.fused_qk_norm_rope_store_fp8`` (kernel/qk_rope_kv.py:165-250)."""

from __future__ import annotations

import torch

from flashrec_b200._lib import call, ptr, require_cuda, stream_ptr


def fused_qk_norm_rope_store_fp8(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    positions: torch.Tensor,
    loc: torch.Tensor,
    q_weight: torch.Tensor,
    k_weight: torch.Tensor,
    eps: float,
    cos_sin_cache: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
) -> bool:
    """In-place NeoX RoPE on Q; RMSNorm Q/K; scatter unscaled e4m3 K/V.

    ``q/k/v`` are ``[T, H, D]`` views (only D must be contiguous, e.g. slices of
    the fused qkv buffer). Caches are ``[slots, H_kv, D]`` e4m3. Returns True;
    unsupported arguments raise instead of asking the caller to fall back.
    """
    require_cuda(q, k, v, positions, loc, q_weight, k_weight, cos_sin_cache, k_cache, v_cache)
    if q.numel() == 0:
        return True
    if k_cache.dtype != torch.float8_e4m3fn or v_cache.dtype != torch.float8_e4m3fn:
        raise TypeError("fused_qk_norm_rope_store_fp8: caches must be float8_e4m3fn")
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise ValueError("fused_qk_norm_rope_store_fp8: q/k/v must be [T, H, D]")
    if q.dtype != torch.bfloat16:
        raise TypeError("fused_qk_norm_rope_store_fp8: bf16 activations only")
    t, n_q, d = (int(s) for s in q.shape)
    n_kv = int(k.shape[1])
    if k.shape[0] != t or v.shape[0] != t or v.shape[1] != n_kv:
        raise ValueError("fused_qk_norm_rope_store_fp8: q/k/v shape mismatch")
    if int(cos_sin_cache.shape[-1]) != d:
        raise ValueError("fused_qk_norm_rope_store_fp8: cos_sin_cache width != head_dim")
    q_src = q
    if q.stride(-1) != 1:
        q = q.contiguous()
    if k.stride(-1) != 1:
        k = k.contiguous()
    if v.stride(-1) != 1:
        v = v.contiguous()
    pos = positions.reshape(-1)[:t].to(dtype=torch.int64).contiguous()
    loc64 = loc.reshape(-1)[:t].to(dtype=torch.int64).contiguous()
    qw = q_weight.reshape(-1).to(device=q.device, dtype=q.dtype).contiguous()
    kw = k_weight.reshape(-1).to(device=q.device, dtype=q.dtype).contiguous()
    cs = cos_sin_cache.to(device=q.device, dtype=torch.float32).contiguous()
    call("fr_qk_norm_rope_kv_fp8", ptr(q), ptr(k), ptr(v), q.stride(0), q.stride(1), k.stride(0), k.stride(1),
         v.stride(0), v.stride(1), ptr(pos), ptr(loc64), ptr(qw), ptr(kw), float(eps), ptr(cs), int(cs.shape[0]),
         ptr(k_cache), ptr(v_cache), k_cache.stride(0), k_cache.stride(1), v_cache.stride(0), v_cache.stride(1),
         t, n_q, n_kv, d, int(k_cache.shape[0]), stream_ptr(q.device))
    if q_src.data_ptr() != q.data_ptr():
        q_src.copy_(q)
    return True


def fp8_qkv_mm_norm_rope_store(
    a_fp8: torch.Tensor,
    w_fp8_kn: torch.Tensor,
    scale_a: torch.Tensor,
    scale_b: torch.Tensor,
    positions: torch.Tensor,
    loc: torch.Tensor,
    q_weight: torch.Tensor,
    k_weight: torch.Tensor,
    eps: float,
    cos_sin_cache: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    n_q: int,
    n_kv: int,
    q_out: torch.Tensor | None = None,
) -> torch.Tensor:
    """The qkv projection (``fp8_scaled_mm`` with bf16 output, kernel/sglops.py:99-140) with
    ``fused_qk_norm_rope_store_fp8`` applied in the GEMM epilogue: returns the normalised, rotated
    Q ``[T, n_q, 128]`` (bf16) and writes K / V (e4m3) into their pool slots; the qkv matrix itself is
    never written. Same bits as the two calls in sequence (head_dim 128, even head counts).
    ``w_fp8_kn`` is the ``[K, N]`` ``.t()`` view of the merged qkv weight."""
    require_cuda(a_fp8, w_fp8_kn, scale_a, scale_b, positions, loc, q_weight, k_weight, cos_sin_cache, k_cache, v_cache)
    if w_fp8_kn.dim() != 2 or w_fp8_kn.stride(0) != 1:
        raise ValueError("fp8_qkv_mm_norm_rope_store: weight must be the column-major [K,N] view of an [N,K] weight")
    t, k = int(a_fp8.shape[0]), int(a_fp8.shape[1])
    d = 128
    if int(w_fp8_kn.shape[1]) != (n_q + 2 * n_kv) * d or int(w_fp8_kn.shape[0]) != k:
        raise ValueError("fp8_qkv_mm_norm_rope_store: weight shape does not match the head counts")
    if k_cache.dtype != torch.float8_e4m3fn or v_cache.dtype != torch.float8_e4m3fn:
        raise TypeError("fp8_qkv_mm_norm_rope_store: caches must be float8_e4m3fn")
    if int(cos_sin_cache.shape[-1]) != d:
        raise ValueError("fp8_qkv_mm_norm_rope_store: cos_sin_cache width != head_dim")
    a = a_fp8 if a_fp8.stride(1) == 1 else a_fp8.contiguous()
    sa = scale_a.reshape(-1).to(torch.float32).contiguous()
    sb = scale_b.reshape(-1).to(torch.float32).contiguous()
    if q_out is None:
        q_out = torch.empty((t, n_q, d), dtype=torch.bfloat16, device=a.device)
    pos = positions.reshape(-1)[:t].to(dtype=torch.int64).contiguous()
    loc64 = loc.reshape(-1)[:t].to(dtype=torch.int64).contiguous()
    qw = q_weight.reshape(-1).to(device=a.device, dtype=torch.bfloat16).contiguous()
    kw = k_weight.reshape(-1).to(device=a.device, dtype=torch.bfloat16).contiguous()
    cs = cos_sin_cache.to(device=a.device, dtype=torch.float32).contiguous()
    call("fr_gemm_fp8_qkv_rope", ptr(a), ptr(w_fp8_kn), ptr(sa), ptr(sb), ptr(q_out), q_out.stride(0), t, int(n_q),
         int(n_kv), d, k, a.stride(0), w_fp8_kn.stride(1), ptr(pos), ptr(loc64), ptr(qw), ptr(kw), float(eps), ptr(cs),
         int(cs.shape[0]), ptr(k_cache), ptr(v_cache), k_cache.stride(0), k_cache.stride(1), v_cache.stride(0),
         v_cache.stride(1), int(k_cache.shape[0]), stream_ptr(a.device))
    return q_out
