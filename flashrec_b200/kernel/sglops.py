"""Element-wise / GEMM wrappers with the reference's ``flashrec.kernel.sglops``
signatures (kernel/sglops.py:34-222), backed by the sm_100a library.

Unlike the reference there is no torch branch: inputs must be CUDA tensors.
"""

from __future__ import annotations

from typing import Optional

import torch

from flashrec_b200 import _lib
from flashrec_b200._lib import call, ptr, require_cuda, stream_ptr

_FP8 = torch.float8_e4m3fn


def _rows2d(x: torch.Tensor, hidden: int) -> torch.Tensor:
    x2 = x.reshape(-1, hidden)
    return x2 if x2.is_contiguous() else x2.contiguous()


def _bf16(x: torch.Tensor, what: str) -> None:
    if x.dtype != torch.bfloat16:
        raise TypeError(f"{what}: expected bfloat16, got {x.dtype}")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm, bf16 in/out (kernel/sglops.py:34-45)."""
    require_cuda(x, weight)
    _bf16(x, "rmsnorm x")
    hidden = int(weight.numel())
    x2 = _rows2d(x, hidden)
    w = weight.reshape(-1).to(device=x.device, dtype=x.dtype).contiguous()
    out = torch.empty_like(x2)
    call("fr_rmsnorm_bf16", ptr(x2), None, ptr(w), float(eps), ptr(out), x2.shape[0], hidden, stream_ptr(x.device))
    return out.view(x.shape)


def fused_add_rmsnorm(
    x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float
) -> tuple[torch.Tensor, torch.Tensor]:
    """``residual += x`` (in place) then RMSNorm(residual) (kernel/sglops.py:48-61)."""
    require_cuda(x, residual, weight)
    _bf16(x, "fused_add_rmsnorm x")
    _bf16(residual, "fused_add_rmsnorm residual")
    hidden = int(weight.numel())
    x2 = _rows2d(x, hidden)
    r2 = residual.reshape(-1, hidden)
    copy_back = not r2.is_contiguous()
    r2c = r2.contiguous() if copy_back else r2
    w = weight.reshape(-1).to(device=x.device, dtype=x.dtype).contiguous()
    out = torch.empty_like(x2)
    call("fr_rmsnorm_bf16", ptr(x2), ptr(r2c), ptr(w), float(eps), ptr(out), x2.shape[0], hidden,
         stream_ptr(x.device))
    if copy_back:
        residual.copy_(r2c.view(residual.shape))
        return out.view(x.shape), residual
    return out.view(x.shape), r2c.view(residual.shape)


def per_token_quant_fp8(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-row e4m3 quantisation; returns (q [rows, hidden], scale [rows, 1]) (kernel/sglops.py:84-96)."""
    require_cuda(x)
    hidden = int(x.shape[-1])
    x2 = _rows2d(x, hidden)
    if x2.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"per_token_quant_fp8: expected bfloat16 or float32, got {x2.dtype}")
    rows = int(x2.shape[0])
    q = torch.empty((rows, hidden), dtype=_FP8, device=x.device)
    s = torch.empty((rows, 1), dtype=torch.float32, device=x.device)
    call("fr_token_quant_fp8", ptr(x2), int(x2.dtype == torch.float32), ptr(q), ptr(s), rows, hidden,
         stream_ptr(x.device))
    return q, s


def fp8_scaled_mm(
    a_fp8: torch.Tensor,
    b_fp8: torch.Tensor,
    scale_a: torch.Tensor,
    scale_b: torch.Tensor,
    out_dtype: torch.dtype,
    bias: Optional[torch.Tensor] = None,
    *,
    block_n: int = 0,
) -> torch.Tensor:
    """a: [M,K] e4m3 row-major, b: [K,N] e4m3 column-major (the ``.t()`` view of an
    [N,K] weight), scale_a: [M,1] or [M], scale_b: [N] (kernel/sglops.py:99-140).
    ``out_dtype`` is bfloat16, or float32 (no bias) for the lm_head logits."""
    require_cuda(a_fp8, b_fp8, scale_a, scale_b, bias)
    if a_fp8.dtype != _FP8 or b_fp8.dtype != _FP8:
        raise TypeError("fp8_scaled_mm: operands must be float8_e4m3fn")
    if b_fp8.dim() != 2 or b_fp8.stride(0) != 1:
        raise ValueError("fp8_scaled_mm: b must be the column-major [K,N] view of an [N,K] weight")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"fp8_scaled_mm: unsupported out_dtype {out_dtype}")
    m, k = int(a_fp8.shape[0]), int(a_fp8.shape[1])
    n = int(b_fp8.shape[1])
    if int(b_fp8.shape[0]) != k:
        raise ValueError("fp8_scaled_mm: inner dimensions differ")
    a = a_fp8 if a_fp8.stride(1) == 1 else a_fp8.contiguous()
    sa = scale_a.reshape(-1).to(torch.float32)
    sb = scale_b.reshape(-1).to(torch.float32)
    if sa.numel() == 1:
        sa = sa.expand(m)
    if sb.numel() == 1:
        sb = sb.expand(n)
    sa = sa.contiguous()
    sb = sb.contiguous()
    if sa.numel() != m or sb.numel() != n:
        raise ValueError("fp8_scaled_mm: scale shapes do not match [M] / [N]")
    bias_c = None
    if bias is not None:
        bias_c = bias.to(dtype=torch.bfloat16).contiguous()
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    call("fr_gemm_fp8_w8a8", ptr(a), ptr(b_fp8), ptr(sa), ptr(sb), ptr(bias_c), ptr(out),
         int(out_dtype == torch.float32), m, n, k, a.stride(0), b_fp8.stride(1), out.stride(0), int(block_n),
         stream_ptr(a.device))
    return out


def fp8_scaled_mm_add_(a_fp8: torch.Tensor, b_fp8: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor,
                       residual: torch.Tensor, block_n: int = 0) -> torch.Tensor:
    """``residual += fp8_scaled_mm(a, b, ..., bf16)`` in place, with the reference's roundings (the
    GEMM output rounded to bf16, then the bf16 sum): the add half of ``fused_add_rmsnorm`` that
    follows the o_proj / down_proj GEMMs (models/qwen3.py:205-214) folded into the GEMM epilogue.
    ``b_fp8`` is the ``[K, N]`` ``.t()`` view of the weight as for ``fp8_scaled_mm``."""
    require_cuda(a_fp8, b_fp8, scale_a, scale_b, residual)
    if b_fp8.dim() != 2 or b_fp8.stride(0) != 1:
        raise ValueError("fp8_scaled_mm_add_: b must be the column-major [K,N] view of an [N,K] weight")
    m, k = int(a_fp8.shape[0]), int(a_fp8.shape[1])
    n = int(b_fp8.shape[1])
    if residual.dtype != torch.bfloat16 or residual.dim() != 2 or tuple(residual.shape) != (m, n) or \
            residual.stride(1) != 1:
        raise ValueError("fp8_scaled_mm_add_: residual must be a bf16 [M, N] matrix with unit column stride")
    a = a_fp8 if a_fp8.stride(1) == 1 else a_fp8.contiguous()
    sa = scale_a.reshape(-1).to(torch.float32).contiguous()
    sb = scale_b.reshape(-1).to(torch.float32).contiguous()
    if sa.numel() != m or sb.numel() != n:
        raise ValueError("fp8_scaled_mm_add_: scale shapes do not match [M] / [N]")
    call("fr_gemm_fp8_w8a8_add", ptr(a), ptr(b_fp8), ptr(sa), ptr(sb), ptr(residual), m, n, k, a.stride(0),
         b_fp8.stride(1), residual.stride(0), int(block_n), stream_ptr(a.device))
    return residual


def interleave_gate_up(weight_nk: torch.Tensor, scale: torch.Tensor, block: int = 128):
    """Regroup the rows of a merged gate_up weight ``[2d, K]`` (gate rows first, then
    up rows, as ``merge_gate_up`` in the reference's models/weight.py lays them out)
    so that every 2*block rows hold ``block`` gate channels followed by the matching
    ``block`` up channels — the layout ``fp8_scaled_mm_silu_mul`` expects."""
    two_d = int(weight_nk.shape[0])
    d = two_d // 2
    if two_d % 2 or d % block:
        raise ValueError(f"intermediate size {d} must be a multiple of {block}")
    idx = torch.arange(d, device=weight_nk.device).view(d // block, block)
    perm = torch.cat((idx, idx + d), dim=1).reshape(-1)
    return weight_nk.index_select(0, perm).contiguous(), scale.reshape(-1).index_select(0, perm).contiguous()


def fp8_scaled_mm_silu_mul(a_fp8, b_interleaved_nk, scale_a, scale_b_interleaved, *, mode: int = 0):
    """gate_up GEMM with SwiGLU in the epilogue: returns ``(y bf16 [M, d], row_amax f32 [M])``,
    bit-identical to ``silu_and_mul(fp8_scaled_mm(...))`` on the un-interleaved weight."""
    require_cuda(a_fp8, b_interleaved_nk, scale_a, scale_b_interleaved)
    m, k = int(a_fp8.shape[0]), int(a_fp8.shape[1])
    n = int(b_interleaved_nk.shape[0])
    y = torch.empty((m, n // 2), dtype=torch.bfloat16, device=a_fp8.device)
    amax = torch.zeros(m, dtype=torch.float32, device=a_fp8.device)
    sa = scale_a.reshape(-1).to(torch.float32).contiguous()
    call("fr_gemm_fp8_silu_mul", ptr(a_fp8), ptr(b_interleaved_nk), ptr(sa), ptr(scale_b_interleaved), ptr(y),
         ptr(amax), m, n, k, a_fp8.stride(0), b_interleaved_nk.stride(0), y.stride(0), int(mode),
         stream_ptr(a_fp8.device))
    return y, amax


def quant_known_amax_fp8(y: torch.Tensor, row_amax: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-row e4m3 quantisation when max|y| per row is already known."""
    require_cuda(y, row_amax)
    rows, d = int(y.shape[0]), int(y.shape[1])
    q = torch.empty((rows, d), dtype=_FP8, device=y.device)
    s = torch.empty((rows, 1), dtype=torch.float32, device=y.device)
    call("fr_quant_known_amax_fp8", ptr(y), ptr(row_amax), ptr(q), ptr(s), rows, d, stream_ptr(y.device))
    return q, s


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    """SwiGLU ``silu(x[..., :d]) * x[..., d:]`` in bf16 (kernel/sglops.py:143-151)."""
    require_cuda(x)
    _bf16(x, "silu_and_mul x")
    last = int(x.shape[-1])
    d = last // 2
    x2 = _rows2d(x, last)
    out = torch.empty((x2.shape[0], d), dtype=x.dtype, device=x.device)
    call("fr_silu_mul_bf16", ptr(x2), ptr(out), x2.shape[0], d, stream_ptr(x.device))
    return out.view(*x.shape[:-1], d)


def _rope_call(positions, query, key, value, loc, k_cache, v_cache, head_size, cos_sin_cache) -> None:
    d = int(head_size)
    t = int(query.shape[0])
    if query.dtype != torch.bfloat16 or key.dtype != torch.bfloat16:
        raise TypeError("rope: bfloat16 activations only")
    if query.dim() != 2 or key.dim() != 2 or query.stride(1) != 1 or key.stride(1) != 1:
        raise ValueError("rope: query / key must be [T, heads * head_size] with unit column stride")
    n_q, n_kv = int(query.shape[1]) // d, int(key.shape[1]) // d
    if int(cos_sin_cache.shape[-1]) != d:
        raise ValueError("rope: cos_sin_cache width != head_size")
    pos = positions.reshape(-1)[:t].to(dtype=torch.int64).contiguous()
    cs = cos_sin_cache.to(device=query.device, dtype=torch.float32).contiguous()
    args_v = (None, 0, 0)
    loc64 = kc = vc = None
    strides_c = (0, 0, 0, 0)
    slots = 0
    if k_cache is not None:
        if k_cache.dtype != _FP8 or v_cache.dtype != _FP8:
            raise TypeError("rope + store: only the float8_e4m3fn pool is supported")
        v2 = value if value.stride(-1) == 1 else value.contiguous()
        if v2.dim() != 2 or int(v2.shape[1]) != n_kv * d:
            raise ValueError("rope + store: value must be [T, kv_heads * head_size]")
        args_v = (v2, v2.stride(0), d)
        loc64 = loc.reshape(-1)[:t].to(torch.int64).contiguous()
        kc = k_cache.view(k_cache.shape[0], -1)
        vc = v_cache.view(v_cache.shape[0], -1)
        strides_c = (kc.stride(0), d, vc.stride(0), d)
        slots = int(kc.shape[0])
    call("fr_rope_neox_inplace", ptr(query), ptr(key), ptr(args_v[0]), query.stride(0), d, key.stride(0), d,
         args_v[1], args_v[2], ptr(pos), ptr(loc64), ptr(cs), int(cs.shape[0]), ptr(kc), ptr(vc), *strides_c, t, n_q,
         n_kv, d, slots, stream_ptr(query.device))


def apply_rope_inplace(positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor, head_size: int,
                       cos_sin_cache: torch.Tensor) -> bool:
    """NeoX rotation of ``query`` [T, Hq * D] and ``key`` [T, Hkv * D] in place (bf16), angles from
    ``cos_sin_cache`` fp32 [max_pos, D] = [cos | sin]; fp32 arithmetic, one rounding to bf16
    (kernel/sglops.py:65-82, which hands the same arguments to sgl-kernel's
    ``apply_rope_with_cos_sin_cache_inplace``). Always returns True: there is no other branch."""
    require_cuda(positions, query, key, cos_sin_cache)
    if query.numel() == 0:
        return True
    _rope_call(positions, query, key, None, None, None, None, head_size, cos_sin_cache)
    return True


def apply_rope_and_store_kv(positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                            loc: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, head_size: int,
                            cos_sin_cache: torch.Tensor) -> bool:
    """``apply_rope_inplace`` plus the KV write of the same tokens in one launch: the rotated key
    (its bf16 value) and ``value`` are converted to e4m3 and stored at ``k_cache[loc]`` /
    ``v_cache[loc]`` (caches ``[slots, Hkv * D]``). The reference's function of this name
    (kernel/sglops.py:155-205) declines an e4m3 pool with bf16 activations and leaves the store to
    ``TokenToKVPool.store``; the bytes written here are the ones that store would write after the
    rotation. Returns True (KV has been written)."""
    require_cuda(positions, query, key, value, loc, k_cache, v_cache, cos_sin_cache)
    if query.numel() == 0:
        return True
    _rope_call(positions, query, key, value, loc, k_cache, v_cache, head_size, cos_sin_cache)
    return True


def store_kv_cache(
    k_cache: torch.Tensor, v_cache: torch.Tensor, loc: torch.Tensor, k: torch.Tensor, v: torch.Tensor
) -> None:
    """k_cache[loc] = k; v_cache[loc] = v. Caches are [slots, H*D] (or [slots, H, D]) e4m3; k/v are
    [n, H*D] bf16 (converted here) or e4m3 already, as ``TokenToKVPool.store`` hands them over
    (kernel/sglops.py:207-222, kvcache/pool.py:121-139)."""
    require_cuda(k_cache, v_cache, loc, k, v)
    if k_cache.dtype != _FP8:
        raise TypeError("store_kv_cache: only the float8_e4m3fn pool is supported")
    n = int(loc.numel())
    if n == 0:
        return
    row = int(k.numel() // n)
    d = 128 if row % 128 == 0 else 64
    h = row // d
    k2 = k.reshape(n, h, d)
    v2 = v.reshape(n, h, d)
    if k2.stride(-1) != 1:
        k2 = k2.contiguous()
    if v2.stride(-1) != 1:
        v2 = v2.contiguous()
    loc64 = loc.reshape(-1).to(torch.int64).contiguous()
    kc = k_cache.view(k_cache.shape[0], -1)
    vc = v_cache.view(v_cache.shape[0], -1)
    if k2.dtype not in (torch.bfloat16, _FP8) or v2.dtype != k2.dtype:
        raise TypeError(f"store_kv_cache: k / v must both be bfloat16 or float8_e4m3fn, got {k2.dtype} / {v2.dtype}")
    call("fr_store_kv_fp8", ptr(k2), ptr(v2), k2.stride(0), k2.stride(1), v2.stride(0), v2.stride(1), ptr(loc64),
         ptr(kc), ptr(vc), kc.stride(0), d, vc.stride(0), d, n, h, d, int(kc.shape[0]), int(k2.dtype == _FP8),
         stream_ptr(k.device))
