"""Fused SwiGLU + per-token e4m3, reference signature of
``flashrec.kernel.silu_fp8.silu_and_mul_per_token_quant_fp8`` (kernel/silu_fp8.py:86-119)."""

from __future__ import annotations

import torch

from flashrec_b200._lib import call, ptr, require_cuda, stream_ptr

_FP8 = torch.float8_e4m3fn


def silu_and_mul_per_token_quant_fp8(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``silu(x[..., :d]) * x[..., d:]`` then per-token e4m3; ``d = last_dim // 2``."""
    require_cuda(x)
    if x.dtype != torch.bfloat16:
        raise TypeError(f"silu_fp8: expected bfloat16, got {x.dtype}")
    last = int(x.shape[-1])
    if last % 2 != 0:
        raise ValueError("silu_fp8: last dimension must be even")
    d = last // 2
    x2 = x.reshape(-1, last)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    rows = int(x2.shape[0])
    y = torch.empty((rows, d), dtype=_FP8, device=x.device)
    scale = torch.empty((rows, 1), dtype=torch.float32, device=x.device)
    call("fr_silu_mul_quant_fp8", ptr(x2), ptr(y), ptr(scale), rows, d, stream_ptr(x.device))
    return y, scale
