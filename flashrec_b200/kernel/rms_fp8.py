"""Fused (add+)RMSNorm -> per-token e4m3, reference signatures of
``flashrec.kernel.rms_fp8`` (kernel/rms_fp8.py:120-145)."""

from __future__ import annotations

import torch

from flashrec_b200._lib import call, ptr, require_cuda, stream_ptr

_FP8 = torch.float8_e4m3fn


def _launch(x, weight, eps, residual):
    require_cuda(x, weight, residual)
    if x.dtype != torch.bfloat16:
        raise TypeError(f"rms_fp8: expected bfloat16 activations, got {x.dtype}")
    hidden = int(weight.numel())
    x2 = x.reshape(-1, hidden)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    rows = int(x2.shape[0])
    w = weight.reshape(-1).to(device=x.device, dtype=x.dtype).contiguous()
    r2 = None
    if residual is not None:
        r2 = residual.reshape(-1, hidden)
        if r2.shape != x2.shape:
            raise ValueError("rms_fp8: residual shape mismatch")
        if not r2.is_contiguous():
            r2 = r2.contiguous()
    q = torch.empty((rows, hidden), dtype=_FP8, device=x.device)
    scale = torch.empty((rows, 1), dtype=torch.float32, device=x.device)
    call("fr_rms_quant_fp8", ptr(x2), ptr(r2), ptr(w), float(eps), ptr(q), ptr(scale), rows, hidden,
         stream_ptr(x.device))
    res_out = None
    if residual is not None:
        if r2.data_ptr() != residual.data_ptr():
            residual.copy_(r2.view(residual.shape))
            res_out = residual
        else:
            res_out = r2.view(residual.shape)
    return q, scale, res_out


def rmsnorm_per_token_quant_fp8(x: torch.Tensor, weight: torch.Tensor, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    q, scale, _ = _launch(x, weight, eps, None)
    return q, scale


def fused_add_rmsnorm_per_token_quant_fp8(
    x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``residual`` is updated in place (residual += x) and returned."""
    return _launch(x, weight, eps, residual)
