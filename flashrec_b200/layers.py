"""Layer-level mirrors of the reference's ``flashrec.layers`` for the FP8 decode
path: ``Linear`` (layers/linear.py:66-172), ``RMSNorm`` (layers/norm.py:14-42)
and the RoPE cos/sin cache of ``RotaryEmbedding`` (layers/rotary.py:18-34).
Same attribute names, argument meaning and call order; the arithmetic runs in
the sm_100a library.
"""

from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from flashrec_b200.kernel.rms_fp8 import (
    fused_add_rmsnorm_per_token_quant_fp8,
    rmsnorm_per_token_quant_fp8,
)
from flashrec_b200.kernel.sglops import (
    fp8_scaled_mm,
    fp8_scaled_mm_add_,
    fused_add_rmsnorm,
    per_token_quant_fp8,
    rmsnorm,
)

_FP8 = torch.float8_e4m3fn


def quantize_weight_fp8(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-output-channel absmax quantisation to e4m3: (q [N,K], scale [N]) (layers/linear.py:26-32)."""
    w = weight if weight.dtype == torch.float32 else weight.float()
    q, s = per_token_quant_fp8(w.contiguous())
    return q, s.reshape(-1)


def as_channel_scale(scale: torch.Tensor, out_features: int, device=None) -> torch.Tensor:
    """Per-tensor scale -> length ``out_features``; per-channel unchanged (layers/linear.py:35-57)."""
    s = scale.detach().to(dtype=torch.float32).reshape(-1)
    if device is not None:
        s = s.to(device=device)
    n = int(s.numel())
    if n == 1:
        return s.expand(out_features).contiguous()
    if n == out_features:
        return s.contiguous()
    raise ValueError(
        f"FP8 weight_scale has {n} values, expected 1 (per-tensor) or {out_features} (per-channel); "
        "block-wise scales are not supported"
    )


class Linear:
    """W8A8 linear layer. ``_fp8_weight`` is the ``[K, N]`` column-major view of the
    stored ``[N, K]`` e4m3 weight, ``_fp8_scale`` is ``[N]`` f32, as in the reference."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False):
        self.in_features = int(in_features)
        self.out_features = int(out_features)
        self.bias: Optional[torch.Tensor] = None
        self._has_bias = bool(bias)
        self._fp8_weight: Optional[torch.Tensor] = None
        self._fp8_scale: Optional[torch.Tensor] = None
        self._use_fp8 = False

    def load(
        self,
        weight: torch.Tensor,
        bias: Optional[torch.Tensor] = None,
        quantize_fp8: bool = False,
        weight_scale: Optional[torch.Tensor] = None,
    ) -> None:
        device = weight.device
        if weight.dtype == torch.uint8 and weight_scale is not None:
            raise NotImplementedError("NVFP4 checkpoints are not supported")
        if weight.dtype == _FP8:
            scale = (
                torch.ones(self.out_features, dtype=torch.float32, device=device)
                if weight_scale is None
                else as_channel_scale(weight_scale, self.out_features, device)
            )
            self._fp8_weight = weight.contiguous().t()
            self._fp8_scale = scale
        elif quantize_fp8:
            q, scale = quantize_weight_fp8(weight)
            self._fp8_weight = q.t()
            self._fp8_scale = scale.to(device=device)
        else:
            raise NotImplementedError("flashrec_b200.Linear implements the FP8 (W8A8) path only")
        self._use_fp8 = True
        if bias is not None:
            self.bias = bias

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.forward(x)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Dynamic per-token quantisation of ``x`` then the FP8 GEMM (layers/linear.py:144-151)."""
        orig = x.shape
        x2 = x.reshape(-1, orig[-1])
        q, a_scale = per_token_quant_fp8(x2)
        out_dtype = x.dtype if x.dtype == torch.bfloat16 else torch.bfloat16
        return self._fp8_mm(q, a_scale, orig, out_dtype)

    def forward_fp8(self, q: torch.Tensor, a_scale: torch.Tensor, orig_shape: tuple, out_dtype: torch.dtype):
        """GEMM from a pre-quantised activation. ``q`` is [M, K] e4m3 (layers/linear.py:134-142)."""
        return self._fp8_mm(q, a_scale, orig_shape, out_dtype)

    def forward_fp8_add_(self, q: torch.Tensor, a_scale: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        """``residual += self(q)`` in place on the bf16 residual stream [M, out_features] (bias-free layers)."""
        if not self._use_fp8:
            raise RuntimeError("Linear.load() has not been called")
        if self.bias is not None:
            raise RuntimeError("forward_fp8_add_: layers with a bias are not supported")
        return fp8_scaled_mm_add_(q, self._fp8_weight, a_scale, self._fp8_scale, residual)

    def _fp8_mm(self, q, a_scale, orig_shape, out_dtype):
        if not self._use_fp8:
            raise RuntimeError("Linear.load() has not been called")
        bias = self.bias.to(dtype=out_dtype) if self.bias is not None else None
        out = fp8_scaled_mm(q, self._fp8_weight, a_scale, self._fp8_scale, out_dtype, bias)
        return out.view(*orig_shape[:-1], self.out_features)


class RMSNorm:
    def __init__(self, hidden_size: int, eps: float = 1e-6, device=None):
        self.weight = torch.ones(hidden_size, dtype=torch.bfloat16, device=device)
        self.eps = float(eps)
        self.hidden_size = int(hidden_size)

    def __call__(self, x, residual=None):
        return self.forward(x, residual)

    def forward(
        self, x: torch.Tensor, residual: Optional[torch.Tensor] = None
    ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
        if residual is None:
            return rmsnorm(x, self.weight, self.eps)
        return fused_add_rmsnorm(x, residual, self.weight, self.eps)

    def quant_fp8(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        """RMSNorm then per-token e4m3. With residual: fused add+norm+quant (layers/norm.py:28-42)."""
        if residual is None:
            return rmsnorm_per_token_quant_fp8(x, self.weight, self.eps)
        return fused_add_rmsnorm_per_token_quant_fp8(x, residual, self.weight, self.eps)


def build_cos_sin_cache(head_dim: int, max_position: int, base: float, device=None) -> torch.Tensor:
    """fp32 ``[max_position, head_dim]`` = ``[cos | sin]`` with ``inv_freq = base^(-2i/D)``,
    computed on the CPU with the reference's exact expression (layers/rotary.py:21-34)
    so that the table is bit-identical, then moved to ``device``."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    t = torch.arange(max_position, dtype=torch.float32)
    freqs = torch.einsum("i,j->ij", t, inv_freq)
    cache = torch.cat((freqs.cos(), freqs.sin()), dim=-1)
    return cache.to(device) if device is not None else cache


class RotaryEmbedding:
    def __init__(self, head_dim: int, max_position: int, base: float, device=None):
        self.head_dim = int(head_dim)
        self.cos_sin_cache = build_cos_sin_cache(head_dim, max_position, base, device)
