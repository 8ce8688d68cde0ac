"""Restricted SID lm_head: mirror of ``RestrictedLMHead`` (logits.py:9-166).

The reference multiplies by the bf16 lm_head rows of the SID range and takes a
fp32 ``log_softmax``. Here the SID rows are quantised per output channel to e4m3
(the W8A8 head the benchmark configurations ask for), the hidden state is
quantised per token like every other Linear input, the logits stay fp32, and
the log-softmax normaliser is — as in the reference — taken over the whole level,
unmasked.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from flashrec_b200._lib import call, ptr, stream_ptr
from flashrec_b200.kernel.sglops import fp8_scaled_mm, per_token_quant_fp8
from flashrec_b200.layers import quantize_weight_fp8


class RestrictedLMHead:
    def __init__(self, special_token_ids: Optional[List[int]], enabled: bool = True):
        self.ids = list(special_token_ids) if special_token_ids else None
        self.enabled = bool(enabled and self.ids)
        self._token_ids: Optional[torch.Tensor] = None
        self._weight: Optional[torch.Tensor] = None        # e4m3 [K_total, H]
        self._scale: Optional[torch.Tensor] = None         # f32 [K_total]
        self._level_weights: Optional[List[torch.Tensor]] = None
        self._level_scales: Optional[List[torch.Tensor]] = None
        self._level_token_ids: Optional[List[torch.Tensor]] = None
        self._codebook_sizes: Optional[List[int]] = None

    # -- reference properties ------------------------------------------------
    @property
    def token_ids(self) -> Optional[torch.Tensor]:
        return self._token_ids

    @property
    def num_tokens(self) -> Optional[int]:
        return None if self._token_ids is None else int(self._token_ids.numel())

    @property
    def ready(self) -> bool:
        return bool(self.enabled and self._weight is not None and self._token_ids is not None)

    @property
    def per_codebook_ready(self) -> bool:
        return bool(self._level_weights)

    @property
    def num_levels(self) -> int:
        return len(self._level_weights) if self._level_weights else 0

    @property
    def max_codebook_k(self) -> int:
        return max(self._codebook_sizes) if self._codebook_sizes else 0

    def codebook_k(self, level: int) -> int:
        if not self._codebook_sizes or level < 0 or level >= len(self._codebook_sizes):
            return 0
        return self._codebook_sizes[level]

    # -- binding ---------------------------------------------------------------
    def bind(self, lm_weight: torch.Tensor) -> None:
        """Slice the SID rows out of the lm_head once and quantise them per channel.

        ``lm_weight`` is [vocab, H] in bf16/fp32."""
        if lm_weight is None or not self.enabled:
            return
        ids = self.ids or []
        vocab = int(lm_weight.shape[0])
        if (not ids) or min(ids) < 0 or max(ids) >= vocab:
            raise ValueError(f"sid_token_range out of range for vocab {vocab}")
        lo, hi = int(ids[0]), int(ids[-1])
        if hi - lo == len(ids) - 1 and all(b - a == 1 for a, b in zip(ids, ids[1:])):
            # one contiguous range: a narrow() view, as the reference takes (logits.py:108-113)
            self._token_ids = torch.arange(lo, hi + 1, dtype=torch.long, device=lm_weight.device)
            rows = lm_weight.narrow(0, lo, len(ids))
        else:
            # scattered ids: gathered once with index_select, as the reference does (logits.py:114-115)
            self._token_ids = torch.tensor(ids, dtype=torch.long, device=lm_weight.device)
            rows = lm_weight.index_select(0, self._token_ids)
        q, s = quantize_weight_fp8(rows)
        self._weight, self._scale = q, s

    def bind_quantized(self, weight_fp8: torch.Tensor, scale: torch.Tensor) -> None:
        """Bind SID rows that are already e4m3 [K_total, H] + f32 [K_total]."""
        ids = self.ids or []
        self._token_ids = torch.tensor(ids, dtype=torch.long, device=weight_fp8.device)
        self._weight, self._scale = weight_fp8.contiguous(), scale.to(torch.float32).contiguous()

    def bind_codebook(self, codebook_sizes: List[int]) -> None:
        """Per-level zero-copy ``narrow()`` views; call after ``bind`` (logits.py:66-90)."""
        if self._weight is None or not self.enabled:
            return
        if sum(codebook_sizes) != self._weight.shape[0]:
            return
        self._codebook_sizes = list(codebook_sizes)
        self._level_weights, self._level_scales, self._level_token_ids = [], [], []
        off = 0
        for size in codebook_sizes:
            self._level_weights.append(self._weight.narrow(0, off, size))
            self._level_scales.append(self._scale.narrow(0, off, size))
            self._level_token_ids.append(self._token_ids.narrow(0, off, size))
            off += size

    # -- compute ---------------------------------------------------------------
    def _logits(self, hidden: torch.Tensor, w: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
        h2 = hidden.reshape(-1, hidden.shape[-1])
        q, a_scale = per_token_quant_fp8(h2)
        return fp8_scaled_mm(q, w.t(), a_scale, s, torch.float32)

    def logits_level(self, hidden: torch.Tensor, level: int):
        """fp32 logits of one level and their row statistics:
        ``(logits [T, K_l], row_max [T], row_logsum [T], token_ids [K_l])``."""
        if not self._level_weights or level < 0 or level >= len(self._level_weights):
            raise RuntimeError("RestrictedLMHead.logits_level requires bind_codebook()")
        logits = self._logits(hidden, self._level_weights[level], self._level_scales[level])
        t, k = logits.shape
        mx = torch.empty(t, dtype=torch.float32, device=logits.device)
        ls = torch.empty(t, dtype=torch.float32, device=logits.device)
        call("fr_logsumexp_rows", ptr(logits), logits.stride(0), ptr(mx), ptr(ls), None, 0, t, k,
             stream_ptr(logits.device))
        return logits, mx, ls, self._level_token_ids[level]

    def _logprobs(self, hidden, w, s, out=None) -> torch.Tensor:
        logits = self._logits(hidden, w, s)
        t, k = logits.shape
        mx = torch.empty(t, dtype=torch.float32, device=logits.device)
        ls = torch.empty(t, dtype=torch.float32, device=logits.device)
        dst = logits if out is None else out
        call("fr_logsumexp_rows", ptr(logits), logits.stride(0), ptr(mx), ptr(ls), ptr(dst), dst.stride(0), t, k,
             stream_ptr(logits.device))
        return dst

    def _restricted_logprobs(self, hidden: torch.Tensor) -> torch.Tensor:
        return self._logprobs(hidden, self._weight, self._scale)

    def compute_level(self, hidden: torch.Tensor, level: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Per-codebook logprobs: GEMM only against the level's rows (logits.py:122-138)."""
        if not self._level_weights or level < 0 or level >= len(self._level_weights):
            if self._weight is None or self._token_ids is None:
                raise RuntimeError("RestrictedLMHead.compute_level requires bind_codebook()")
            return self._restricted_logprobs(hidden), self._token_ids
        return (
            self._logprobs(hidden, self._level_weights[level], self._level_scales[level]),
            self._level_token_ids[level],
        )

    def compute_into(self, hidden: torch.Tensor, lm_weight, out: torch.Tensor) -> torch.Tensor:
        """Write restricted logprobs into ``out`` [T, K] fp32 (logits.py:140-155)."""
        del lm_weight
        if self._weight is None or self._token_ids is None:
            raise RuntimeError("RestrictedLMHead.compute_into requires bind()")
        return self._logprobs(hidden, self._weight, self._scale, out=out)

    def compute(self, hidden: torch.Tensor, lm_weight=None):
        """Return (logprobs [T, K], candidate_token_ids)."""
        if self._weight is None and lm_weight is not None:
            self.bind(lm_weight)
        if not self.ready:
            raise RuntimeError("RestrictedLMHead is not bound / not enabled")
        return self._restricted_logprobs(hidden), self._token_ids


def topk_rows(x: torch.Tensor, k: int, row_max=None, row_logsum=None):
    """Per-row sorted top-k (values, int64 indices); ties -> smaller index. With the
    row statistics given, the values are log-probs. Stands in for ``torch.topk(...,
    sorted=True)`` on the expand path (scheduler/scheduler.py:1476-1482)."""
    x2 = x.reshape(-1, x.shape[-1])
    rows, cols = x2.shape
    vals = torch.empty((rows, k), dtype=torch.float32, device=x.device)
    idx = torch.empty((rows, k), dtype=torch.int64, device=x.device)
    call("fr_topk_rows", ptr(x2), x2.stride(0), ptr(row_max), ptr(row_logsum), ptr(vals), ptr(idx), rows, cols,
         int(k), stream_ptr(x.device))
    return vals.view(*x.shape[:-1], k), idx.view(*x.shape[:-1], k)
