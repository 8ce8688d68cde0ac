"""Beam selection with stop tokens and sampling noise: a mirror of the reference's ``search/select.py``
(``SelectResult``, ``FinalSelect``, ``joint_select`` :98-161, ``select_final_topk`` :164-179) and of the two
samplers of ``search/expand.py`` (``apply_temperature`` :61-70, ``gumbel_like`` :73-79), on this library's
selection kernels. The reference calls these once per request with ``[num_rows]`` / ``[num_rows, C]`` tensors;
here a leading group dimension is accepted as well (``[G, num_rows]`` / ``[G, num_rows, C]``), one CTA per group,
and every output then carries the same leading dimension.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from flashrec_b200._lib import call, load, ptr, require_cuda, stream_ptr


@dataclass
class SelectResult:
    """Fixed-shape outputs of one expansion step: survivor slots are valid in ``[0, num_survivors)``,
    finished slots in ``[0, num_finished)``, the rest are zero."""

    next_tokens: torch.Tensor        # [K] int64
    parent_idx: torch.Tensor         # [K] int64, row of the input frontier
    new_cum_logprobs: torch.Tensor   # [K] float32
    num_survivors: torch.Tensor      # [] int64
    fin_tokens: torch.Tensor         # [C] int64
    fin_parent_idx: torch.Tensor     # [C] int64
    fin_cum_logprobs: torch.Tensor   # [C] float32
    num_finished: torch.Tensor       # [] int64


@dataclass
class FinalSelect:
    tokens: torch.Tensor        # [K] int64
    parent_idx: torch.Tensor    # [K] int64
    cum_logprobs: torch.Tensor  # [K] float32


def _prep(cum_logprobs, top_logprobs, top_tokens, perturb):
    require_cuda(cum_logprobs, top_logprobs, top_tokens)
    grouped = top_logprobs.dim() == 3
    lp = top_logprobs if grouped else top_logprobs.unsqueeze(0)
    g, r, c = (int(x) for x in lp.shape)
    lp = lp.to(torch.float32).contiguous()
    cum = cum_logprobs.reshape(g, r).to(torch.float32).contiguous()
    tok = top_tokens.reshape(g, r, c).to(torch.int64).contiguous()
    pt = None
    if perturb is not None:
        require_cuda(perturb)
        pt = perturb.reshape(g, r, c).to(torch.float32).contiguous()
    return grouped, g, r, c, cum, lp, tok, pt


def joint_select(
    cum_logprobs: torch.Tensor,
    top_logprobs: torch.Tensor,
    top_tokens: torch.Tensor,
    stop_token_ids: torch.Tensor,
    beam_width: int,
    perturb: Optional[torch.Tensor] = None,
) -> SelectResult:
    """One expansion step: walk the ``C`` best of the ``rows x C`` extensions in score order; stop-token candidates
    finish, the others survive while fewer than ``beam_width`` survivors precede them. ``perturb`` is added for
    ranking only. Pass an empty ``stop_token_ids`` tensor for no stop check. No host synchronisation."""
    grouped, g, r, c, cum, lp, tok, pt = _prep(cum_logprobs, top_logprobs, top_tokens, perturb)
    k = int(beam_width)
    dev = lp.device
    stop = stop_token_ids.to(device=dev, dtype=torch.int64).contiguous()
    ws = torch.empty(int(load().fr_joint_select_workspace_bytes(g, c)), dtype=torch.uint8, device=dev)
    out = SelectResult(
        next_tokens=torch.empty((g, k), dtype=torch.int64, device=dev),
        parent_idx=torch.empty((g, k), dtype=torch.int64, device=dev),
        new_cum_logprobs=torch.empty((g, k), dtype=torch.float32, device=dev),
        num_survivors=torch.empty((g,), dtype=torch.int64, device=dev),
        fin_tokens=torch.empty((g, c), dtype=torch.int64, device=dev),
        fin_parent_idx=torch.empty((g, c), dtype=torch.int64, device=dev),
        fin_cum_logprobs=torch.empty((g, c), dtype=torch.float32, device=dev),
        num_finished=torch.empty((g,), dtype=torch.int64, device=dev),
    )
    call("fr_joint_select", ptr(out.next_tokens), ptr(out.parent_idx), ptr(out.new_cum_logprobs), ptr(out.num_survivors),
         ptr(out.fin_tokens), ptr(out.fin_parent_idx), ptr(out.fin_cum_logprobs), ptr(out.num_finished), ptr(cum), ptr(lp),
         ptr(tok), ptr(pt), ptr(stop) if stop.numel() else None, int(stop.numel()), ptr(ws), int(ws.numel()), g, r, c, k,
         stream_ptr(dev))
    if not grouped:
        out = SelectResult(*(getattr(out, f).reshape(getattr(out, f).shape[1:]) for f in out.__dataclass_fields__))
    return out


def select_final_topk(
    cum_logprobs: torch.Tensor,
    top_logprobs: torch.Tensor,
    top_tokens: torch.Tensor,
    beam_width: int,
    perturb: Optional[torch.Tensor] = None,
) -> FinalSelect:
    """The step that ends by length: the best ``beam_width`` extensions, in order, all finished."""
    grouped, g, r, c, cum, lp, tok, pt = _prep(cum_logprobs, top_logprobs, top_tokens, perturb)
    k = int(beam_width)
    dev = lp.device
    tokens = torch.empty((g, k), dtype=torch.int64, device=dev)
    parent = torch.empty((g, k), dtype=torch.int64, device=dev)
    vals = torch.empty((g, k), dtype=torch.float32, device=dev)
    idx = torch.empty((g, k), dtype=torch.int64, device=dev)
    call("fr_select_final_topk", ptr(tokens), ptr(parent), ptr(vals), ptr(idx), ptr(cum), ptr(lp), ptr(tok), ptr(pt),
         g, r, c, k, stream_ptr(dev))
    if not grouped:
        tokens, parent, vals = tokens[0], parent[0], vals[0]
    return FinalSelect(tokens=tokens, parent_idx=parent, cum_logprobs=vals)


def apply_temperature(logprobs: torch.Tensor, temperature: float) -> torch.Tensor:
    """``log_softmax(logits / T)`` from log-softmax rows (a second log-softmax removes the per-row constant);
    ``T <= 0`` and ``T == 1`` return the input. The row statistics come from ``fr_logsumexp_rows``."""
    if temperature is None or temperature <= 0.0 or abs(temperature - 1.0) < 1e-6:
        return logprobs
    require_cuda(logprobs)
    x = (logprobs.to(torch.float32) / float(temperature)).contiguous()
    rows = x.reshape(-1, x.shape[-1])
    out = torch.empty_like(rows)
    mx = torch.empty(rows.shape[0], dtype=torch.float32, device=x.device)
    ls = torch.empty_like(mx)
    call("fr_logsumexp_rows", ptr(rows), rows.stride(0), ptr(mx), ptr(ls), ptr(out), out.stride(0), int(rows.shape[0]),
         int(rows.shape[1]), stream_ptr(x.device))
    return out.reshape(x.shape)


def gumbel_like(x: torch.Tensor) -> torch.Tensor:
    """Standard Gumbel(0, 1) noise of ``x``'s shape (float32): added to log-probs before a top-k it turns the
    selection into sampling without replacement. The uniform draws come from torch's generator."""
    eps = torch.finfo(torch.float32).tiny
    u = torch.rand_like(x, dtype=torch.float32).clamp_min(eps)
    return -torch.log(-torch.log(u))
