"""Trie mask / advance / expand and the fused mask+top-K+expand step, with the
reference's ``flashrec.kernel.beam_trie`` signatures (kernel/beam_trie.py:82-690).

Differences from the reference, all on purpose:
  * no torch fallback — the CUDA library is the only path;
  * the trie argument may be the reference's dense ``allow_table`` /
    ``next_node`` tensors, or a :class:`flashrec_b200.trie.DeviceTrie` (dense,
    sorted-key CSR or per-node bitmap), so CSR catalogs take the fused kernel too;
  * beam widths up to 4096 (the reference kernel stops at 512).
"""

from __future__ import annotations

import ctypes
from typing import NamedTuple, Optional, Sequence, Union

import torch

from flashrec_b200 import _lib
from flashrec_b200._lib import FrTrie, call, ptr, require_cuda, stream_ptr

_NEG_INF = float("-inf")


class GenrecFusedResult(NamedTuple):
    vals: torch.Tensor
    parents: torch.Tensor
    tokens: torch.Tensor
    indices: torch.Tensor
    token_ids: Optional[torch.Tensor]
    node_ids: Optional[torch.Tensor]


def _as_allow_u8(allow_table: torch.Tensor) -> torch.Tensor:
    return allow_table.view(torch.uint8) if allow_table.dtype == torch.bool else allow_table


def make_dense_trie(
    allow_table: torch.Tensor, next_node: Optional[torch.Tensor], token_base: int, invalid_node: int
) -> tuple[FrTrie, list]:
    """``fr_trie`` descriptor over the reference's dense tables; the returned
    list keeps the tensors the descriptor points at alive."""
    allow = _as_allow_u8(allow_table)
    if not allow.is_contiguous():
        allow = allow.contiguous()
    keep = [allow]
    tr = FrTrie()
    tr.kind = _lib.FR_TRIE_DENSE
    tr.allow = allow.data_ptr()
    tr.n_rows = int(allow.shape[0])
    tr.vsz = int(allow.shape[1])
    tr.token_base = int(token_base)
    tr.invalid_node = int(invalid_node)
    if next_node is not None:
        if next_node.dtype not in (torch.int32, torch.int64):
            raise TypeError("next_node must be int32 or int64")
        nn = next_node if next_node.is_contiguous() else next_node.contiguous()
        keep.append(nn)
        tr.next = nn.data_ptr()
        tr.next_is_i32 = int(nn.dtype == torch.int32)
    return tr, keep


def _resolve_trie(trie_or_table, next_node, token_base, invalid_node):
    """Accept a DeviceTrie-like object (has ``.descriptor()``) or dense tensors."""
    if trie_or_table is None:
        return None, []
    if hasattr(trie_or_table, "descriptor"):
        return trie_or_table.descriptor(), [trie_or_table]
    return make_dense_trie(trie_or_table, next_node, token_base, invalid_node)


def _i64(t: torch.Tensor) -> torch.Tensor:
    t = t if t.dtype == torch.int64 else t.to(torch.int64)
    return t if t.is_contiguous() else t.contiguous()


def _f32(t: torch.Tensor) -> torch.Tensor:
    t = t if t.dtype == torch.float32 else t.to(torch.float32)
    return t if t.is_contiguous() else t.contiguous()


def trie_mask_candidates(
    scores: torch.Tensor,
    cand_tokens: torch.Tensor,
    node_ids: torch.Tensor,
    allow_table,
    token_base: int,
    out: Optional[torch.Tensor] = None,
    neg_inf: float = _NEG_INF,
) -> torch.Tensor:
    """scores[r, c] kept where ``cand_tokens[r, c]`` continues node ``node_ids[r]``, else ``neg_inf``."""
    require_cuda(scores, cand_tokens, node_ids)
    tr, keep = _resolve_trie(allow_table, None, token_base, 0)
    s_in = _f32(scores)
    if out is None:
        out = torch.empty_like(s_in)
    rows, cols = int(s_in.shape[0]), int(s_in.shape[1])
    # converted copies stay bound to names until the launch has been issued: a temporary freed
    # before the call could be handed to the next conversion by the caching allocator
    tok_c, nodes_c = _i64(cand_tokens), _i64(node_ids)
    call("fr_trie_mask", ptr(out), ptr(s_in), ptr(tok_c), ptr(nodes_c), ctypes.byref(tr),
         float(neg_inf), rows, cols, stream_ptr(scores.device))
    del keep, tok_c, nodes_c
    return out


def trie_advance_nodes(
    node_ids: torch.Tensor,
    parents: torch.Tensor,
    tokens: torch.Tensor,
    next_node,
    token_base: int,
    invalid_node: int,
    out: Optional[torch.Tensor] = None,
    allow_table: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``next[node_ids[parents[i]], tokens[i]]`` with the reference's sentinels.

    ``next_node`` is the dense table (then ``allow_table`` is not needed) or a DeviceTrie."""
    require_cuda(node_ids, parents, tokens)
    if hasattr(next_node, "descriptor"):
        tr, keep = next_node.descriptor(), [next_node]
    else:
        if next_node.dtype not in (torch.int32, torch.int64):
            raise TypeError("next_node must be int32 or int64")
        nn = next_node if next_node.is_contiguous() else next_node.contiguous()
        keep = [nn]
        tr = FrTrie()
        tr.kind = _lib.FR_TRIE_DENSE
        tr.next = nn.data_ptr()
        tr.next_is_i32 = int(nn.dtype == torch.int32)
        # advance never reads the allow table; any non-null device pointer satisfies the descriptor check
        tr.allow = allow_table.data_ptr() if allow_table is not None else nn.data_ptr()
        tr.n_rows = int(nn.shape[0])
        tr.vsz = int(nn.shape[1])
        tr.token_base = int(token_base)
        tr.invalid_node = int(invalid_node)
    nodes = _i64(node_ids)
    par = _i64(parents.to(device=node_ids.device)).view(-1)
    tok = _i64(tokens.to(device=node_ids.device)).view(-1)
    if out is None:
        out = torch.empty_like(par)
    if nodes.dim() == 1:
        n, bw, k = 1, int(nodes.shape[0]), int(par.numel())
    else:
        n, bw = int(nodes.shape[0]), int(nodes.shape[1])
        k = int(par.numel()) // max(n, 1)
    call("fr_trie_advance", ptr(out), ptr(nodes), ptr(par), ptr(tok), ctypes.byref(tr), n, bw, k,
         stream_ptr(node_ids.device))
    del keep
    return out.view(parents.shape) if nodes.dim() > 1 else out


def trie_advance_nodes_batched(node_ids, parents, tokens, next_node, token_base, invalid_node, out=None):
    return trie_advance_nodes(node_ids, parents, tokens, next_node, token_base, invalid_node, out)


def beam_expand_token_ids(
    token_ids: torch.Tensor,
    parents: torch.Tensor,
    new_tokens: torch.Tensor,
    col: int,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Gather parent token rows and write the new token column. ``token_ids`` is
    ``[bw, width]`` or ``[n, bw, width]`` int64."""
    require_cuda(token_ids, parents, new_tokens)
    tid = _i64(token_ids)
    if tid.dim() == 2:
        n, (bw, width) = 1, tid.shape
    else:
        n, bw, width = tid.shape
    col = int(col)
    if col >= width:  # the reference pads one column in this case
        tid = torch.nn.functional.pad(tid, (0, 1))
        width += 1
    par = _i64(parents.to(device=tid.device)).reshape(-1)
    tok = _i64(new_tokens.to(device=tid.device)).reshape(-1)
    if out is None or out.data_ptr() == tid.data_ptr() or tuple(out.shape) != tuple(tid.shape):
        out = torch.empty_like(tid)
    call("fr_beam_expand", ptr(out), ptr(tid), ptr(par), ptr(tok), int(n), int(bw), int(width), col,
         stream_ptr(tid.device))
    return out


def _canonical_device(device: torch.device) -> torch.device:
    device = torch.device(device)
    if device.type == "cuda" and device.index is None and torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return device


class GenrecFusedWorkspace:
    """Grow-only named buffers + ping-pong planes (kernel/beam_trie.py:247-299)."""

    def __init__(self) -> None:
        self._bufs: dict = {}

    def get(self, name: str, shape: tuple, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        shape = tuple(int(x) for x in shape)
        device = _canonical_device(device)
        t = self._bufs.get(name)
        tail = shape[1:]
        same_tail = (
            t is not None
            and t.dtype == dtype
            and t.device == device
            and t.ndim == len(shape)
            and tuple(int(x) for x in t.shape[1:]) == tail
        )
        if t is None or not same_tail or int(t.size(0)) < shape[0]:
            grown = list(shape)
            if same_tail:
                grown[0] = max(shape[0], int(t.size(0)))
            t = torch.empty(*grown, dtype=dtype, device=device)
            self._bufs[name] = t
        return t[: shape[0]]

    def get_filled(self, name, shape, dtype, device, value) -> torch.Tensor:
        prev = self._bufs.get(name)
        view = self.get(name, shape, dtype, device)
        full = self._bufs[name]
        if prev is None or prev.data_ptr() != full.data_ptr() or prev.shape != full.shape:
            full.fill_(value)
        return view

    def pair(self, name, shape, dtype, device) -> tuple[torch.Tensor, torch.Tensor]:
        return self.get(f"{name}_a", shape, dtype, device), self.get(f"{name}_b", shape, dtype, device)


def tensors_alias(a: torch.Tensor, b: torch.Tensor) -> bool:
    return (
        a.dtype == b.dtype
        and a.device == b.device
        and tuple(a.shape) == tuple(b.shape)
        and a.data_ptr() == b.data_ptr()
        and a.stride() == b.stride()
    )


def _pingpong_io(ws, name, user, dtype, device):
    """Never gather from the plane being written (kernel/beam_trie.py:355-373)."""
    shape = tuple(int(x) for x in user.shape)
    a, b = ws.pair(name, shape, dtype, device)
    if tensors_alias(user, a):
        return a, b
    if tensors_alias(user, b):
        return b, a
    dst = b if user.data_ptr() == a.data_ptr() else a
    return user, dst


def _col_i32(col: Union[int, torch.Tensor], n: int, device, ws: GenrecFusedWorkspace) -> torch.Tensor:
    out = ws.get("col", (n,), torch.int32, device)
    if isinstance(col, torch.Tensor):
        src = col.to(device=device, dtype=torch.int32).reshape(-1)
        if int(src.numel()) == 1:
            out.copy_(src.expand(n))
        elif int(src.numel()) >= n:
            out.copy_(src[:n])
        else:
            raise ValueError(f"col length {int(src.numel())} < n={n}")
    else:
        out.fill_(int(col))
    return out


def genrec_mask_topk_expand(
    cum: torch.Tensor,
    top_logprobs: torch.Tensor,
    top_tokens: torch.Tensor,
    *,
    select_k: int,
    node_ids: Optional[torch.Tensor] = None,
    allow_table=None,
    token_base: int = 0,
    token_ids: Optional[torch.Tensor] = None,
    col: Union[int, torch.Tensor] = 0,
    next_node: Optional[torch.Tensor] = None,
    invalid_node: int = 0,
    do_expand: Optional[torch.Tensor] = None,
    apply_mask: bool = True,
    apply_expand: bool = True,
    apply_advance: bool = True,
    inplace: bool = False,
    workspace: Optional[GenrecFusedWorkspace] = None,
) -> GenrecFusedResult:
    """Mask + sorted top-K + optional expand/advance in one launch.

    ``cum`` [N,BW] f32; ``top_logprobs`` [N,BW,C] f32; ``top_tokens`` [N,BW,C]
    int64. Token / node planes are written to a ping-pong workspace plane that
    never aliases the input (``inplace`` is accepted for signature parity and
    ignored, as in the reference's CUDA path)."""
    del inplace
    require_cuda(cum, top_logprobs, top_tokens, node_ids, token_ids)
    n, bw = int(cum.shape[0]), int(cum.shape[1])
    c = int(top_logprobs.shape[2])
    k = int(select_k)
    device = cum.device
    ws = workspace if workspace is not None else GenrecFusedWorkspace()
    tr, keep = _resolve_trie(allow_table, next_node, token_base, invalid_node)
    do_mask = bool(apply_mask and node_ids is not None and tr is not None)
    do_exp = bool(apply_expand and token_ids is not None)
    has_next = tr is not None and (tr.kind != _lib.FR_TRIE_DENSE or tr.next)
    do_adv = bool(apply_advance and do_mask and do_exp and has_next)
    out_vals = ws.get("vals", (n, k), torch.float32, device)
    out_parents = ws.get("parents", (n, k), torch.int64, device)
    out_tokens = ws.get("sel_tokens", (n, k), torch.int64, device)
    out_indices = ws.get("indices", (n, k), torch.int64, device)
    scratch = ws.get("scratch", (n, bw * c), torch.float32, device) if do_mask else None
    node_in = _i64(node_ids) if do_mask else None
    tok_in = tok_out = None
    do_t = col_t = None
    if do_exp:
        tok_in, tok_out = _pingpong_io(ws, "tok", _i64(token_ids), torch.int64, device)
        if do_expand is not None:
            do_t = do_expand.to(device=device, dtype=torch.uint8).reshape(-1).contiguous()
        col_t = _col_i32(col, n, device, ws)
    node_out = None
    if do_adv:
        node_in, node_out = _pingpong_io(ws, "node", node_in, torch.int64, device)
    # converted inputs stay bound to names until the launch has been issued (a temporary freed
    # earlier could be reused by the next conversion before the kernel reads it)
    cum_c, lp_c, tok_c = _f32(cum), _f32(top_logprobs), _i64(top_tokens)
    call("fr_mask_topk_expand", ptr(out_vals), ptr(out_parents), ptr(out_tokens), ptr(out_indices), None,
         ptr(scratch), ptr(cum_c), ptr(lp_c), ptr(tok_c), ptr(node_in), ptr(tok_in),
         ptr(tok_out), ptr(node_out), ptr(do_t), ptr(col_t), ctypes.byref(tr) if tr is not None else None,
         n, bw, c, k, int(tok_in.shape[2]) if do_exp else 0, int(do_mask), int(do_exp), int(do_adv),
         stream_ptr(device))
    del keep, cum_c, lp_c, tok_c
    return GenrecFusedResult(
        vals=out_vals,
        parents=out_parents,
        tokens=out_tokens,
        indices=out_indices,
        token_ids=tok_out if do_exp else None,
        node_ids=node_out if do_adv else None,
    )


def call_genrec_cuda(
    out_vals: torch.Tensor,
    out_parents: torch.Tensor,
    out_tokens: torch.Tensor,
    out_indices: torch.Tensor,
    scratch: torch.Tensor,
    cum: torch.Tensor,
    top_logprobs: torch.Tensor,
    top_tokens: torch.Tensor,
    node_in: torch.Tensor,
    allow_u8,
    tok_in: torch.Tensor,
    tok_out: torch.Tensor,
    next_node: Optional[torch.Tensor],
    node_out: torch.Tensor,
    do_exp: torch.Tensor,
    token_base: int,
    invalid_node: int,
    col_t: torch.Tensor,
    apply_mask: int = 1,
    apply_expand: int = 1,
    apply_advance: int = 1,
) -> bool:
    """Launch into caller-owned buffers; nothing is allocated, so the call can be
    captured in a CUDA graph (kernel/beam_trie.py:633-684)."""
    tr, keep = _resolve_trie(allow_u8, next_node, token_base, invalid_node)
    n, bw = int(cum.shape[0]), int(cum.shape[1])
    c = int(top_logprobs.shape[2])
    k = int(out_vals.shape[1])
    call("fr_mask_topk_expand", ptr(out_vals), ptr(out_parents), ptr(out_tokens), ptr(out_indices), None,
         ptr(scratch), ptr(cum), ptr(top_logprobs), ptr(top_tokens), ptr(node_in), ptr(tok_in), ptr(tok_out),
         ptr(node_out), ptr(do_exp), ptr(col_t), ctypes.byref(tr) if tr is not None else None, n, bw, c, k,
         int(tok_in.shape[2]), int(apply_mask), int(apply_expand), int(apply_advance), stream_ptr(cum.device))
    del keep
    return True


def try_load_beam_trie() -> bool:
    """True when the CUDA library is loadable and a GPU is present."""
    if not torch.cuda.is_available():
        return False
    try:
        _lib.load()
    except Exception:
        return False
    return True
