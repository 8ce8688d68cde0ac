"""KV pool, slot-table bookkeeping and the decode attention backend: mirrors of
``TokenToKVPool`` (kvcache/pool.py:66-139), ``gather_kv_indices``
(attention/kv_indices.py:63-132), ``remap_by_parents`` (scheduler/kv_remap.py:30-66) and ``AttentionBackend`` (attention/flashinfer.py)
for the FP8 decode path.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch

from flashrec_b200 import _lib
from flashrec_b200._lib import call, ptr, require_cuda, stream_ptr
from flashrec_b200.kernel.sglops import store_kv_cache

_FP8 = torch.float8_e4m3fn


class TokenToKVPool:
    """Physical KV: e4m3 ``[num_tokens, num_kv_heads, head_dim]`` per layer; slot 0 is
    a dummy that is never handed out (kvcache/pool.py:66-114). ``page_size`` only
    sets the allocation granularity (slot = page * page_size + offset); the byte
    layout is the reference's page-size-1 layout."""

    def __init__(self, num_layers, num_tokens, num_kv_heads, head_dim, dtype, device, page_size: int = 1):
        if dtype != _FP8:
            raise NotImplementedError("flashrec_b200 implements the float8_e4m3fn KV pool only")
        self.num_layers = int(num_layers)
        self.num_tokens = int(num_tokens)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.dtype = dtype
        self.device = torch.device(device)
        self.page_size = int(page_size)
        self.row_dim = self.num_kv_heads * self.head_dim
        shape = (self.num_tokens, self.num_kv_heads, self.head_dim)
        self.k = [torch.zeros(shape, dtype=torch.uint8, device=device).view(_FP8) for _ in range(num_layers)]
        self.v = [torch.zeros(shape, dtype=torch.uint8, device=device).view(_FP8) for _ in range(num_layers)]
        first = self.page_size if self.page_size > 1 else 1  # page 0 / slot 0 reserved
        self._free: List[int] = list(range(first, self.num_tokens))
        self.last_alloc_cpu: List[int] = []

    def available_size(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> Optional[torch.Tensor]:
        n = int(n)
        if n <= 0:
            self.last_alloc_cpu = []
            return torch.empty(0, dtype=torch.int64, device=self.device)
        if n > len(self._free):
            self.last_alloc_cpu = []
            return None
        idx = self._free[-n:]
        del self._free[-n:]
        self.last_alloc_cpu = idx
        return torch.tensor(idx, dtype=torch.int64, device=self.device)

    def free(self, indices) -> None:
        ids = indices.tolist() if isinstance(indices, torch.Tensor) else list(indices)
        self._free.extend(int(i) for i in ids if int(i) > 0)

    def k_cache(self, layer_id: int) -> torch.Tensor:
        return self.k[layer_id]

    def v_cache(self, layer_id: int) -> torch.Tensor:
        return self.v[layer_id]

    def store(self, layer_id: int, k: torch.Tensor, v: torch.Tensor, loc: torch.Tensor) -> None:
        n = int(loc.numel())
        if n == 0:
            return
        store_kv_cache(
            self.k[layer_id].view(-1, self.row_dim),
            self.v[layer_id].view(-1, self.row_dim),
            loc,
            k.reshape(n, self.row_dim),
            v.reshape(n, self.row_dim),
        )


def gather_kv_indices(
    req_to_token: torch.Tensor,
    rows: torch.Tensor,
    seq_lens: Union[Sequence[int], torch.Tensor],
    out: Optional[torch.Tensor] = None,
    total: Optional[int] = None,
    indptr_out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Concatenated slot ids of each row's ``[:seq_len]`` prefix (int32).

    With ``out`` and ``indptr_out`` given and ``seq_lens`` an int32 device tensor,
    nothing is allocated and nothing syncs (graph-capturable); otherwise ``total``
    is obtained from the host copy of ``seq_lens`` as the reference does."""
    require_cuda(req_to_token, rows)
    device = req_to_token.device
    if req_to_token.dtype != torch.int32:
        raise TypeError("req_to_token must be int32")
    rows = rows.reshape(-1).to(device=device, dtype=torch.int64)
    n = int(rows.numel())
    if n == 0:
        return torch.empty(0, dtype=torch.int32, device=device) if out is None else out[:0]
    if isinstance(seq_lens, torch.Tensor):
        sl = seq_lens.reshape(-1)[:n].to(device=device, dtype=torch.int32).contiguous()
        if total is None and out is None:
            total = int(sl.sum().item())
    else:
        seq_list = [int(x) for x in seq_lens]
        if len(seq_list) != n:
            raise ValueError("rows and seq_lens length mismatch")
        if total is None:
            total = int(sum(seq_list))
        sl = torch.tensor(seq_list, dtype=torch.int32, device=device)
    if int(sl.numel()) != n:
        raise ValueError("rows and seq_lens length mismatch")
    if out is None:
        out = torch.empty(max(int(total), 0), dtype=torch.int32, device=device)
    elif out.dtype != torch.int32:
        raise TypeError("out must be int32")
    cap = int(out.numel()) if total is None else min(int(total), int(out.numel()))
    if indptr_out is None:
        indptr_out = torch.empty(n + 1, dtype=torch.int32, device=device)
    call("fr_gather_kv_indices", ptr(req_to_token), req_to_token.stride(0), ptr(rows), ptr(sl), ptr(indptr_out),
         ptr(out), n, cap, stream_ptr(device))
    return out.reshape(-1)[:cap] if total is not None else out


def kv_table_step(
    req_to_token: torch.Tensor,
    rows: torch.Tensor,
    seq_lens: torch.Tensor,
    out: torch.Tensor,
    indptr_out: torch.Tensor,
    *,
    new_slot: Optional[torch.Tensor] = None,
    parents_rel: Optional[torch.Tensor] = None,
    prefix_len: Optional[torch.Tensor] = None,
    group_indptr: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """The slot-table work of one decode tick for a whole wave, in one call:
    ``remap_by_parents`` of every request (scheduler/kv_remap.py:30-66) with last
    tick's ``parents_rel``, the batched ``write_decode`` of this tick's ``new_slot``
    (scheduler/scheduler.py:1305-1310) and ``gather_kv_indices``
    (attention/kv_indices.py:63-132). ``seq_lens`` (int32, device) are the lengths
    after the tick; the decode window of a row is ``[prefix_len, seq_len - 1)``
    (``[prefix_len, seq_len)`` without ``new_slot``). Everything is a device tensor
    given by the caller: nothing allocates or syncs (graph-capturable)."""
    require_cuda(req_to_token, rows, seq_lens, out, indptr_out)
    if req_to_token.dtype != torch.int32 or seq_lens.dtype != torch.int32 or rows.dtype != torch.int64:
        raise TypeError("req_to_token / seq_lens must be int32 and rows int64")
    if out.dtype != torch.int32 or indptr_out.dtype != torch.int32:
        raise TypeError("out / indptr_out must be int32")
    n = int(rows.numel())
    if int(seq_lens.numel()) != n or int(indptr_out.numel()) < n + 1:
        raise ValueError("seq_lens / indptr_out do not match rows")
    for name, t, dt in (("new_slot", new_slot, torch.int64), ("parents_rel", parents_rel, torch.int64),
                        ("prefix_len", prefix_len, torch.int32)):
        if t is not None and (t.dtype != dt or int(t.numel()) != n or not t.is_contiguous()):
            raise TypeError(f"{name} must be a contiguous {dt} tensor of {n} elements")
    n_groups = 0
    if parents_rel is not None:
        if group_indptr is None or prefix_len is None or group_indptr.dtype != torch.int32:
            raise TypeError("parents_rel needs prefix_len and an int32 group_indptr")
        n_groups = int(group_indptr.numel()) - 1
    call("fr_kv_table_step", ptr(req_to_token), req_to_token.stride(0), int(req_to_token.shape[0]),
         int(req_to_token.shape[1]), ptr(rows), ptr(group_indptr), n_groups, ptr(parents_rel), ptr(prefix_len),
         ptr(seq_lens), ptr(new_slot), ptr(indptr_out), ptr(out), n, int(out.numel()), stream_ptr(req_to_token.device))
    return out


def copy_prefill_to_beams_many(req_to_token: torch.Tensor, srcs: torch.Tensor, beam_rows: torch.Tensor,
                               m: int) -> None:
    """``table[beam_rows[r, b], :m] = table[srcs[r], :m]``: a prefill row's slots handed
    to all beams of its request (ModelEngine.copy_prefill_to_beams_many,
    engine/engine.py:252-274; ``m`` is the reference's ``max(seq_lens)``)."""
    require_cuda(req_to_token, srcs, beam_rows)
    if req_to_token.dtype != torch.int32 or srcs.dtype != torch.int64 or beam_rows.dtype != torch.int64:
        raise TypeError("req_to_token must be int32, srcs / beam_rows int64")
    if beam_rows.dim() != 2 or int(beam_rows.shape[0]) != int(srcs.numel()) or not beam_rows.is_contiguous():
        raise ValueError("beam_rows must be a contiguous [n_requests, beam_width] tensor")
    if not 0 <= int(m) <= int(req_to_token.shape[1]):
        raise ValueError("m exceeds the table width")
    call("fr_kv_table_fanout", ptr(req_to_token), req_to_token.stride(0), int(req_to_token.shape[0]), ptr(srcs),
         ptr(beam_rows), int(beam_rows.shape[0]), int(beam_rows.shape[1]), int(m), stream_ptr(req_to_token.device))


class AttentionBackend:
    """Decode attention over the e4m3 pool. ``prepare`` plans (finds each group's
    shared slot prefix on the device); ``forward`` stores nothing when
    ``skip_store`` is set (the fused rope kernel already wrote K/V)."""

    def __init__(self, kv_pool: TokenToKVPool, num_qo_heads: int, num_kv_heads: int, head_dim: int,
                 max_shared_len: int = 0, keep_prefix: bool = False):
        self.kv_pool = kv_pool
        self.num_qo_heads = int(num_qo_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.n_rep = self.num_qo_heads // self.num_kv_heads
        self._group_rows: Optional[torch.Tensor] = None
        self._prefill_scratch: Optional[torch.Tensor] = None
        self._shared_len: Optional[torch.Tensor] = None
        self._max_group_rows = 0
        self._n_groups = 0
        # longest shared prefix the tensor-core path should cover (0 = use the kernel without scratch)
        self.max_shared_len = int(max_shared_len)
        self._scratch: Optional[torch.Tensor] = None
        # keep_prefix: one scratch buffer per layer, so that the widened shared prefix written at
        # the first decode step of a set of requests is reused by their later steps
        # (``prepare(batch, reuse_prefix=True)``) instead of being widened again every step
        self.keep_prefix = bool(keep_prefix) and self.max_shared_len > 0
        self._layer_scratch: dict = {}
        self._scratch_bytes = 0
        self._prepared_len: Optional[torch.Tensor] = None
        self._reuse = False

    def set_groups(self, group_rows: torch.Tensor, max_group_rows: int) -> None:
        """``group_rows`` int32 [n_groups + 1]: rows [g[i], g[i+1]) are the beams of one request."""
        self._group_rows = group_rows.to(dtype=torch.int32).contiguous()
        self._n_groups = int(group_rows.numel()) - 1
        self._max_group_rows = int(max_group_rows)
        if self._shared_len is None or self._shared_len.numel() < self._n_groups:
            self._shared_len = torch.zeros(self._n_groups, dtype=torch.int32, device=group_rows.device)
        if self.max_shared_len > 0:
            need = int(_lib.load().fr_decode_attn_scratch_bytes(self._n_groups, self.num_kv_heads, self.max_shared_len))
            if need > self._scratch_bytes:
                self._layer_scratch.clear()
            self._scratch_bytes = max(self._scratch_bytes, need)
            if not self.keep_prefix and (self._scratch is None or self._scratch.numel() < need):
                self._scratch = torch.empty(need, dtype=torch.uint8, device=group_rows.device)
            if self.keep_prefix and (self._prepared_len is None or self._prepared_len.numel() < self._n_groups):
                self._prepared_len = torch.zeros(self._n_groups, dtype=torch.int32, device=group_rows.device)
        self._reuse = False

    def _scratch_for(self, layer_id: int, device) -> Optional[torch.Tensor]:
        if not self.keep_prefix:
            return self._scratch
        buf = self._layer_scratch.get(layer_id)
        if buf is None:
            buf = torch.empty(self._scratch_bytes, dtype=torch.uint8, device=device)
            self._layer_scratch[layer_id] = buf
        return buf

    def prepare(self, batch, reuse_prefix: bool = False) -> None:
        """Plan the step. ``reuse_prefix`` (needs ``keep_prefix``): the rows are later decode steps
        of the requests of the previous ``prepare``; their prompt slots and KV bytes are unchanged,
        so each layer widens only the prefix tokens that call had not covered yet."""
        if batch.kv_indices is None or batch.kv_indptr is None:
            return
        reuse = bool(reuse_prefix) and self.keep_prefix and self._shared_len is not None
        if reuse:
            self._prepared_len.copy_(self._shared_len[: self._prepared_len.numel()])
        self._reuse = reuse
        if self._group_rows is None:
            n = int(batch.kv_indptr.numel()) - 1
            self.set_groups(torch.arange(n + 1, dtype=torch.int32, device=batch.kv_indptr.device), 1)
        call("fr_decode_attn_plan", ptr(batch.kv_indptr), ptr(batch.kv_indices), ptr(self._group_rows),
             self._n_groups, self._max_group_rows, ptr(self._shared_len), stream_ptr(batch.kv_indptr.device))

    def _forward_prefill(self, q, kc, vc, batch, out) -> torch.Tensor:
        """Causal attention of the extend tokens over each request's slot list (the new tokens' K/V
        are in the pool already): the prefill branch of ``AttentionBackend.forward``
        (attention/flashinfer.py:351-378; mask of ``_sdpa``, attention/flashinfer.py:380-431)."""
        ext = [int(x) for x in (batch.extend_seq_lens or [])]
        n_req = len(ext)
        if n_req == 0 or batch.qo_indptr is None or batch.kv_indptr is None or batch.kv_indices is None:
            raise ValueError("a prefill batch needs extend_seq_lens, qo_indptr, kv_indptr and kv_indices")
        pre = [int(x) for x in (batch.extend_prefix_lens or [0] * n_req)]
        max_ext, max_kv = max(ext), max(e + p for e, p in zip(ext, pre))
        need = int(_lib.load().fr_decode_attn_scratch_bytes(n_req, self.num_kv_heads, max_kv))
        if self._prefill_scratch is None or self._prefill_scratch.numel() < need:
            self._prefill_scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
        scratch = self._prefill_scratch
        call("fr_prefill_attn_fp8", ptr(q), q.stride(0), q.stride(1), ptr(kc), ptr(vc), kc.stride(0), kc.stride(1),
             vc.stride(0), vc.stride(1), ptr(batch.qo_indptr), ptr(batch.kv_indptr), ptr(batch.kv_indices), ptr(out),
             out.stride(0), int(q.shape[0]), n_req, self.num_qo_heads, self.num_kv_heads, self.head_dim, max_ext,
             max_kv, self.kv_pool.num_tokens, float(self.head_dim) ** -0.5, ptr(scratch), int(scratch.numel()),
             stream_ptr(q.device))
        return out

    def forward(self, q, k, v, layer_id: int, batch, skip_store: bool = False, out=None) -> torch.Tensor:
        """q: [T, Hq, D] bf16 (may be a strided view); returns [T, Hq, D] bf16."""
        require_cuda(q)
        if not skip_store:
            self.kv_pool.store(layer_id, k, v, batch.out_cache_loc)
        t = int(q.shape[0])
        if out is None:
            out = torch.empty((t, self.num_qo_heads, self.head_dim), dtype=torch.bfloat16, device=q.device)
        kc = self.kv_pool.k[layer_id]
        vc = self.kv_pool.v[layer_id]
        if batch.is_prefill:
            return self._forward_prefill(q, kc, vc, batch, out)
        scratch = self._scratch_for(layer_id, q.device) if self.max_shared_len > 0 else None
        args = (ptr(q), q.stride(0), q.stride(1), ptr(kc), ptr(vc), kc.stride(0), kc.stride(1),
                vc.stride(0), vc.stride(1), ptr(batch.kv_indptr), ptr(batch.kv_indices), ptr(self._group_rows),
                ptr(self._shared_len), ptr(out), out.stride(0), t, self._n_groups, self.num_qo_heads,
                self.num_kv_heads, self.head_dim, self._max_group_rows, self.kv_pool.num_tokens,
                float(self.head_dim) ** -0.5, ptr(scratch), int(scratch.numel()) if scratch is not None else 0,
                self.max_shared_len)
        if self._reuse:
            call("fr_decode_attn_reuse_fp8", *args, ptr(self._prepared_len), stream_ptr(q.device))
        else:
            call("fr_decode_attn_fp8", *args, stream_ptr(q.device))
        return out
