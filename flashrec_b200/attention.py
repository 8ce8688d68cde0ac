"""KV pool, slot-table bookkeeping and the decode attention backend: mirrors of
``TokenToKVPool`` (kvcache/pool.py:66-139), ``gather_kv_indices``
(attention/kv_indices.py:63-132), ``remap_by_parents`` (scheduler/kv_remap.py:30-66) and ``AttentionBackend`` (attention/flashinfer.py)
for the FP8 decode path.
"""

from __future__ import annotations

import itertools
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
    """Attention over the e4m3 pool with the reference's ``AttentionBackend`` interface
    (attention/flashinfer.py:75-238): ``prepare`` / ``forward`` and, for decode steps replayed from CUDA
    graphs, ``init_graph_wrappers`` / ``graph_bufs`` / ``begin_graph_decode`` / ``end_graph_decode``.

    ``backend`` and ``fi_backend`` are accepted so that the reference's engine can construct this class
    (engine/engine.py:120-127) and are otherwise ignored: there is one implementation, this library's.

    Beams of one request share their prompt slots. The kernels exploit that when they know which rows
    belong together: either ``set_groups`` (explicit), or ``beam_width`` (rows ``[i * bw, (i + 1) * bw)`` of a
    batch whose row count is a multiple of ``bw`` form a group, which is how the reference lays out a decode
    batch and pads it for graph replay, config.py:220-238); otherwise every row is its own group and the
    result is the same. The shared slot prefix itself is found on the device by ``prepare``.

    Kernel choice: the tcgen05 path needs scratch memory for the widened shared prefixes. It is used when
    the longest slot list is known on the host — ``max_shared_len`` given, the batch carries the reference's
    ``seq_lens_cpu``, or the graph buffers were sized by ``init_graph_wrappers`` — and the scratch stays under
    ``scratch_limit_bytes``; otherwise the kernel without scratch (``mma.sync``) runs. Both agree within the
    bf16 tolerance."""

    def __init__(self, kv_pool: TokenToKVPool, num_qo_heads: int, num_kv_heads: int, head_dim: int,
                 backend: str = "flashinfer", fi_backend: str = "fa2", *, max_shared_len: int = 0,
                 keep_prefix: bool = False, beam_width: int = 0, scratch_limit_bytes: int = 8 << 30):
        self.kv_pool = kv_pool
        self.num_qo_heads = int(num_qo_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.n_rep = max(self.num_qo_heads // max(self.num_kv_heads, 1), 1)
        self.device = kv_pool.device
        self.backend = backend
        self.fi_backend = str(fi_backend or "fa2")
        self.q_dtype = torch.bfloat16
        self.prefill_overlap_ok = True  # prefill and decode share no planning workspace here
        # the reference's engine captures decode graphs only when this is not None (engine/engine.py:326)
        self._fi_decode = self
        self._fi_prefill = self
        self.beam_width = int(beam_width)
        self.scratch_limit_bytes = int(scratch_limit_bytes)
        self._group_rows: Optional[torch.Tensor] = None
        self._groups_explicit = False
        self._prefill_scratch: Optional[torch.Tensor] = None
        self._shared_len: Optional[torch.Tensor] = None
        self._max_group_rows = 0
        self._n_groups = 0
        # longest shared prefix the tensor-core path should cover (0 = decide per batch, see the class text)
        self.max_shared_len = int(max_shared_len)
        self._act_cap = 0
        self._act_scratch: Optional[torch.Tensor] = None
        self._scratch: Optional[torch.Tensor] = None
        # keep_prefix: one scratch buffer per layer, so that the widened shared prefix written at
        # the first decode step of a set of requests is reused by their later steps
        # (``prepare(batch, reuse_prefix=True)``) instead of being widened again every step
        self.keep_prefix = bool(keep_prefix) and self.max_shared_len > 0
        self._layer_scratch: dict = {}
        self._scratch_bytes = 0
        self._prepared_len: Optional[torch.Tensor] = None
        self._reuse = False
        # slot lists of the prepared batch (set by ``prepare``; graph replays keep pointing at static buffers)
        self._cur_indptr: Optional[torch.Tensor] = None
        self._cur_indices: Optional[torch.Tensor] = None
        self._own_indptr: Optional[torch.Tensor] = None
        self._graph_bufs: dict = {}
        self._graph_bs: Optional[int] = None
        self._graph_max_seq = 0
        self._auto_groups: dict = {}

    # -- groups -------------------------------------------------------------------------------------
    def set_groups(self, group_rows: torch.Tensor, max_group_rows: int) -> None:
        """``group_rows`` int32 [n_groups + 1]: rows [g[i], g[i+1]) are the beams of one request."""
        self._groups_explicit = True
        self._set_groups(group_rows, max_group_rows)

    def _set_groups(self, group_rows: torch.Tensor, max_group_rows: int) -> None:
        self._group_rows = group_rows.to(dtype=torch.int32).contiguous()
        self._n_groups = int(group_rows.numel()) - 1
        self._max_group_rows = int(max_group_rows)
        if self._shared_len is None or self._shared_len.numel() < self._n_groups:
            self._shared_len = torch.zeros(self._n_groups, dtype=torch.int32, device=group_rows.device)
        if self.max_shared_len > 0:
            self._size_scratch(self.max_shared_len, group_rows.device)
            if self.keep_prefix and (self._prepared_len is None or self._prepared_len.numel() < self._n_groups):
                self._prepared_len = torch.zeros(self._n_groups, dtype=torch.int32, device=group_rows.device)
        self._reuse = False

    def _size_scratch(self, shared_len: int, device) -> bool:
        need = int(_lib.load().fr_decode_attn_scratch_bytes(self._n_groups, self.num_kv_heads, int(shared_len)))
        if self.max_shared_len <= 0 and need > self.scratch_limit_bytes:
            return False
        if need > self._scratch_bytes:
            self._layer_scratch.clear()
        self._scratch_bytes = max(self._scratch_bytes, need)
        if not self.keep_prefix and (self._scratch is None or self._scratch.numel() < need):
            self._scratch = torch.empty(need, dtype=torch.uint8, device=device)
        return True

    def _groups_for(self, n: int, device) -> None:
        """Groups of a batch of ``n`` rows when none were set explicitly: ``beam_width`` rows per group
        if that divides ``n``, else one row per group. Cached per row count (static under graph replay)."""
        bw = self.beam_width if self.beam_width > 0 and n % self.beam_width == 0 else 1
        key = (n, bw)
        g = self._auto_groups.get(key)
        if g is None:
            g = torch.arange(n // bw + 1, dtype=torch.int32, device=device) * bw
            self._auto_groups[key] = g
        if self._group_rows is not g:
            self._set_groups(g, bw)

    def _graph_plan_buffers(self, bufs: dict, device) -> None:
        """Under graph replay every pointer the captured ``forward`` reads must stay where it was at
        capture: the group's shared-length array and the scratch of the tensor-core path live with
        the batch size's static buffers and are allocated once, on the first ``prepare`` for that size."""
        if "shared_len" not in bufs:
            bufs["shared_len"] = torch.zeros(self._n_groups, dtype=torch.int32, device=device)
            bufs["scratch"] = None
            if self.max_shared_len <= 0 and self._graph_max_seq > 0:
                need = int(_lib.load().fr_decode_attn_scratch_bytes(self._n_groups, self.num_kv_heads,
                                                                    self._graph_max_seq))
                if need <= self.scratch_limit_bytes:
                    bufs["scratch"] = torch.empty(need, dtype=torch.uint8, device=device)
        self._shared_len = bufs["shared_len"]

    def _scratch_for(self, layer_id: int, device) -> Optional[torch.Tensor]:
        if not self.keep_prefix:
            return self._scratch
        buf = self._layer_scratch.get(layer_id)
        if buf is None:
            buf = torch.empty(self._scratch_bytes, dtype=torch.uint8, device=device)
            self._layer_scratch[layer_id] = buf
        return buf

    # -- CUDA-graph decode (static slot-list buffers per captured batch size) --------------------
    def init_graph_wrappers(self, capture_bs: List[int], max_seq_len: int) -> None:
        """Static ``indptr`` / ``indices`` / ``last`` buffers per captured batch size, as the reference
        allocates for its per-size FlashInfer wrappers (attention/flashinfer.py:143-183); ``prepare``
        writes them outside the graph, the captured ``forward`` reads them on replay."""
        max_seq_len = max(int(max_seq_len), 1)
        self._graph_max_seq = max(self._graph_max_seq, max_seq_len)
        for bs in capture_bs:
            bs = int(bs)
            if bs <= 0 or bs in self._graph_bufs:
                continue
            self._graph_bufs[bs] = {
                "indptr": torch.zeros(bs + 1, dtype=torch.int32, device=self.device),
                "indices": torch.zeros(bs * max_seq_len, dtype=torch.int32, device=self.device),
                "last": torch.ones(bs, dtype=torch.int32, device=self.device),
            }

    def graph_bufs(self, bs: int) -> Optional[dict]:
        return self._graph_bufs.get(int(bs))

    def begin_graph_decode(self, bs: int) -> None:
        if int(bs) not in self._graph_bufs:
            raise RuntimeError(f"no CUDA-graph buffers for bs={bs}")
        self._graph_bs = int(bs)

    def end_graph_decode(self) -> None:
        self._graph_bs = None

    # -- planning -------------------------------------------------------------------------------------
    def _decode_lists(self, batch, n: int):
        """(indptr, indices) int32 device tensors of a decode batch. The reference's batch carries the
        flat ``kv_indices`` and the lengths only (core.py:81-101): the running sum is then taken on the
        device, into the graph buffers while a graph batch size is active."""
        kv = batch.kv_indices.view(-1)
        if kv.dtype != torch.int32:
            kv = kv.to(torch.int32)
        bufs = self._graph_bufs.get(self._graph_bs) if self._graph_bs is not None else None
        given = getattr(batch, "kv_indptr", None)
        lens = None
        if given is None:
            lens = batch.seq_lens.view(-1)[:n]
            if lens.dtype != torch.int32:
                lens = lens.to(torch.int32)
        if bufs is not None:
            indptr, indices = bufs["indptr"], bufs["indices"]
            if given is not None:
                indptr[: n + 1].copy_(given.view(-1)[: n + 1], non_blocking=True)
            else:
                torch.cumsum(lens, dim=0, out=indptr[1: n + 1])
            nidx = int(kv.numel())
            if nidx > 0 and kv.data_ptr() != indices.data_ptr():
                indices[:nidx].copy_(kv, non_blocking=True)
            return indptr, indices
        if given is not None:
            return given, kv
        if self._own_indptr is None or self._own_indptr.numel() < n + 1:
            self._own_indptr = torch.zeros(n + 1, dtype=torch.int32, device=kv.device)
        torch.cumsum(lens, dim=0, out=self._own_indptr[1: n + 1])
        return self._own_indptr, kv

    def _host_max_len(self, batch, n: int) -> int:
        """Longest slot list of the batch if the host knows it without a device read, else 0."""
        sl_cpu = getattr(batch, "seq_lens_cpu", None)
        if sl_cpu is not None and sl_cpu.device.type == "cpu" and n > 0:
            return int(sl_cpu.view(-1)[:n].max())
        return 0

    def prepare(self, batch, reuse_prefix: bool = False) -> None:
        """Plan the step, outside any graph (all layers share the plan): slot-list offsets, the rows'
        groups and each group's shared slot prefix (found on the device). ``reuse_prefix`` (needs
        ``keep_prefix``): the rows are later decode steps of the requests of the previous ``prepare``;
        their prompt slots and KV bytes are unchanged, so each layer widens only the prefix tokens that
        call had not covered yet. A batch without ``kv_indices`` is left alone, as in the reference
        (attention/flashinfer.py:201-209)."""
        if batch.kv_indices is None:
            return
        if batch.is_prefill:
            return  # the prefill kernel takes its lists straight from the batch
        n = int(batch.n_rows)
        indptr, indices = self._decode_lists(batch, n)
        self._cur_indptr, self._cur_indices = indptr, indices
        if not self._groups_explicit:
            self._groups_for(n, indptr.device)
        bufs = self._graph_bufs.get(self._graph_bs) if self._graph_bs is not None else None
        if bufs is not None:
            self._graph_plan_buffers(bufs, indptr.device)
        if self.max_shared_len > 0:
            self._act_cap = self.max_shared_len
            self._act_scratch = None if self.keep_prefix else self._scratch
        elif bufs is not None:
            self._act_scratch = bufs["scratch"]
            self._act_cap = self._graph_max_seq if self._act_scratch is not None else 0
        else:
            want = self._host_max_len(batch, n)
            ok = want > 0 and self._size_scratch(want, indptr.device)
            self._act_cap = want if ok else 0
            self._act_scratch = self._scratch if ok else None
        reuse = bool(reuse_prefix) and self.keep_prefix and self._shared_len is not None
        if reuse:
            self._prepared_len.copy_(self._shared_len[: self._prepared_len.numel()])
        self._reuse = reuse
        call("fr_decode_attn_plan", ptr(indptr), ptr(indices), ptr(self._group_rows),
             self._n_groups, self._max_group_rows, ptr(self._shared_len), stream_ptr(indptr.device))

    def _forward_prefill(self, q, kc, vc, batch, out) -> torch.Tensor:
        """Causal attention of the extend tokens over each request's slot list (the new tokens' K/V
        are in the pool already): the prefill branch of ``AttentionBackend.forward``
        (attention/flashinfer.py:351-378; mask of ``_sdpa``, attention/flashinfer.py:380-431).
        ``qo_indptr`` / ``kv_indptr`` are taken from the batch when it has them; the reference's batch
        carries ``extend_seq_lens`` and ``seq_lens_cpu`` instead, from which they are summed on the host."""
        ext = [int(x) for x in (batch.extend_seq_lens or [])]
        n_req = len(ext)
        if n_req == 0 or batch.kv_indices is None:
            raise ValueError("a prefill batch needs extend_seq_lens and kv_indices")
        pre = [int(x) for x in (batch.extend_prefix_lens or [0] * n_req)]
        qo = getattr(batch, "qo_indptr", None)
        if qo is None:
            qo = torch.tensor([0] + list(itertools.accumulate(ext)), dtype=torch.int32).to(q.device, non_blocking=True)
        kv_indptr = getattr(batch, "kv_indptr", None)
        if kv_indptr is None:
            lens = [e + p for e, p in zip(ext, pre)]
            kv_indptr = torch.tensor([0] + list(itertools.accumulate(lens)), dtype=torch.int32).to(q.device,
                                                                                                 non_blocking=True)
        kv_indices = batch.kv_indices.view(-1)
        if kv_indices.dtype != torch.int32:
            kv_indices = kv_indices.to(torch.int32)
        max_ext, max_kv = max(ext), max(e + p for e, p in zip(ext, pre))
        need = int(_lib.load().fr_decode_attn_scratch_bytes(n_req, self.num_kv_heads, max_kv))
        if self._prefill_scratch is None or self._prefill_scratch.numel() < need:
            self._prefill_scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
        scratch = self._prefill_scratch
        call("fr_prefill_attn_fp8", ptr(q), q.stride(0), q.stride(1), ptr(kc), ptr(vc), kc.stride(0), kc.stride(1),
             vc.stride(0), vc.stride(1), ptr(qo), ptr(kv_indptr), ptr(kv_indices), ptr(out),
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
        if self._cur_indptr is None or self._cur_indices is None:
            raise RuntimeError("AttentionBackend.forward: prepare(batch) has not been called for a decode batch")
        shared_cap = self._act_cap
        scratch = None
        if shared_cap > 0:
            scratch = self._scratch_for(layer_id, q.device) if self.keep_prefix else self._act_scratch
        args = (ptr(q), q.stride(0), q.stride(1), ptr(kc), ptr(vc), kc.stride(0), kc.stride(1),
                vc.stride(0), vc.stride(1), ptr(self._cur_indptr), ptr(self._cur_indices), ptr(self._group_rows),
                ptr(self._shared_len), ptr(out), out.stride(0), t, self._n_groups, self.num_qo_heads,
                self.num_kv_heads, self.head_dim, self._max_group_rows, self.kv_pool.num_tokens,
                float(self.head_dim) ** -0.5, ptr(scratch), int(scratch.numel()) if scratch is not None else 0,
                shared_cap)
        if self._reuse:
            call("fr_decode_attn_reuse_fp8", *args, ptr(self._prepared_len), stream_ptr(q.device))
        else:
            call("fr_decode_attn_fp8", *args, stream_ptr(q.device))
        return out
