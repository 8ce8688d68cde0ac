"""Decode-side driver of trie-constrained SID beam search: the device work of
one engine tick in the reference (``BeamRecEngine._forward_decode`` and
``_expand_decode_body``, scheduler/scheduler.py:1261-1456; ``DecodeGraphRunner``,
engine/graph.py:85-517), sequenced for a fixed wave of requests.

Per step: one slot-table call (the rows' decode windows re-parented by the
previous step's parents, this step's KV slots appended, the flat slot lists
gathered), the model body, the SID head of the step's level and the fused beam
step. Before the first step every beam row receives its request's prompt slots.
Each step is captured once in a CUDA graph (rows = requests x beam width, a
multiple of the beam width as in ``resolved_cuda_graph_sizes``, config.py:220-238)
and replayed.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from flashrec_b200._lib import call, ptr, stream_ptr
from flashrec_b200.attention import AttentionBackend, TokenToKVPool, copy_prefill_to_beams_many, kv_table_step
from flashrec_b200.decoder import ForwardBatch, Qwen3Config, Qwen3ForCausalLM
from flashrec_b200.kernel.beam_trie import GenrecFusedResult
from flashrec_b200.kernel.sglops import per_token_quant_fp8
from flashrec_b200.logits import RestrictedLMHead

_FP8 = torch.float8_e4m3fn


@dataclass
class BeamStepOut:
    vals: torch.Tensor      # [N, K] f32 cumulative scores, sorted descending
    parents: torch.Tensor   # [N, K] i64 beam index of the parent
    tokens: torch.Tensor    # [N, K] i64 chosen token
    indices: torch.Tensor   # [N, K] i64 flat candidate index b * width + code
    child: torch.Tensor     # [N, K] i64 trie node after the step


def sid_beam_step(
    cum: torch.Tensor,
    logits: torch.Tensor,
    row_max: torch.Tensor,
    row_logsum: torch.Tensor,
    node_ids: Optional[torch.Tensor],
    trie,
    level_tok_base: int,
    select_k: int,
    *,
    token_ids_in: Optional[torch.Tensor] = None,
    token_ids_out: Optional[torch.Tensor] = None,
    node_ids_out: Optional[torch.Tensor] = None,
    col: Optional[torch.Tensor] = None,
    out: Optional[BeamStepOut] = None,
    idx_base: int = 0,
    idx_width: int = 0,
) -> BeamStepOut:
    """One full-width beam step straight from the level's fp32 logits.

    ``cum`` [N,BW] f32; ``logits`` [N*BW, K_l] f32 with row statistics;
    ``node_ids`` [N,BW] i64; ``trie`` a DeviceTrie (or None = unconstrained).
    If the token planes are given (distinct; in [N,BW,L], out [N,max(BW,K),L] i64) the winners'
    token rows are expanded and ``node_ids_out`` receives the advanced nodes."""
    n, bw = int(cum.shape[0]), int(cum.shape[1])
    kl = int(logits.shape[1])
    k = int(select_k)
    dev = cum.device
    if out is None:
        out = BeamStepOut(
            vals=torch.empty((n, k), dtype=torch.float32, device=dev),
            parents=torch.empty((n, k), dtype=torch.int64, device=dev),
            tokens=torch.empty((n, k), dtype=torch.int64, device=dev),
            indices=torch.empty((n, k), dtype=torch.int64, device=dev),
            child=torch.empty((n, k), dtype=torch.int64, device=dev),
        )
    tr = trie.descriptor() if trie is not None else None
    do_exp = token_ids_in is not None and token_ids_out is not None
    do_adv = do_exp and node_ids is not None and node_ids_out is not None and trie is not None
    call("fr_sid_beam_step", ptr(out.vals), ptr(out.parents), ptr(out.tokens), ptr(out.indices), ptr(out.child),
         ptr(cum), ptr(logits), logits.stride(0), ptr(row_max), ptr(row_logsum), ptr(node_ids), ptr(token_ids_in),
         ptr(token_ids_out), ptr(node_ids_out), None, ptr(col), ctypes.byref(tr) if tr is not None else None,
         int(level_tok_base), int(idx_base), int(idx_width), n, bw, kl, k,
         int(token_ids_in.shape[2]) if do_exp else 0, int(do_exp), int(do_adv), stream_ptr(dev))
    return out


class SidHeadWorkspace:
    """Grow-only device buffer for ``sid_head_topk`` (tile statistics, candidate lists, row masks)."""

    def __init__(self):
        self.buf: Optional[torch.Tensor] = None

    def get(self, n: int, bw: int, level_width: int, cand_capacity: int, device) -> torch.Tensor:
        from flashrec_b200._lib import load

        need = int(load().fr_sid_head_topk_workspace_bytes(int(n), int(bw), int(level_width), int(cand_capacity)))
        if need < 0:
            raise ValueError("sid_head_topk: bad workspace dimensions")
        if self.buf is None or self.buf.numel() < need or self.buf.device != torch.device(device):
            self.buf = torch.empty(need, dtype=torch.uint8, device=device)
        return self.buf


def sid_head_topk(
    cum: torch.Tensor,
    hidden_fp8: torch.Tensor,
    hidden_scale: torch.Tensor,
    weight_fp8: torch.Tensor,
    weight_scale: torch.Tensor,
    node_ids: Optional[torch.Tensor],
    trie,
    level_tok_base: int,
    select_k: int,
    workspace: SidHeadWorkspace,
    *,
    cand_capacity: Optional[int] = None,
    token_ids_in: Optional[torch.Tensor] = None,
    token_ids_out: Optional[torch.Tensor] = None,
    node_ids_out: Optional[torch.Tensor] = None,
    col: Optional[torch.Tensor] = None,
    out: Optional[BeamStepOut] = None,
    idx_base: int = 0,
    idx_width: int = 0,
    level: Optional[int] = None,
    phase: int = 0,
    row_max: Optional[torch.Tensor] = None,
    row_logsum: Optional[torch.Tensor] = None,
    out_records: Optional[torch.Tensor] = None,
) -> BeamStepOut:
    """The level's head GEMM and the beam step in one call (``fr_sid_head_topk``): the fp32 logits are never
    written, only per-row statistics and the trie-legal candidates leave the GEMM. ``hidden_fp8`` e4m3
    ``[N*BW, H]`` with ``hidden_scale`` (``per_token_quant_fp8`` of the final hidden states), ``weight_fp8`` the
    level's e4m3 head rows ``[K_l, H]`` with ``weight_scale``; the rest as ``sid_beam_step``. ``cand_capacity``:
    candidate records per request; by default the trie's bound for ``level`` (or beams x level width)."""
    n, bw = int(cum.shape[0]), int(cum.shape[1])
    kl, h = int(weight_fp8.shape[0]), int(weight_fp8.shape[1])
    k = int(select_k)
    dev = cum.device
    if cand_capacity is None:
        if trie is not None and level is not None and hasattr(trie, "candidate_bound"):
            cand_capacity = trie.candidate_bound(int(level), bw)
        else:
            cand_capacity = bw * kl
    if out is None:
        out = BeamStepOut(
            vals=torch.empty((n, k), dtype=torch.float32, device=dev),
            parents=torch.empty((n, k), dtype=torch.int64, device=dev),
            tokens=torch.empty((n, k), dtype=torch.int64, device=dev),
            indices=torch.empty((n, k), dtype=torch.int64, device=dev),
            child=torch.empty((n, k), dtype=torch.int64, device=dev),
        )
    ws = workspace.get(n, bw, kl, cand_capacity, dev)
    tr = trie.descriptor() if trie is not None else None
    do_exp = token_ids_in is not None and token_ids_out is not None
    do_adv = do_exp and node_ids is not None and node_ids_out is not None and trie is not None
    sa = hidden_scale.reshape(-1)
    sw = weight_scale.reshape(-1)
    call("fr_sid_head_topk", ptr(out.vals), ptr(out.parents), ptr(out.tokens), ptr(out.indices), ptr(out.child),
         ptr(out_records), ptr(hidden_fp8), ptr(sa), hidden_fp8.stride(0), ptr(weight_fp8), ptr(sw), weight_fp8.stride(0), h, ptr(cum),
         ptr(node_ids), ptr(token_ids_in), ptr(token_ids_out), ptr(node_ids_out), None, ptr(col),
         ctypes.byref(tr) if tr is not None else None, int(level_tok_base), int(idx_base), int(idx_width), n, bw, kl, k,
         int(token_ids_in.shape[2]) if do_exp else 0, int(do_exp), int(do_adv), int(phase), ptr(row_max),
         ptr(row_logsum), ptr(ws), int(ws.numel()), int(cand_capacity), stream_ptr(dev))
    return out


class SidDecodeEngine:
    """A wave of ``n_requests`` requests x ``beam_width`` beams decoding ``len(sizes)``
    SID levels with a Qwen3-shaped FP8 model. Weights are random (N(0, 0.02)), the
    prompt KV is synthetic e4m3 data laid out as a prefill would have left it:
    requests share the slots of a common prompt prefix (a radix-cache hit), every
    beam of a request shares the request's prompt slots.

    With ``sharded_head`` (a :class:`flashrec_b200.sharded_head.ShardedSidHead` over a process group of equal
    engines) the model body stays data-parallel over the ranks' own requests and the SID head is split by
    token range: every step all-gathers the ranks' quantised final hidden rows, runs the head on the rank's
    code range for ALL requests, and merges the shards' winners, so every rank holds the beam state of all
    requests and continues with its own. With a ``data_seed`` the weights come from ``seed`` alone (the same
    on every rank) and prompts and KV fill from ``data_seed``."""

    def __init__(
        self,
        cfg: Qwen3Config,
        n_requests: int,
        beam_width: int,
        prompt_lens: Sequence[int],
        sizes: Sequence[int],
        token_base: int,
        trie,
        device,
        *,
        shared_prefix: int = 0,
        page_size: int = 16,
        seed: int = 0,
        use_graphs: bool = True,
        keep_prefix: bool = True,
        fuse_rope_gemm: bool = True,
        level0_from_prefill: bool = False,
        fused_head: bool = True,
        sharded_head=None,
        data_seed: Optional[int] = None,
    ):
        self.cfg = cfg
        self.device = torch.device(device)
        self.n = int(n_requests)
        self.bw = int(beam_width)
        self.rows = self.n * self.bw
        self.sizes = [int(s) for s in sizes]
        self.steps = len(self.sizes)
        self.token_base = int(token_base)
        self.trie = trie
        self.use_graphs = bool(use_graphs)
        self.prompt_lens = [int(p) for p in prompt_lens]
        assert len(self.prompt_lens) == self.n
        self.shared_prefix = int(shared_prefix)
        self.seed = int(seed)
        self.data_seed = self.seed if data_seed is None else int(data_seed)
        self.sharded = sharded_head
        self.world = int(sharded_head.world) if sharded_head is not None else 1
        self.rank = int(sharded_head.rank) if sharded_head is not None else 0
        self.n_total = self.n * self.world
        if sharded_head is not None:
            if level0_from_prefill or trie is None or not fused_head:
                raise ValueError("the sharded head runs the fused, trie-constrained decode steps only")
            if any(int(k) % self.world for k in sizes):
                raise ValueError("every level width must be divisible by the number of head shards")
        # the reference's flow: level 0 is chosen from the prefill's last-token logits (one row per
        # request, init_from_prefill_batch, search/expand.py:168-237) and only levels 1.. are decode steps
        self.first_step = 1 if level0_from_prefill else 0
        self.prefill_hidden: Optional[torch.Tensor] = None
        dev = self.device
        g = torch.Generator(device=dev)
        g.manual_seed(self.data_seed)

        # ---- KV pool: [page 0 dummy][shared prefix][per-request prompts][decode slots] ----
        uniq_prompt = shared_prefix + sum(max(p - shared_prefix, 0) for p in self.prompt_lens)
        decode_slots = self.rows * self.steps
        num_tokens = page_size + uniq_prompt + decode_slots
        num_tokens = (num_tokens + page_size - 1) // page_size * page_size
        self.pool = TokenToKVPool(cfg.num_hidden_layers, num_tokens, cfg.num_key_value_heads, cfg.head_dim, _FP8, dev,
                                  page_size=page_size)
        n_prompt_slots = uniq_prompt
        for layer in range(cfg.num_hidden_layers):  # synthetic "prefill" contents
            for cache in (self.pool.k[layer], self.pool.v[layer]):
                blk = torch.randn((n_prompt_slots, cfg.num_key_value_heads, cfg.head_dim), generator=g, device=dev,
                                  dtype=torch.float32)
                cache[page_size: page_size + n_prompt_slots].copy_(blk.to(torch.bfloat16).to(_FP8))
        # slot table: row -> slot ids, like ReqToTokenPool.req_to_token (kvcache/pool.py:142-183): the
        # beam rows first, then one prefill row per request whose slots every wave hands to its beams
        self.max_seq = max(self.prompt_lens) + self.steps
        table = torch.zeros((self.rows + self.n, self.max_seq), dtype=torch.int32)
        shared = torch.arange(page_size, page_size + shared_prefix, dtype=torch.int32)
        cursor = page_size + shared_prefix
        for r, plen in enumerate(self.prompt_lens):
            own = torch.arange(cursor, cursor + max(plen - shared_prefix, 0), dtype=torch.int32)
            cursor += int(own.numel())
            table[self.rows + r, :plen] = torch.cat((shared[: min(plen, shared_prefix)], own))
        self.req_to_token = table.to(dev)
        self.prefill_rows = torch.arange(self.rows, self.rows + self.n, dtype=torch.int64, device=dev)
        self.decode_slot_base = page_size + uniq_prompt
        plen_rows = torch.tensor(self.prompt_lens, dtype=torch.int64).repeat_interleave(self.bw)
        self.prompt_len_rows = plen_rows.to(dev)
        self.prefix_len_rows = self.prompt_len_rows.to(torch.int32)
        self.rows_idx = torch.arange(self.rows, dtype=torch.int64, device=dev)
        self.group_indptr = torch.arange(self.n + 1, dtype=torch.int32, device=dev) * self.bw

        # ---- model + head ----------------------------------------------------------------
        self.attn = AttentionBackend(self.pool, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                                     max_shared_len=max(self.prompt_lens) + self.steps, keep_prefix=keep_prefix)
        self.attn.set_groups(self.group_indptr, self.bw)
        self.model = Qwen3ForCausalLM(cfg, self.attn, dev, fuse_rope_gemm=fuse_rope_gemm)
        self.model.init_random(seed=seed + 1)
        sid_total = sum(self.sizes)
        gw = g
        if sharded_head is not None or data_seed is not None:  # the same head on every rank, whatever its prompts drew from g
            gw = torch.Generator(device=dev)
            gw.manual_seed(seed + 2)
        sid_w = torch.randn((sid_total, cfg.hidden_size), generator=gw, device=dev, dtype=torch.float32) * 0.02
        self.head = RestrictedLMHead(list(range(self.token_base, self.token_base + sid_total)))
        from flashrec_b200.layers import quantize_weight_fp8

        self.head.bind_quantized(*quantize_weight_fp8(sid_w))
        self.head.bind_codebook(self.sizes)
        self.level_tok_base = [self.token_base + sum(self.sizes[:l]) for l in range(self.steps)]

        # ---- static step buffers ------------------------------------------------------------
        i64 = dict(dtype=torch.int64, device=dev)
        self.input_ids = torch.zeros(self.rows, **i64)
        self.positions = torch.zeros(self.rows, **i64)
        self.out_cache_loc = torch.zeros(self.rows, **i64)
        self.seq_lens = torch.zeros(self.rows, dtype=torch.int32, device=dev)
        total_idx = sum(self.prompt_lens) * self.bw + self.rows * self.steps
        self.kv_indices = torch.zeros(total_idx, dtype=torch.int32, device=dev)
        self.kv_indptr = torch.zeros(self.rows + 1, dtype=torch.int32, device=dev)
        # beam state of all requests of the group (n_total == n without a sharded head); this engine's own
        # requests are the rows [rank * n, (rank + 1) * n) of it
        nt = self.n_total
        own = slice(self.rank * self.n, (self.rank + 1) * self.n)
        self.g_cum = torch.zeros((nt, self.bw), dtype=torch.float32, device=dev)
        self.g_node_planes = [torch.zeros((nt, self.bw), **i64) for _ in range(2)]
        self.g_tok_planes = [torch.zeros((nt, self.bw, self.steps), **i64) for _ in range(2)]
        self.g_col = torch.zeros(nt, dtype=torch.int32, device=dev)
        self.g_outs = [
            BeamStepOut(
                vals=torch.empty((nt, self.bw), dtype=torch.float32, device=dev),
                parents=torch.empty((nt, self.bw), **i64), tokens=torch.empty((nt, self.bw), **i64),
                indices=torch.empty((nt, self.bw), **i64), child=torch.empty((nt, self.bw), **i64))
            for _ in range(self.steps)
        ]
        self.cum = self.g_cum[own]
        self.node_planes = [t[own] for t in self.g_node_planes]
        self.tok_planes = [t[own] for t in self.g_tok_planes]
        self.col = self.g_col[own]
        self.outs = [BeamStepOut(vals=o.vals[own], parents=o.parents[own], tokens=o.tokens[own],
                                 indices=o.indices[own], child=o.child[own]) for o in self.g_outs]
        # pinned host staging for the per-step inputs and the final result
        self.h_loc = torch.empty((self.steps, self.rows), dtype=torch.int64).pin_memory()
        for s in range(self.steps):
            self.h_loc[s] = self.decode_slot_base + s * self.rows + torch.arange(self.rows)
        self.d_loc = self.h_loc.to(dev)  # device-resident copy for runs that exclude host traffic
        self.h_vals = torch.empty((self.n, self.bw), dtype=torch.float32).pin_memory()
        self.h_tokens = torch.empty((self.n, self.bw, self.steps), dtype=torch.int64).pin_memory()
        self._cum0 = torch.zeros((self.n, 1), dtype=torch.float32, device=dev)
        self._node0 = torch.zeros((self.n, 1), **i64)
        self._tok0 = torch.zeros((self.n, 1, self.steps), **i64)
        # head GEMM + statistics + trie mask + top-K without the fp32 logits matrix (fr_sid_head_topk); the
        # three-call flow (GEMM -> row statistics -> beam step) stays as the other branch
        self.fused_head = bool(fused_head) and trie is not None and self.bw % 32 == 0
        self.head_ws = SidHeadWorkspace()
        self.cand_caps = [trie.candidate_bound(l, self.bw) for l in range(self.steps)] if self.fused_head else []
        self.graphs: List[Optional[torch.cuda.CUDAGraph]] = [None] * self.steps
        self.kernel_launches_per_step: List[int] = [0] * self.steps
        self.reset()

    # ------------------------------------------------------------------------------------
    def reset(self) -> None:
        """Beam state before the first step: one live beam per request at the trie root, every
        beam row holding its request's prompt slots (engine/engine.py:252-274)."""
        copy_prefill_to_beams_many(self.req_to_token, self.prefill_rows, self.rows_idx.view(self.n, self.bw),
                                   max(self.prompt_lens))
        self.g_cum.fill_(float("-inf"))
        self.g_cum[:, 0] = 0.0
        self.g_node_planes[0].zero_()
        self.g_tok_planes[0].zero_()
        self.input_ids.fill_(self.token_base)  # stand-in for the last prompt token
        self.positions.copy_(self.prompt_len_rows)
        self.seq_lens.copy_((self.prompt_len_rows + 1).to(torch.int32))

    def _level0_from_prefill(self) -> None:
        """Level 0 from the last prompt token of every request: one logits row per request, the
        top ``beam_width`` legal first codes become the request's beams (init_from_prefill_batch,
        search/expand.py:168-237, with the candidate set widened to the whole level). Same kernels as
        a decode step, with one input beam per request."""
        if self.prefill_hidden is None:
            raise RuntimeError("level0_from_prefill needs prefill() first")
        logits, mx, ls, _ = self.head.logits_level(self.prefill_hidden, 0)
        self.col.fill_(0)
        out = sid_beam_step(self._cum0, logits, mx, ls, self._node0, self.trie, self.level_tok_base[0], self.bw,
                            token_ids_in=self._tok0, token_ids_out=self.tok_planes[1],
                            node_ids_out=self.node_planes[1], col=self.col, out=self.outs[0])
        self.cum.copy_(out.vals)
        if self.trie is None:
            self.node_planes[1].fill_(-1)
        self.input_ids.copy_(out.tokens.reshape(-1))

    def _step_body(self, s: int) -> None:
        """Device work of decode step ``s`` (level ``s``); allocation-stable, capturable."""
        src, dst = s & 1, (s & 1) ^ 1
        # slot table: the windows follow last step's parents (scheduler/kv_remap.py:30-66), this step's
        # slots go in (scheduler.py:1305-1310), the flat slot list of the attention call comes out
        kv_table_step(self.req_to_token, self.rows_idx, self.seq_lens, self.kv_indices, self.kv_indptr,
                      new_slot=self.out_cache_loc,
                      parents_rel=self.outs[s - 1].parents.view(-1) if s > 0 else None,
                      prefix_len=self.prefix_len_rows, group_indptr=self.group_indptr)
        batch = ForwardBatch(input_ids=self.input_ids, req_pool_indices=self.rows_idx, seq_lens=self.seq_lens,
                             positions=self.positions, out_cache_loc=self.out_cache_loc, kv_indices=self.kv_indices,
                             kv_indptr=self.kv_indptr)
        self.attn.prepare(batch, reuse_prefix=s > self.first_step)
        hidden = self.model.forward(batch)
        self.g_col.fill_(s)
        if self.sharded is not None:
            # the ranks' hidden rows (e4m3 + scales) in rank order, then the head on this rank's codes of
            # the level for every request of the group; the merged winners land in the group's state
            h8, h_scale = per_token_quant_fp8(hidden)
            gh, gs = self.sharded.gather_hidden(h8, h_scale.reshape(-1))
            kl = self.sizes[s]
            lo, hi = kl // self.world * self.rank, kl // self.world * (self.rank + 1)
            local = (gh, gs, self.head._level_weights[s][lo:hi], self.head._level_scales[s][lo:hi])
            self.sharded.step(self.g_cum, local, self.g_node_planes[src], self.trie, self.level_tok_base[s], kl,
                              self.bw, level=s, token_ids_in=self.g_tok_planes[src],
                              token_ids_out=self.g_tok_planes[dst], node_ids_out=self.g_node_planes[dst],
                              col=self.g_col, out=self.g_outs[s])
            out = self.outs[s]
            self.g_cum.copy_(self.g_outs[s].vals)
        elif self.fused_head:
            h8, h_scale = per_token_quant_fp8(hidden)
            out = sid_head_topk(self.cum, h8, h_scale, self.head._level_weights[s], self.head._level_scales[s],
                                self.node_planes[src], self.trie, self.level_tok_base[s], self.bw, self.head_ws,
                                cand_capacity=self.cand_caps[s], token_ids_in=self.tok_planes[src],
                                token_ids_out=self.tok_planes[dst], node_ids_out=self.node_planes[dst], col=self.col,
                                out=self.outs[s])
        else:
            logits, mx, ls, _ = self.head.logits_level(hidden, s)
            out = sid_beam_step(self.cum, logits, mx, ls, self.node_planes[src], self.trie, self.level_tok_base[s],
                                self.bw, token_ids_in=self.tok_planes[src], token_ids_out=self.tok_planes[dst],
                                node_ids_out=self.node_planes[dst], col=self.col, out=self.outs[s])
        # state of the next step (the window remap by out.parents is deferred to its table call, as
        # scheduler.py:1590-1610 defers it)
        if self.sharded is None:
            self.cum.copy_(out.vals)
        if self.trie is None:
            self.node_planes[dst].fill_(-1)
        self.input_ids.copy_(out.tokens.reshape(-1))
        self.positions.add_(1)
        self.seq_lens.add_(1)

    def capture(self) -> None:
        """Warm up and capture one CUDA graph per step."""
        if not self.use_graphs:
            return
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            self.run(host_io=False, _eager=True)  # warm-up: module loading, attribute setting
        torch.cuda.current_stream(self.device).wait_stream(stream)
        torch.cuda.synchronize(self.device)
        self.reset()
        for s in range(self.first_step, self.steps):
            self.out_cache_loc.copy_(self.h_loc[s], non_blocking=True)
            gph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gph):
                self._step_body(s)
            self.graphs[s] = gph
        torch.cuda.synchronize(self.device)
        self.reset()

    def run(self, host_io: bool = True, _eager: bool = False) -> None:
        """One wave: all decode steps. With ``host_io`` the per-step slot ids come
        from pinned host memory and the final beams are read back to the host."""
        self.reset()
        if self.first_step:
            self._level0_from_prefill()
        for s in range(self.first_step, self.steps):
            if host_io:
                self.out_cache_loc.copy_(self.h_loc[s], non_blocking=True)
            else:
                self.out_cache_loc.copy_(self.d_loc[s])
            if self.graphs[s] is not None and not _eager:
                self.graphs[s].replay()
            else:
                self._step_body(s)
        if host_io:
            last = self.steps & 1
            self.h_vals.copy_(self.cum, non_blocking=True)
            self.h_tokens.copy_(self.tok_planes[last], non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()

    def prefill(self, chunk_tokens: Optional[int] = None) -> torch.Tensor:
        """Run the model over the prompts (seeded random token ids) so that the pool holds their real
        K/V instead of the synthetic fill. Request 0 computes the shared prefix, the others take it as a
        cached prefix (a radix hit; ``extend_prefix_lens``, core.py:81-101) and extend only their own tokens.
        By default everything is one extend batch. With ``chunk_tokens`` every request extends at most that
        many tokens per pass (chunked prefill, for prompts that do not fit one batch): each pass is an extend
        batch over what the earlier passes left in the pool; the other requests join in the pass in which
        request 0 completes the shared prefix (inside a layer K/V are written before attention reads them).
        Eager, like the reference's prefill. Returns the hidden state of each request's last prompt token,
        ``[n_requests, hidden]`` (engine/engine.py:286-303)."""
        dev = self.device
        sp = self.shared_prefix
        pre = [0 if r == 0 else min(sp, p) for r, p in enumerate(self.prompt_lens)]
        if min(p - q for p, q in zip(self.prompt_lens, pre)) <= 0:
            raise ValueError("every request needs at least one token of its own after the shared prefix")
        g = torch.Generator().manual_seed(self.data_seed + 17)
        shared_ids = torch.randint(0, self.token_base, (sp,), generator=g)
        full_ids = []
        for r, plen in enumerate(self.prompt_lens):
            own = torch.randint(0, self.token_base, (plen - min(sp, plen),), generator=g)
            full_ids.append(torch.cat((shared_ids[: min(sp, plen)], own)))
        table = self.req_to_token[self.rows:].cpu()
        chunk = int(chunk_tokens) if chunk_tokens else max(self.prompt_lens)
        if chunk <= 0:
            raise ValueError("chunk_tokens must be positive")
        # the pass in which request 0 has the whole shared prefix in the pool: the others start there
        first_pass = [0] + [max(0, -(-min(sp, self.prompt_lens[0]) // chunk) - 1)] * (self.n - 1)
        done = list(pre)  # tokens of each request already in the pool
        last_hidden = torch.empty((self.n, self.cfg.hidden_size), dtype=torch.bfloat16, device=dev)
        self.prefill_tokens = 0
        k = 0
        while any(d < p for d, p in zip(done, self.prompt_lens)):
            reqs = [r for r in range(self.n) if done[r] < self.prompt_lens[r] and k >= first_pass[r]]
            ext = [min(chunk, self.prompt_lens[r] - done[r]) for r in reqs]
            seq_l = [done[r] + e for r, e in zip(reqs, ext)]
            rows = self.prefill_rows[torch.tensor(reqs, dtype=torch.int64, device=dev)]
            seq = torch.tensor(seq_l, dtype=torch.int32, device=dev)
            kv_indices = torch.empty(sum(seq_l), dtype=torch.int32, device=dev)
            kv_indptr = torch.empty(len(reqs) + 1, dtype=torch.int32, device=dev)
            kv_table_step(self.req_to_token, rows, seq, kv_indices, kv_indptr)  # plain gather
            loc = torch.cat([table[r, done[r]: done[r] + e] for r, e in zip(reqs, ext)]).to(torch.int64)
            qo = torch.zeros(len(reqs) + 1, dtype=torch.int32)
            qo[1:] = torch.cumsum(torch.tensor(ext), 0)
            batch = ForwardBatch(
                input_ids=torch.cat([full_ids[r][done[r]: done[r] + e] for r, e in zip(reqs, ext)]).to(dev),
                req_pool_indices=rows, seq_lens=seq,
                positions=torch.cat([torch.arange(done[r], done[r] + e) for r, e in zip(reqs, ext)]).to(dev),
                out_cache_loc=loc.to(dev), is_prefill=True, kv_indices=kv_indices, kv_indptr=kv_indptr,
                extend_prefix_lens=[done[r] for r in reqs], extend_seq_lens=ext, qo_indptr=qo.to(dev))
            hidden = self.model.forward(batch)
            last = self.model.last_token_hidden(hidden, batch)
            for i, (r, e) in enumerate(zip(reqs, ext)):
                done[r] += e
                if done[r] == self.prompt_lens[r]:
                    last_hidden[r] = last[i]
            self.prefill_tokens += int(qo[-1])
            k += 1
        self.prefill_passes = k
        self.prefill_hidden = last_hidden
        return self.prefill_hidden

    # results of the last run (device tensors)
    @property
    def final_tokens(self) -> torch.Tensor:
        return self.tok_planes[self.steps & 1]

    @property
    def final_nodes(self) -> torch.Tensor:
        return self.node_planes[self.steps & 1]
