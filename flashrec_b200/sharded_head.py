"""Token-range-sharded SID head step across ranks (one process per GPU).

Each rank owns the codes ``[lo, hi)`` of every level: its slice of the head rows, and of the level's
candidates. The model body runs data-parallel (each rank on its own requests); the head needs every row
on every rank, so the step starts with the ranks' quantised hidden rows being gathered. Per level:

  0. all-gather of the e4m3 hidden rows and their scales (skipped when the caller already has all rows)
  1. local head GEMM on the rank's codes: row statistics of those codes + the trie-legal candidates
     (``fr_sid_head_topk`` phase 1; the logits are never written)
  2. ONE all-gather of the statistics, ``[2, rows]`` floats per rank  ->  statistics of the full row
  3. local beam step over the rank's candidates with the full row's normaliser (phase 2); the winners
     leave as 16-byte records {score, flat index, child node}
  4. ONE all-gather of the records, ``[N, K]`` x 16 bytes per rank
  5. every rank merges the ``world`` sorted lists into the same global top-K and applies expand /
     advance, so all ranks continue with identical beam state.

The collectives are plain ``torch.distributed`` all-gathers (NCCL on GPUs): the data lands in local memory
before any kernel reads it. The arithmetic is delegated to an ``ops`` object: :class:`CudaHeadOps` calls the
C-ABI kernels; tests inject a CPU implementation to exercise the protocol with the gloo backend.
"""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(width: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous code range of ``rank``; the remainder goes to the first ranks."""
    base, rem = divmod(int(width), int(world))
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class CudaHeadOps:
    """The arithmetic of the sharded step on the local GPU (C-ABI kernels). ``local`` is the tuple
    ``(hidden_fp8 [rows, H], hidden_scale [rows], w_local e4m3 [hi - lo, H], s_local f32 [hi - lo])``."""

    def __init__(self):
        from flashrec_b200.sid_decode import SidHeadWorkspace

        self.ws = SidHeadWorkspace()
        self._cap = None

    def _capacity(self, trie, level, bw, width):
        if trie is not None and level is not None and hasattr(trie, "candidate_bound"):
            return trie.candidate_bound(int(level), bw)
        return bw * width

    def local_stats(self, cum, local, node_ids, trie, level_tok_base, lo, level_width, level):
        from flashrec_b200.sid_decode import sid_head_topk

        h8, hs, w, s = local
        n, bw = int(cum.shape[0]), int(cum.shape[1])
        self._cap = self._capacity(trie, level, bw, int(w.shape[0]))
        stats = torch.empty((2, n * bw), dtype=torch.float32, device=cum.device)
        sid_head_topk(cum, h8, hs, w, s, node_ids, trie, level_tok_base, 1, self.ws, cand_capacity=self._cap,
                      idx_base=lo, idx_width=level_width, phase=1, row_max=stats[0], row_logsum=stats[1])
        return stats

    def combine_stats(self, all_stats: torch.Tensor):
        from flashrec_b200._lib import call, ptr, stream_ptr

        s, _, t = all_stats.shape
        out = torch.empty((2, t), dtype=torch.float32, device=all_stats.device)
        # shard s holds its maxima at all_stats[s, 0] and its log-sums at all_stats[s, 1]: stride 2 * t
        call("fr_lse_combine_shards", ptr(all_stats), ptr(all_stats[0, 1]), ptr(out[0]), ptr(out[1]), s, t, 2 * t,
             stream_ptr(all_stats.device))
        return out[0], out[1]

    def local_step(self, cum, local, mx, ls, node_ids, trie, level_tok_base, k, lo, level_width):
        from flashrec_b200.sid_decode import sid_head_topk

        h8, hs, w, s = local
        n = int(cum.shape[0])
        rec = torch.empty((n, int(k), 4), dtype=torch.int32, device=cum.device)
        sid_head_topk(cum, h8, hs, w, s, node_ids, trie, level_tok_base, k, self.ws, cand_capacity=self._cap,
                      idx_base=lo, idx_width=level_width, phase=2, row_max=mx, row_logsum=ls, out_records=rec)
        return rec

    def merge(self, all_rec, node_ids, token_ids_in, token_ids_out, node_ids_out, col, level_tok_base, idx_width, trie,
              bw, out=None):
        from flashrec_b200._lib import call, ptr, stream_ptr
        from flashrec_b200.sid_decode import BeamStepOut

        s, n, k, _ = all_rec.shape
        dev = all_rec.device
        if out is None:
            out = BeamStepOut(*(torch.empty((n, k), dtype=dt, device=dev)
                                for dt in (torch.float32, torch.int64, torch.int64, torch.int64, torch.int64)))
        tr = trie.descriptor() if trie is not None else None
        do_exp = token_ids_in is not None and token_ids_out is not None
        call("fr_topk_merge_shards", ptr(out.vals), ptr(out.parents), ptr(out.tokens), ptr(out.indices),
             ptr(out.child), None, None, None, ptr(all_rec), ptr(node_ids), ptr(token_ids_in), ptr(token_ids_out),
             ptr(node_ids_out), None, ptr(col), ctypes.byref(tr) if tr is not None else None, int(level_tok_base),
             int(idx_width), s, n, int(bw), k, int(token_ids_in.shape[2]) if do_exp else 0, int(do_exp),
             int(do_exp and node_ids_out is not None and node_ids is not None), stream_ptr(dev))
        return out


class ShardedSidHead:
    def __init__(self, ops=None, group: Optional[dist.ProcessGroup] = None):
        self.ops = ops if ops is not None else CudaHeadOps()
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def _all_gather(self, t: torch.Tensor) -> torch.Tensor:
        t = t.contiguous()
        out = torch.empty((self.world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out.view((self.world * int(t.shape[0]),) + tuple(t.shape[1:])) if t.dim() else out,
                                    t, group=self.group)
        return out

    def gather_hidden(self, hidden_fp8_local: torch.Tensor, scale_local: torch.Tensor):
        """Step 0: every rank's quantised hidden rows, in rank order (e4m3 bytes travel as uint8)."""
        h = self._all_gather(hidden_fp8_local.view(torch.uint8))
        s = self._all_gather(scale_local.reshape(-1))
        return h.view(-1, h.shape[-1]).view(hidden_fp8_local.dtype), s.view(-1)

    def step(self, cum, local, node_ids, trie, level_tok_base: int, level_width: int, select_k: int, *, level=None,
             token_ids_in=None, token_ids_out=None, node_ids_out=None, col=None, out=None):
        """``local``: what this rank's ``ops`` compute from (:class:`CudaHeadOps`: the hidden rows of ALL
        requests and the rank's head rows). Every rank must own shards of equal width. ``out``: a
        ``BeamStepOut`` of ``[N, K]`` buffers to write the merged result into (CUDA ops only)."""
        if level_width % self.world != 0:
            raise ValueError("level width must be divisible by the world size")
        lo, hi = shard_range(level_width, self.rank, self.world)
        stats = self.ops.local_stats(cum, local, node_ids, trie, level_tok_base, lo, level_width, level)
        mx, ls = self.ops.combine_stats(self._all_gather(stats))
        rec = self.ops.local_step(cum, local, mx, ls, node_ids, trie, level_tok_base, select_k, lo, level_width)
        if out is None:  # (stand-in ops of the CPU protocol test take no buffers)
            return self.ops.merge(self._all_gather(rec), node_ids, token_ids_in, token_ids_out, node_ids_out, col,
                                  level_tok_base, level_width, trie, int(cum.shape[1]))
        return self.ops.merge(self._all_gather(rec), node_ids, token_ids_in, token_ids_out, node_ids_out, col,
                              level_tok_base, level_width, trie, int(cum.shape[1]), out=out)
