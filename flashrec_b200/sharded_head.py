"""Token-range-sharded SID head step across ranks (one process per GPU).

Each rank owns the codes ``[lo, hi)`` of every level (its slice of the lm_head
rows and of the level's logits). Per step:

  1. local row statistics (max, log-sum-exp) of the local logits slice
  2. all-gather of the statistics  ->  statistics of the full row
  3. local beam step over the local codes (global normaliser, global flat indices)
  4. all-gather of the local winners (score, flat index, child node)
  5. every rank merges the ``world`` sorted lists into the same global top-K and
     applies expand / advance, so all ranks continue with identical beam state.

The collectives are plain ``torch.distributed`` all-gathers (NCCL on GPUs): the
exchanged records are tiny (``rows * 8`` and ``N * K * 20`` bytes per rank) and
land in local memory before any kernel reads them. The arithmetic is delegated
to an ``ops`` object: :class:`CudaHeadOps` calls the C-ABI kernels; tests inject
a CPU implementation to exercise the protocol with the gloo backend.
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
    """The arithmetic of the sharded step on the local GPU (C-ABI kernels)."""

    def local_stats(self, logits: torch.Tensor):
        from flashrec_b200._lib import call, ptr, stream_ptr

        t, k = logits.shape
        mx = torch.empty(t, dtype=torch.float32, device=logits.device)
        ls = torch.empty(t, dtype=torch.float32, device=logits.device)
        call("fr_logsumexp_rows", ptr(logits), logits.stride(0), ptr(mx), ptr(ls), None, 0, t, k,
             stream_ptr(logits.device))
        return mx, ls

    def combine_stats(self, all_mx: torch.Tensor, all_ls: torch.Tensor):
        from flashrec_b200._lib import call, ptr, stream_ptr

        s, t = all_mx.shape
        mx = torch.empty(t, dtype=torch.float32, device=all_mx.device)
        ls = torch.empty(t, dtype=torch.float32, device=all_mx.device)
        call("fr_lse_combine_shards", ptr(all_mx), ptr(all_ls), ptr(mx), ptr(ls), s, t, stream_ptr(all_mx.device))
        return mx, ls

    def local_step(self, cum, logits, mx, ls, node_ids, trie, level_tok_base, k, idx_base, idx_width):
        from flashrec_b200.sid_decode import sid_beam_step

        o = sid_beam_step(cum, logits, mx, ls, node_ids, trie, level_tok_base, k, idx_base=idx_base,
                          idx_width=idx_width)
        return o.vals, o.indices, o.child

    def merge(self, all_vals, all_idx, all_child, node_ids, token_ids_in, token_ids_out, node_ids_out, col,
              level_tok_base, idx_width):
        from flashrec_b200._lib import call, ptr, stream_ptr
        from flashrec_b200.sid_decode import BeamStepOut

        s, n, k = all_vals.shape
        bw = int(node_ids.shape[1])
        dev = all_vals.device
        out = BeamStepOut(*(torch.empty((n, k), dtype=dt, device=dev)
                            for dt in (torch.float32, torch.int64, torch.int64, torch.int64, torch.int64)))
        do_exp = token_ids_in is not None
        call("fr_topk_merge_shards", ptr(out.vals), ptr(out.parents), ptr(out.tokens), ptr(out.indices),
             ptr(out.child), ptr(all_vals), ptr(all_idx), ptr(all_child), ptr(node_ids), ptr(token_ids_in),
             ptr(token_ids_out), ptr(node_ids_out), None, ptr(col), int(level_tok_base), int(idx_width), s, n, bw, k,
             int(token_ids_in.shape[2]) if do_exp else 0, int(do_exp), int(do_exp and node_ids_out is not None),
             stream_ptr(dev))
        return out


class ShardedSidHead:
    def __init__(self, ops=None, group: Optional[dist.ProcessGroup] = None):
        self.ops = ops if ops is not None else CudaHeadOps()
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def _all_gather(self, t: torch.Tensor) -> torch.Tensor:
        t = t.contiguous()
        out = torch.empty((self.world * int(t.shape[0]),) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=self.group)
        return out.view((self.world,) + tuple(t.shape))

    def step(self, cum, local_logits, node_ids, trie, level_tok_base: int, level_width: int, select_k: int, *,
             token_ids_in=None, token_ids_out=None, node_ids_out=None, col=None):
        """``local_logits`` [N*BW, hi-lo] are this rank's columns of the level's logits;
        every rank must pass shards of equal width (pad the level if necessary)."""
        lo, hi = shard_range(level_width, self.rank, self.world)
        if int(local_logits.shape[1]) != hi - lo:
            raise ValueError("local_logits width does not match this rank's shard")
        if level_width % self.world != 0:
            raise ValueError("level width must be divisible by the world size")
        smx, sls = self.ops.local_stats(local_logits)
        mx, ls = self.ops.combine_stats(self._all_gather(smx), self._all_gather(sls))
        vals, idx, child = self.ops.local_step(cum, local_logits, mx, ls, node_ids, trie, level_tok_base, select_k,
                                               lo, level_width)
        return self.ops.merge(self._all_gather(vals), self._all_gather(idx), self._all_gather(child), node_ids,
                              token_ids_in, token_ids_out, node_ids_out, col, level_tok_base, level_width)
