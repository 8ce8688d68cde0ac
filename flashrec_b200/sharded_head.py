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
              level_tok_base, idx_width, trie=None, beam_width=None):
        from flashrec_b200._lib import call, ptr, stream_ptr
        from flashrec_b200.sid_decode import BeamStepOut

        s, n, k = all_vals.shape
        bw = int(beam_width) if beam_width is not None else int(node_ids.shape[1])
        dev = all_vals.device
        tr = trie.descriptor() if trie is not None else None
        out = BeamStepOut(*(torch.empty((n, k), dtype=dt, device=dev)
                            for dt in (torch.float32, torch.int64, torch.int64, torch.int64, torch.int64)))
        do_exp = token_ids_in is not None
        call("fr_topk_merge_shards", ptr(out.vals), ptr(out.parents), ptr(out.tokens), ptr(out.indices),
             ptr(out.child), ptr(all_vals), ptr(all_idx), ptr(all_child), ptr(node_ids), ptr(token_ids_in),
             ptr(token_ids_out), ptr(node_ids_out), None, ptr(col), ctypes.byref(tr) if tr is not None else None,
             int(level_tok_base), int(idx_width), s, n, bw, k,
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
                              token_ids_in, token_ids_out, node_ids_out, col, level_tok_base, level_width,
                              trie=trie, beam_width=int(cum.shape[1]))


def _main() -> None:
    """Self-check and timing of the sharded head on real GPUs, one rank per GPU:

        python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
            --master-port P -m flashrec_b200.sharded_head [--requests 16 --beam 2048 ...]

    A wide-beam catalog search shaped like the largest baseline configuration (4 levels x 4096 codes,
    Zipf-skewed 10M-item catalog, 2048 beams): every level is decoded through the sharded protocol and,
    on the same inputs and row statistics, through the unsharded beam step; all ranks must end in the
    unsharded result bit for bit. Prints one JSON line (rank 0) with the step times (CUDA events, max over ranks)."""
    import argparse
    import json
    import os

    import numpy as np

    from flashrec_b200.kernel.sglops import fp8_scaled_mm, per_token_quant_fp8
    from flashrec_b200.layers import quantize_weight_fp8
    from flashrec_b200.sid_decode import sid_beam_step
    from flashrec_b200.trie import build_trie_device

    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=16)
    ap.add_argument("--beam", type=int, default=2048)
    ap.add_argument("--levels", type=int, default=4)
    ap.add_argument("--width", type=int, default=4096)
    ap.add_argument("--items", type=int, default=10_000_000)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--reps", type=int, default=5)
    args = ap.parse_args()

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    n, bw, L, kl, base = args.requests, args.beam, args.levels, args.width, 151_936
    sizes = [kl] * L
    rng = np.random.default_rng(0)  # the same catalog, weights and hidden states on every rank
    cols = [np.minimum(rng.zipf(1.1, args.items) - 1, kl - 1) if l < 2 else rng.integers(0, kl, args.items)
            for l in range(L)]
    trie = build_trie_device(torch.from_numpy(np.stack(cols, 1).astype(np.int32)).to(dev), sizes, base)
    g = torch.Generator(device=dev).manual_seed(1)
    w = torch.randn((L * kl, args.hidden), generator=g, device=dev) * 0.02
    wq, ws = quantize_weight_fp8(w)
    del w
    head = ShardedSidHead()
    lo, hi = shard_range(kl, rank, world)

    def planes():
        cum = torch.full((n, bw), float("-inf"), device=dev)
        cum[:, 0] = 0.0
        return (cum, torch.zeros((n, bw), dtype=torch.int64, device=dev),
                torch.zeros((n, bw, L), dtype=torch.int64, device=dev))

    cum_s, node_s, tok_s = planes()
    cum_u, node_u, tok_u = planes()
    ok = True
    stat_gap = 0.0
    t_sharded, t_unsharded = [], []
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    for lv in range(L):
        hidden = (torch.randn((n * bw, args.hidden), generator=g, device=dev)).to(torch.bfloat16)
        a_q, a_s = per_token_quant_fp8(hidden)
        rows = slice(lv * kl + lo, lv * kl + hi)
        local = fp8_scaled_mm(a_q, wq[rows].t(), a_s, ws.reshape(-1)[rows], torch.float32)  # this rank's columns
        full = torch.empty((world, n * bw, hi - lo), dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(full.view(-1, hi - lo), local)
        full = full.permute(1, 0, 2).reshape(n * bw, kl).contiguous()
        col = torch.full((n,), lv, dtype=torch.int32, device=dev)
        for rep in range(args.reps + 1):  # the first repetition warms up
            tok_o, node_o = torch.zeros_like(tok_s), torch.zeros_like(node_s)
            dist.barrier()
            e0, e1 = ev(), ev()
            e0.record()
            out_s = head.step(cum_s, local, node_s, trie, base + lv * kl, kl, bw, token_ids_in=tok_s,
                              token_ids_out=tok_o, node_ids_out=node_o, col=col)
            e1.record()
            torch.cuda.synchronize()
            if rep:
                t_sharded.append(e0.elapsed_time(e1))
        # unsharded on the same logits: timed with its own one-pass row statistics, then (for the bit-exact
        # comparison) run with the statistics the protocol combines from the shards: the two normalisers
        # agree to rounding only, since they sum the row in different orders
        ops = head.ops
        for rep in range(args.reps + 1):
            tok_r, node_r = torch.zeros_like(tok_u), torch.zeros_like(node_u)
            e0, e1 = ev(), ev()
            e0.record()
            mx, ls = ops.local_stats(full)
            out_1 = sid_beam_step(cum_u, full, mx, ls, node_u, trie, base + lv * kl, bw, token_ids_in=tok_u,
                                  token_ids_out=tok_r, node_ids_out=node_r, col=col)
            e1.record()
            torch.cuda.synchronize()
            if rep:
                t_unsharded.append(e0.elapsed_time(e1))
        smx, sls = ops.local_stats(local)
        cmx, cls_ = ops.combine_stats(head._all_gather(smx), head._all_gather(sls))
        tok_r, node_r = torch.zeros_like(tok_u), torch.zeros_like(node_u)
        out_u = sid_beam_step(cum_u, full, cmx, cls_, node_u, trie, base + lv * kl, bw, token_ids_in=tok_u,
                              token_ids_out=tok_r, node_ids_out=node_r, col=col)
        fin = torch.isfinite(out_u.vals) & torch.isfinite(out_1.vals)
        stat_gap = max(stat_gap, float((out_u.vals[fin] - out_1.vals[fin]).abs().max().item()) if fin.any() else 0.0)
        ok = ok and torch.equal(out_s.vals, out_u.vals) and torch.equal(out_s.tokens, out_u.tokens)
        ok = ok and torch.equal(out_s.parents, out_u.parents) and torch.equal(tok_o, tok_r)
        ok = ok and torch.equal(node_o, node_r)
        cum_s, node_s, tok_s = out_s.vals.clone(), node_o, tok_o
        cum_u, node_u, tok_u = out_u.vals.clone(), node_r, tok_r
    live = torch.isfinite(cum_s)
    flags = torch.tensor([int(ok), int((node_s[live] == -1).all())], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    t = torch.tensor([sum(t_sharded) / args.reps, sum(t_unsharded) / args.reps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({
            "check": "sharded SID head == unsharded, all ranks, all levels", "equal": bool(flags[0].item()),
            "complete_sids_reached": bool(flags[1].item()), "n_gpus": world, "requests": n, "beam_width": bw,
            "levels": L, "level_width": kl, "catalog_items": int(trie.arrays.n_items), "trie_nodes": trie.n_nodes,
            "live_beams": int(live.sum().item()),
            "ms_sharded_head_all_levels": float(t[0].item()), "ms_unsharded_head_all_levels": float(t[1].item()),
            "max_score_gap_vs_one_pass_statistics": stat_gap,
            "note": "head step only (statistics, exchange, beam step, merge); logits GEMM excluded from both"}))
    dist.barrier()
    dist.destroy_process_group()
    if not flags[0].item():
        raise SystemExit(1)


if __name__ == "__main__":
    _main()
