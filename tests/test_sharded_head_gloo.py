"""Host protocol of the token-range-sharded SID head on CPU ranks (gloo,
world_size 2): one all-gather of the statistics, local steps, one all-gather of the 16-byte winner
records, merge.
The arithmetic is injected from the CPU oracle; the GPU kernels behind the same
protocol are checked bit for bit against the unsharded step in
tests/test_gpu_attn_head.py::test_merge_shards_equals_unsharded."""

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sid_oracle as O


class OracleHeadOps:
    """CPU stand-in for CudaHeadOps: ``local`` is the rank's slice of the level's fp32 logits."""

    def __init__(self, otr):
        self.otr = otr

    def local_stats(self, cum, local, node_ids, trie, level_tok_base, lo, level_width, level):
        return torch.stack(O.row_stats(local))  # [2, rows]

    def combine_stats(self, all_stats):
        all_mx, all_ls = all_stats[:, 0], all_stats[:, 1]
        mx = all_mx.amax(dim=0)
        return mx, torch.log(torch.exp(all_ls + (all_mx - mx)).sum(dim=0))

    def local_step(self, cum, logits, mx, ls, node_ids, trie, level_tok_base, k, idx_base, idx_width):
        n, bw = cum.shape
        w = logits.shape[1]
        lp = O.logprobs_from_stats(logits, mx, ls).view(n, bw, w)
        toks = (level_tok_base + idx_base + torch.arange(w))[None, None, :].expand(n, bw, w)
        r = O.mask_topk_expand(cum, lp, toks, k, node_ids=node_ids, trie=self.otr, apply_expand=False)
        gidx = r["parents"] * idx_width + idx_base + (r["indices"] % w)
        gidx = torch.where(torch.isfinite(r["vals"]), gidx, torch.zeros_like(gidx))
        # the 16-byte record of the exchange: {score bits, flat index, child low, child high}
        rec = torch.empty((n, k, 4), dtype=torch.int32)
        rec[..., 0] = r["vals"].contiguous().view(torch.int32)
        rec[..., 1] = gidx.to(torch.int32)
        rec[..., 2] = (r["child"] & 0xffffffff).to(torch.int64).view(torch.int64).to(torch.int32)
        rec[..., 3] = (r["child"] >> 32).to(torch.int32)
        return rec

    def merge(self, all_rec, node_ids, tin, tout, nout, col, level_tok_base, idx_width, trie, bw):
        s, n, k, _ = all_rec.shape
        all_vals = all_rec[..., 0].contiguous().view(torch.float32)
        all_idx = all_rec[..., 1].to(torch.int64) & 0xffffffff
        all_child = (all_rec[..., 3].to(torch.int64) << 32) | (all_rec[..., 2].to(torch.int64) & 0xffffffff)
        out = dict(vals=torch.empty(n, k), idx=torch.empty(n, k, dtype=torch.int64),
                   child=torch.empty(n, k, dtype=torch.int64))
        for i in range(n):
            v = all_vals[:, i].reshape(-1).numpy()
            ix = all_idx[:, i].reshape(-1).numpy()
            ch = all_child[:, i].reshape(-1).numpy()
            live = np.isfinite(v)
            order = np.lexsort((ix[live], -v[live].astype(np.float64)))[:k]
            m = order.shape[0]
            out["vals"][i] = float("-inf")
            out["idx"][i] = 0
            out["child"][i] = 0
            out["vals"][i, :m] = torch.from_numpy(v[live][order])
            out["idx"][i, :m] = torch.from_numpy(ix[live][order])
            out["child"][i, :m] = torch.from_numpy(ch[live][order])
        return out


def _case():
    from flashrec_b200.trie import build_trie_arrays

    rng = np.random.default_rng(5)
    n, bw, kl = 2, 24, 64
    sizes, base = [kl, kl], 300
    arrays = build_trie_arrays(np.stack([rng.integers(0, kl, 900) for _ in sizes], 1), sizes, base)
    otr = O.OracleTrie(arrays.csr_keys, arrays.edge_child, arrays.vsz, base, arrays.invalid_node)
    n1 = int(arrays.level_start[2] - arrays.level_start[1])
    nodes = torch.from_numpy(rng.integers(1, 1 + n1, (n, bw)))
    cum = torch.from_numpy(rng.standard_normal((n, bw)).astype(np.float32))
    cum[1, 10:] = float("-inf")
    logits = torch.from_numpy(rng.standard_normal((n * bw, kl)).astype(np.float32))
    return otr, nodes, cum, logits, base + kl, kl, bw


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flashrec_b200.sharded_head import ShardedSidHead, shard_range

        otr, nodes, cum, logits, tok_base, kl, bw = _case()
        lo, hi = shard_range(kl, rank, world)
        head = ShardedSidHead(ops=OracleHeadOps(otr))
        out = head.step(cum, logits[:, lo:hi].contiguous(), nodes, None, tok_base, kl, bw)
        q.put((rank, out["vals"].numpy(), out["idx"].numpy(), out["child"].numpy()))
    finally:
        dist.destroy_process_group()


def test_shard_ranges_partition_the_level():
    from flashrec_b200.sharded_head import shard_range

    for width, world in ((8192, 8), (4096, 8), (10, 3), (5, 8)):
        spans = [shard_range(width, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == width
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1


def test_sharded_step_equals_unsharded_gloo_world2():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    otr, nodes, cum, logits, tok_base, kl, bw = _case()
    ref = O.sid_beam_step(cum, logits, nodes, otr, tok_base, bw)
    for rank, vals, idx, child in results:
        live = np.isfinite(ref["vals"].numpy())
        assert np.array_equal(np.isfinite(vals), live)
        assert np.allclose(vals[live], ref["vals"].numpy()[live], atol=1e-5)
        assert np.array_equal(idx[live], ref["indices"].numpy()[live])
        assert np.array_equal(child[live], ref["child"].numpy()[live])
    assert np.array_equal(results[0][2], results[1][2])  # every rank ends with the same beams
