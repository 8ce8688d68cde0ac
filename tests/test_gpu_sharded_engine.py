"""The decode engine with the SID head split by token range over two GPUs (NCCL): model body data-parallel
over the ranks' own requests, hidden rows all-gathered, head on the rank's code range for all requests,
winners merged. Needs two GPUs (skipped otherwise); the host protocol alone runs on CPU ranks in
tests/test_sharded_head_gloo.py."""

import datetime
import os
import socket
import traceback

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=90))
    try:
        _body(rank, world, dev, dist, q)
    except Exception:  # the parent fails the test with this text instead of waiting for a result
        q.put(("error", rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def _body(rank, world, dev, dist, q):
    from flashrec_b200 import device_status
    from flashrec_b200.decoder import Qwen3Config
    from flashrec_b200.sharded_head import ShardedSidHead
    from flashrec_b200.sid_decode import SidDecodeEngine
    from flashrec_b200.trie import build_trie_device

    rng = np.random.default_rng(3)
    sizes, base = [256, 256, 256], 1000
    items = np.unique(rng.integers(0, 256, (30000, 3)), axis=0).astype(np.int32)
    trie = build_trie_device(torch.from_numpy(items).to(dev), sizes, base, layout="csr")
    cfg = Qwen3Config(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=128, max_position_embeddings=256, vocab_size=base + sum(sizes))
    n, bw = 2, 64
    plens = [40 + 7 * rank, 55 + 3 * rank]
    kw = dict(shared_prefix=16, page_size=16, seed=0, data_seed=rank)
    sh = SidDecodeEngine(cfg, n, bw, plens, sizes, base, trie, dev, sharded_head=ShardedSidHead(), **kw)
    sh.prefill()
    sh.run(host_io=False, _eager=True)
    eager = (sh.cum.clone(), sh.tok_planes[sh.steps & 1].clone(), sh.g_cum.clone())
    sh.capture()
    sh.run(host_io=True)
    torch.cuda.synchronize()
    assert device_status() == (0, 0)
    # graph replay == eager, and every rank holds the same state of the whole group
    assert torch.equal(sh.cum, eager[0]) and torch.equal(sh.tok_planes[sh.steps & 1], eager[1])
    both = [torch.empty_like(sh.g_cum) for _ in range(world)]
    dist.all_gather(both, sh.g_cum.contiguous())
    assert all(torch.equal(b, both[0]) for b in both)
    nodes = sh.final_nodes
    assert int(((nodes != -1) & torch.isfinite(sh.cum)).sum()) == 0  # complete, legal SIDs only
    # the same requests through the unsharded engine with the same weights
    un = SidDecodeEngine(cfg, n, bw, plens, sizes, base, trie, dev, **kw)
    un.prefill()
    un.run(host_io=False, _eager=True)
    torch.cuda.synchronize()
    q.put((rank, sh.cum.cpu().numpy(), sh.tok_planes[sh.steps & 1].cpu().numpy(), un.cum.cpu().numpy(),
           un.tok_planes[un.steps & 1].cpu().numpy()))
    sh.graphs = [None] * sh.steps  # captured NCCL work goes before the process group does
    torch.cuda.synchronize()
    dist.barrier()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_head_engine_equals_the_unsharded_engine_on_two_gpus():
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in procs:
            results.append(q.get(timeout=240))
            assert results[-1][0] != "error", results[-1][2]
    finally:
        for p in procs:
            p.join(timeout=30 if len(results) == len(procs) and results[-1][0] != "error" else 1)
            if p.is_alive():
                p.terminate()
    assert all(p.exitcode == 0 for p in procs)
    for rank, cum_s, tok_s, cum_u, tok_u in results:
        for r in range(cum_s.shape[0]):
            live_s, live_u = np.isfinite(cum_s[r]), np.isfinite(cum_u[r])
            assert live_s.sum() == live_u.sum() and live_s.sum() > 0
            sid_s = {tuple(t): v for t, v in zip(tok_s[r][live_s].tolist(), cum_s[r][live_s].tolist())}
            sid_u = {tuple(t): v for t, v in zip(tok_u[r][live_u].tolist(), cum_u[r][live_u].tolist())}
            common = set(sid_s) & set(sid_u)
            # the shards' combined normaliser differs from the one-pass one by rounding: the beams agree except
            # where scores tie within that rounding at the cut
            assert len(common) >= 0.95 * len(sid_u), (rank, r, len(common), len(sid_u))
            assert max(abs(sid_s[k] - sid_u[k]) for k in common) < 2e-2
            assert tuple(tok_s[r][0]) == tuple(tok_u[r][0]) or abs(cum_s[r][0] - cum_u[r][0]) < 1e-3
