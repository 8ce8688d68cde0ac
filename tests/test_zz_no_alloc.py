"""The workspace-free variant of the fused beam step.

Some hosts bind the C ABI from a decode worker that has no allocator to ask for
a workspace: the server's device memory is split up once at start-up, and a tick
must not wait on cudaMalloc. ``fr_mask_topk_expand_static`` serves them from a
fixed array inside the library. This file checks, through the C ABI, that it
returns exactly what ``fr_mask_topk_expand`` returns, on two calls in a row (the
array is shared and keeps the previous call's contents), and that an oversized
request is refused. It is collected last on purpose."""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, n, bw, c, k, L):
    from flashrec_b200.trie import build_trie_arrays, trie_to_device

    rng = np.random.default_rng(seed)
    sizes, base = (16, 16, 16), 900
    arrays = build_trie_arrays(np.stack([rng.integers(0, s, 500) for s in sizes], 1), list(sizes), base)
    trie = trie_to_device(arrays, "csr", DEV)
    n1 = int(arrays.level_start[2] - arrays.level_start[1])
    t = lambda a: torch.from_numpy(a).to(DEV)  # noqa: E731
    cum = t(rng.standard_normal((n, bw)).astype(np.float32))
    lp = torch.sort(t(rng.standard_normal((n, bw, c)).astype(np.float32)), dim=-1, descending=True).values.contiguous()
    tok = t(rng.integers(base + 16, base + 32, (n, bw, c)))
    nodes = t(rng.integers(1, 1 + n1, (n, bw)))
    token_ids = t(rng.integers(base, base + 16, (n, bw, L)))
    col = torch.full((n,), 1, dtype=torch.int32, device=DEV)
    return trie, cum, lp, tok, nodes, token_ids, col


def _run(entry, with_scratch, trie, cum, lp, tok, nodes, token_ids, col, k, masked=True):
    from flashrec_b200._lib import call, ptr, stream_ptr

    n, bw, c = lp.shape
    L = token_ids.shape[2]
    i64 = dict(dtype=torch.int64, device=DEV)
    outs = dict(vals=torch.empty((n, k), device=DEV), parents=torch.empty((n, k), **i64),
                tokens=torch.empty((n, k), **i64), indices=torch.empty((n, k), **i64),
                child=torch.empty((n, k), **i64), tok_out=torch.zeros_like(token_ids), node_out=torch.zeros_like(nodes))
    tr = trie.descriptor()
    head = [ptr(outs["vals"]), ptr(outs["parents"]), ptr(outs["tokens"]), ptr(outs["indices"]), ptr(outs["child"])]
    scratch = [ptr(torch.empty(n * bw * c, device=DEV))] if with_scratch else []
    call(entry, *head, *scratch, ptr(cum), ptr(lp), ptr(tok), ptr(nodes), ptr(token_ids), ptr(outs["tok_out"]),
         ptr(outs["node_out"]), None, ptr(col), ctypes.byref(tr), n, bw, c, k, L, int(masked), 1, int(masked),
         stream_ptr(torch.device(DEV)))
    torch.cuda.synchronize()
    return outs


def test_static_scratch_entry_matches_the_workspace_entry_twice():
    for seed, shape in ((1, (3, 64, 24, 64, 3)), (2, (2, 128, 40, 100, 4))):  # second call: other sizes, same array
        n, bw, c, k, L = shape
        args = _case(seed, n, bw, c, k, L)
        ref = _run("fr_mask_topk_expand", True, *args, k)
        got = _run("fr_mask_topk_expand_static", False, *args, k)
        for name in ref:
            assert torch.equal(ref[name], got[name]), (seed, name)


def test_static_scratch_entry_refuses_oversized_requests():
    from flashrec_b200 import FlashRecKernelError

    args = _case(3, 1, 8, 4, 8, 2)
    trie, cum, lp, tok, nodes, token_ids, col = args
    from flashrec_b200._lib import call, ptr, stream_ptr

    tr = trie.descriptor()
    with pytest.raises(FlashRecKernelError, match="FR_ERR_UNSUPPORTED"):
        # claims N*BW*C = 4 * 2048 * 512 floats > 2 Mi: rejected before any pointer is touched
        call("fr_mask_topk_expand_static", None, None, None, None, None, ptr(cum), ptr(lp), ptr(tok), ptr(nodes), None,
             None, None, None, None, ctypes.byref(tr), 4, 2048, 512, 8, 0, 1, 0, 0, stream_ptr(torch.device(DEV)))


def test_static_scratch_entry_unmasked_step_matches_and_has_no_size_limit():
    """Without masking the fixed array is never touched: the two entries agree, and a step larger
    than the array (N*BW*C = 2.25 Mi candidates) is served instead of refused."""
    args = _case(4, 2, 64, 16, 48, 3)
    ref = _run("fr_mask_topk_expand", True, *args, 48, masked=False)
    got = _run("fr_mask_topk_expand_static", False, *args, 48, masked=False)
    for name in ("vals", "parents", "tokens", "indices", "tok_out"):
        assert torch.equal(ref[name], got[name]), name
    n, bw, c, k = 9, 512, 512, 512
    g = torch.Generator(device=DEV).manual_seed(5)
    cum = torch.randn((n, bw), generator=g, device=DEV)
    lp = torch.randn((n, bw, c), generator=g, device=DEV)
    tok = torch.randint(0, 1000, (n, bw, c), generator=g, device=DEV)
    trie = args[0]
    big_ref = _run("fr_mask_topk_expand", True, trie, cum, lp, tok, torch.zeros((n, bw), dtype=torch.int64, device=DEV),
                   torch.zeros((n, bw, 2), dtype=torch.int64, device=DEV),
                   torch.zeros(n, dtype=torch.int32, device=DEV), k, masked=False)
    big = _run("fr_mask_topk_expand_static", False, trie, cum, lp, tok,
               torch.zeros((n, bw), dtype=torch.int64, device=DEV),
               torch.zeros((n, bw, 2), dtype=torch.int64, device=DEV), torch.zeros(n, dtype=torch.int32, device=DEV), k,
               masked=False)
    for name in ("vals", "parents", "tokens", "indices"):
        assert torch.equal(big_ref[name], big[name]), name
