"""GPU parity of the selection step with stop tokens and rank noise (``flashrec_b200.search``) against the
reference-written fixture and the CPU oracle: every output slot, bit for bit."""

import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import sid_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FIELDS = ("next_tokens", "parent_idx", "new_cum_logprobs", "num_survivors", "fin_tokens", "fin_parent_idx",
          "fin_cum_logprobs", "num_finished")


def test_joint_select_and_final_topk_equal_the_reference_fixture():
    from flashrec_b200.search import apply_temperature, joint_select, select_final_topk

    g = load_golden("select")
    for i in range(int(g["n_cases"])):
        cum, lp, tok, pert = (torch.from_numpy(g[f"c{i}_{n}"]).to(DEV) for n in ("cum", "lp", "tok", "pert"))
        st, k = torch.from_numpy(g[f"c{i}_stop"]).to(DEV), int(g[f"c{i}_k"])
        for tag, pt in (("plain", None), ("noise", pert)):
            r = joint_select(cum, lp, tok, st, k, perturb=pt)
            for f in FIELDS:
                assert np.array_equal(getattr(r, f).cpu().numpy(), g[f"c{i}_{tag}_{f}"]), (i, tag, f)
            if f"c{i}_{tag}_final_tokens" in g.files:
                kk = g[f"c{i}_{tag}_final_tokens"].shape[0]
                fr = select_final_topk(cum, lp, tok, kk, perturb=pt)
                assert np.array_equal(fr.tokens.cpu().numpy(), g[f"c{i}_{tag}_final_tokens"])
                assert np.array_equal(fr.parent_idx.cpu().numpy(), g[f"c{i}_{tag}_final_parent"])
                assert np.array_equal(fr.cum_logprobs.cpu().numpy(), g[f"c{i}_{tag}_final_cum"])
        t = apply_temperature(lp, 0.7)
        assert np.allclose(t.cpu().numpy(), g[f"c{i}_temp"], atol=2e-6)
        assert apply_temperature(lp, 1.0) is lp and apply_temperature(lp, 0.0) is lp


@pytest.mark.parametrize("groups,rows,cand,k,n_stop", [(3, 512, 1024, 512, 2), (1, 64, 4096, 64, 0), (5, 7, 33, 50, 30),
                                                       (2, 128, 256, 128, 300)])
def test_joint_select_batched_groups_against_the_oracle(groups, rows, cand, k, n_stop):
    """Several groups per launch (one CTA each), the bench's width (512 beams x 1024 candidates), the widest
    candidate list (4096), more slots than survivors, no stop tokens, and a stop set where nearly every
    candidate finishes; with Gumbel rank noise."""
    from flashrec_b200.search import gumbel_like, joint_select, select_final_topk

    gen = torch.Generator().manual_seed(groups * 1000 + cand)
    cum = torch.randn(groups, rows, generator=gen)
    cum[0, rows // 2:] = float("-inf") if rows > 8 else cum[0, rows // 2:]  # dead beams rank last
    lp = torch.log_softmax(torch.randn(groups, rows, cand, generator=gen), dim=-1)
    vocab = 400
    tok = torch.randint(0, vocab, (groups, rows, cand), generator=gen)
    stop = torch.randperm(vocab, generator=gen)[:n_stop]
    noise = gumbel_like(lp.to(DEV))
    assert noise.shape == lp.shape and noise.dtype == torch.float32 and torch.isfinite(noise).all()
    for pt in (None, noise):
        got = joint_select(cum.to(DEV), lp.to(DEV), tok.to(DEV), stop.to(DEV), k, perturb=pt)
        for gi in range(groups):
            ref = O.joint_select(cum[gi], lp[gi], tok[gi], stop, k, None if pt is None else pt[gi].cpu())
            for f in FIELDS:
                assert torch.equal(getattr(got, f)[gi].cpu(), torch.as_tensor(ref[f])), (gi, f)
        kk = min(k, cand)
        fin = select_final_topk(cum.to(DEV), lp.to(DEV), tok.to(DEV), kk, perturb=pt)
        for gi in range(groups):
            ref = O.select_final_topk(cum[gi], lp[gi], tok[gi], kk, None if pt is None else pt[gi].cpu())
            assert torch.equal(fin.tokens[gi].cpu(), ref["tokens"]) and torch.equal(fin.parent_idx[gi].cpu(), ref["parent_idx"])
            assert torch.equal(fin.cum_logprobs[gi].cpu(), ref["cum_logprobs"])


def test_joint_select_ties_rank_by_flat_index_and_graph_capture():
    from flashrec_b200.search import joint_select

    cum = torch.zeros(4)
    lp = torch.full((4, 8), -1.0)
    lp[2, 3] = -0.5
    tok = torch.arange(32).reshape(4, 8)
    stop = torch.tensor([1, 19])
    ref = O.joint_select(cum, lp, tok, stop, 5)
    d = [t.to(DEV) for t in (cum, lp, tok, stop)]
    got = joint_select(*d, 5)  # eager first (allocations), then the same call inside a graph
    gph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gph):
        got2 = joint_select(*d, 5)
    gph.replay()
    torch.cuda.synchronize()
    for r in (got, got2):
        for f in FIELDS:
            assert torch.equal(getattr(r, f).cpu(), torch.as_tensor(ref[f])), f


def test_joint_select_argument_limits():
    """More candidates per row than the select supports is refused before any launch; zero groups is a no-op."""
    from flashrec_b200 import FlashRecKernelError
    from flashrec_b200.search import joint_select

    cum = torch.zeros(1, 2, device=DEV)
    lp = torch.zeros(1, 2, 4100, device=DEV)
    tok = torch.zeros(1, 2, 4100, dtype=torch.int64, device=DEV)
    with pytest.raises(FlashRecKernelError):
        joint_select(cum, lp, tok, torch.empty(0, dtype=torch.int64, device=DEV), 2)
    with pytest.raises(FlashRecKernelError):
        joint_select(cum.cpu(), lp.cpu(), tok.cpu(), torch.empty(0, dtype=torch.int64), 2)  # no CPU path
    out = joint_select(torch.zeros(0, 2, device=DEV), torch.zeros(0, 2, 8, device=DEV),
                       torch.zeros(0, 2, 8, dtype=torch.int64, device=DEV), torch.empty(0, dtype=torch.int64, device=DEV), 2)
    assert out.next_tokens.shape == (0, 2) and out.num_survivors.shape == (0,)
