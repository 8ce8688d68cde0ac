"""Prefill (extend) attention on the GPU through the C ABI: against the fixture made with the
reference's SDPA prefill branch, against the CPU oracle on ragged batches, and against the decode
path (the last prompt token computed by a prefill equals the same token computed as a decode step)."""

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits, fp8_from_bits
from oracle import sid_oracle as O
from test_oracle_golden import _prefill_fixture

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FP8 = torch.float8_e4m3fn


def _run_prefill(q, kc, vc, ext, pre, kv_indices, hq, hkv):
    from flashrec_b200.attention import AttentionBackend, TokenToKVPool
    from flashrec_b200.decoder import ForwardBatch

    pool = TokenToKVPool(1, kc.shape[0], hkv, 128, FP8, DEV)
    pool.k[0].copy_(kc.to(DEV))
    pool.v[0].copy_(vc.to(DEV))
    be = AttentionBackend(pool, hq, hkv, 128)
    seq = [e + p for e, p in zip(ext, pre)]
    qo = torch.tensor(np.concatenate(([0], np.cumsum(ext))), dtype=torch.int32, device=DEV)
    kv = torch.tensor(np.concatenate(([0], np.cumsum(seq))), dtype=torch.int32, device=DEV)
    t = int(q.shape[0])
    batch = ForwardBatch(input_ids=torch.zeros(t, dtype=torch.int64, device=DEV), req_pool_indices=None,
                         seq_lens=torch.tensor(seq, dtype=torch.int32, device=DEV),
                         positions=torch.zeros(t, dtype=torch.int64), out_cache_loc=torch.zeros(t, dtype=torch.int64),
                         is_prefill=True, kv_indices=kv_indices.to(DEV), kv_indptr=kv, extend_prefix_lens=list(pre),
                         extend_seq_lens=list(ext), qo_indptr=qo)
    return be.forward(q.to(DEV), None, None, 0, batch, skip_store=True), qo.cpu(), kv.cpu()


def test_prefill_attention_golden_reference():
    g, qo, kv = _prefill_fixture()
    out, _, _ = _run_prefill(bf16_from_bits(g["q"]), fp8_from_bits(g["k_cache"]), fp8_from_bits(g["v_cache"]),
                             g["ext"].tolist(), g["pre"].tolist(), torch.from_numpy(g["kv_indices"]), 2, 1)
    ref = bf16_from_bits(g["out"]).float()
    assert torch.allclose(out.float().cpu(), ref, rtol=2e-2, atol=2e-2)  # bf16 attention output: 2e-2


@pytest.mark.parametrize("hq,hkv,ext,pre", [
    (16, 8, [200, 1, 64, 65, 7], [0, 0, 0, 0, 0]),        # plain causal; tile-edge and single-token prompts
    (16, 8, [33, 128, 1, 90], [64, 17, 300, 1]),          # cached prefixes (radix hits), incl. a 1-token extend
    (8, 8, [150, 40], [0, 70]),
    (8, 2, [100, 31], [5, 0]),
    (8, 1, [70, 20, 16], [0, 130, 3]),
    (16, 8, [1024, 700], [0, 324]),                       # the longest prompts of the bench workload
])
def test_prefill_attention_vs_oracle(hq, hkv, ext, pre):
    rng = np.random.default_rng(hq * 100 + hkv + len(ext))
    seq = [e + p for e, p in zip(ext, pre)]
    slots = sum(seq) + 16
    kc = torch.from_numpy(rng.standard_normal((slots, hkv, 128)).astype(np.float32)).bfloat16().to(FP8)
    vc = torch.from_numpy(rng.standard_normal((slots, hkv, 128)).astype(np.float32)).bfloat16().to(FP8)
    kvi = torch.from_numpy((rng.permutation(slots - 1)[: sum(seq)] + 1).astype(np.int32))
    q = torch.from_numpy(rng.standard_normal((sum(ext), hq, 128)).astype(np.float32)).bfloat16()
    out, qo, kv = _run_prefill(q, kc, vc, ext, pre, kvi, hq, hkv)
    ref = O.prefill_attention(q, kc, vc, qo, kv, kvi, hq // hkv).float()
    err = (out.float().cpu() - ref).abs().max() / ref.abs().max()
    assert err < 2e-2, err
    # the first token of a request without a prefix sees one key: its output is that key's V row
    for g in range(len(ext)):
        if pre[g] == 0:
            v0 = vc[int(kvi[int(kv[g])])].float().repeat_interleave(hq // hkv, dim=0)
            assert torch.allclose(out[int(qo[g])].float().cpu(), v0, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("tc", [True, False])
def test_model_prefill_then_decode_is_consistent(tc):
    """Whole model: the hidden state of the last prompt token from one prefill of L tokens against the
    same token run as a decode step on top of a prefill of the first L - 1 tokens, and
    ``last_token_hidden`` picks each request's last row. With the tcgen05 decode path (``tc``) both routes
    run the same tile arithmetic on the same K/V bytes: the hidden states are equal bit for bit."""
    from flashrec_b200.attention import AttentionBackend, TokenToKVPool
    from flashrec_b200.decoder import ForwardBatch, Qwen3Config, Qwen3ForCausalLM

    cfg = Qwen3Config(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                      intermediate_size=1024, num_hidden_layers=2, max_position_embeddings=512, vocab_size=700)
    lens = [97, 30, 200]
    pool = TokenToKVPool(cfg.num_hidden_layers, 1024, cfg.num_key_value_heads, cfg.head_dim, FP8, DEV)
    attn = AttentionBackend(pool, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                            max_shared_len=256 if tc else 0)
    model = Qwen3ForCausalLM(cfg, attn, DEV)
    model.init_random(seed=4)
    g = torch.Generator().manual_seed(9)
    ids = [torch.randint(0, 700, (n,), generator=g) for n in lens]
    starts = np.concatenate(([1], 1 + np.cumsum(lens)[:-1]))  # each request's slots are consecutive, from slot 1
    slots = [torch.arange(int(s), int(s) + n) for s, n in zip(starts, lens)]

    def prefill(upto):  # prefill of the first `upto[r]` tokens of every request
        ext = list(upto)
        qo = torch.tensor(np.concatenate(([0], np.cumsum(ext))), dtype=torch.int32, device=DEV)
        batch = ForwardBatch(
            input_ids=torch.cat([i[:n] for i, n in zip(ids, ext)]).to(DEV), req_pool_indices=None,
            seq_lens=torch.tensor(ext, dtype=torch.int32, device=DEV),
            positions=torch.cat([torch.arange(n) for n in ext]).to(DEV),
            out_cache_loc=torch.cat([s[:n] for s, n in zip(slots, ext)]).to(DEV), is_prefill=True,
            kv_indices=torch.cat([s[:n] for s, n in zip(slots, ext)]).to(torch.int32).to(DEV), kv_indptr=qo,
            extend_prefix_lens=[0] * len(ext), extend_seq_lens=ext, qo_indptr=qo)
        hidden = model.forward(batch)
        return hidden, model.last_token_hidden(hidden, batch)

    hidden_full, last_full = prefill(lens)
    offs = np.cumsum(lens) - 1
    assert torch.equal(last_full, hidden_full[torch.from_numpy(offs).to(DEV)])
    kv_full = [pool.k[l].clone() for l in range(cfg.num_hidden_layers)]
    for l in range(cfg.num_hidden_layers):
        pool.k[l].zero_()
        pool.v[l].zero_()
    prefill([n - 1 for n in lens])
    n = len(lens)
    indptr = torch.tensor(np.concatenate(([0], np.cumsum(lens))), dtype=torch.int32, device=DEV)
    attn.set_groups(torch.arange(n + 1, dtype=torch.int32, device=DEV), 1)
    batch = ForwardBatch(input_ids=torch.stack([i[-1] for i in ids]).to(DEV), req_pool_indices=None,
                         seq_lens=torch.tensor(lens, dtype=torch.int32, device=DEV),
                         positions=torch.tensor([x - 1 for x in lens], device=DEV),
                         out_cache_loc=torch.stack([s[-1] for s in slots]).to(DEV),
                         kv_indices=torch.cat(slots).to(torch.int32).to(DEV), kv_indptr=indptr)
    attn.prepare(batch)
    last_dec = model.forward(batch)
    if tc:
        assert torch.equal(last_dec, last_full)
    else:
        # the kernel without scratch (mma.sync, bf16 P) against the tcgen05 one: each is within 2e-2 of the
        # oracle on its own, but per-token FP8 re-quantisation after the attention turns last-bit differences
        # into e4m3 rounding flips (6 % of an element), so the whole-model bound is loose: it catches a wrong
        # mask or a wrong slot (errors of order 1), not rounding
        d = (last_dec.float() - last_full.float()).abs()
        assert d.max() / last_full.float().abs().max() < 0.15 and d.mean() / last_full.float().abs().mean() < 0.1
    # both routes wrote the same layer-0 K bytes (layer 0's keys do not depend on attention; the GEMMs run at
    # different row counts, so allow the odd rounding tie to fall the other way)
    diff = (pool.k[0].view(torch.uint8) != kv_full[0].view(torch.uint8)).float().mean().item()
    assert diff < 1e-3, diff


def test_extend_over_cached_prefix_equals_full_prefill():
    """A request that takes another request's first 40 tokens as a cached prefix (their K/V written by that
    request in the same batch) ends in the hidden state of prefilling all of its tokens itself."""
    from flashrec_b200.attention import AttentionBackend, TokenToKVPool
    from flashrec_b200.decoder import ForwardBatch, Qwen3Config, Qwen3ForCausalLM

    cfg = Qwen3Config(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                      intermediate_size=1024, num_hidden_layers=2, max_position_embeddings=512, vocab_size=700)
    pool = TokenToKVPool(cfg.num_hidden_layers, 1024, cfg.num_key_value_heads, cfg.head_dim, FP8, DEV)
    attn = AttentionBackend(pool, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim)
    model = Qwen3ForCausalLM(cfg, attn, DEV)
    model.init_random(seed=6)
    g = torch.Generator().manual_seed(2)
    shared, sp = torch.randint(0, 700, (40,), generator=g), 40
    ids = [torch.cat((shared, torch.randint(0, 700, (n,), generator=g))) for n in (50, 85)]

    def run(reqs):  # reqs: (token ids, cached prefix length, slot list of all its tokens)
        ext = [len(i) - p for i, p, _ in reqs]
        qo = torch.tensor(np.concatenate(([0], np.cumsum(ext))), dtype=torch.int32, device=DEV)
        kv = torch.tensor(np.concatenate(([0], np.cumsum([len(i) for i, _, _ in reqs]))), dtype=torch.int32, device=DEV)
        batch = ForwardBatch(
            input_ids=torch.cat([i[p:] for i, p, _ in reqs]).to(DEV), req_pool_indices=None,
            seq_lens=torch.tensor([len(i) for i, _, _ in reqs], dtype=torch.int32, device=DEV),
            positions=torch.cat([torch.arange(p, len(i)) for i, p, _ in reqs]).to(DEV),
            out_cache_loc=torch.cat([sl[p:] for _, p, sl in reqs]).to(DEV), is_prefill=True,
            kv_indices=torch.cat([sl for _, _, sl in reqs]).to(torch.int32).to(DEV), kv_indptr=kv,
            extend_prefix_lens=[p for _, p, _ in reqs], extend_seq_lens=ext, qo_indptr=qo)
        return model.last_token_hidden(model.forward(batch), batch)

    s0 = torch.arange(1, 1 + len(ids[0]))
    s1 = torch.cat((s0[:sp], torch.arange(200, 200 + len(ids[1]) - sp)))
    both = run([(ids[0], 0, s0), (ids[1], sp, s1)])
    alone = run([(ids[1], 0, torch.arange(500, 500 + len(ids[1])))])
    d = (both[1].float() - alone[0].float()).abs()
    assert d.max() / alone.float().abs().max() < 1e-1 and d.mean() / alone.float().abs().mean() < 2e-2


def test_prefill_attention_empty_request_and_unaligned_lengths():
    """A request without extend tokens in the batch contributes nothing and disturbs nobody; key counts that
    are not multiples of the 64-token tile and a query count that is not a multiple of the 64-row tile."""
    hq, hkv = 16, 8
    ext, pre = [5, 0, 67, 1], [59, 10, 62, 0]
    rng = np.random.default_rng(1)
    seq = [e + p for e, p in zip(ext, pre)]
    slots = sum(seq) + 8
    kc = torch.from_numpy(rng.standard_normal((slots, hkv, 128)).astype(np.float32)).bfloat16().to(FP8)
    vc = torch.from_numpy(rng.standard_normal((slots, hkv, 128)).astype(np.float32)).bfloat16().to(FP8)
    kvi = torch.from_numpy((rng.permutation(slots - 1)[: sum(seq)] + 1).astype(np.int32))
    q = torch.from_numpy(rng.standard_normal((sum(ext), hq, 128)).astype(np.float32)).bfloat16()
    out, qo, kv = _run_prefill(q, kc, vc, ext, pre, kvi, hq, hkv)
    ref = O.prefill_attention(q, kc, vc, qo, kv, kvi, hq // hkv).float()
    assert (out.float().cpu() - ref).abs().max() / ref.abs().max() < 2e-2
    assert torch.isfinite(out.float()).all()


@pytest.mark.parametrize("chunk", [64, 5, 1000])
def test_chunked_prefill_leaves_the_same_pool_as_one_batch(chunk):
    """``SidDecodeEngine.prefill(chunk_tokens=...)``: every request extends at most ``chunk`` tokens per pass over
    what the earlier passes left in the pool (chunk 5 is shorter than the 16-token shared prefix: the other
    requests wait for request 0 to finish it). Layer 0's K bytes depend on no attention and must equal the
    one-batch prefill exactly; deeper layers and the last-token hidden states see attention computed over a
    cached prefix instead of inside one batch (same arithmetic, other tile boundaries): nearly all e4m3 bytes
    equal, hidden states within the attention tolerance. A chunk that covers every prompt is the one-batch run."""
    from flashrec_b200.decoder import Qwen3Config
    from flashrec_b200.sid_decode import SidDecodeEngine
    from flashrec_b200.trie import build_trie_arrays, trie_to_device

    cfg = Qwen3Config(hidden_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                      intermediate_size=512, num_hidden_layers=3, max_position_embeddings=512, vocab_size=1000 + 64)
    rng = np.random.default_rng(2)
    sizes, base = [32, 32], 1000
    trie = trie_to_device(build_trie_arrays(np.stack([rng.integers(0, 32, 300) for _ in sizes], 1), sizes, base), "csr", DEV)
    prompts = [97, 30, 200]

    def run(chunk_tokens):
        eng = SidDecodeEngine(cfg, 3, 32, prompts, sizes, base, trie, DEV, shared_prefix=16, seed=3, use_graphs=False)
        h = eng.prefill(chunk_tokens=chunk_tokens).clone()
        table = eng.req_to_token[eng.rows:].cpu()
        slots = torch.cat([table[r, :p] for r, p in enumerate(prompts)]).to(torch.int64).to(DEV)
        kv = [(eng.pool.k[l][slots].view(torch.uint8).clone(), eng.pool.v[l][slots].view(torch.uint8).clone())
              for l in range(cfg.num_hidden_layers)]
        return h, kv, eng

    h1, kv1, e1 = run(None)
    h2, kv2, e2 = run(chunk)
    assert e1.prefill_passes == 1 and e1.prefill_tokens == e2.prefill_tokens == 97 + (30 - 16) + (200 - 16)
    if chunk >= max(prompts):
        assert e2.prefill_passes == 1 and torch.equal(h1, h2)
        assert all(torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) for a, b in zip(kv1, kv2))
        return
    assert e2.prefill_passes >= -(-(200 - 16) // chunk)  # the longest request extends 184 tokens of its own
    assert torch.equal(kv1[0][0], kv2[0][0]) and torch.equal(kv1[0][1], kv2[0][1])
    for l in range(1, cfg.num_hidden_layers):
        for a, b in zip(kv1[l], kv2[l]):
            assert (a != b).float().mean() < 0.05, l
    d = (h1.float() - h2.float()).abs()
    assert d.max() / h1.float().abs().max() < 0.15 and d.mean() / h1.float().abs().mean() < 2e-2
