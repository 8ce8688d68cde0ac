"""Drop-in checks against the reference engine itself (installed unmodified under ``oracle/_ref``):

1. the reference's own GPU tests for this path, run with this library's kernels swapped in at the
   reference's function boundary (``tests/refshim.py``): in each of them the CUDA side is now this
   library and the expected side is still the reference's own torch code;
2. the reference's ``Qwen3ForCausalLM`` (its modules, its weight loading) with the kernels and the
   attention backend swapped in, one decode step captured and replayed by the reference's own
   ``DecodeGraphRunner`` at 2 x beam width rows, against this repository's ``decoder.py`` — bit for bit.
"""

import numpy as np
import pytest
import torch

import refshim

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not refshim.available(), reason="oracle/_ref not installed")]
DEV = "cuda:0"
FP8 = torch.float8_e4m3fn

# (reference test file, class, test) — the CUDA-gated tests of the kernels on this path
REFERENCE_TESTS = [
    ("test_rms_fp8", "TestRmsFp8", "test_rmsnorm_quant_matches_sequential"),
    ("test_rms_fp8", "TestRmsFp8", "test_fused_add_quant_matches_sequential"),
    ("test_rms_fp8", "TestRmsFp8", "test_shared_qkv_quant_matches_three_linears"),
    ("test_silu_fp8", "TestSiluFp8", "test_silu_quant_matches_sequential"),
    ("test_qk_rope_kv", "TestQkRopeKv", "test_fused_matches_sequential_fp8_store"),
    ("test_mlp", "TestSiluAndMul", "test_cuda_matches_cpu"),
    ("test_kv_pool", "TestGatherAndPool", "test_gather_gpu_seq_lens_with_total"),
    ("test_expand", "TestExpand", "test_genrec_cuda_matches_pytorch"),
    ("test_expand", "TestExpand", "test_genrec_cuda_skips_masked_heads"),
    ("test_expand", "TestExpand", "test_genrec_cuda_production_shape"),
    ("test_expand", "TestExpand", "test_workspace_canonicalizes_cuda_device"),
    ("test_expand", "TestExpand", "test_genrec_cuda_pingpong_flips_and_matches_cpu"),
    ("test_graph_expand", "TestGraphExpand", "test_fill_topk_tokens_matches_advanced_index"),
    ("test_graph_expand", "TestGraphExpand", "test_graph_replay_matches_eager_and_clone_survives"),
    ("test_graph_expand", "TestGraphExpand", "test_graph_flip_kernel_matches_eager"),
    ("test_graph_expand", "TestGraphExpand", "test_single_request_graph_replay_keeps_beam_diversity"),
    ("test_trie_csr", "TestTrieCsrParity", "test_mask_candidates_matches_dense"),
    ("test_trie_csr", "TestTrieCsrParity", "test_advance_matches_dense"),
]


@pytest.mark.parametrize("stem,cls,name", REFERENCE_TESTS, ids=[f"{s}::{n}" for s, _, n in REFERENCE_TESTS])
def test_reference_own_test_passes_with_this_library_swapped_in(stem, cls, name):
    mod = refshim.load_reference_test_module(stem)
    obj = getattr(mod, cls)()
    fn = getattr(obj, name)
    if stem == "test_trie_csr":  # the module's pytest fixture, called by hand
        fn(mod.trie_pair.__wrapped__() if hasattr(mod.trie_pair, "__wrapped__") else _trie_pair(mod))
    else:
        fn()
    torch.cuda.synchronize()


def _trie_pair(mod):
    import random

    rng = random.Random(7)
    device = torch.device("cuda")
    seqs = mod._random_sequences(rng, 120)
    dense, csr = mod._build_pair(seqs, device)
    return rng, device, seqs, dense, csr


def test_reference_model_and_graph_runner_with_swapped_kernels_equal_this_decoder_bitwise():
    """The reference's model classes + its CUDA-graph runner on top of this library, against decoder.py."""
    refshim.install()
    import flashrec.models.qwen3 as RQ
    from flashrec.core import ForwardBatch as RefBatch
    from flashrec.engine.graph import DecodeGraphRunner

    from flashrec_b200.attention import AttentionBackend, TokenToKVPool
    from flashrec_b200.core import ForwardBatch
    from flashrec_b200.decoder import Qwen3Config, Qwen3ForCausalLM
    from flashrec_b200.layers import quantize_weight_fp8

    H, HQ, HKV, D, I, L, V = 512, 4, 2, 128, 1024, 2, 600
    bw, rows, prompt, slots = 64, 128, 40, 2048
    g = torch.Generator().manual_seed(9)
    w = [dict(qkv=0.02 * torch.randn((HQ + 2 * HKV) * D, H, generator=g), o=0.02 * torch.randn(H, HQ * D, generator=g),
              gate_up=0.02 * torch.randn(2 * I, H, generator=g), down=0.02 * torch.randn(H, I, generator=g),
              ln1=1 + 0.1 * torch.randn(H, generator=g), ln2=1 + 0.1 * torch.randn(H, generator=g),
              qn=1 + 0.1 * torch.randn(D, generator=g), kn=1 + 0.1 * torch.randn(D, generator=g)) for _ in range(L)]
    embed = (0.02 * torch.randn(V, H, generator=g)).bfloat16()
    final = 1 + 0.1 * torch.randn(H, generator=g)
    kv0 = [(torch.randn(slots, HKV, D, generator=g).bfloat16().to(FP8), torch.randn(slots, HKV, D, generator=g).bfloat16().to(FP8))
           for _ in range(L)]

    def fresh_pool():
        pool = TokenToKVPool(L, slots, HKV, D, FP8, torch.device(DEV))
        for i, (k, v) in enumerate(kv0):
            pool.k[i].copy_(k.to(DEV))
            pool.v[i].copy_(v.to(DEV))
        return pool

    # two requests x 64 beams: each request's beams share its 40 prompt slots, one own slot per row
    ids = torch.randint(0, V, (rows,), generator=g)
    own = torch.arange(1000, 1000 + rows)
    lists = torch.cat([torch.cat([torch.arange(1 + r * prompt, 1 + (r + 1) * prompt).repeat(bw, 1),
                                  own[r * bw:(r + 1) * bw, None]], dim=1) for r in range(2)]).to(torch.int32)
    positions = torch.full((rows,), prompt)

    # ---- this repository's decoder -------------------------------------------------------------------
    cfg = Qwen3Config(hidden_size=H, num_attention_heads=HQ, num_key_value_heads=HKV, head_dim=D, intermediate_size=I,
                      num_hidden_layers=L, max_position_embeddings=256, vocab_size=V)
    pool_a = fresh_pool()
    attn_a = AttentionBackend(pool_a, HQ, HKV, D, beam_width=bw, max_shared_len=prompt + 1)
    mine = Qwen3ForCausalLM(cfg, attn_a, DEV, fuse_residual=False, fuse_rope_gemm=False)
    for layer, lw in zip(mine.layers, w):
        layer.self_attn.qkv_proj.load(lw["qkv"].to(DEV), quantize_fp8=True)
        layer.self_attn.o_proj.load(lw["o"].to(DEV), quantize_fp8=True)
        layer.mlp.gate_up_proj.load(lw["gate_up"].to(DEV), quantize_fp8=True)
        layer.mlp.down_proj.load(lw["down"].to(DEV), quantize_fp8=True)
        layer.mlp.prepare_fused()
        layer.input_layernorm.weight.copy_(lw["ln1"].to(DEV))
        layer.post_attention_layernorm.weight.copy_(lw["ln2"].to(DEV))
        layer.self_attn.q_norm.weight.copy_(lw["qn"].to(DEV))
        layer.self_attn.k_norm.weight.copy_(lw["kn"].to(DEV))
    mine.norm.weight.copy_(final.to(DEV))
    mine.embed_tokens = embed.to(DEV)
    batch_a = ForwardBatch(input_ids=ids.to(DEV), req_pool_indices=None,
                           seq_lens=torch.full((rows,), prompt + 1, dtype=torch.int32, device=DEV),
                           positions=positions.to(DEV), out_cache_loc=own.to(DEV), kv_indices=lists.reshape(-1).to(DEV),
                           kv_indptr=(torch.arange(rows + 1, dtype=torch.int32) * (prompt + 1)).to(DEV))
    attn_a.prepare(batch_a)
    want = mine.forward(batch_a).clone()

    # ---- the reference's model + graph runner, kernels and attention backend swapped in ---------------
    rcfg = RQ.Qwen3Config(hidden_size=H, intermediate_size=I, num_hidden_layers=L, num_attention_heads=HQ,
                          num_key_value_heads=HKV, head_dim=D, vocab_size=V, rms_norm_eps=1e-6, rope_theta=1e6,
                          max_position_embeddings=256, tie_word_embeddings=True)
    pool_b = fresh_pool()
    attn_b = AttentionBackend(pool_b, HQ, HKV, D, backend="flashinfer", fi_backend="fa2", beam_width=bw)
    theirs = RQ.Qwen3ForCausalLM(rcfg, attn_b, torch.device(DEV), torch.bfloat16)
    for layer, lw in zip(theirs.layers, w):
        for lin, key in ((layer.self_attn.qkv_proj, "qkv"), (layer.self_attn.o_proj, "o"),
                         (layer.mlp.gate_up_proj, "gate_up"), (layer.mlp.down_proj, "down")):
            q8, s8 = quantize_weight_fp8(lw[key].to(DEV))  # the same e4m3 bytes and scales as above
            lin.load(q8, weight_scale=s8)
        layer.input_layernorm.weight.data.copy_(lw["ln1"].bfloat16().to(DEV))
        layer.post_attention_layernorm.weight.data.copy_(lw["ln2"].bfloat16().to(DEV))
        layer.self_attn.q_norm.weight.data.copy_(lw["qn"].bfloat16().to(DEV))
        layer.self_attn.k_norm.weight.data.copy_(lw["kn"].bfloat16().to(DEV))
    theirs.norm.weight.data.copy_(final.bfloat16().to(DEV))
    theirs.embed_tokens.weight.data = embed.to(DEV)
    # the cos / sin table is an input of the kernels: give both sides the same one (the reference fills it
    # with the device's cos / sin, this repository with the host's; the two differ in the last bit)
    theirs.rotary.cos_sin_cache.copy_(mine.rotary.cos_sin_cache)
    max_seq = 64
    attn_b.init_graph_wrappers([rows], max_seq)
    runner = DecodeGraphRunner(device=torch.device(DEV), max_bs=rows, max_seq_len=max_seq, capture_bs=[rows], attn=attn_b)
    with torch.inference_mode():
        runner.capture(lambda b: theirs(b), attn_b.prepare)
        assert rows in runner.graphs, "the reference's runner captured no graph for this batch size"
        seq_cpu = torch.full((rows,), prompt + 1, dtype=torch.int32)
        batch_b = RefBatch(input_ids=ids.to(DEV), req_pool_indices=torch.zeros(rows, dtype=torch.int64, device=DEV),
                           seq_lens=seq_cpu.to(DEV), seq_lens_cpu=seq_cpu, positions=positions.to(DEV),
                           out_cache_loc=own.to(DEV), is_prefill=False, kv_indices=lists.reshape(-1).to(DEV))
        got, fused = runner.replay(batch_b, attn_b.prepare)
        got = got.clone()
        # eager through the same objects (no graph) gives the same bits
        attn_b.prepare(batch_b)
        eager = theirs(batch_b).clone()
    torch.cuda.synchronize()
    assert fused is None
    assert torch.equal(eager, want), float((eager.float() - want.float()).abs().max())
    assert torch.equal(got, want), float((got.float() - want.float()).abs().max())
    for i in range(L):  # and the KV pools hold the same bytes (slot 0 is the dummy slot the runner's warm-up writes)
        assert torch.equal(pool_a.k[i][1:].view(torch.uint8), pool_b.k[i][1:].view(torch.uint8))
        assert torch.equal(pool_a.v[i][1:].view(torch.uint8), pool_b.v[i][1:].view(torch.uint8))


def _write_checkpoint(path, cfg, seed, prequantised):
    """A tiny Hugging Face style Qwen3 directory: split q / k / v and gate / up matrices, either bf16 or e4m3 with
    a per-channel ``weight_scale`` (stored as [N, 1], [N] or [1]: every form the loaders accept)."""
    import json

    from safetensors.torch import save_file

    from oracle import sid_oracle as O

    g = torch.Generator().manual_seed(seed)
    H, D, I = cfg["hidden_size"], cfg["head_dim"], cfg["intermediate_size"]
    HQ, HKV, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["vocab_size"]
    tensors = {"model.embed_tokens.weight": (0.02 * torch.randn(V, H, generator=g)).bfloat16(),
               "model.norm.weight": (1 + 0.1 * torch.randn(H, generator=g)).bfloat16()}
    for li in range(cfg["num_hidden_layers"]):
        pre = f"model.layers.{li}."
        mats = {"self_attn.q_proj": (HQ * D, H), "self_attn.k_proj": (HKV * D, H), "self_attn.v_proj": (HKV * D, H),
                "self_attn.o_proj": (H, HQ * D), "mlp.gate_proj": (I, H), "mlp.up_proj": (I, H), "mlp.down_proj": (H, I)}
        for j, (name, (n, k)) in enumerate(mats.items()):
            w = 0.02 * torch.randn(n, k, generator=g)
            if prequantised:
                q8, s = O.quantize_weight_fp8(w)
                tensors[pre + name + ".weight"] = q8
                s = s.reshape(-1).float()
                key = ".weight_scale_inv" if j % 3 == 2 else ".weight_scale"  # both spellings name the scale
                tensors[pre + name + key] = s.reshape(-1, 1) if j % 2 == 0 else s
            else:
                tensors[pre + name + ".weight"] = w.bfloat16()
        for name, n in (("input_layernorm", H), ("post_attention_layernorm", H), ("self_attn.q_norm", D), ("self_attn.k_norm", D)):
            tensors[pre + name + ".weight"] = (1 + 0.1 * torch.randn(n, generator=g)).bfloat16()
    path.mkdir(parents=True, exist_ok=True)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(path / "model.safetensors"))
    (path / "config.json").write_text(json.dumps(cfg))
    return tensors


@pytest.mark.parametrize("prequantised", [True, False])
def test_checkpoint_loading_equals_the_reference_loader(tmp_path, prequantised):
    """``flashrec_b200.weights.load_weights`` against the reference's ``load_weights`` (models/weight.py:116-263) on the
    same checkpoint directory: merged qkv / gate_up matrices and their scales, o / down, norms, embedding — equal
    byte for byte, for a pre-quantised e4m3 checkpoint (scales concatenated, nothing requantised) and for a bf16
    checkpoint quantised at load; and the loaded model's decode step equals the reference model's.
    The bf16 case loads the reference model on the CPU: that is the arithmetic this library reproduces (on a GPU
    torch turns the reference's ``amax / 448`` into a multiplication by the rounded reciprocal, which moves one
    scale in a few hundred by one ulp, so the reference's own GPU and CPU loads do not agree with each other)."""
    refshim.install()
    import flashrec.models.qwen3 as RQ
    from flashrec.models.weight import load_hf_config as ref_config
    from flashrec.models.weight import load_weights as ref_load

    from flashrec_b200.attention import AttentionBackend, TokenToKVPool
    from flashrec_b200.core import ForwardBatch
    from flashrec_b200.decoder import Qwen3ForCausalLM
    from flashrec_b200.weights import load_hf_config, load_weights

    raw = dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=2,
               num_key_value_heads=1, head_dim=128, vocab_size=300, rms_norm_eps=1e-6, rope_theta=1e6,
               max_position_embeddings=128, tie_word_embeddings=True)
    _write_checkpoint(tmp_path, raw, 21, prequantised)
    cfg, rcfg = load_hf_config(str(tmp_path)), ref_config(str(tmp_path))
    dev = torch.device(DEV)
    slots, rows, prompt = 256, 64, 9
    pools = [TokenToKVPool(cfg.num_hidden_layers, slots, cfg.num_key_value_heads, 128, FP8, dev) for _ in range(2)]
    attn_a = AttentionBackend(pools[0], cfg.num_attention_heads, cfg.num_key_value_heads, 128, beam_width=rows)
    attn_b = AttentionBackend(pools[1], cfg.num_attention_heads, cfg.num_key_value_heads, 128, beam_width=rows)
    mine = Qwen3ForCausalLM(cfg, attn_a, dev, fuse_residual=False, fuse_rope_gemm=False)
    ref_dev = dev if prequantised else torch.device("cpu")
    theirs = RQ.Qwen3ForCausalLM(rcfg, attn_b, ref_dev, torch.bfloat16)
    load_weights(mine, str(tmp_path), dev, torch.bfloat16, quantize_fp8=not prequantised)
    ref_load(theirs, str(tmp_path), ref_dev, torch.bfloat16, quantize_fp8=not prequantised)
    for a, b in zip(mine.layers, theirs.layers):
        for x, y in ((a.self_attn.qkv_proj, b.self_attn.qkv_proj), (a.self_attn.o_proj, b.self_attn.o_proj),
                     (a.mlp.gate_up_proj, b.mlp.gate_up_proj), (a.mlp.down_proj, b.mlp.down_proj)):
            assert x._fp8_weight.shape == y._fp8_weight.shape
            assert torch.equal(x._fp8_weight.contiguous().view(torch.uint8).cpu(), y._fp8_weight.contiguous().view(torch.uint8).cpu())
            assert torch.equal(x._fp8_scale.reshape(-1).cpu(), y._fp8_scale.reshape(-1).float().cpu())
        for x, y in ((a.input_layernorm, b.input_layernorm), (a.post_attention_layernorm, b.post_attention_layernorm),
                     (a.self_attn.q_norm, b.self_attn.q_norm), (a.self_attn.k_norm, b.self_attn.k_norm)):
            assert torch.equal(x.weight.cpu(), y.weight.data.cpu())
    assert torch.equal(mine.norm.weight.cpu(), theirs.norm.weight.data.cpu())
    assert torch.equal(mine.embed_tokens.cpu(), theirs.embed_tokens.weight.data.cpu())
    assert mine.lm_head_weight is mine.embed_tokens  # tied: the checkpoint has no lm_head
    if not prequantised:
        return
    # one decode step of both models on the same batch (each on its own, equally filled pool)
    g = torch.Generator().manual_seed(4)
    for p in pools:
        for li in range(cfg.num_hidden_layers):
            p.k[li][1:1 + prompt].copy_(torch.randn(prompt, 1, 128, generator=torch.Generator().manual_seed(li)).bfloat16().to(FP8))
            p.v[li][1:1 + prompt].copy_(torch.randn(prompt, 1, 128, generator=torch.Generator().manual_seed(50 + li)).bfloat16().to(FP8))
    ids = torch.randint(0, cfg.vocab_size, (rows,), generator=g).to(dev)
    own = torch.arange(100, 100 + rows)
    lists = torch.cat([torch.arange(1, 1 + prompt).repeat(rows, 1), own[:, None]], dim=1).to(torch.int32)
    theirs.rotary.cos_sin_cache.copy_(mine.rotary.cos_sin_cache)
    outs = []
    for model, attn in ((mine, attn_a), (theirs, attn_b)):
        batch = ForwardBatch(input_ids=ids, req_pool_indices=None,
                             seq_lens=torch.full((rows,), prompt + 1, dtype=torch.int32, device=dev),
                             positions=torch.full((rows,), prompt, device=dev), out_cache_loc=own.to(dev),
                             kv_indices=lists.reshape(-1).to(dev),
                             kv_indptr=(torch.arange(rows + 1, dtype=torch.int32) * (prompt + 1)).to(dev))
        attn.prepare(batch)
        with torch.inference_mode():
            outs.append((model.forward(batch) if model is mine else model(batch)).clone())
    assert torch.equal(outs[0], outs[1])


def test_reference_expand_step_with_stop_tokens_on_the_swapped_selection_kernels():
    """The reference's own ``expand_step`` (search/expand.py:240-372) in its stop-token branch and its
    end-by-length branch, on CUDA tensors with ``joint_select`` / ``select_final_topk`` swapped for this
    library's (``fr_joint_select``, ``fr_select_final_topk``), against the same calls on the CPU with the
    reference's own selection: beams, scores, token planes and finished sequences equal step by step; and
    with a fixed Gumbel noise tensor (sampling without replacement) the two sides still agree."""
    refshim.install()
    import torch.nn.functional as F
    import flashrec.search.expand as RE
    from flashrec.search.expand import expand_step, init_from_prefill

    g = torch.Generator().manual_seed(5)
    vocab, bw, cand = 50, 8, 16
    lp0 = F.log_softmax(torch.randn(vocab, generator=g), -1)
    steps = [(torch.stack([torch.randperm(vocab, generator=g)[:cand] for _ in range(bw)]),
              F.log_softmax(torch.randn(bw, cand, generator=g), -1)) for _ in range(3)]
    noise = [-torch.log(-torch.log(torch.rand(bw, cand, generator=g).clamp_min(1e-20))) for _ in range(3)]
    stops = [3, 7, 11, 19]

    def run(device, temperature):
        bl = init_from_prefill(lp0.to(device), beam_width=bw, beam_candidates=cand, max_new_tokens=4, prompt_len=1)
        trace = []
        for i, (tt, tl) in enumerate(steps):
            if temperature > 0:  # the same noise on both sides instead of each device's own generator
                fixed = noise[i].to(device)
                RE.gumbel_like = lambda x, fixed=fixed: fixed
            rows = int(bl.cum_logprobs.shape[0])
            par = expand_step(bl, tt[:rows].to(device), tl[:rows].to(device), bw, stop_token_ids=stops, ignore_eos=False,
                              will_finish=(i == 2), temperature=temperature)
            trace.append((None if par is None else par.cpu(), bl.last_tokens.cpu(), bl.cum_logprobs.cpu(),
                          bl.token_ids[: bl.last_tokens.shape[0]].cpu()))
        return trace, [(tuple(s.tokens), round(s.cum_logprob, 5)) for s in bl.completed]

    keep = RE.gumbel_like
    try:
        for temperature in (0.0, 1.0):
            cpu_trace, cpu_done = run(torch.device("cpu"), temperature)
            gpu_trace, gpu_done = run(torch.device(DEV), temperature)
            assert cpu_done == gpu_done and len(cpu_done) > 0
            for a, b in zip(cpu_trace, gpu_trace):
                assert (a[0] is None) == (b[0] is None)
                if a[0] is not None:
                    assert torch.equal(a[0], b[0])
                assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])
    finally:
        RE.gumbel_like = keep
