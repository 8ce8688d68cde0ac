"""Benchmark of the quantized SID decode step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one decode wave of the hot path: 32 concurrent requests x 512
beams = 16384 beam rows through a 28-layer Qwen3-1.7B-shaped FP8 model, the
SID head and the trie-constrained beam step, for each of the 3 SID levels.
Metric: beam rows decoded per second (rows x levels / time), whole job.

  value  device-timed (CUDA events), inputs resident in HBM, CUDA-graph replay
  e2e    same wave driven from pinned host buffers: per-step slot ids copied
         host->device, final beams (scores + SID tokens) copied device->host
  roofline      the gate_up FP8 GEMM with the SwiGLU epilogue (dominant kernel), timed alone
  cpu_baseline  the reference engine's own torch CPU path for the same step, a bounded sample
                (also what --impl reference times)

With --gpus N > 1 (launched by torch.distributed.run) every rank runs its own
replica on its own requests (requests never interact): weak scaling, no
data-path collective; the time is the max over ranks.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "sid_decode_beam_rows_per_s"
UNIT = "beam-rows/s"
WORKLOAD = dict(
    workload="qwen3-1.7b-shaped 28-layer FP8 W8A8 decode, fp8 KV, 3-level SID (3x8192), 1M-item CSR trie",
    requests=32, beam_width=512, levels=3, prompt_len="uniform[128,1024]", shared_prefix=64,
    l2_policy="working set (1.4 GB weights + activations) far larger than the 126 MB L2",
)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="config4", choices=["config4", "config5"],
                    help="config4 (default): 32 requests x 512 beams, 3 x 8192 codes, 1M items, prompts 128-1024. "
                         "config5: the widest configuration as one replica per GPU: 2048 beams, 4 x 4096 codes, 10M "
                         "Zipf items, prompts 1024-4096 (give --requests; 64 requests over the GPUs of a box is the "
                         "stated concurrency)")
    ap.add_argument("--requests", type=int, default=32)
    ap.add_argument("--beam", type=int, default=512)
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--items", type=int, default=1_000_000)
    ap.add_argument("--trie", default="csr", choices=["csr", "bitmap"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--level0-from-prefill", action="store_true",
                    help="the reference's flow: level 0 from the prefill's last-token logits, decode steps for the "
                         "other levels only (not the default workload, which runs all three levels as decode steps)")
    ap.add_argument("--no-prefill", action="store_true",
                    help="leave the prompt K/V as the synthetic fill instead of running the prefill pass")
    ap.add_argument("--no-fuse-rope-gemm", action="store_true",
                    help="run QK-norm + RoPE + KV write as their own kernel instead of in the qkv GEMM's epilogue")
    ap.add_argument("--no-fused-head", action="store_true",
                    help="run the SID head as GEMM -> row statistics -> beam step (fp32 logits in HBM) instead of the "
                         "fused head call")
    ap.add_argument("--head-compare", action="store_true",
                    help="time the SID head + beam step of every level at the bench's sizes, fused call against the "
                         "three-call flow, CSR and bitmap tries, and exit")
    ap.add_argument("--config5", action="store_true",
                    help="only run the token-range-sharded head step of the widest configuration (the `config5` object "
                         "of the JSON line, which multi-GPU runs always carry) and print it")
    ap.add_argument("--no-config5", action="store_true", help="leave the `config5` object out of a multi-GPU line")
    ap.add_argument("--sharded-head", action="store_true",
                    help="N > 1: one group of N x --requests requests; the model body data-parallel over the ranks' "
                         "own requests, the SID head split by token range over the ranks (NCCL all-gathers of the "
                         "hidden rows, the row statistics and the winners) instead of independent replicas")
    ap.add_argument("--attn-compare", action="store_true",
                    help="time one layer's decode attention on the bench's slot lists beside FlashInfer's paged "
                         "decode kernel (a library comparison) and exit")
    ap.add_argument("--ref-kernels", type=int, default=0, metavar="ROWS",
                    help="time the reference's own GPU kernels for this path (its Triton kernels and its beam_trie CUDA "
                         "source JIT-built through tvm_ffi, from the install under oracle/_ref) beside this library's at "
                         "ROWS rows and exit")
    ap.add_argument("--profile-prefill", action="store_true",
                    help="run one prefill pass between cudaProfilerStart/Stop and exit (for ncu --profile-from-start off)")
    ap.add_argument("--profile-wave", action="store_true",
                    help="run one eager (non-graph) wave between cudaProfilerStart/Stop and exit (for ncu "
                         "--profile-from-start off)")
    ap.add_argument("--gemm-shapes", type=int, default=0, metavar="ROWS",
                    help="time the FP8 GEMM of every layer shape at ROWS rows (this library and cuBLASLt) and exit")
    ap.add_argument("--profile-kernels", action="store_true",
                    help="launch each hot kernel once at the wave's shapes (random inputs) between "
                         "cudaProfilerStart/Stop and exit (for ncu --set full --profile-from-start off)")
    return ap.parse_args()


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._thr = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits"],
                    capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thr.join(timeout=10)

    def summary(self):
        sm = [int(s[0]) for s in self.samples if s and s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for s in self.samples if len(s) >= 6 for i in range(4) if s[2 + i] == "Active"})
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ---------------------------------------------------------------------------
# workload construction (seeded, synthetic)
# ---------------------------------------------------------------------------
def make_catalog(items: int, sizes, seed=0):
    import numpy as np

    rng = np.random.default_rng(seed)
    return np.stack([rng.integers(0, s, items) for s in sizes], axis=1)


def prompt_lengths(n: int, seed: int, lo: int = 128, hi: int = 1024):
    import numpy as np

    rng = np.random.default_rng(1000 + seed)
    return [int(x) for x in rng.integers(lo, hi + 1, n)]


def make_zipf_catalog(items: int, sizes, seed=0):
    """Popular first and second codes (Zipf 1.1), uniform deeper codes: a few nodes with thousands of children."""
    import numpy as np

    rng = np.random.default_rng(seed)
    cols = [np.minimum(rng.zipf(1.1, items) - 1, s - 1) if l < 2 else rng.integers(0, s, items)
            for l, s in enumerate(sizes)]
    return np.stack(cols, axis=1)


# ---------------------------------------------------------------------------
# CPU baseline = the --impl reference arm: the reference's own torch CPU path
# ---------------------------------------------------------------------------
REF_DIR = ROOT / "oracle" / "_ref"


def bench_config(args, world: int, rows: int, decode_steps: int):
    """The ``config`` object of the JSON line: the workload only, so that both arms print the same object
    (measured quantities such as the per-GPU value or the number of distinct catalog items are top-level keys)."""
    return dict(WORKLOAD, requests=args.requests, beam_width=args.beam, layers=args.layers,
                catalog_items=args.items, trie=args.trie,
                parallelism=WORKLOAD.get("parallelism", f"dp{world}"), rows_per_gpu=rows,
                decode_steps_per_wave=decode_steps)


class ReferenceCpuStep:
    """One decode step of the hot path through the UNMODIFIED reference engine on the host cores (its torch
    branch: sgl-kernel is absent, so every ``flashrec.kernel.sglops`` wrapper computes in torch, and its
    attention backend takes SDPA), installed under ``oracle/_ref`` by ``oracle/Makefile``:

      body   ``Qwen3DecoderLayer.forward`` (models/qwen3.py:198-215) of ONE layer for ``rows_body`` beam rows of
             one request over a 256-token prompt: ``RMSNorm.quant_fp8``, ``Linear.forward_fp8`` (torch._scaled_mm
             on the CPU), the KV store into the e4m3 ``TokenToKVPool``, ``AttentionBackend._sdpa``,
             ``silu_and_mul_per_token_quant_fp8``. One thing is substituted: ``RotaryEmbedding.forward``'s torch
             formula raises on a CPU (it multiplies 64-wide cos / sin into 128-wide heads), so the rotation comes
             from the oracle's restatement of the reference's Triton kernel.
      head   ``RestrictedLMHead.compute_level`` (bf16, as the reference keeps the head) for a whole request of
             ``beam`` rows, per-beam ``torch.topk`` of 2 x beam candidates and ``expand_step`` with the reference's
             CSR ``BeamValidPathTrie`` (search/expand.py:240-372).

    The step time of a request is extrapolated: body x layers x (beam / rows_body) + head. Falls back to the
    oracle port of the same ops (``kind`` "port") when ``oracle/_ref`` is not there."""

    def __init__(self, beam: int, sizes, items: int, layers: int, rows_body: int = 8):
        import numpy as np
        import torch

        self.torch = torch
        self.beam, self.layers, self.rows = int(beam), int(layers), int(rows_body)
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        self.kind = "reference" if (REF_DIR / "flashrec" / "__init__.py").exists() else "port"
        if self.kind == "port":
            self._port = lambda: cpu_baseline_port(beam, sizes, items, layers)
            return
        if str(REF_DIR) not in sys.path:
            sys.path.insert(0, str(REF_DIR))
        from flashrec.attention.flashinfer import AttentionBackend
        from flashrec.core import ForwardBatch
        from flashrec.kvcache.pool import TokenToKVPool
        from flashrec.layers import rotary as ref_rotary
        from flashrec.logits import RestrictedLMHead
        from flashrec.models.qwen3 import Qwen3Config, Qwen3DecoderLayer
        from flashrec.search import trie as trie_mod
        from flashrec.search.expand import expand_step, init_from_prefill_batch
        from flashrec.search.trie import BeamValidPathTrie

        from oracle import sid_oracle as O

        def rope_forward(self_, positions, query, key):  # see the class text
            return O.rope_neox(positions, query, key, self_.head_dim, self_.cos_sin_cache)

        ref_rotary.RotaryEmbedding.forward = rope_forward
        g = torch.Generator().manual_seed(0)
        H, HQ, HKV, D, I = 2048, 16, 8, 128, 6144
        rows, plen = self.rows, 256
        cfg = Qwen3Config(hidden_size=H, intermediate_size=I, num_hidden_layers=1, num_attention_heads=HQ,
                          num_key_value_heads=HKV, head_dim=D, vocab_size=32, rms_norm_eps=1e-6, rope_theta=1e6,
                          max_position_embeddings=plen + 8, tie_word_embeddings=True)
        dev = torch.device("cpu")
        pool = TokenToKVPool(1, plen + rows + 1, HKV, D, torch.float8_e4m3fn, dev)
        pool.k[0][1:plen + 1] = torch.randn(plen, HKV, D, generator=g).bfloat16().to(torch.float8_e4m3fn)
        pool.v[0][1:plen + 1] = torch.randn(plen, HKV, D, generator=g).bfloat16().to(torch.float8_e4m3fn)
        attn = AttentionBackend(pool, HQ, HKV, D, backend="flashinfer")
        rot = ref_rotary.RotaryEmbedding(D, plen + 8, 1e6, device=dev)
        layer = Qwen3DecoderLayer(cfg, 0, attn, rot)
        for lin, (n_out, n_in) in ((layer.self_attn.qkv_proj, ((HQ + 2 * HKV) * D, H)), (layer.self_attn.o_proj, (H, HQ * D)),
                                   (layer.mlp.gate_up_proj, (2 * I, H)), (layer.mlp.down_proj, (H, I))):
            lin.load(0.02 * torch.randn(n_out, n_in, generator=g), quantize_fp8=True)
        loc = torch.arange(plen + 1, plen + 1 + rows)
        lists = torch.cat([torch.cat((torch.arange(1, plen + 1), loc[i:i + 1])) for i in range(rows)]).to(torch.int32)
        seq = torch.full((rows,), plen + 1, dtype=torch.int64)
        self._batch = ForwardBatch(input_ids=torch.zeros(rows, dtype=torch.int64), req_pool_indices=torch.zeros(rows, dtype=torch.int64),
                                   seq_lens=seq, seq_lens_cpu=seq.clone(), positions=torch.full((rows,), plen),
                                   out_cache_loc=loc, is_prefill=False, kv_indices=lists)
        self._layer = layer
        self._x = torch.randn(rows, H, generator=g).bfloat16()
        # head of a whole request: bf16 SID rows, the reference's trie in its CSR layout
        sid_total, base = int(sum(sizes)), 0
        head = RestrictedLMHead(list(range(sid_total)))
        head.bind((0.02 * torch.randn(sid_total, H, generator=g)).bfloat16())
        head.bind_codebook(list(sizes))
        cat = make_catalog(min(items, 200_000), sizes)
        offs = np.concatenate([[0], np.cumsum(sizes)])
        tr = BeamValidPathTrie(mode="trie")
        tr.max_depth = len(sizes)
        for it in cat.tolist():
            toks = [int(base + offs[l] + it[l]) for l in range(len(sizes))]
            for dd in range(len(sizes)):
                tr.children.setdefault(tuple(toks[:dd]), set()).add(toks[dd])
        tr.all_tokens = set(range(sid_total))
        tr.finalize_index(token_base=base, vocab_size=sid_total)
        saved = trie_mod._DENSE_MAX_CELLS
        trie_mod._DENSE_MAX_CELLS = 0  # the CSR cache, as the 1M-item catalog takes
        try:
            tr._ensure_gpu_cache(dev)
        finally:
            trie_mod._DENSE_MAX_CELLS = saved
        self._trie, self._head = tr, head
        self._hidden = torch.randn(self.beam, H, generator=g).bfloat16()
        lp0, ids0 = head.compute_level(self._hidden[:1], 0)
        self._init = lambda: init_from_prefill_batch(lp0, self.beam, min(2 * self.beam, sizes[0]), len(sizes), [plen],
                                                     valid_path=tr, candidate_token_ids=ids0)[0]
        self._expand_step = expand_step
        self.catalog_items = int(cat.shape[0])

    def sample(self):
        """(beam rows per second, description) of one extrapolated request step."""
        if self.kind == "port":
            v, _, desc = self._port()
            return v, desc
        torch = self.torch
        with torch.inference_mode():
            t0 = time.perf_counter()
            self._layer(self._x, self._x.clone(), self._batch)
            t_layer = time.perf_counter() - t0
            bl = self._init()
            t0 = time.perf_counter()
            lp, ids = self._head.compute_level(self._hidden, 1)
            c = min(2 * self.beam, int(lp.shape[1]))
            vals, idx = torch.topk(lp, c, dim=-1, largest=True, sorted=True)
            self._expand_step(bl, ids[idx], vals, self.beam, valid_path=self._trie)
            t_head = time.perf_counter() - t0
        per_request_step = t_layer * self.layers * (self.beam / self.rows) + t_head
        desc = (f"reference engine (torch CPU branch, {self.cores} threads): Qwen3DecoderLayer.forward of 1 layer for "
                f"{self.rows} beam rows over a 256-token prompt {t_layer:.2f}s, x {self.layers} layers x "
                f"{self.beam}/{self.rows} rows (extrapolated); RestrictedLMHead.compute_level + top-{c} + expand_step "
                f"with the CSR trie ({self.catalog_items} items) for one request of {self.beam} beams {t_head:.2f}s; "
                "rotation from the oracle (the reference's torch RoPE raises on a CPU)")
        return self.beam / per_request_step, desc


def cpu_baseline_port(beam: int, sizes, items: int, layers: int, budget_rows: int = 64):
    """The oracle's restatement of one decode step on the host cores, used when the reference install is
    not there: `budget_rows` beam rows of one request (prompt 256) through ONE
    decoder layer, one SID head level and one beam step; the layer time is
    multiplied by the layer count. Returns (beam_rows_per_s, cores, description)."""
    import numpy as np
    import torch

    from oracle import sid_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    H, HQ, HKV, D, I = 2048, 16, 8, 128, 6144
    rows, plen = budget_rows, 256
    w = {k: O.quantize_weight_fp8(0.02 * torch.randn(n, kk, generator=g))
         for k, (n, kk) in dict(qkv=(4096, H), o=(H, H), gate_up=(2 * I, H), down=(H, I), head=(sizes[0], H)).items()}
    norms = dict(input=torch.ones(H, dtype=torch.bfloat16), post=torch.ones(H, dtype=torch.bfloat16),
                 q=torch.ones(D, dtype=torch.bfloat16), k=torch.ones(D, dtype=torch.bfloat16))
    cs = O.build_cos_sin_cache(D, plen + 8, 1e6)
    slots = plen + rows + 1
    kc = torch.randn(slots, HKV, D, generator=g).bfloat16().to(O.FP8)
    vc = torch.randn(slots, HKV, D, generator=g).bfloat16().to(O.FP8)
    x = torch.randn(rows, H, generator=g).bfloat16()
    pos = torch.full((rows,), plen)
    loc = torch.arange(plen + 1, plen + 1 + rows)
    indptr = torch.arange(rows + 1, dtype=torch.int32) * (plen + 1)
    indices = torch.cat([torch.cat((torch.arange(1, plen + 1), loc[i:i + 1])) for i in range(rows)]).to(torch.int32)
    from flashrec_b200.trie import build_trie_arrays  # host-side numpy builder, no GPU involved

    arrays = build_trie_arrays(make_catalog(min(items, 200_000), sizes), list(sizes), 151_936)
    otr = O.OracleTrie(arrays.csr_keys, arrays.edge_child, arrays.vsz, arrays.token_base, arrays.invalid_node)

    def layer(x, residual):
        return O.decoder_layer(x, residual, w, norms, pos, loc, cs, kc, vc, indptr, indices, HQ, HKV, D)

    def head_and_step(h):
        hq, hs = O.per_token_quant_fp8(h)
        logits = O.fp8_logits_f32(hq, w["head"][0], hs, w["head"][1])
        cum = torch.zeros(1, rows)
        nodes = torch.zeros(1, rows, dtype=torch.int64)
        return O.sid_beam_step(cum, logits, nodes, otr, arrays.token_base, rows)

    layer(x, x.clone())  # warm-up
    t0 = time.perf_counter()
    h, r = layer(x, x.clone())
    t_layer = time.perf_counter() - t0
    t0 = time.perf_counter()
    head_and_step(h)
    t_head = time.perf_counter() - t0
    per_step = t_layer * layers + t_head
    desc = (f"oracle port: {rows} beam rows of one request (prompt 256): 1 decoder layer timed {t_layer:.3f}s x {layers} "
            f"layers (extrapolated) + head level and beam step {t_head:.3f}s")
    return rows / per_step, cores, desc


def run_reference_arm(args):
    """``--impl reference``: rank 0 alone times the reference's CPU implementation of the step; each step is
    one bounded sample (see ReferenceCpuStep)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sizes = [8192] * 3
    ref = ReferenceCpuStep(args.beam, sizes, args.items, args.layers)
    for _ in range(max(0, min(args.warmup, 1))):
        ref.sample()
    vals, desc = [], ""
    t0 = time.perf_counter()
    for _ in range(max(1, min(args.steps, 3))):
        v, desc = ref.sample()
        vals.append(v)
    wall = time.perf_counter() - t0
    v = statistics.median(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": wall / len(vals) * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> bf16 on the host (torch)", "data": "synthetic",
        "config": bench_config(args, max(args.gpus, 1), args.requests * args.beam, len(sizes)),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": ref.cores, "kind": ref.kind, "sample": desc,
                         "samples_timed": len(vals)},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------
def dram_traffic_of_dominant_kernel(rows: int):
    """DRAM bytes per launch of the dominant kernel, from the text summary of its ncu capture (the
    ``dram__bytes_read.sum`` / ``dram__bytes_write.sum`` rows of one launch at 16384 rows), scaled by the row
    count. ``None`` when no capture summary is present: the number is never made up."""
    import re

    src = ROOT / "profiles" / "gate_up_gemm_dram_traffic.txt"
    if not src.exists():
        return None, "no ncu capture summary found"
    vals = {}
    for line in src.read_text().splitlines():
        m = re.match(r"\s*(dram__bytes_(?:read|write)\.sum)\s+([0-9.eE+]+)\s*(\w*)", line)
        if m:
            mult = {"": 1.0, "byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}.get(m.group(3), 1.0)
            vals[m.group(1)] = float(m.group(2)) * mult
    if len(vals) != 2:
        return None, "ncu capture summary unreadable"
    return sum(vals.values()) * rows / 16384.0, ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch at "
                                                  "M=16384 (capture summary under profiles/), scaled to this row count")


def time_gemms(torch, rows: int, iters: int = 10):
    """FP8 GEMM roofline figures, timed alone with CUDA events on the launch stream:
    (a) the dominant kernel of the wave, the gate_up GEMM with the SwiGLU epilogue, at the
    wave's row count; (b) the four linear-layer shapes of one decoder layer back to back
    (plain GEMMs), with cuBLASLt on the same shapes beside it. Between timed launches of (a)
    a 256 MB buffer is rewritten, so its operands come from HBM, not from L2."""
    from flashrec_b200.kernel.sglops import fp8_scaled_mm, fp8_scaled_mm_silu_mul, interleave_gate_up

    dev = torch.device("cuda", torch.cuda.current_device())
    shapes = [("qkv", 4096, 2048), ("o", 2048, 2048), ("gate_up", 12288, 2048), ("down", 2048, 6144)]
    ops, flops = [], 0.0
    for name, n, k in shapes:
        a = torch.randn(rows, k, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, k, device=dev).to(torch.float8_e4m3fn)
        sa = (torch.rand(rows, 1, device=dev) + 0.5) / 45.0  # gate / up values of order 1
        sb = torch.rand(n, device=dev) + 0.5
        ops.append((a, b, sa, sb))
        flops += 2.0 * rows * n * k
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # (a) dominant kernel
    a, b, sa, sb = ops[2]
    wi, si = interleave_gate_up(b, sb)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(3):
        fp8_scaled_mm_silu_mul(a, wi, sa, si)
    torch.cuda.synchronize()
    # the kernel alone between the events: output and row-maximum buffers exist beforehand (the wrapper would
    # allocate them and launch a fill inside the timed region)
    from flashrec_b200._lib import call, ptr, stream_ptr

    y = torch.empty((rows, 12288 // 2), dtype=torch.bfloat16, device=dev)
    amax = torch.zeros(rows, dtype=torch.float32, device=dev)
    sa_flat = sa.reshape(-1).to(torch.float32).contiguous()
    fused_ms = []
    for _ in range(iters):
        flush.zero_()
        amax.zero_()
        e0.record()
        call("fr_gemm_fp8_silu_mul", ptr(a), ptr(wi), ptr(sa_flat), ptr(si), ptr(y), ptr(amax), rows, 12288, 2048,
             a.stride(0), wi.stride(0), y.stride(0), 0, stream_ptr(dev))
        e1.record()
        torch.cuda.synchronize()
        fused_ms.append(e0.elapsed_time(e1))
    del y, amax
    fused_sec = sum(fused_ms) / len(fused_ms) / 1e3
    fused_flops = 2.0 * rows * 12288 * 2048
    del flush, wi, si
    # (b) the four layer shapes
    for a, b, sa, sb in ops:  # warm-up
        fp8_scaled_mm(a, b.t(), sa, sb, torch.bfloat16)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        for a, b, sa, sb in ops:
            fp8_scaled_mm(a, b.t(), sa, sb, torch.bfloat16)
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / 1e3 / iters
    lib = None
    try:  # cuBLASLt FP8 on the same shapes, for orientation only
        one = torch.ones((), device=dev)
        for a, b, sa, sb in ops:
            torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb.view(1, -1), out_dtype=torch.bfloat16)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(iters):
            for a, b, sa, sb in ops:
                torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb.view(1, -1), out_dtype=torch.bfloat16)
        e1.record()
        torch.cuda.synchronize()
        lib = flops / (e0.elapsed_time(e1) / 1e3 / iters) / 1e12
        del one
    except Exception:
        lib = None
    return fused_flops, fused_sec, flops, sec, lib


def gemm_shapes(rows: int, emit: bool = True):
    """FP8 GEMM time of every linear-layer shape of the step at ``rows`` rows (512 = the decode
    step of a single request), this library and cuBLASLt (``torch._scaled_mm``) side by side:
    20 launches per CUDA graph, two replays timed with CUDA events (weights stay L2-resident)."""
    import torch

    from flashrec_b200.kernel.sglops import fp8_scaled_mm

    dev = torch.device("cuda", torch.cuda.current_device())
    fp8 = torch.float8_e4m3fn
    shapes = {"qkv": (4096, 2048), "o": (2048, 2048), "gate_up": (12288, 2048), "down": (2048, 6144),
              "config1": (6144, 2048), "sid_head_level": (8192, 2048)}
    out = {}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def graph_us(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(20):
                fn()
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / 40

    for name, (n, k) in shapes.items():
        a = torch.randn(rows, k, device=dev).to(fp8)
        b = torch.randn(n, k, device=dev).to(fp8)
        sa = torch.rand(rows, 1, device=dev) + 0.5
        sb = torch.rand(n, device=dev) + 0.5
        flops = 2.0 * rows * n * k
        us = graph_us(lambda: fp8_scaled_mm(a, b.t(), sa, sb, torch.bfloat16))
        lib = graph_us(lambda: torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb.view(1, -1),
                                                out_dtype=torch.bfloat16))
        out[name] = {"N": n, "K": k, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1),
                     "cublaslt_us": round(lib, 2), "cublaslt_tflops": round(flops / lib / 1e6, 1)}
    if emit:
        print(json.dumps({"gemm_shapes_rows": rows, "shapes": out}))
    return out


def profile_kernels(rows: int):
    """One launch of every hot kernel at the bench shapes, for a small ncu capture
    (about 1.5 GB resident, each kernel a fraction of a millisecond)."""
    import torch

    from flashrec_b200.kernel.qk_rope_kv import fp8_qkv_mm_norm_rope_store, fused_qk_norm_rope_store_fp8
    from flashrec_b200.kernel.rms_fp8 import fused_add_rmsnorm_per_token_quant_fp8
    from flashrec_b200.kernel.sglops import (fp8_scaled_mm, fp8_scaled_mm_silu_mul, per_token_quant_fp8,
                                             quant_known_amax_fp8)
    from flashrec_b200.kernel.silu_fp8 import silu_and_mul_per_token_quant_fp8
    from flashrec_b200.layers import build_cos_sin_cache

    dev = torch.device("cuda", torch.cuda.current_device())
    fp8 = torch.float8_e4m3fn
    a = torch.randn(rows, 2048, device=dev).to(fp8)
    b = torch.randn(12288, 2048, device=dev).mul_(0.05).to(fp8)
    sa = torch.rand(rows, 1, device=dev) * 0.02 + 0.01
    sb = torch.rand(12288, device=dev) * 0.02 + 0.01
    h = torch.randn(rows, 2048, device=dev).bfloat16()
    r = torch.randn(rows, 2048, device=dev).bfloat16()
    w = torch.ones(2048, device=dev).bfloat16()
    gu = torch.randn(rows, 12288, device=dev).bfloat16()
    qkv = torch.randn(rows, 32, 128, device=dev).bfloat16()
    cs = build_cos_sin_cache(128, 2048, 1e6, device=dev)
    pos = torch.randint(0, 2048, (rows,), device=dev)
    pos_req = torch.randint(128, 1025, (max(rows // 512, 1),), device=dev).repeat_interleave(min(rows, 512))[:rows]
    loc = torch.arange(1, rows + 1, device=dev)
    kc = torch.zeros(rows + 16, 8, 128, dtype=torch.uint8, device=dev).view(fp8)
    vc = torch.zeros_like(kc)
    hw = torch.ones(128, device=dev).bfloat16()

    def once():
        y, am = fp8_scaled_mm_silu_mul(a, b, sa, sb)                      # gate_up GEMM + SwiGLU epilogue
        quant_known_amax_fp8(y, am)
        fp8_scaled_mm(a, b.t(), sa, sb, torch.bfloat16)                   # plain GEMM, CTA pairs
        fp8_scaled_mm(a, b.t(), sa, sb, torch.bfloat16, block_n=256)      # plain GEMM, one CTA per tile
        fused_add_rmsnorm_per_token_quant_fp8(h, r, w, 1e-6)
        per_token_quant_fp8(h)
        silu_and_mul_per_token_quant_fp8(gu)                              # unfused SwiGLU quantiser
        fused_qk_norm_rope_store_fp8(qkv[:, :16], qkv[:, 16:24], qkv[:, 24:], pos, loc, hw, hw, 1e-6, cs, kc, vc)
        # qkv GEMM with QK-norm + RoPE + KV write in its epilogue (rows of a request share a position)
        fp8_qkv_mm_norm_rope_store(a, b[:4096].t(), sa, sb[:4096], pos_req, loc, hw, hw, 1e-6, cs, kc, vc, 16, 8)

    for _ in range(2):
        once()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    once()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(json.dumps({"profiled": "kernels", "rows": rows}))


def ref_kernels_compare(rows: int):
    """The reference's own GPU kernels for this path beside this library's, same inputs, same harness (20
    launches per CUDA graph, two replays timed with CUDA events; outputs allocated inside the graph by both
    sides, as their wrappers do). The reference comes unmodified from ``oracle/_ref``: its Triton kernels
    (kernel/rms_fp8.py:29-61, silu_fp8.py:29-72, qk_rope_kv.py:28-155, attention/kv_indices.py:20-42), its torch
    branch where it has no kernel of its own (``per_token_quant_fp8`` without sgl-kernel), and
    ``kernel/csrc/beam_trie.cuh`` JIT-built through tvm_ffi. Prints one JSON line; an entry the box cannot run
    is recorded as unavailable with the error."""
    import numpy as np
    import torch

    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    dev = torch.device("cuda", torch.cuda.current_device())
    fp8 = torch.float8_e4m3fn
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def graph_us(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(20):
                fn()
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / 40

    out = {}

    def compare(name, mine, theirs, nbytes):
        rec = {"algorithmic_bytes": nbytes}
        try:
            rec["this_library_us"] = round(graph_us(mine), 2)
            rec["this_library_GBps"] = round(nbytes / rec["this_library_us"] / 1e3, 1)
        except Exception as exc:
            rec["this_library_error"] = repr(exc)[:200]
        try:
            rec["reference_us"] = round(graph_us(theirs), 2)
            rec["reference_GBps"] = round(nbytes / rec["reference_us"] / 1e3, 1)
        except Exception as exc:
            rec["reference_unavailable"] = "unavailable on this box: " + repr(exc)[:200]
        out[name] = rec

    import flashrec_b200.attention as b_att
    import flashrec_b200.kernel.beam_trie as b_trie
    import flashrec_b200.kernel.qk_rope_kv as b_rope
    import flashrec_b200.kernel.rms_fp8 as b_rms
    import flashrec_b200.kernel.sglops as b_sgl
    import flashrec_b200.kernel.silu_fp8 as b_silu

    try:
        import flashrec.attention.kv_indices as r_kvi
        import flashrec.kernel.beam_trie as r_trie
        import flashrec.kernel.qk_rope_kv as r_rope
        import flashrec.kernel.rms_fp8 as r_rms
        import flashrec.kernel.sglops as r_sgl
        import flashrec.kernel.silu_fp8 as r_silu
    except Exception as exc:
        print(json.dumps({"ref_kernels_rows": rows, "reference_unavailable": "unavailable on this box: " + repr(exc)[:300]}))
        return

    H, I, HQ, HKV, D = 2048, 6144, 16, 8, 128
    x = torch.randn(rows, H, device=dev).bfloat16()
    res = torch.randn(rows, H, device=dev).bfloat16()
    w = torch.ones(H, device=dev).bfloat16()
    compare("rmsnorm_per_token_quant_fp8", lambda: b_rms.rmsnorm_per_token_quant_fp8(x, w, 1e-6),
            lambda: r_rms.rmsnorm_per_token_quant_fp8(x, w, 1e-6), rows * H * 3 + rows * 4)
    compare("fused_add_rmsnorm_per_token_quant_fp8", lambda: b_rms.fused_add_rmsnorm_per_token_quant_fp8(x, res, w, 1e-6),
            lambda: r_rms.fused_add_rmsnorm_per_token_quant_fp8(x, res, w, 1e-6), rows * H * 7 + rows * 4)
    compare("per_token_quant_fp8", lambda: b_sgl.per_token_quant_fp8(x), lambda: r_sgl.per_token_quant_fp8(x),
            rows * H * 3 + rows * 4)
    gu = torch.randn(rows, 2 * I, device=dev).bfloat16()
    compare("silu_and_mul_per_token_quant_fp8", lambda: b_silu.silu_and_mul_per_token_quant_fp8(gu),
            lambda: r_silu.silu_and_mul_per_token_quant_fp8(gu), rows * (2 * I * 2 + I + 4))
    qkv = torch.randn(rows, HQ + 2 * HKV, D, device=dev).bfloat16()
    from flashrec_b200.layers import build_cos_sin_cache

    cs = build_cos_sin_cache(D, 2048, 1e6, device=dev)
    pos = torch.randint(0, 2048, (rows,), device=dev)
    loc = torch.arange(1, rows + 1, device=dev)
    kc = torch.zeros(rows + 16, HKV, D, dtype=torch.uint8, device=dev).view(fp8)
    vc = torch.zeros_like(kc)
    hw = torch.ones(D, device=dev).bfloat16()
    rope_args = (qkv[:, :HQ], qkv[:, HQ:HQ + HKV], qkv[:, HQ + HKV:], pos, loc, hw, hw, 1e-6, cs, kc, vc)
    compare("fused_qk_norm_rope_store_fp8", lambda: b_rope.fused_qk_norm_rope_store_fp8(*rope_args),
            lambda: r_rope.fused_qk_norm_rope_store_fp8(*rope_args),
            rows * ((HQ + 2 * HKV) * D * 2 + HQ * D * 2 + 2 * HKV * D + 16))
    # slot-list gather: rows x ~600 slots
    rng = np.random.default_rng(0)
    lens = torch.from_numpy(rng.integers(128, 1025, max(rows // 512, 1)).repeat(min(rows, 512))[:rows].astype(np.int32)).to(dev)
    table = torch.randint(1, 60000, (rows, 1040), dtype=torch.int32, device=dev)
    ridx = torch.arange(rows, device=dev)
    total = int(lens.sum().item())
    buf = torch.empty(total, dtype=torch.int32, device=dev)
    compare("gather_kv_indices", lambda: b_att.gather_kv_indices(table, ridx, lens, out=buf, total=total),
            lambda: r_kvi.gather_kv_indices(table, ridx, lens, out=buf, total=total), total * 8 + rows * 16)
    # fused mask + top-k + expand + advance on a dense trie (the reference kernel's limit: 512 beams)
    n, bw, c, L, vsz, nodes_n = max(rows // 512, 1), min(rows, 512), 128, 3, 192, 4096
    g = torch.Generator(device=dev).manual_seed(0)
    allow = (torch.rand(nodes_n + 1, vsz, generator=g, device=dev) > 0.5)
    nxt = torch.randint(0, nodes_n, (nodes_n + 1, vsz), generator=g, device=dev)
    cum = torch.randn(n, bw, generator=g, device=dev)
    lp = torch.sort(torch.randn(n, bw, c, generator=g, device=dev), dim=-1, descending=True).values.contiguous()
    tok = torch.randint(1000, 1000 + vsz, (n, bw, c), generator=g, device=dev)
    node = torch.randint(0, nodes_n, (n, bw), generator=g, device=dev)
    tids = torch.randint(1000, 1000 + vsz, (n, bw, L), generator=g, device=dev)
    kw = dict(select_k=bw, node_ids=node, allow_table=allow, token_base=1000, token_ids=tids, col=1, next_node=nxt,
              invalid_node=nodes_n)
    ws_b, ws_r = b_trie.GenrecFusedWorkspace(), r_trie.GenrecFusedWorkspace()
    loaded = False
    try:
        loaded = bool(r_trie.try_load_beam_trie())
    except Exception:
        loaded = False
    compare("genrec_mask_topk_expand", lambda: b_trie.genrec_mask_topk_expand(cum, lp, tok, workspace=ws_b, **kw),
            (lambda: r_trie.genrec_mask_topk_expand(cum, lp, tok, workspace=ws_r, **kw)) if loaded else
            (lambda: (_ for _ in ()).throw(RuntimeError("beam_trie.cuh did not build through tvm_ffi"))),
            n * bw * c * (4 + 8) * 2)
    out["genrec_mask_topk_expand"]["shape"] = f"N={n} BW={bw} C={c} dense trie {nodes_n} x {vsz}"
    # selection with stop tokens and Gumbel rank noise: every request in one launch here, one call per request in
    # the reference (torch ops: topk, isin, cumsum, scatter), as its expand_step calls it
    import flashrec_b200.search as b_sel
    try:
        import flashrec.search.select as r_sel
    except Exception:
        r_sel = None
    cj = 256
    lpj = torch.log_softmax(torch.randn(n, bw, cj, generator=g, device=dev), dim=-1)
    tkj = torch.randint(0, 4000, (n, bw, cj), generator=g, device=dev)
    stop = torch.arange(0, 40, device=dev)
    pert = b_sel.gumbel_like(lpj)

    def ref_joint():
        if r_sel is None:
            raise RuntimeError("flashrec.search.select not importable")
        for i in range(n):
            r_sel.joint_select(cum[i], lpj[i], tkj[i], stop, bw, perturb=pert[i])

    compare("joint_select", lambda: b_sel.joint_select(cum, lpj, tkj, stop, bw, perturb=pert), ref_joint,
            n * bw * cj * (4 + 8 + 4))
    if "reference_us" not in out["joint_select"]:
        # the reference's version cannot be captured (torch.isin synchronises): time it eagerly, 20 calls between events
        try:
            for _ in range(3):
                ref_joint()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(20):
                ref_joint()
            e1.record()
            torch.cuda.synchronize()
            out["joint_select"].pop("reference_unavailable", None)
            out["joint_select"]["reference_us"] = round(e0.elapsed_time(e1) * 1e3 / 20, 2)
            out["joint_select"]["reference_note"] = "eager launches (not capturable in a CUDA graph)"
        except Exception as exc:
            out["joint_select"]["reference_unavailable"] = "unavailable on this box: " + repr(exc)[:200]
    out["joint_select"]["shape"] = f"{n} requests x {bw} rows x {cj} candidates, 40 stop tokens, rank noise"
    print(json.dumps({"ref_kernels_rows": rows, "kernels": out}))


def head_compare(requests: int, beam: int, items: int, iters: int = 10):
    """SID head + beam step of each level at the bench's sizes (requests x beam rows, hidden 2048, 3 x 8192
    codes, the bench's catalog), with the beam state the previous level left: the fused call
    (``fr_sid_head_topk``: no logits matrix) beside the three-call flow (fp32 logits GEMM -> row statistics ->
    beam step), for the CSR and the bitmap trie. CUDA events around each flow, a 256 MB buffer rewritten between
    repetitions, median. Prints one JSON line."""
    import numpy as np
    import torch

    from flashrec_b200.kernel.sglops import per_token_quant_fp8
    from flashrec_b200.layers import quantize_weight_fp8
    from flashrec_b200.logits import RestrictedLMHead
    from flashrec_b200.sid_decode import SidHeadWorkspace, sid_beam_step, sid_head_topk
    from flashrec_b200.trie import build_trie_device

    dev = torch.device("cuda", torch.cuda.current_device())
    sizes, base, hidden = [8192] * 3, 151_936, 2048
    n, bw = requests, beam
    cat = torch.from_numpy(np.ascontiguousarray(make_catalog(items, sizes), dtype=np.int32)).to(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    wq, wsc = quantize_weight_fp8(torch.randn((sum(sizes), hidden), generator=g, device=dev) * 0.02)
    head = RestrictedLMHead(list(range(base, base + sum(sizes))))
    head.bind_quantized(wq, wsc)
    head.bind_codebook(sizes)
    hs = [torch.randn((n * bw, hidden), generator=g, device=dev).to(torch.bfloat16) for _ in sizes]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn):
        for _ in range(3):
            out = fn()
        torch.cuda.synchronize()
        ms = []
        for _ in range(iters):
            flush.zero_()
            e0.record()
            out = fn()
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        return out, statistics.median(ms) * 1e3

    res = {"head_compare": True, "rows": n * bw, "requests": n, "beam_width": bw, "level_width": sizes[0],
           "hidden": hidden, "layouts": {}}
    for layout in ("csr", "bitmap"):
        trie = build_trie_device(cat, sizes, base, layout=layout)
        cum = torch.full((n, bw), float("-inf"), device=dev)
        cum[:, 0] = 0.0
        nodes = torch.zeros((n, bw), dtype=torch.int64, device=dev)
        toks = torch.zeros((n, bw, 3), dtype=torch.int64, device=dev)
        wsp = SidHeadWorkspace()
        levels = []
        for lv in range(3):
            col = torch.full((n,), lv, dtype=torch.int32, device=dev)
            tok_o, node_o = torch.zeros_like(toks), torch.zeros_like(nodes)

            def unfused():
                lg, mx, ls, _ = head.logits_level(hs[lv], lv)
                return sid_beam_step(cum, lg, mx, ls, nodes, trie, base + lv * sizes[0], bw, token_ids_in=toks,
                                     token_ids_out=tok_o, node_ids_out=node_o, col=col)

            def fused():
                q, sc = per_token_quant_fp8(hs[lv])
                return sid_head_topk(cum, q, sc, head._level_weights[lv], head._level_scales[lv], nodes, trie,
                                     base + lv * sizes[0], bw, wsp, level=lv, token_ids_in=toks, token_ids_out=tok_o,
                                     node_ids_out=node_o, col=col)

            _, us_u = timed(unfused)
            out, us_f = timed(fused)
            levels.append({"level": lv, "three_calls_us": round(us_u, 1), "fused_us": round(us_f, 1),
                           "candidate_capacity_per_request": trie.candidate_bound(lv, bw),
                           "live_beams": int(torch.isfinite(cum).sum().item())})
            cum, nodes, toks = out.vals.clone(), node_o, tok_o
        res["layouts"][layout] = levels
        del trie
    print(json.dumps(res))


def config5_head(dist, dev, rank: int, world: int, requests: int = 16, beam: int = 2048, levels: int = 4,
                 width: int = 4096, items: int = 10_000_000, hidden: int = 2048, reps: int = 3):
    """The one exchange step of the scope, at the widest baseline configuration's shape: 4 levels x 4096
    codes, a Zipf-skewed 10M-item catalog (CSR trie built on every GPU), 2048 beams, ``requests`` requests
    whose beam state every rank holds. The SID head is split by token range over the ``world`` ranks
    (``flashrec_b200.sharded_head``: local fused head on the rank's codes, one all-gather of row statistics,
    one of 16-byte winner records, merge) and timed per level beside the unsharded fused head on one GPU, with
    and without the all-gather of the ranks' quantised hidden rows that a data-parallel model body needs
    first. CUDA events, max over ranks. Also checks that every rank's merged result equals the unsharded
    step on the same (combined) row statistics, bit for bit. Returns a dict for the JSON line."""
    import numpy as np
    import torch

    from flashrec_b200.kernel.sglops import per_token_quant_fp8
    from flashrec_b200.layers import quantize_weight_fp8
    from flashrec_b200.sharded_head import ShardedSidHead, shard_range
    from flashrec_b200.sid_decode import BeamStepOut, SidHeadWorkspace, sid_head_topk
    from flashrec_b200.trie import build_trie_device

    n, bw, L, kl, base = requests, beam, levels, width, 151_936
    sizes = [kl] * L
    rng = np.random.default_rng(0)  # the same catalog, weights and hidden states on every rank
    cols = [np.minimum(rng.zipf(1.1, items) - 1, kl - 1) if l < 2 else rng.integers(0, kl, items) for l in range(L)]
    trie = build_trie_device(torch.from_numpy(np.stack(cols, 1).astype(np.int32)).to(dev), sizes, base)
    g = torch.Generator(device=dev).manual_seed(1)
    wq, ws = quantize_weight_fp8(torch.randn((L * kl, hidden), generator=g, device=dev) * 0.02)
    ws = ws.reshape(-1)
    sharded = world > 1
    head = ShardedSidHead() if sharded else None
    lo, hi = shard_range(kl, rank, world)
    rows = n * bw
    my_rows = slice(rank * rows // world, (rank + 1) * rows // world)
    i64 = dict(dtype=torch.int64, device=dev)

    def planes():
        cum = torch.full((n, bw), float("-inf"), device=dev)
        cum[:, 0] = 0.0
        return cum, torch.zeros((n, bw), **i64), torch.zeros((n, bw, L), **i64)

    cum, node, tok = planes()
    ws_full = SidHeadWorkspace()
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    t_un, t_sh, t_shx = [], [], []
    t_un_g, t_sh_g = [], []  # the same steps replayed as CUDA graphs (kernels and NCCL collectives captured)
    graph_note = None
    equal = True

    def timed_graph(fn, sink, lv):
        """Capture one call of ``fn`` and time ``reps`` replays; on any capture problem record why and go on.
        The ranks agree on the outcome before anyone replays, so a rank whose capture failed leaves nobody
        waiting in a collective."""
        nonlocal graph_note
        if graph_note is not None:
            return
        gr, why = None, None
        try:
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                fn()
        except Exception as exc:
            gr, why = None, repr(exc)[:160]
        ok = torch.tensor([0 if gr is None else 1], dtype=torch.int32, device=dev)
        if dist is not None:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            graph_note = "graph capture unavailable: " + (why or "failed on another rank")
            return
        for rep_i in range(reps + 1):
            barrier()
            e0, e1 = ev(), ev()
            e0.record()
            gr.replay()
            e1.record()
            torch.cuda.synchronize()
            if rep_i:
                sink.append((lv, e0.elapsed_time(e1)))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for lv in range(L):
        hid = torch.randn((rows, hidden), generator=g, device=dev).to(torch.bfloat16)
        h8, hs = per_token_quant_fp8(hid)
        wl, sl = wq[lv * kl:(lv + 1) * kl], ws[lv * kl:(lv + 1) * kl]
        col = torch.full((n,), lv, dtype=torch.int32, device=dev)
        tb = base + lv * kl
        cap = trie.candidate_bound(lv, bw)
        # unsharded fused head, everything on this GPU
        for rep in range(reps + 1):
            tok_u, node_u = torch.zeros_like(tok), torch.zeros_like(node)
            barrier()
            e0, e1 = ev(), ev()
            e0.record()
            out_u = sid_head_topk(cum, h8, hs.reshape(-1), wl, sl, node, trie, tb, bw, ws_full, cand_capacity=cap,
                                  token_ids_in=tok, token_ids_out=tok_u, node_ids_out=node_u, col=col)
            e1.record()
            torch.cuda.synchronize()
            if rep:
                t_un.append((lv, e0.elapsed_time(e1)))
        tok_g, node_g = torch.zeros_like(tok), torch.zeros_like(node)
        timed_graph(lambda: sid_head_topk(cum, h8, hs.reshape(-1), wl, sl, node, trie, tb, bw, ws_full, cand_capacity=cap,
                                          token_ids_in=tok, token_ids_out=tok_g, node_ids_out=node_g, col=col),
                    t_un_g, lv)
        if sharded:
            local = (h8, hs.reshape(-1), wl[lo:hi], sl[lo:hi])
            for rep in range(reps + 1):
                tok_s, node_s = torch.zeros_like(tok), torch.zeros_like(node)
                barrier()
                e0, e1 = ev(), ev()
                e0.record()
                out_s = head.step(cum, local, node, trie, tb, kl, bw, level=lv, token_ids_in=tok, token_ids_out=tok_s,
                                  node_ids_out=node_s, col=col)
                e1.record()
                torch.cuda.synchronize()
                if rep:
                    t_sh.append((lv, e0.elapsed_time(e1)))
            tok_sg, node_sg = torch.zeros_like(tok), torch.zeros_like(node)
            timed_graph(lambda: head.step(cum, local, node, trie, tb, kl, bw, level=lv, token_ids_in=tok,
                                          token_ids_out=tok_sg, node_ids_out=node_sg, col=col), t_sh_g, lv)
            # the same with the hidden rows of a data-parallel body gathered first
            h8_my, hs_my = h8[my_rows].contiguous(), hs.reshape(-1)[my_rows].contiguous()
            for rep in range(reps + 1):
                tok_x, node_x = torch.zeros_like(tok), torch.zeros_like(node)
                barrier()
                e0, e1 = ev(), ev()
                e0.record()
                gh, gs = head.gather_hidden(h8_my, hs_my)
                out_x = head.step(cum, (gh, gs, wl[lo:hi], sl[lo:hi]), node, trie, tb, kl, bw, level=lv, token_ids_in=tok,
                                  token_ids_out=tok_x, node_ids_out=node_x, col=col)
                e1.record()
                torch.cuda.synchronize()
                if rep:
                    t_shx.append((lv, e0.elapsed_time(e1)))
            equal = equal and torch.equal(out_x.vals, out_s.vals) and torch.equal(tok_x, tok_s)
            # bit-exact check: the unsharded step on the statistics the protocol combined
            stats = head.ops.local_stats(cum, local, node, trie, tb, lo, kl, lv)
            cmx, cls_ = head.ops.combine_stats(head._all_gather(stats))
            tok_r, node_r = torch.zeros_like(tok), torch.zeros_like(node)
            sid_head_topk(cum, h8, hs.reshape(-1), wl, sl, node, trie, tb, bw, ws_full, cand_capacity=cap, phase=1)
            ref = sid_head_topk(cum, h8, hs.reshape(-1), wl, sl, node, trie, tb, bw, ws_full, cand_capacity=cap, phase=2,
                                row_max=cmx, row_logsum=cls_, token_ids_in=tok, token_ids_out=tok_r, node_ids_out=node_r,
                                col=col)
            equal = equal and torch.equal(out_s.vals, ref.vals) and torch.equal(out_s.tokens, ref.tokens)
            equal = equal and torch.equal(out_s.parents, ref.parents) and torch.equal(tok_s, tok_r)
            equal = equal and torch.equal(node_s, node_r)
            cum, node, tok = out_s.vals.clone(), node_s, tok_s
        else:
            cum, node, tok = out_u.vals.clone(), node_u, tok_u

    def total_ms(ts):
        if not ts:
            return None
        per_level = [sum(t for l, t in ts if l == lv) / reps for lv in range(L)]
        t = torch.tensor(per_level, device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [round(float(x), 4) for x in t.tolist()]

    live = torch.isfinite(cum)
    flags = torch.tensor([int(equal), int((node[live] == -1).all().item())], device=dev)
    if dist is not None:
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    un, sh, shx = total_ms(t_un), total_ms(t_sh), total_ms(t_shx)
    un_g, sh_g = total_ms(t_un_g), total_ms(t_sh_g)
    return {
        "workload": "head step of the widest configuration: token-range-sharded SID head, NCCL all-gathers",
        "requests": n, "beam_width": bw, "levels": L, "level_width": kl, "catalog_items": int(trie.arrays.n_items),
        "trie_nodes": trie.n_nodes, "n_gpus": world,
        "head_ms_per_level_unsharded_one_gpu": un, "head_ms_all_levels_unsharded_one_gpu": round(sum(un), 4),
        "head_ms_per_level_sharded": sh, "head_ms_all_levels_sharded": round(sum(sh), 4) if sh else None,
        "head_ms_all_levels_sharded_with_hidden_all_gather": round(sum(shx), 4) if shx else None,
        "graph_replay": {"head_ms_per_level_unsharded_one_gpu": un_g,
                         "head_ms_all_levels_unsharded_one_gpu": round(sum(un_g), 4) if un_g else None,
                         "head_ms_per_level_sharded": sh_g,
                         "head_ms_all_levels_sharded": round(sum(sh_g), 4) if sh_g else None, "note": graph_note},
        "sharded_equals_unsharded_bitwise_on_shared_statistics": bool(flags[0].item()) if sharded else None,
        "complete_sids_reached": bool(flags[1].item()),
        "collectives_per_level": "1 x statistics [2, rows] f32 + 1 x winner records [N, K] x 16 B (+ 2 for the hidden "
                                 "rows of a data-parallel body)",
    }


def attn_compare(requests: int, beam: int, iters: int = 10):
    """The decode attention of one layer on the bench's slot lists (requests x beam rows, prompts
    U[128,1024] shared by a request's beams, one own slot per row), timed between L2 flushes: this
    library's shared-prefix tcgen05 path (widening pass + attention kernel) beside FlashInfer's paged
    decode kernel called the way the reference calls it (page_size 1, e4m3 KV, bf16 Q; library code, a
    comparison only). Prints one JSON line."""
    import numpy as np
    import torch

    from flashrec_b200.attention import AttentionBackend, TokenToKVPool
    from flashrec_b200.decoder import ForwardBatch

    dev = torch.device("cuda", torch.cuda.current_device())
    hq, hkv, d = 16, 8, 128
    plens = prompt_lengths(requests, 0)
    rows = requests * beam
    slots = 16 + sum(plens) + rows
    pool = TokenToKVPool(1, slots, hkv, d, torch.float8_e4m3fn, dev)
    g = torch.Generator(device=dev).manual_seed(0)
    for c in (pool.k[0], pool.v[0]):
        c.copy_(torch.randn(c.shape, generator=g, device=dev).to(torch.bfloat16).to(torch.float8_e4m3fn))
    lists, cursor = [], 16
    for r, p in enumerate(plens):
        prefix = np.arange(cursor, cursor + p, dtype=np.int32)
        cursor += p
        own = np.arange(cursor, cursor + beam, dtype=np.int32)
        cursor += beam
        lists.append(np.concatenate([np.tile(prefix, (beam, 1)), own[:, None]], axis=1).reshape(-1))
    lens = np.repeat(np.asarray(plens) + 1, beam)
    indptr = torch.from_numpy(np.concatenate(([0], np.cumsum(lens))).astype(np.int32)).to(dev)
    indices = torch.from_numpy(np.concatenate(lists)).to(dev)
    q = torch.randn((rows, hq, d), generator=g, device=dev).to(torch.bfloat16)
    be = AttentionBackend(pool, hq, hkv, d, max_shared_len=max(plens) + 1)
    be.set_groups(torch.arange(requests + 1, dtype=torch.int32, device=dev) * beam, beam)
    batch = ForwardBatch(input_ids=None, req_pool_indices=None, seq_lens=torch.from_numpy(lens.astype(np.int32)).to(dev),
                         positions=None, out_cache_loc=None, kv_indices=indices, kv_indptr=indptr)
    be.prepare(batch)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn):
        for _ in range(3):
            out = fn()
        torch.cuda.synchronize()
        ms = []
        for _ in range(iters):
            flush.zero_()
            e0.record()
            out = fn()
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        return out, statistics.median(ms) * 1e3

    mine, us_mine = timed(lambda: be.forward(q, None, None, 0, batch, skip_store=True))
    res = {"attn_compare": True, "rows": rows, "requests": requests, "beam_width": beam,
           "keys_per_row_mean": float(lens.mean()), "this_library_us": us_mine,
           "this_library": "shared_kv_prepare_kernel + decode_attn_tc_kernel (tcgen05, shared prefix once per request)"}
    try:
        from flashinfer import BatchDecodeWithPagedKVCacheWrapper

        ws = torch.zeros(128 << 20, dtype=torch.uint8, device=dev)
        kv = (pool.k[0].unsqueeze(1), pool.v[0].unsqueeze(1))
        last = torch.ones(rows, dtype=torch.int32, device=dev)
        for tc in (True, False):
            w = BatchDecodeWithPagedKVCacheWrapper(ws, kv_layout="NHD", use_tensor_cores=tc)
            w.plan(indptr, indices, last, hq, hkv, d, 1, pos_encoding_mode="NONE", q_data_type=torch.bfloat16,
                   kv_data_type=torch.float8_e4m3fn)
            ref, us = timed(lambda: w.run(q, kv))
            key = "flashinfer_tensor_cores_us" if tc else "flashinfer_cuda_cores_us"
            res[key] = us
            res[key.replace("_us", "_max_abs_diff")] = float((ref.float() - mine.float()).abs().max().item())
    except Exception as exc:  # the library may be unable to build or load its kernel here
        res["flashinfer_unavailable"] = repr(exc)[:300]
    print(json.dumps(res))


def main():
    args = parse()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.attn_compare:
        import torch

        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        attn_compare(args.requests, args.beam)
        return
    if args.head_compare:
        import torch

        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        head_compare(args.requests, args.beam, args.items)
        return
    if args.gemm_shapes:
        import torch

        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        gemm_shapes(args.gemm_shapes)
        return
    if args.ref_kernels:
        import torch

        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        ref_kernels_compare(args.ref_kernels)
        return
    if args.profile_kernels:
        import torch

        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        profile_kernels(args.requests * args.beam)
        return
    import numpy as np
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    from flashrec_b200 import _lib, device_status
    from flashrec_b200.decoder import Qwen3Config
    from flashrec_b200.sid_decode import SidDecodeEngine
    from flashrec_b200.trie import build_trie_device

    _lib.load()  # fails loudly if the CUDA library is missing
    if args.config5:
        c5 = config5_head(dist, dev, rank, world)
        if rank == 0:
            print(json.dumps({"config5": c5}))
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return
    sizes = [8192] * 3
    token_base = 151_936
    p_lo, p_hi = 128, 1024
    if args.workload == "config5":
        sizes, p_lo, p_hi = [4096] * 4, 1024, 4096
        args.beam = 2048 if args.beam == 512 else args.beam
        args.items = 10_000_000 if args.items == 1_000_000 else args.items
        WORKLOAD.update(workload="qwen3-1.7b-shaped 28-layer FP8 W8A8 decode, fp8 KV, 4-level SID (4x4096), 10M-item "
                                 "Zipf catalog (CSR trie), one replica per GPU", levels=4,
                        prompt_len="uniform[1024,4096]")
    cfg = Qwen3Config(num_hidden_layers=args.layers)
    catalog = make_zipf_catalog(args.items, sizes) if args.workload == "config5" else make_catalog(args.items, sizes)
    # sort-based build on the GPU, straight into the layout the beam step reads
    trie = build_trie_device(torch.from_numpy(np.ascontiguousarray(catalog, dtype=np.int32)).to(dev), sizes,
                             token_base, layout=args.trie)
    arrays = trie.arrays
    sharded = None
    if args.sharded_head:
        if dist is None:
            raise SystemExit("--sharded-head needs more than one rank (torchrun)")
        from flashrec_b200.sharded_head import ShardedSidHead

        sharded = ShardedSidHead()
        WORKLOAD.update(parallelism=f"dp{world} body + token-range-sharded SID head (NCCL)",
                        requests_in_group=args.requests * world)
    eng = SidDecodeEngine(cfg, args.requests, args.beam, prompt_lengths(args.requests, rank, p_lo, p_hi), sizes, token_base, trie,
                          dev, shared_prefix=64, page_size=16, seed=0 if sharded is not None else rank,
                          fuse_rope_gemm=not args.no_fuse_rope_gemm, level0_from_prefill=args.level0_from_prefill,
                          fused_head=not args.no_fused_head, sharded_head=sharded,
                          data_seed=rank if sharded is not None else None)
    # Prefill of the prompts (eager, one extend batch): the decode waves below then read real K/V. Timed on
    # its own; it is not part of `value` (the metric is the decode step).
    prefill = None
    if not args.no_prefill or args.level0_from_prefill:
        eng.prefill()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.prefill()
        e1.record()
        torch.cuda.synchronize()
        pms = e0.elapsed_time(e1)
        prefill = {"tokens": eng.prefill_tokens, "ms": pms, "tokens_per_s": eng.prefill_tokens / pms * 1e3,
                   "note": f"prompts U[{p_lo},{p_hi}], 64-token shared prefix computed once (cached prefix for the rest)"}
    if args.profile_prefill:
        eng.prefill()
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        eng.prefill()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled_prefill_tokens": eng.prefill_tokens}))
        return
    # count this library's kernel launches in one eager wave
    counter = {"n": 0}
    orig_call = _lib.call
    # entries that launch more than one kernel per call (scan + gather + write-back; widening + attention;
    # plan initialisation + plan); every other entry launches one
    kernels_per_call = {"fr_gather_kv_indices": 2, "fr_kv_table_step": 3, "fr_decode_attn_fp8": 2,
                        "fr_decode_attn_reuse_fp8": 2, "fr_decode_attn_plan": 2}

    def counting_call(name, *a):
        counter["n"] += kernels_per_call.get(name, 1)
        return orig_call(name, *a)

    import flashrec_b200.attention as m_att
    import flashrec_b200.decoder as m_dec
    import flashrec_b200.kernel.qk_rope_kv as m_rope
    import flashrec_b200.kernel.rms_fp8 as m_rms
    import flashrec_b200.kernel.sglops as m_sgl
    import flashrec_b200.kernel.silu_fp8 as m_silu
    import flashrec_b200.logits as m_log
    import flashrec_b200.sid_decode as m_sid

    mods = [m_att, m_dec, m_rope, m_rms, m_sgl, m_silu, m_log, m_sid]
    # (the fused head call: row-mask pass for CSR tries + GEMM + statistics combine + beam step)
    kernels_per_call["fr_sid_head_topk"] = 3 if args.trie == "bitmap" else 4
    for m in mods:
        m.call = counting_call
    eng.run(host_io=False, _eager=True)
    torch.cuda.synchronize()
    launches_per_wave = counter["n"]
    for m in mods:
        m.call = orig_call
    if args.profile_wave:
        eng.run(host_io=False, _eager=True)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        eng.run(host_io=False, _eager=True)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled_wave_launches": launches_per_wave}))
        return
    eng.capture()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(host_io: bool, k: int) -> float:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(k):
            eng.run(host_io=host_io)
        e1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        sec = e0.elapsed_time(e1) / 1e3
        if host_io:
            sec = max(sec, wall)  # the wave ends with a host-visible result
        if dist is not None:
            t = torch.tensor([sec], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        return sec

    for _ in range(max(args.warmup, 3)):
        eng.run(host_io=False)
    with ClockSampler(local) as clk:
        sec = timed(False, args.steps)
        sec_e2e = timed(True, args.steps)
    barrier()
    code, site = device_status()
    rows_levels = args.requests * args.beam * (len(sizes) - eng.first_step)  # decode steps x rows
    value = world * rows_levels * args.steps / sec
    e2e_value = world * rows_levels * args.steps / sec_e2e
    h2d = eng.rows * 8 * eng.steps
    d2h = eng.h_vals.numel() * 4 + eng.h_tokens.numel() * 8

    # legality of the produced beams (illegal-SID rate must be 0)
    nodes = eng.final_nodes
    live = torch.isfinite(eng.cum)
    illegal = int(((nodes != -1) & live).sum().item())

    line = None
    if rank == 0:
        fused_flops, fused_sec, flops, gsec, lib_tf = time_gemms(torch, eng.rows)
        peaks = {}
        pk = ROOT / "MEASURED_PEAKS.json"
        if pk.exists():
            peaks = json.loads(pk.read_text())
        bf16_burst = float(peaks.get("bf16_tflops", 1590.0))
        peak_fp8 = 2.0 * bf16_burst
        achieved = fused_flops / fused_sec / 1e12
        traffic, traffic_src = dram_traffic_of_dominant_kernel(eng.rows)
        roof = {
            "bound": "tensor", "achieved": achieved, "peak": peak_fp8, "unit": "TFLOP/s",
            "frac": achieved / peak_fp8, "traffic": traffic,
            "kernel": "gemm_fp8_pair_kernel<bf16, EPI=1> (gate_up GEMM + SwiGLU epilogue, M=%d N=12288 K=2048; "
                      "35 %% of the wave)" % eng.rows,
            "us_per_launch": fused_sec * 1e6,
            "peak_source": ("2 x measured bf16 burst (MEASURED_PEAKS.json)" if peaks else "2 x fallback 1.59 PFLOP/s")
            + "; nominal dense FP8 4500",
            "traffic_source": traffic_src,
            "layer_gemms_tflops": flops / gsec / 1e12,
            "layer_gemms": "plain qkv+o+gate_up+down at M=%d, 4 launches back to back" % eng.rows,
            "cublaslt_fp8_tflops_same_shapes": lib_tf,
        }
        # the second baseline metric is quoted at 512 rows (one request): per-shape time, PFLOP/s and fraction of
        # the same peak, with cuBLASLt's FP8 GEMM on the same shapes in the same run beside it
        try:
            m512 = gemm_shapes(512, emit=False)
            roof["m512"] = {k: {"us": v["us"], "tflops": v["tflops"], "frac": round(v["tflops"] / peak_fp8, 4),
                                "cublaslt_us": v["cublaslt_us"], "cublaslt_tflops": v["cublaslt_tflops"]}
                            for k, v in m512.items()}
        except Exception as exc:  # a library comparison must not take the bench line down
            roof["m512"] = {"error": repr(exc)[:200]}
        cpu = None
        if not args.no_cpu_baseline and world == 1:
            # one bounded sample on the host cores; only in the single-process run, where nothing else loads them
            try:
                ref = ReferenceCpuStep(args.beam, sizes, args.items, args.layers)
                v, desc = ref.sample()
                cpu = {"value": v, "unit": UNIT, "cores": ref.cores, "kind": ref.kind, "sample": desc}
            except Exception as exc:  # the host-side baseline must not take the GPU line down
                cpu = {"value": None, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "reference",
                       "sample": "failed: " + repr(exc)[:200]}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32 (bf16 activations)",
            "data": "synthetic",
            "config": bench_config(args, world, eng.rows, eng.steps - eng.first_step),
            "value_per_gpu": value / world, "catalog_items_distinct": int(arrays.n_items),
            "clocks": clk.summary(),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": sec_e2e / args.steps * 1e3},
            "gpu_launches": launches_per_wave * args.steps,
            "roofline": roof,
            "cpu_baseline": cpu,
            "prefill": prefill,
            "illegal_sid_beams": illegal,
            "device_status": [code, site],
        }
    c5 = None
    if world > 1 and not args.no_config5:
        # the one path with a real exchange: all ranks take part, after the replicas' timed region
        del eng
        torch.cuda.empty_cache()
        try:
            c5 = config5_head(dist, dev, rank, world)
        except Exception as exc:  # keep the replicas' line even if the exchange path fails on this rank
            c5 = {"error": repr(exc)[:300]}
    if rank == 0:
        if c5 is not None:
            line["config5"] = c5
        print(json.dumps(line), flush=True)
    if dist is not None:
        # captured graphs that hold NCCL work go before the communicator does
        eng = None
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
