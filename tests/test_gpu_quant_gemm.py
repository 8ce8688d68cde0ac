"""GPU parity: quantisers and the FP8 GEMM against the CPU oracle and the
reference's golden outputs. Bit-exact for e4m3 bytes / scales / bf16 residuals;
GEMM within 2e-2 relative (bf16 output)."""

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits, bits8, bits16, fp8_from_bits, load_golden
from oracle import sid_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _eq_bytes(a: torch.Tensor, b: torch.Tensor):
    assert np.array_equal(bits8(a), bits8(b))


@pytest.mark.parametrize("rows,hidden", [(8, 2048), (5, 384), (33, 1024), (3, 4096), (1, 8), (17, 6144)])
def test_rms_quant_bit_exact(rows, hidden):
    from flashrec_b200.kernel.rms_fp8 import fused_add_rmsnorm_per_token_quant_fp8, rmsnorm_per_token_quant_fp8

    g = torch.Generator().manual_seed(rows * 131 + hidden)
    x = torch.randn(rows, hidden, generator=g).bfloat16()
    r = torch.randn(rows, hidden, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16()
    q_ref, s_ref = O.rmsnorm_quant_fp8(x, w, 1e-6)
    q, s = rmsnorm_per_token_quant_fp8(x.to(DEV), w.to(DEV), 1e-6)
    _eq_bytes(q, q_ref)
    assert torch.equal(s.cpu(), s_ref)
    q2_ref, s2_ref, r2_ref = O.rmsnorm_quant_fp8(x, w, 1e-6, residual=r.clone())
    r_dev = r.to(DEV)
    q2, s2, r2 = fused_add_rmsnorm_per_token_quant_fp8(x.to(DEV), r_dev, w.to(DEV), 1e-6)
    _eq_bytes(q2, q2_ref)
    assert torch.equal(s2.cpu(), s2_ref)
    assert np.array_equal(bits16(r2), bits16(r2_ref))
    assert r2.data_ptr() == r_dev.data_ptr()  # updated in place


def test_rms_quant_golden_reference_bytes():
    from flashrec_b200.kernel.rms_fp8 import fused_add_rmsnorm_per_token_quant_fp8, rmsnorm_per_token_quant_fp8
    from flashrec_b200.kernel.sglops import fused_add_rmsnorm, rmsnorm

    g = load_golden("rms_quant")
    for tag in ("a", "b"):
        x, r, w = (bf16_from_bits(g[f"{tag}_{n}"]).to(DEV) for n in ("x", "r", "w"))
        q, s = rmsnorm_per_token_quant_fp8(x, w, 1e-6)
        assert np.array_equal(bits8(q), g[f"{tag}_q"]) and np.array_equal(s.cpu().numpy(), g[f"{tag}_s"])
        assert np.array_equal(bits16(rmsnorm(x, w, 1e-6)), g[f"{tag}_y"])
        q2, s2, r2 = fused_add_rmsnorm_per_token_quant_fp8(x, r.clone(), w, 1e-6)
        assert np.array_equal(bits8(q2), g[f"{tag}_q_res"]) and np.array_equal(s2.cpu().numpy(), g[f"{tag}_s_res"])
        assert np.array_equal(bits16(r2), g[f"{tag}_r_out"])
        y3, r3 = fused_add_rmsnorm(x, r.clone(), w, 1e-6)
        assert np.array_equal(bits16(r3), g[f"{tag}_r_out"])


@pytest.mark.parametrize("rows,hidden", [(6, 2048), (7, 72), (2, 12288)])
def test_token_quant_bit_exact(rows, hidden):
    from flashrec_b200.kernel.sglops import per_token_quant_fp8

    g = torch.Generator().manual_seed(hidden)
    x = (3 * torch.randn(rows, hidden, generator=g)).bfloat16()
    x[0, :] = 0  # all-zero row: amax clamps to 1e-12
    q_ref, s_ref = O.per_token_quant_fp8(x)
    q, s = per_token_quant_fp8(x.to(DEV))
    _eq_bytes(q, q_ref)
    assert torch.equal(s.cpu(), s_ref)
    assert s.shape == (rows, 1)
    # fp32 input (weight quantisation)
    wf = 0.02 * torch.randn(rows, hidden, generator=g)
    qw_ref, sw_ref = O.quantize_weight_fp8(wf)
    from flashrec_b200.layers import quantize_weight_fp8

    qw, sw = quantize_weight_fp8(wf.to(DEV))
    _eq_bytes(qw, qw_ref)
    assert torch.equal(sw.cpu(), sw_ref)


def test_empty_inputs():
    from flashrec_b200.kernel.sglops import per_token_quant_fp8
    from flashrec_b200.kernel.silu_fp8 import silu_and_mul_per_token_quant_fp8

    q, s = per_token_quant_fp8(torch.empty(0, 256, dtype=torch.bfloat16, device=DEV))
    assert q.shape == (0, 256) and s.shape == (0, 1)
    q, s = silu_and_mul_per_token_quant_fp8(torch.empty(0, 512, dtype=torch.bfloat16, device=DEV))
    assert q.shape == (0, 256)


@pytest.mark.parametrize("rows,d", [(4, 6144), (9, 1024), (3, 136), (2, 16384)])
def test_silu_quant_bit_exact(rows, d):
    from flashrec_b200.kernel.sglops import silu_and_mul
    from flashrec_b200.kernel.silu_fp8 import silu_and_mul_per_token_quant_fp8

    g = torch.Generator().manual_seed(d)
    x = (2 * torch.randn(rows, 2 * d, generator=g)).bfloat16()
    x[0, :8] = torch.tensor([-100.0, -88.0, 88.0, 1e-30, -1e-30, 0.0, 30.0, -30.0]).bfloat16()
    q_ref, s_ref = O.silu_mul_quant_fp8(x)
    q, s = silu_and_mul_per_token_quant_fp8(x.to(DEV))
    _eq_bytes(q, q_ref)
    assert torch.equal(s.cpu(), s_ref)
    assert np.array_equal(bits16(silu_and_mul(x.to(DEV))), bits16(O.silu_and_mul(x)))


def test_silu_quant_golden_close_to_reference():
    from flashrec_b200.kernel.silu_fp8 import silu_and_mul_per_token_quant_fp8

    g = load_golden("quant_silu")
    q, s = silu_and_mul_per_token_quant_fp8(bf16_from_bits(g["gu"]).to(DEV))
    assert (bits8(q) != g["q_silu"]).mean() < 1e-3  # torch's float32 exp vs exact silu
    assert np.allclose(s.cpu().numpy(), g["s_silu"], rtol=1e-2)


GEMM_SHAPES = [
    # M, N, K, block_n
    (128, 256, 128, 256),
    (128, 128, 256, 128),
    (128, 64, 384, 64),
    (24, 96, 256, 0),
    (512, 512, 2048, 0),
    (200, 1000, 1040, 128),
    (300, 328, 144, 256),
    (1, 8, 16, 64),
    # 512 = CTA pairs (cluster of 2) on 256 x 256 tiles
    (512, 512, 2048, 512),
    (300, 328, 144, 512),
    (1000, 768, 256, 512),
    (130, 2048, 6144, 512),
    # 1024 = split-K over a cluster (256 x 256 tile per cluster, partial tiles summed through
    # distributed shared memory); 0 picks it by itself for few rows
    (512, 2048, 6144, 1024),   # 8 CTAs per tile
    (512, 4096, 2048, 0),      # 4 CTAs per tile (auto)
    (300, 328, 144, 1024),     # ragged everywhere, K tail, a single k-split
    (37, 200, 2048, 1024),     # N not a multiple of 4 pieces' row, one row block
    (1000, 768, 256, 1024),
    # 1024 + 128 / 1024 + 256: split-K with the tile width named (128 x 128 or 128 x 256 per cluster)
    (512, 2048, 6144, 1152),   # 2 CTAs per 128-wide tile
    (256, 2048, 6144, 1152),   # 4 CTAs per tile
    (128, 1024, 2048, 1152),   # 8 CTAs per tile
    (300, 328, 144, 1152),     # ragged, a single k-split
    (37, 200, 2048, 1152),
    (512, 2048, 6144, 1280),
    (256, 2048, 6144, 0),      # auto: the plan's cost model picks the narrow tile here
]


@pytest.mark.parametrize("m,n,k,bn", GEMM_SHAPES)
def test_gemm_fp8_vs_oracle(m, n, k, bn):
    from flashrec_b200 import device_status
    from flashrec_b200.kernel.sglops import fp8_scaled_mm

    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = 0.02 * torch.randn(n, k, generator=g)
    aq, asc = O.per_token_quant_fp8(a)
    wq, wsc = O.quantize_weight_fp8(w)
    ref = O.fp8_scaled_mm(aq, wq, asc, wsc).float()
    out = fp8_scaled_mm(aq.to(DEV), wq.to(DEV).t(), asc.to(DEV), wsc.to(DEV), torch.bfloat16, block_n=bn)
    torch.cuda.synchronize()
    assert device_status() == (0, 0)
    got = out.float().cpu()
    denom = ref.abs().max().clamp(min=1e-6)
    assert ((got - ref).abs().max() / denom) < 2e-2
    # fp32 output (lm_head logits): one rounding only, much tighter
    ref32 = O.fp8_logits_f32(aq, wq, asc, wsc)
    out32 = fp8_scaled_mm(aq.to(DEV), wq.to(DEV).t(), asc.to(DEV), wsc.to(DEV), torch.float32, block_n=bn)
    assert torch.allclose(out32.cpu(), ref32, rtol=1e-5, atol=1e-6 * float(ref32.abs().max()))


def test_gemm_exact_accumulation_small_integers():
    """Operands that are small integers make every partial sum exact, so the
    tensor-core result must equal the integer matmul exactly."""
    from flashrec_b200.kernel.sglops import fp8_scaled_mm

    g = torch.Generator().manual_seed(1)
    m, n, k = 256, 384, 512
    a = torch.randint(-3, 4, (m, k), generator=g).float()
    b = torch.randint(-3, 4, (n, k), generator=g).float()
    ref = a @ b.t()
    ones_m = torch.ones(m, 1, device=DEV)
    ones_n = torch.ones(n, device=DEV)
    for bn in (64, 128, 256, 512, 1024, 1152, 1280):
        out = fp8_scaled_mm(a.to(torch.float8_e4m3fn).to(DEV), b.to(torch.float8_e4m3fn).to(DEV).t(), ones_m, ones_n,
                            torch.float32, block_n=bn)
        assert torch.equal(out.cpu(), ref), f"block_n={bn}"


def test_linear_golden_and_bias():
    from flashrec_b200.layers import Linear

    g = load_golden("linear_fp8")
    lin = Linear(256, 96)
    lin.load(torch.from_numpy(g["w"]).to(DEV), quantize_fp8=True)
    assert np.array_equal(bits8(lin._fp8_weight.t()), g["wq"])
    assert np.array_equal(lin._fp8_scale.cpu().numpy(), g["wscale"])
    y = lin.forward_fp8(fp8_from_bits(g["xq"]).to(DEV), torch.from_numpy(g["xs"]).to(DEV), (24, 256), torch.bfloat16)
    ref = bf16_from_bits(g["y"]).float()
    assert ((y.float().cpu() - ref).abs().max() / ref.abs().max()) < 2e-2
    y2 = lin(bf16_from_bits(g["x"]).to(DEV))  # dynamic activation quantisation path
    assert torch.equal(y2, y)
    lin.bias = torch.randn(96, device=DEV).bfloat16()
    yb = lin(bf16_from_bits(g["x"]).to(DEV))
    assert torch.allclose(yb.float(), (y + lin.bias).float(), atol=1e-2)


def test_bad_arguments_raise():
    from flashrec_b200 import FlashRecKernelError
    from flashrec_b200.kernel.sglops import fp8_scaled_mm, per_token_quant_fp8

    with pytest.raises(FlashRecKernelError):
        per_token_quant_fp8(torch.zeros(4, 64, dtype=torch.bfloat16))  # CPU tensor: no fallback
    a = torch.zeros(8, 24, device=DEV).to(torch.float8_e4m3fn)  # K % 16 != 0
    b = torch.zeros(16, 24, device=DEV).to(torch.float8_e4m3fn)
    with pytest.raises(FlashRecKernelError):
        fp8_scaled_mm(a, b.t(), torch.ones(8, 1, device=DEV), torch.ones(16, device=DEV), torch.bfloat16)


@pytest.mark.parametrize("m,d,k", [(200, 256, 512), (128, 1024, 256), (37, 128, 2048)])
def test_gemm_silu_epilogue_equals_unfused_bit_for_bit(m, d, k):
    """gate_up GEMM with SwiGLU in the epilogue + known-amax quantiser == GEMM -> fused SwiGLU quantiser."""
    from flashrec_b200.kernel.sglops import (fp8_scaled_mm, fp8_scaled_mm_silu_mul, interleave_gate_up,
                                             quant_known_amax_fp8, silu_and_mul)
    from flashrec_b200.kernel.silu_fp8 import silu_and_mul_per_token_quant_fp8

    g = torch.Generator().manual_seed(m + d)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = 0.05 * torch.randn(2 * d, k, generator=g)
    aq, asc = O.per_token_quant_fp8(a)
    wq, wsc = O.quantize_weight_fp8(w)
    aq, asc, wq, wsc = aq.to(DEV), asc.to(DEV), wq.to(DEV), wsc.to(DEV)
    gu = fp8_scaled_mm(aq, wq.t(), asc, wsc, torch.bfloat16, block_n=256)
    q_ref, s_ref = silu_and_mul_per_token_quant_fp8(gu)
    wi, si = interleave_gate_up(wq, wsc)
    y, amax = fp8_scaled_mm_silu_mul(aq, wi, asc, si, mode=1)
    assert np.array_equal(bits16(y), bits16(silu_and_mul(gu)))
    y2, amax2 = fp8_scaled_mm_silu_mul(aq, wi, asc, si, mode=2)  # CTA pairs
    assert torch.equal(y2, y) and torch.equal(amax2, amax)
    q, s = quant_known_amax_fp8(y, amax)
    assert np.array_equal(bits8(q), bits8(q_ref)) and torch.equal(s, s_ref)
    # and against the CPU oracle of the unfused reference order
    qo, so = O.silu_mul_quant_fp8(gu.cpu())
    assert np.array_equal(bits8(q), bits8(qo)) and torch.equal(s.cpu(), so)


@pytest.mark.parametrize("case", ["zero_rows", "wide_gates", "tiny_channel_scales", "huge_row_scales"])
def test_gemm_silu_epilogue_corner_inputs(case):
    """The SwiGLU epilogue keeps bit parity with GEMM -> SwiGLU where its shortcuts do not apply: all-zero
    rows, gates far into both tails, and scales outside the range its FMA-pipe bf16 rounding covers."""
    from flashrec_b200.kernel.sglops import fp8_scaled_mm, fp8_scaled_mm_silu_mul, interleave_gate_up, silu_and_mul

    m, d, k = 300, 256, 512
    g = torch.Generator().manual_seed(7)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = 0.05 * torch.randn(2 * d, k, generator=g)
    if case == "zero_rows":
        a[5:40] = 0
        a[257:] = 0
    if case == "wide_gates":
        w = 2.0 * torch.randn(2 * d, k, generator=g)  # gate values of a few tens, both signs
    aq, asc = O.per_token_quant_fp8(a)
    wq, wsc = O.quantize_weight_fp8(w)
    if case == "tiny_channel_scales":
        wsc[::7] = 1e-30
        wsc[3::11] = 1e-41  # subnormal scale: subnormal gate / up values
    if case == "huge_row_scales":
        asc[::5] = 3e30
        wsc[::3] = 1e6
    aq, asc, wq, wsc = aq.to(DEV), asc.to(DEV), wq.to(DEV), wsc.to(DEV)
    gu = fp8_scaled_mm(aq, wq.t(), asc, wsc, torch.bfloat16, block_n=256)
    ref = silu_and_mul(gu)
    wi, si = interleave_gate_up(wq, wsc)
    for mode in (1, 2):
        y, amax = fp8_scaled_mm_silu_mul(aq, wi, asc, si, mode=mode)
        assert np.array_equal(bits16(y), bits16(ref)), (case, mode)
        finite = torch.isfinite(ref.float()).all(dim=1)
        want = ref.float().abs().amax(dim=1)
        assert torch.equal(amax.flatten()[finite], want[finite]), (case, mode)


@pytest.mark.parametrize("m,n,k,block_n", [(300, 512, 256, 0), (37, 200, 128, 64), (128, 256, 2048, 256),
                                           (700, 1024, 384, 512), (513, 200, 512, 512), (4100, 2048, 256, 0),
                                           (512, 2048, 6144, 1024), (300, 200, 384, 1024), (512, 2048, 2048, 0),
                                           (512, 2048, 6144, 1152), (300, 200, 384, 1152), (256, 2048, 6144, 1280)])
def test_gemm_add_into_residual_equals_gemm_then_bf16_add(m, n, k, block_n):
    """fr_gemm_fp8_w8a8_add == GEMM (bf16 out) followed by the bf16 add of fused_add_rmsnorm, bit for bit,
    through the single-CTA kernels (hint 64 / 256 / auto) and the CTA-pair kernel (hint 512, ragged edges)."""
    from flashrec_b200.kernel.sglops import fp8_scaled_mm, fp8_scaled_mm_add_

    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = 0.05 * torch.randn(n, k, generator=g)
    res = torch.randn(m, n, generator=g).bfloat16()
    aq, asc = O.per_token_quant_fp8(a)
    wq, wsc = O.quantize_weight_fp8(w)
    aq, asc, wq, wsc = aq.to(DEV), asc.to(DEV), wq.to(DEV), wsc.to(DEV)
    x = fp8_scaled_mm(aq, wq.t(), asc, wsc, torch.bfloat16, block_n=block_n)
    want = (x.float() + res.to(DEV).float()).bfloat16()
    # a padded residual matrix: row pitch larger than N, columns beyond N must stay untouched
    pitch = (n + 15) // 8 * 8
    buf = torch.full((m, pitch), 7.0, dtype=torch.bfloat16, device=DEV)
    buf[:, :n] = res.to(DEV)
    out = fp8_scaled_mm_add_(aq, wq.t(), asc, wsc, buf[:, :n], block_n=block_n)
    assert out.data_ptr() == buf.data_ptr()
    assert np.array_equal(bits16(buf[:, :n].contiguous()), bits16(want))
    assert (buf[:, n:] == 7.0).all()


@pytest.mark.parametrize("t,n_q,n_kv,k", [(300, 4, 2, 512), (37, 2, 2, 256), (1100, 16, 8, 2048)])
def test_qkv_gemm_with_norm_rope_kv_epilogue_equals_the_two_calls(t, n_q, n_kv, k):
    """fr_gemm_fp8_qkv_rope == qkv GEMM (bf16) -> fused_qk_norm_rope_store_fp8: Q bits, K / V pool bytes,
    untouched slots; rows with out-of-range slots are skipped."""
    from flashrec_b200.kernel.qk_rope_kv import fp8_qkv_mm_norm_rope_store, fused_qk_norm_rope_store_fp8
    from flashrec_b200.kernel.sglops import fp8_scaled_mm

    d = 128
    g = torch.Generator().manual_seed(t + n_q)
    a = torch.randn(t, k, generator=g).bfloat16()
    w = 0.05 * torch.randn((n_q + 2 * n_kv) * d, k, generator=g)
    aq, asc = O.per_token_quant_fp8(a)
    wq, wsc = O.quantize_weight_fp8(w)
    aq, asc, wq, wsc = aq.to(DEV), asc.to(DEV), wq.to(DEV), wsc.to(DEV)
    qw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16().to(DEV)
    kw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16().to(DEV)
    cs = O.build_cos_sin_cache(d, 400, 1e6).to(DEV)
    pos = torch.randint(0, 400, (t,), generator=g).to(DEV)
    slots = t + 20
    loc = (torch.randperm(slots - 1, generator=g)[:t] + 1)
    loc[0] = -5          # outside the pool: no write
    loc[t // 2] = slots  # outside the pool: no write
    loc = loc.to(DEV)

    def pools():
        kc = torch.full((slots, n_kv, d), 0x11, dtype=torch.uint8, device=DEV).view(torch.float8_e4m3fn)
        return kc, kc.clone()

    qkv = fp8_scaled_mm(aq, wq.t(), asc, wsc, torch.bfloat16, block_n=256).view(t, n_q + 2 * n_kv, d)
    kc_ref, vc_ref = pools()
    fused_qk_norm_rope_store_fp8(qkv[:, :n_q], qkv[:, n_q:n_q + n_kv], qkv[:, n_q + n_kv:], pos, loc, qw, kw, 1e-6, cs,
                                 kc_ref, vc_ref)
    kc, vc = pools()
    q = fp8_qkv_mm_norm_rope_store(aq, wq.t(), asc, wsc, pos, loc, qw, kw, 1e-6, cs, kc, vc, n_q, n_kv)
    assert q.shape == (t, n_q, d)
    assert np.array_equal(bits16(q), bits16(qkv[:, :n_q].contiguous()))
    assert np.array_equal(bits8(kc), bits8(kc_ref)) and np.array_equal(bits8(vc), bits8(vc_ref))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_one_process_drives_a_second_gpu():
    """Kernels that opt in to more than 48 KB of dynamic shared memory (every tcgen05 GEMM variant, the wide beam
    step) launched on cuda:0 and then on cuda:1 from one process: the opt-in is per device, so a cache keyed by
    process would leave the second device without it (launch failure). Same bits on both devices."""
    from flashrec_b200 import device_status
    from flashrec_b200.kernel.sglops import (fp8_scaled_mm, fp8_scaled_mm_add_, fp8_scaled_mm_silu_mul,
                                             interleave_gate_up, per_token_quant_fp8)
    from flashrec_b200.layers import quantize_weight_fp8
    from flashrec_b200.sid_decode import sid_beam_step

    g = torch.Generator().manual_seed(3)
    x = torch.randn(1024, 512, generator=g).bfloat16()
    w = 0.05 * torch.randn(1024, 512, generator=g)
    res = torch.randn(1024, 1024, generator=g).bfloat16()
    logits = torch.randn(2 * 64, 4096, generator=g)
    outs = []
    for dev in ("cuda:0", "cuda:1"):
        with torch.cuda.device(dev):
            q, s = per_token_quant_fp8(x.to(dev))
            wq, ws = quantize_weight_fp8(w.to(dev))
            y = fp8_scaled_mm(q, wq.t(), s, ws, torch.bfloat16)               # pair kernel (M = 1024)
            y512 = fp8_scaled_mm(q[:512], wq.t(), s[:512], ws, torch.bfloat16)  # one CTA per tile
            wi, si = interleave_gate_up(wq, ws)
            ys, amax = fp8_scaled_mm_silu_mul(q, wi, s, si)
            r = res.to(dev).clone()
            fp8_scaled_mm_add_(q, wq.t(), s, ws, r)
            lg = logits.to(dev)
            mx = lg.amax(dim=-1)
            ls = torch.log(torch.exp(lg - mx[:, None]).sum(-1))
            cum = torch.zeros(2, 64, device=dev)
            st = sid_beam_step(cum, lg, mx, ls, None, None, 0, 2048)           # K = 2048: wide shared memory
            torch.cuda.synchronize()
            assert device_status() == (0, 0)
            outs.append([t.cpu() for t in (y, y512, ys, amax, r, st.vals, st.indices)])
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("m,n,k", [(512, 4096, 2048), (512, 2048, 2048), (300, 4096, 256), (1000, 2048, 384), (129, 4096, 128)])
def test_few_row_gemms_equal_across_tilings(m, n, k):
    """A decode step of one request (a few hundred rows): whatever tiling the library picks, plain and
    add-into-residual outputs must equal, bit for bit, the one-CTA-per-tile kernel (tile hint 128 / 64) and the
    256 x 256 pair kernel (hint 512), with ragged last row blocks; and the oracle within the GEMM tolerance."""
    from flashrec_b200.kernel.sglops import fp8_scaled_mm, fp8_scaled_mm_add_, per_token_quant_fp8
    from flashrec_b200.layers import quantize_weight_fp8

    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).bfloat16()
    w = 0.05 * torch.randn(n, k, generator=g)
    res = torch.randn(m, n, generator=g).bfloat16()
    q, s = per_token_quant_fp8(x.to(DEV))
    wq, ws = quantize_weight_fp8(w.to(DEV))
    y = fp8_scaled_mm(q, wq.t(), s, ws, torch.bfloat16)
    for hint in (64, 128, 512):
        assert torch.equal(y, fp8_scaled_mm(q, wq.t(), s, ws, torch.bfloat16, block_n=hint)), hint
    ref = O.fp8_scaled_mm(q.cpu(), wq.cpu(), s.cpu(), ws.cpu()).float()
    assert ((y.float().cpu() - ref).abs().max() / ref.abs().max()) < 2e-2
    want = (y.float() + res.to(DEV).float()).bfloat16()
    for hint in (0, 64, 128, 512):
        r = res.to(DEV).clone()
        fp8_scaled_mm_add_(q, wq.t(), s, ws, r, block_n=hint)
        assert torch.equal(r, want), hint
