// Activation quantisers of the FP8 decode step: one pass over HBM per row,
// emitting e4m3 bytes plus one fp32 scale per row.
//
//   fr_rms_quant_fp8        RMSNorm.quant_fp8 (layers/norm.py:28-42) =
//                           rmsnorm / fused_add_rmsnorm (kernel/sglops.py:34-61)
//                           followed by per_token_quant_fp8 (kernel/sglops.py:84-96)
//   fr_token_quant_fp8      per_token_quant_fp8 (kernel/sglops.py:84-96) and
//                           quantize_weight_fp8 (layers/linear.py:26-32)
//   fr_silu_mul_quant_fp8   silu_and_mul_per_token_quant_fp8 (kernel/silu_fp8.py:86-119)
//   fr_rmsnorm_bf16         rmsnorm / fused_add_rmsnorm (kernel/sglops.py:34-61)
//   fr_silu_mul_bf16        silu_and_mul (kernel/sglops.py:143-151)
//
// Numerics follow the reference's torch path, including its intermediate
// bf16 roundings: the normalised row is rounded to bf16 before the amax and
// the division by the scale; silu and the gate*up product are each rounded to
// bf16. The only deliberate difference is the sum of squares, accumulated in
// fp64 and rounded once (order independent), where torch adds in fp32.
#include "fr_common.cuh"

namespace fr {

constexpr int kWarpsPerCta = 4;  // 128-thread CTAs: at ~96 registers per thread five of them fit on an SM (20 warps) where two 256-thread CTAs give 16

// ---------------------------------------------------------------------------
// One warp per row, hidden = 256 * VPL, whole row held in registers.
// ---------------------------------------------------------------------------
template <int VPL, bool NORM, bool RESID, bool QUANT>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
row_warp_kernel(const uint4* __restrict__ x, uint4* __restrict__ resid, const uint4* __restrict__ w, float eps,
                uint2* __restrict__ q, float* __restrict__ scale, uint4* __restrict__ y_out, int rows) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  constexpr int kVecPerRow = VPL * 32;
  const uint4* xr = x + static_cast<size_t>(row) * kVecPerRow;

  uint4 v[VPL];
#pragma unroll
  for (int j = 0; j < VPL; ++j) v[j] = __ldg(xr + j * 32 + lane);

  if constexpr (RESID) {
    uint4* rr = resid + static_cast<size_t>(row) * kVecPerRow;
    // every residual load is issued before the first store to the same array (the
    // compiler cannot reorder them itself), so the row costs one memory round trip
    uint4 r[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) r[j] = rr[j * 32 + lane];
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      uint32_t* xv = reinterpret_cast<uint32_t*>(&v[j]);
      const uint32_t* rv = reinterpret_cast<const uint32_t*>(&r[j]);
#pragma unroll
      for (int t = 0; t < 4; ++t) xv[t] = add_bf16x2(rv[t], xv[t]);  // residual + x, rounded to bf16
    }
#pragma unroll
    for (int j = 0; j < VPL; ++j) rr[j * 32 + lane] = v[j];
  }

  float amax = 0.f;
  if constexpr (NORM) {
    // four independent chains: a lane's 8 * VPL fp64 FMAs in one chain are the longest dependent
    // sequence of the kernel when few rows are in flight (a decode step of one request)
    double s4[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const uint32_t* xv = reinterpret_cast<const uint32_t*>(&v[j]);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const double a = static_cast<double>(bf16lo(xv[t])), b = static_cast<double>(bf16hi(xv[t]));
        s4[t] = fma(a, a, s4[t]);  // the squares are exact (8-bit significands)
        s4[t] = fma(b, b, s4[t]);
      }
    }
    double ss = warp_sum((s4[0] + s4[1]) + (s4[2] + s4[3]));
    const float var = static_cast<float>(ss / static_cast<double>(VPL * 256));
    const float rstd = rsqrt_rn(__fadd_rn(var, eps));
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      uint4 wv = __ldg(w + j * 32 + lane);
      uint32_t* xv = reinterpret_cast<uint32_t*>(&v[j]);
      const uint32_t* wp = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float a = __fmul_rn(__fmul_rn(bf16lo(xv[t]), rstd), bf16lo(wp[t]));
        float b = __fmul_rn(__fmul_rn(bf16hi(xv[t]), rstd), bf16hi(wp[t]));
        xv[t] = pack_bf16(a, b);
      }
    }
  }

  if constexpr (!QUANT) {
    uint4* yr = y_out + static_cast<size_t>(row) * kVecPerRow;
#pragma unroll
    for (int j = 0; j < VPL; ++j) yr[j * 32 + lane] = v[j];
    return;
  } else {
    uint32_t am2 = 0;  // running max |.| of both bf16 lanes
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const uint32_t* xv = reinterpret_cast<const uint32_t*>(&v[j]);
#pragma unroll
      for (int t = 0; t < 4; ++t) am2 = absmax_bf16x2(am2, xv[t]);
    }
    amax = warp_max(fmaxf(bf16lo(am2), bf16hi(am2)));
    const float s = row_scale(amax);
    const float inv = __fdiv_rn(1.0f, s);
    const float sf = finite_or_zero(s);
    uint2* qr = q + static_cast<size_t>(row) * kVecPerRow;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const uint32_t* xv = reinterpret_cast<const uint32_t*>(&v[j]);
      uint2 o;
      o.x = pack_e4m3x4(quant_div_fast(bf16lo(xv[0]), sf, inv), quant_div_fast(bf16hi(xv[0]), sf, inv), quant_div_fast(bf16lo(xv[1]), sf, inv),
                        quant_div_fast(bf16hi(xv[1]), sf, inv));
      o.y = pack_e4m3x4(quant_div_fast(bf16lo(xv[2]), sf, inv), quant_div_fast(bf16hi(xv[2]), sf, inv), quant_div_fast(bf16lo(xv[3]), sf, inv),
                        quant_div_fast(bf16hi(xv[3]), sf, inv));
      qr[j * 32 + lane] = o;
    }
    if (lane == 0) scale[row] = s;
  }
}

// ---------------------------------------------------------------------------
// Generic: one CTA per row, any hidden that is a multiple of 8; the row is
// staged in dynamic shared memory (hidden * 2 bytes) so HBM is read once.
// ---------------------------------------------------------------------------
constexpr int kBlockRowThreads = 256;

__device__ __forceinline__ double block_sum(double v, double* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  double t = 0.0;
  for (int i = 0; i < kBlockRowThreads / 32; ++i) t += red[i];  // fixed order
  return t;
}

__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = red[0];
  for (int i = 1; i < kBlockRowThreads / 32; ++i) t = fmaxf(t, red[i]);
  return t;
}

template <bool NORM, bool RESID, bool QUANT>
__global__ void __launch_bounds__(kBlockRowThreads)
row_block_kernel(const uint4* __restrict__ x, uint4* __restrict__ resid, const uint4* __restrict__ w, float eps,
                 uint2* __restrict__ q, float* __restrict__ scale, uint4* __restrict__ y_out, int hidden) {
  extern __shared__ uint4 row_smem[];
  __shared__ double red_d[kBlockRowThreads / 32];
  __shared__ float red_f[kBlockRowThreads / 32];
  const int row = blockIdx.x;
  const int nvec = hidden >> 3;
  const uint4* xr = x + static_cast<size_t>(row) * nvec;
  double ss = 0.0;
  for (int i = threadIdx.x; i < nvec; i += kBlockRowThreads) {
    uint4 v = __ldg(xr + i);
    uint32_t* xv = reinterpret_cast<uint32_t*>(&v);
    if constexpr (RESID) {
      uint4* rr = resid + static_cast<size_t>(row) * nvec;
      uint4 r = rr[i];
      const uint32_t* rv = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
      for (int t = 0; t < 4; ++t)
        xv[t] = pack_bf16(__fadd_rn(bf16lo(rv[t]), bf16lo(xv[t])), __fadd_rn(bf16hi(rv[t]), bf16hi(xv[t])));
      rr[i] = v;
    }
    if constexpr (NORM) {
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float a = bf16lo(xv[t]), b = bf16hi(xv[t]);
        ss += static_cast<double>(a * a);
        ss += static_cast<double>(b * b);
      }
    }
    row_smem[i] = v;
  }
  float amax = 0.f;
  if constexpr (NORM) {
    ss = block_sum(ss, red_d);
    const float var = static_cast<float>(ss / static_cast<double>(hidden));
    const float rstd = rsqrt_rn(__fadd_rn(var, eps));
    for (int i = threadIdx.x; i < nvec; i += kBlockRowThreads) {
      uint4 v = row_smem[i];
      uint4 wv = __ldg(w + i);
      uint32_t* xv = reinterpret_cast<uint32_t*>(&v);
      const uint32_t* wp = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float a = __fmul_rn(__fmul_rn(bf16lo(xv[t]), rstd), bf16lo(wp[t]));
        float b = __fmul_rn(__fmul_rn(bf16hi(xv[t]), rstd), bf16hi(wp[t]));
        xv[t] = pack_bf16(a, b);
        amax = fmaxf(amax, fmaxf(fabsf(round_bf16(a)), fabsf(round_bf16(b))));
      }
      if constexpr (QUANT) row_smem[i] = v;
      else y_out[static_cast<size_t>(row) * nvec + i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < nvec; i += kBlockRowThreads) {
      uint4 v = row_smem[i];
      const uint32_t* xv = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int t = 0; t < 4; ++t) amax = fmaxf(amax, fmaxf(fabsf(bf16lo(xv[t])), fabsf(bf16hi(xv[t]))));
    }
  }
  if constexpr (QUANT) {
    amax = block_max(amax, red_f);
    const float s = row_scale(amax);
    const float inv = __fdiv_rn(1.0f, s);
    const float sf = finite_or_zero(s);
    uint2* qr = q + static_cast<size_t>(row) * nvec;
    for (int i = threadIdx.x; i < nvec; i += kBlockRowThreads) {
      uint4 v = row_smem[i];
      const uint32_t* xv = reinterpret_cast<const uint32_t*>(&v);
      uint2 o;
      o.x = pack_e4m3x4(quant_div_fast(bf16lo(xv[0]), sf, inv), quant_div_fast(bf16hi(xv[0]), sf, inv), quant_div_fast(bf16lo(xv[1]), sf, inv),
                        quant_div_fast(bf16hi(xv[1]), sf, inv));
      o.y = pack_e4m3x4(quant_div_fast(bf16lo(xv[2]), sf, inv), quant_div_fast(bf16hi(xv[2]), sf, inv), quant_div_fast(bf16lo(xv[3]), sf, inv),
                        quant_div_fast(bf16hi(xv[3]), sf, inv));
      qr[i] = o;
    }
    if (threadIdx.x == 0) scale[row] = s;
  }
}

// fp32 input rows (load-time weight quantisation); no bf16 rounding anywhere.
__global__ void __launch_bounds__(kBlockRowThreads)
row_quant_f32_kernel(const float4* __restrict__ x, uint32_t* __restrict__ q, float* __restrict__ scale, int hidden) {
  __shared__ float red_f[kBlockRowThreads / 32];
  const int row = blockIdx.x;
  const int nvec = hidden >> 2;
  const float4* xr = x + static_cast<size_t>(row) * nvec;
  float amax = 0.f;
  for (int i = threadIdx.x; i < nvec; i += kBlockRowThreads) {
    float4 v = __ldg(xr + i);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
  amax = block_max(amax, red_f);
  const float s = row_scale(amax);
    const float inv = __fdiv_rn(1.0f, s);
    const float sf = finite_or_zero(s);
  uint32_t* qr = q + static_cast<size_t>(row) * nvec;
  for (int i = threadIdx.x; i < nvec; i += kBlockRowThreads) {
    float4 v = __ldg(xr + i);
    qr[i] = pack_e4m3x4(quant_div_fast(v.x, sf, inv), quant_div_fast(v.y, sf, inv), quant_div_fast(v.z, sf, inv), quant_div_fast(v.w, sf, inv));
  }
  if (threadIdx.x == 0) scale[row] = s;
}

// ---------------------------------------------------------------------------
// SwiGLU: silu(gate) * up, both rounded to bf16 as the torch bf16 path does.
// ---------------------------------------------------------------------------
template <int NV, bool QUANT>
__global__ void __launch_bounds__(kBlockRowThreads)
silu_mul_kernel(const uint4* __restrict__ x, uint2* __restrict__ q, float* __restrict__ scale,
                uint4* __restrict__ y_out, int d, const uint16_t* __restrict__ silu_table) {
  __shared__ float red_f[kBlockRowThreads / 32];
  const int row = blockIdx.x;
  const int nvec = d >> 3;
  const uint4* gate = x + static_cast<size_t>(row) * nvec * 2;
  const uint4* up = gate + nvec;
  // all loads of the row are issued before any arithmetic (2 * NV 16-byte loads in flight per thread)
  uint4 g[NV], u[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = j * kBlockRowThreads + threadIdx.x;
    g[j] = make_uint4(0, 0, 0, 0);
    u[j] = make_uint4(0, 0, 0, 0);
    if (i < nvec) {
      g[j] = __ldcs(gate + i);  // streamed once
      u[j] = __ldcs(up + i);
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    uint32_t* yv = reinterpret_cast<uint32_t*>(&g[j]);  // the product overwrites the gate registers
    const uint32_t* uv = reinterpret_cast<const uint32_t*>(&u[j]);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      yv[t] = silu_mul_pack(yv[t], uv[t], silu_table);
      amax = fmaxf(amax, fmaxf(fabsf(bf16lo(yv[t])), fabsf(bf16hi(yv[t]))));
    }
    if constexpr (!QUANT) {
      const int i = j * kBlockRowThreads + threadIdx.x;
      if (i < nvec) y_out[static_cast<size_t>(row) * nvec + i] = g[j];
    }
  }
  if constexpr (QUANT) {
    amax = block_max(amax, red_f);
    const float s = row_scale(amax);
    const float inv = __fdiv_rn(1.0f, s);
    const float sf = finite_or_zero(s);
    uint2* qr = q + static_cast<size_t>(row) * nvec;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = j * kBlockRowThreads + threadIdx.x;
      if (i < nvec) {
        const uint32_t* xv = reinterpret_cast<const uint32_t*>(&g[j]);
        uint2 o;
        o.x = pack_e4m3x4(quant_div_fast(bf16lo(xv[0]), sf, inv), quant_div_fast(bf16hi(xv[0]), sf, inv),
                          quant_div_fast(bf16lo(xv[1]), sf, inv), quant_div_fast(bf16hi(xv[1]), sf, inv));
        o.y = pack_e4m3x4(quant_div_fast(bf16lo(xv[2]), sf, inv), quant_div_fast(bf16hi(xv[2]), sf, inv),
                          quant_div_fast(bf16lo(xv[3]), sf, inv), quant_div_fast(bf16hi(xv[3]), sf, inv));
        qr[i] = o;
      }
    }
    if (threadIdx.x == 0) scale[row] = s;
  }
}

// Rows whose max|y| is already known (written by the fused GEMM epilogue):
// pure streaming quantiser, 16-byte loads / 8-byte stores, grid-stride.
template <int NV>
__global__ void __launch_bounds__(256)
quant_known_amax_kernel(const uint4* __restrict__ y, const float* __restrict__ row_amax, uint2* __restrict__ q,
                        float* __restrict__ scale, int vec_per_row) {
  const int row = blockIdx.x;
  const uint4* yr = y + static_cast<size_t>(row) * vec_per_row;
  uint4 v[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = j * 256 + threadIdx.x;
    v[j] = make_uint4(0, 0, 0, 0);
    if (i < vec_per_row) v[j] = __ldcs(yr + i);
  }
  const float s = row_scale(__ldg(row_amax + row));
  const float inv = __fdiv_rn(1.0f, s);
  const float sf = finite_or_zero(s);
  uint2* qr = q + static_cast<size_t>(row) * vec_per_row;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = j * 256 + threadIdx.x;
    if (i < vec_per_row) {
      const uint32_t xv[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
      uint2 o;
      o.x = pack_e4m3x4(quant_div_fast(bf16lo(xv[0]), sf, inv), quant_div_fast(bf16hi(xv[0]), sf, inv),
                        quant_div_fast(bf16lo(xv[1]), sf, inv), quant_div_fast(bf16hi(xv[1]), sf, inv));
      o.y = pack_e4m3x4(quant_div_fast(bf16lo(xv[2]), sf, inv), quant_div_fast(bf16hi(xv[2]), sf, inv),
                        quant_div_fast(bf16lo(xv[3]), sf, inv), quant_div_fast(bf16hi(xv[3]), sf, inv));
      qr[i] = o;
    }
  }
  if (threadIdx.x == 0) scale[row] = s;
}

// ---------------------------------------------------------------------------
// host-side dispatch
// ---------------------------------------------------------------------------
template <bool NORM, bool RESID, bool QUANT>
static int launch_rows(const void* x, void* resid, const void* w, float eps, void* q, float* scale, void* y,
                       int rows, int hidden, cudaStream_t stream) {
  if (rows == 0) return FR_OK;
  const uint4* xp = static_cast<const uint4*>(x);
  uint4* rp = static_cast<uint4*>(resid);
  const uint4* wp = static_cast<const uint4*>(w);
  uint2* qp = static_cast<uint2*>(q);
  uint4* yp = static_cast<uint4*>(y);
  const int grid_w = ceil_div(rows, kWarpsPerCta);
  switch (hidden) {
    case 1024:
      row_warp_kernel<4, NORM, RESID, QUANT><<<grid_w, kWarpsPerCta * 32, 0, stream>>>(xp, rp, wp, eps, qp, scale, yp, rows);
      return launch_status();
    case 2048:
      row_warp_kernel<8, NORM, RESID, QUANT><<<grid_w, kWarpsPerCta * 32, 0, stream>>>(xp, rp, wp, eps, qp, scale, yp, rows);
      return launch_status();
    case 4096:
      row_warp_kernel<16, NORM, RESID, QUANT><<<grid_w, kWarpsPerCta * 32, 0, stream>>>(xp, rp, wp, eps, qp, scale, yp, rows);
      return launch_status();
    default:
      break;
  }
  const size_t smem = static_cast<size_t>(hidden) * 2;
  FR_CHECK_SUPPORTED(smem <= 200 * 1024);
  auto kern = row_block_kernel<NORM, RESID, QUANT>;
  if (smem > 40 * 1024) {  // leave room for the kernel's static shared memory
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return FR_ERR_CUDA;
  }
  kern<<<rows, kBlockRowThreads, smem, stream>>>(xp, rp, wp, eps, qp, scale, yp, hidden);
  return launch_status();
}

}  // namespace fr

using namespace fr;

extern "C" int fr_rms_quant_fp8(const void* x, void* residual, const void* weight, float eps, void* q_out,
                                float* scale_out, int rows, int hidden, cudaStream_t stream) {
  FR_CHECK_ARG(rows >= 0 && hidden > 0 && hidden % 8 == 0);
  if (rows == 0) return FR_OK;
  FR_CHECK_ARG(x && weight && q_out && scale_out);
  FR_CHECK_ARG(aligned16(x) && aligned16(weight) && aligned16(q_out) && (!residual || aligned16(residual)));
  if (residual) return launch_rows<true, true, true>(x, residual, weight, eps, q_out, scale_out, nullptr, rows, hidden, stream);
  return launch_rows<true, false, true>(x, nullptr, weight, eps, q_out, scale_out, nullptr, rows, hidden, stream);
}

extern "C" int fr_rmsnorm_bf16(const void* x, void* residual, const void* weight, float eps, void* y_out, int rows,
                               int hidden, cudaStream_t stream) {
  FR_CHECK_ARG(rows >= 0 && hidden > 0 && hidden % 8 == 0);
  if (rows == 0) return FR_OK;
  FR_CHECK_ARG(x && weight && y_out);
  FR_CHECK_ARG(aligned16(x) && aligned16(weight) && aligned16(y_out) && (!residual || aligned16(residual)));
  if (residual) return launch_rows<true, true, false>(x, residual, weight, eps, nullptr, nullptr, y_out, rows, hidden, stream);
  return launch_rows<true, false, false>(x, nullptr, weight, eps, nullptr, nullptr, y_out, rows, hidden, stream);
}

extern "C" int fr_token_quant_fp8(const void* x, int x_is_f32, void* q_out, float* scale_out, int rows, int hidden,
                                  cudaStream_t stream) {
  FR_CHECK_ARG(rows >= 0 && hidden > 0);
  if (rows == 0) return FR_OK;
  FR_CHECK_ARG(x && q_out && scale_out && aligned16(x) && aligned16(q_out));
  if (x_is_f32) {
    FR_CHECK_ARG(hidden % 4 == 0);
    row_quant_f32_kernel<<<rows, kBlockRowThreads, 0, stream>>>(static_cast<const float4*>(x),
                                                               static_cast<uint32_t*>(q_out), scale_out, hidden);
    return launch_status();
  }
  FR_CHECK_ARG(hidden % 8 == 0);
  return launch_rows<false, false, true>(x, nullptr, nullptr, 0.f, q_out, scale_out, nullptr, rows, hidden, stream);
}

template <bool QUANT>
static int launch_silu(const void* x, void* q, float* scale, void* y, int rows, int d, cudaStream_t stream) {
  const uint4* xp = static_cast<const uint4*>(x);
  uint2* qp = static_cast<uint2*>(q);
  uint4* yp = static_cast<uint4*>(y);
  const int nv = ceil_div(d >> 3, kBlockRowThreads);
  const uint16_t* table = silu_table_ptr(stream);
  if (!table) return FR_ERR_CUDA;
  switch (nv) {
    case 1: silu_mul_kernel<1, QUANT><<<rows, kBlockRowThreads, 0, stream>>>(xp, qp, scale, yp, d, table); break;
    case 2: silu_mul_kernel<2, QUANT><<<rows, kBlockRowThreads, 0, stream>>>(xp, qp, scale, yp, d, table); break;
    case 3: silu_mul_kernel<3, QUANT><<<rows, kBlockRowThreads, 0, stream>>>(xp, qp, scale, yp, d, table); break;
    case 4: silu_mul_kernel<4, QUANT><<<rows, kBlockRowThreads, 0, stream>>>(xp, qp, scale, yp, d, table); break;
    case 5: case 6: silu_mul_kernel<6, QUANT><<<rows, kBlockRowThreads, 0, stream>>>(xp, qp, scale, yp, d, table); break;
    case 7: case 8: silu_mul_kernel<8, QUANT><<<rows, kBlockRowThreads, 0, stream>>>(xp, qp, scale, yp, d, table); break;
    default: return FR_ERR_UNSUPPORTED;  // d > 16384
  }
  return launch_status();
}

extern "C" int fr_silu_mul_quant_fp8(const void* x, void* q_out, float* scale_out, int rows, int d,
                                     cudaStream_t stream) {
  FR_CHECK_ARG(rows >= 0 && d > 0 && d % 8 == 0);
  if (rows == 0) return FR_OK;
  FR_CHECK_ARG(x && q_out && scale_out && aligned16(x) && aligned16(q_out));
  return launch_silu<true>(x, q_out, scale_out, nullptr, rows, d, stream);
}

extern "C" int fr_silu_mul_bf16(const void* x, void* y_out, int rows, int d, cudaStream_t stream) {
  FR_CHECK_ARG(rows >= 0 && d > 0 && d % 8 == 0);
  if (rows == 0) return FR_OK;
  FR_CHECK_ARG(x && y_out && aligned16(x) && aligned16(y_out));
  return launch_silu<false>(x, nullptr, nullptr, y_out, rows, d, stream);
}

extern "C" int fr_quant_known_amax_fp8(const void* y, const float* row_amax, void* q_out, float* scale_out, int rows,
                                       int d, cudaStream_t stream) {
  FR_CHECK_ARG(rows >= 0 && d > 0 && d % 8 == 0);
  if (rows == 0) return FR_OK;
  FR_CHECK_ARG(y && row_amax && q_out && scale_out && aligned16(y) && aligned16(q_out));
  const uint4* yp = static_cast<const uint4*>(y);
  uint2* qp = static_cast<uint2*>(q_out);
  const int vec = d / 8;
  switch (ceil_div(vec, 256)) {
    case 1: quant_known_amax_kernel<1><<<rows, 256, 0, stream>>>(yp, row_amax, qp, scale_out, vec); break;
    case 2: quant_known_amax_kernel<2><<<rows, 256, 0, stream>>>(yp, row_amax, qp, scale_out, vec); break;
    case 3: quant_known_amax_kernel<3><<<rows, 256, 0, stream>>>(yp, row_amax, qp, scale_out, vec); break;
    case 4: quant_known_amax_kernel<4><<<rows, 256, 0, stream>>>(yp, row_amax, qp, scale_out, vec); break;
    case 5: case 6: case 7: case 8:
      quant_known_amax_kernel<8><<<rows, 256, 0, stream>>>(yp, row_amax, qp, scale_out, vec); break;
    default: return FR_ERR_UNSUPPORTED;  // d > 16384
  }
  return launch_status();
}
