// Row-wise pieces of the SID lm_head that sit between the FP8 logits GEMM and
// the beam step:
//
//   fr_logsumexp_rows      max and log-sum-exp of each fp32 logits row, optionally
//                          the full log-softmax (F.log_softmax in
//                          RestrictedLMHead._restricted_logprobs / compute_level,
//                          logits.py:118-138)
//   fr_topk_rows           per-row sorted top-k, the candidate pre-selection of the
//                          reference's expand path (torch.topk in
//                          scheduler/scheduler.py:1476-1482, engine/graph.py:185-194)
//   fr_lse_combine_shards  merges per-shard row statistics when the level's token
//                          range is split over GPUs
//
// log-prob convention everywhere: lp = (x - max) - log(sum exp(x - max)), the
// order of operations of a fused CPU log_softmax.
#include "fr_common.cuh"
#include "sid_head.cuh"
#include "topk_select.cuh"

namespace fr {
namespace head {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
logsumexp_kernel(const float* __restrict__ x, int64_t ld, float* __restrict__ row_max, float* __restrict__ row_logsum,
                 float* __restrict__ lp_out, int64_t ldo, int cols) {
  __shared__ float red[kThreads / 32];
  const int row = blockIdx.x;
  const float* xr = x + static_cast<int64_t>(row) * ld;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < cols; i += kThreads) mx = fmaxf(mx, xr[i]);
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
  for (int i = 1; i < kThreads / 32; ++i) mx = fmaxf(mx, red[i]);
  __syncthreads();
  float sum = 0.f;
  for (int i = threadIdx.x; i < cols; i += kThreads) sum += expf(xr[i] - mx);
  sum = warp_sum(sum);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = 0.f;
  for (int i = 0; i < kThreads / 32; ++i) sum += red[i];
  const float ls = logf(sum);
  if (threadIdx.x == 0) {
    row_max[row] = mx;
    row_logsum[row] = ls;
  }
  if (lp_out) {
    float* o = lp_out + static_cast<int64_t>(row) * ldo;
    for (int i = threadIdx.x; i < cols; i += kThreads) o[i] = __fsub_rn(__fsub_rn(xr[i], mx), ls);
  }
}

// The same statistics for rows that fit the CTA's registers (cols <= 1024 * VPT, cols and ld multiples of 4,
// 16-byte aligned rows): one pass over HBM with 16-byte loads, the row kept in registers between the maximum,
// the sum and the optional log-prob write. Same arithmetic per element as logsumexp_kernel; the sum's order
// differs (it is only compared within a tolerance anywhere).
template <int VPT>
__global__ void __launch_bounds__(kThreads)
logsumexp_vec_kernel(const float* __restrict__ x, int64_t ld, float* __restrict__ row_max, float* __restrict__ row_logsum,
                     float* __restrict__ lp_out, int64_t ldo, int cols) {
  __shared__ float red[kThreads / 32];
  const int row = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + static_cast<int64_t>(row) * ld);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = cols >> 2;
  float4 v[VPT];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * kThreads;
    v[i] = idx < nvec ? __ldg(xr + idx) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    mx = fmaxf(mx, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
  }
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int i = 1; i < kThreads / 32; ++i) mx = fmaxf(mx, red[i]);
  __syncthreads();
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    sum += (expf(v[i].x - mx) + expf(v[i].y - mx)) + (expf(v[i].z - mx) + expf(v[i].w - mx));  // exp(-inf) = 0
  sum = warp_sum(sum);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = 0.f;
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) sum += red[i];
  const float ls = logf(sum);
  if (threadIdx.x == 0) {
    row_max[row] = mx;
    row_logsum[row] = ls;
  }
  if (lp_out) {
    float4* o = reinterpret_cast<float4*>(lp_out + static_cast<int64_t>(row) * ldo);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * kThreads;
      if (idx < nvec)
        o[idx] = make_float4(__fsub_rn(__fsub_rn(v[i].x, mx), ls), __fsub_rn(__fsub_rn(v[i].y, mx), ls),
                             __fsub_rn(__fsub_rn(v[i].z, mx), ls), __fsub_rn(__fsub_rn(v[i].w, mx), ls));
    }
  }
}

__global__ void __launch_bounds__(kThreads)
topk_rows_kernel(const float* __restrict__ x, int64_t ld, const float* __restrict__ row_max,
                 const float* __restrict__ row_logsum, float* __restrict__ vals, int64_t* __restrict__ idx, int cols,
                 int k, int kp2) {
  extern __shared__ __align__(16) uint8_t dyn[];
  __shared__ topk::SelectSmem sm;
  uint64_t* win = reinterpret_cast<uint64_t*>(dyn);        // [kp2]
  float* v = reinterpret_cast<float*>(win + kp2);          // [cols]
  const int row = blockIdx.x;
  const float* xr = x + static_cast<int64_t>(row) * ld;
  const bool xf = row_max != nullptr && row_logsum != nullptr;
  const float mx = xf ? row_max[row] : 0.f, ls = xf ? row_logsum[row] : 0.f;
  for (int i = threadIdx.x; i < cols; i += kThreads) {
    const float t = xr[i];
    v[i] = xf ? __fsub_rn(__fsub_rn(t, mx), ls) : t;
  }
  __syncthreads();
  const int nvalid = topk::radix_select_topk<kThreads>(
      [&](auto&& f) {
        for (int i = threadIdx.x; i < cols; i += kThreads) f(topk::compose(v[i], static_cast<uint32_t>(i)));
      },
      k, win, kp2, sm);
  for (int j = threadIdx.x; j < k; j += kThreads) {
    const size_t o = static_cast<size_t>(row) * k + j;
    if (j < nvalid) {
      vals[o] = topk::composite_score(win[j]);
      idx[o] = static_cast<int64_t>(topk::composite_index(win[j]));
    } else {
      vals[o] = -INFINITY;
      idx[o] = 0;
    }
  }
}

__global__ void lse_combine_kernel(const float* __restrict__ smax, const float* __restrict__ slog,
                                   float* __restrict__ row_max, float* __restrict__ row_logsum, int S, int rows,
                                   int64_t stride) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float mx, ls;
  lse_combine(smax + r, slog + r, S, stride, mx, ls);
  row_max[r] = mx;
  row_logsum[r] = ls;
}

}  // namespace head
}  // namespace fr

using namespace fr;

extern "C" int fr_logsumexp_rows(const float* logits, int64_t ld, float* row_max, float* row_logsum,
                                 float* logprobs_out, int64_t ldo, int rows, int cols, cudaStream_t stream) {
  FR_CHECK_ARG(rows >= 0 && cols > 0 && ld >= cols);
  if (rows == 0) return FR_OK;
  FR_CHECK_ARG(logits && row_max && row_logsum && (!logprobs_out || ldo >= cols));
  const bool vec = cols % 4 == 0 && ld % 4 == 0 && aligned16(logits) && cols <= 8 * 1024 &&
                   (!logprobs_out || (ldo % 4 == 0 && aligned16(logprobs_out)));
  if (vec) {
    const int vpt = ceil_div(cols, 4 * head::kThreads);
#define FR_LSE_CASE(V)                                                                                              \
  head::logsumexp_vec_kernel<V><<<rows, head::kThreads, 0, stream>>>(logits, ld, row_max, row_logsum, logprobs_out, \
                                                                     ldo, cols)
    if (vpt <= 1) FR_LSE_CASE(1);
    else if (vpt <= 2) FR_LSE_CASE(2);
    else if (vpt <= 4) FR_LSE_CASE(4);
    else FR_LSE_CASE(8);
#undef FR_LSE_CASE
    return launch_status();
  }
  head::logsumexp_kernel<<<rows, head::kThreads, 0, stream>>>(logits, ld, row_max, row_logsum, logprobs_out, ldo, cols);
  return launch_status();
}

extern "C" int fr_topk_rows(const float* x, int64_t ld, const float* row_max, const float* row_logsum,
                            float* vals_out, int64_t* idx_out, int rows, int cols, int k, cudaStream_t stream) {
  FR_CHECK_ARG(rows >= 0 && cols > 0 && k > 0 && ld >= cols);
  if (rows == 0) return FR_OK;
  FR_CHECK_ARG(x && vals_out && idx_out);
  FR_CHECK_SUPPORTED(k <= cols && k <= 8192 && cols <= 49152);
  int kp2 = 1;
  while (kp2 < k) kp2 <<= 1;
  const size_t smem = static_cast<size_t>(kp2) * 8 + static_cast<size_t>(cols) * 4;
  FR_CHECK_SUPPORTED(smem <= 200 * 1024);
  if (smem > 32 * 1024) {  // static shared memory of the kernel counts towards the 48 KiB default limit
    if (cudaFuncSetAttribute(head::topk_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return FR_ERR_CUDA;
  }
  head::topk_rows_kernel<<<rows, head::kThreads, smem, stream>>>(x, ld, row_max, row_logsum, vals_out, idx_out, cols,
                                                                 k, kp2);
  return launch_status();
}

extern "C" int fr_lse_combine_shards(const float* shard_max, const float* shard_logsum, float* row_max,
                                     float* row_logsum, int S, int rows, int64_t shard_stride, cudaStream_t stream) {
  FR_CHECK_ARG(S > 0 && rows >= 0 && (shard_stride == 0 || shard_stride >= rows));
  if (rows == 0) return FR_OK;
  FR_CHECK_ARG(shard_max && shard_logsum && row_max && row_logsum);
  head::lse_combine_kernel<<<ceil_div(rows, 256), 256, 0, stream>>>(shard_max, shard_logsum, row_max, row_logsum, S,
                                                                   rows, shard_stride > 0 ? shard_stride : rows);
  return launch_status();
}
