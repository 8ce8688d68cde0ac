// Decode attention over the e4m3 KV pool, page size 1 (one slot per token):
//
//     out[r, h, :] = softmax(q[r, h, :] . K[idx_r, h / G, :]^T * sm_scale) . V[idx_r, h / G, :]
//
// with idx_r = indices[indptr[r] : indptr[r+1]] and G = Hq / Hkv. Stands in for
// AttentionBackend.forward's decode branch (attention/flashinfer.py:212-238,
// FlashInfer BatchDecodeWithPagedKVCacheWrapper with page_size 1, NHD layout,
// no positional encoding, scale head_dim^-0.5, :245-260) and its SDPA
// restatement (attention/flashinfer.py:380-431).
//
// Beam-search structure exploited here: the rows (beams) of one request all
// start with the request's prompt slots and differ only in a few trailing decode
// slots. Rows are therefore handed over in GROUPS; fr_decode_attn_plan finds, on
// the device, the longest slot prefix common to every row of a group. For that
// shared prefix one CTA treats (beams x G query heads) of one KV head as the M
// dimension of a tensor-core contraction against K/V tiles that are read ONCE
// per CTA (mma.sync m16n8k16 bf16, e4m3 K/V widened to bf16 while staging to
// shared memory, fp32 online softmax). The per-row tail (<= a handful of slots)
// is folded in afterwards with scalar FMAs on the same accumulators. A row that
// shares nothing simply has everything in its tail, so any slot list is valid
// input.
#include "fr_common.cuh"

namespace fr {
namespace attn {

constexpr int kD = 128;
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kQPerCta = kWarps * 16;  // query vectors (beam x head-in-group) per CTA
constexpr int kTileN = 64;             // KV tokens per tile
constexpr int kRowPad = kD + 8;        // bf16 elements per staged K/V row (272 B: conflict-free ldmatrix)

struct Params {
  const __nv_bfloat16* q;
  int64_t q_t, q_h;
  const uint8_t* kc;
  const uint8_t* vc;
  int64_t ck_s, ck_h, cv_s, cv_h;
  const int32_t* indptr;
  const int32_t* indices;
  const int32_t* group_rows;
  const int32_t* shared_len;
  __nv_bfloat16* out;
  int64_t o_t;
  int n_rows, n_groups, hq, hkv, num_slots;
  float scale_log2;  // sm_scale * log2(e)
};

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// 16 e4m3 bytes -> 16 bf16 (exact), written as two 16-byte shared stores.
__device__ __forceinline__ void widen16(const uint4& in, __nv_bfloat16* dst) {
  const uint32_t w[4] = {in.x, in.y, in.z, in.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] & 0xffffu), __NV_E4M3);
    __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] >> 16), __NV_E4M3);
    float2 f01 = __half22float2(*reinterpret_cast<__half2*>(&h01));
    float2 f23 = __half22float2(*reinterpret_cast<__half2*>(&h23));
    o[2 * i] = pack_bf16(f01.x, f01.y);
    o[2 * i + 1] = pack_bf16(f23.x, f23.y);
  }
  uint4* d4 = reinterpret_cast<uint4*>(dst);
  d4[0] = make_uint4(o[0], o[1], o[2], o[3]);
  d4[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t v) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(v), __NV_E4M3);
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}

template <int G>
__global__ void __launch_bounds__(kThreads) decode_attn_kernel(Params p) {
  __shared__ __align__(16) __nv_bfloat16 Ks[kTileN * kRowPad];
  __shared__ __align__(16) __nv_bfloat16 Vs[kTileN * kRowPad];
  __shared__ int32_t slot_s[kTileN];

  constexpr int kBeamsPerCta = kQPerCta / G;
  const int grp = blockIdx.z;
  const int kvh = blockIdx.y;
  const int row0 = p.group_rows[grp];
  const int rows_in_group = p.group_rows[grp + 1] - row0;
  const int beam0 = blockIdx.x * kBeamsPerCta;
  if (beam0 >= rows_in_group) return;
  const int ls = p.shared_len[grp];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  // the two query vectors (fragment rows g and g+8) this thread co-owns
  int qrow[2], qhead[2];
  bool qlive[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int qv = warp * 16 + g + 8 * half;
    const int beam = beam0 + qv / G;
    qlive[half] = beam < rows_in_group;
    qrow[half] = row0 + (qlive[half] ? beam : 0);
    qhead[half] = kvh * G + qv % G;
  }

  // Q as mma A fragments: qa[ks][0..3] for the 16-wide k-step ks
  uint32_t qa[kD / 16][4];
#pragma unroll
  for (int ks = 0; ks < kD / 16; ++ks) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const __nv_bfloat16* qp = p.q + qrow[half] * p.q_t + qhead[half] * p.q_h + ks * 16 + 2 * t;
      uint32_t v0 = 0, v1 = 0;
      if (qlive[half]) {
        v0 = *reinterpret_cast<const uint32_t*>(qp);
        v1 = *reinterpret_cast<const uint32_t*>(qp + 8);
      }
      qa[ks][half] = v0;
      qa[ks][2 + half] = v1;
    }
  }

  float o[kD / 8][4];
#pragma unroll
  for (int i = 0; i < kD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  const int32_t* shared_idx = p.indices + p.indptr[row0];  // first row's list holds the shared prefix

  for (int n0 = 0; n0 < ls; n0 += kTileN) {
    const int ntok = min(kTileN, ls - n0);
    __syncthreads();  // previous tile fully consumed
    if (threadIdx.x < kTileN) {
      int32_t s = threadIdx.x < ntok ? shared_idx[n0 + threadIdx.x] : 0;
      s = s < 0 ? 0 : (s >= p.num_slots ? p.num_slots - 1 : s);
      slot_s[threadIdx.x] = s;
    }
    __syncthreads();
    // stage K and V: 8 chunks of 16 bytes per token, chunk index fastest across lanes
    for (int i = threadIdx.x; i < kTileN * 8; i += kThreads) {
      const int tok = i >> 3, ch = i & 7;
      uint4 kraw = make_uint4(0, 0, 0, 0), vraw = make_uint4(0, 0, 0, 0);
      if (tok < ntok) {
        const int64_t s = slot_s[tok];
        kraw = __ldg(reinterpret_cast<const uint4*>(p.kc + s * p.ck_s + kvh * p.ck_h + ch * 16));
        vraw = __ldg(reinterpret_cast<const uint4*>(p.vc + s * p.cv_s + kvh * p.cv_h + ch * 16));
      }
      widen16(kraw, Ks + tok * kRowPad + ch * 16);
      widen16(vraw, Vs + tok * kRowPad + ch * 16);
    }
    __syncthreads();

    // S = Q K^T for this warp's 16 query vectors x 64 tokens
    float s_acc[kTileN / 8][4];
#pragma unroll
    for (int j = 0; j < kTileN / 8; ++j) s_acc[j][0] = s_acc[j][1] = s_acc[j][2] = s_acc[j][3] = 0.f;
    const uint32_t ks_base = static_cast<uint32_t>(__cvta_generic_to_shared(Ks));
    const uint32_t vs_base = static_cast<uint32_t>(__cvta_generic_to_shared(Vs));
#pragma unroll
    for (int j = 0; j < kTileN / 8; ++j) {
#pragma unroll
      for (int kp = 0; kp < kD / 32; ++kp) {
        // four 8x8 matrices: (tokens 8j.., dims 32kp + 0 / 8 / 16 / 24)
        uint32_t b[4];
        const int mrow = 8 * j + (lane & 7);
        const int mcol = 32 * kp + 8 * (lane >> 3);
        ldmatrix_x4(b, ks_base + (mrow * kRowPad + mcol) * 2);
        mma_bf16_16816(s_acc[j], qa[2 * kp], b[0], b[1]);
        mma_bf16_16816(s_acc[j], qa[2 * kp + 1], b[2], b[3]);
      }
    }
    // scale, mask the ragged end of the last tile, online softmax
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < kTileN / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = 8 * j + 2 * t + (e & 1);
        float v = s_acc[j][e] * p.scale_log2;
        if (col >= ntok) v = -INFINITY;
        s_acc[j][e] = v;
        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
      }
    }
    float corr[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float mx = tile_max[half];
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[half], mx);  // finite: every tile has >= 1 live token
      corr[half] = exp2f(m_run[half] - m_new);
      m_run[half] = m_new;
      l_run[half] *= corr[half];
    }
#pragma unroll
    for (int i = 0; i < kD / 8; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0];
      o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    uint32_t pa[kTileN / 16][4];
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < kTileN / 8; ++j) {
      const float p0 = exp2f(s_acc[j][0] - m_run[0]);
      const float p1 = exp2f(s_acc[j][1] - m_run[0]);
      const float p2 = exp2f(s_acc[j][2] - m_run[1]);
      const float p3 = exp2f(s_acc[j][3] - m_run[1]);
      // the bf16-rounded probabilities feed both the row sum and P.V
      const uint32_t lo = pack_bf16(p0, p1), hi = pack_bf16(p2, p3);
      psum[0] += bf16lo(lo) + bf16hi(lo);
      psum[1] += bf16lo(hi) + bf16hi(hi);
      pa[j >> 1][(j & 1) * 2 + 0] = lo;
      pa[j >> 1][(j & 1) * 2 + 1] = hi;
    }
    l_run[0] += psum[0];
    l_run[1] += psum[1];
    // O += P V
#pragma unroll
    for (int kk = 0; kk < kTileN / 16; ++kk) {
#pragma unroll
      for (int dn = 0; dn < kD / 16; ++dn) {
        // four 8x8 matrices: (tokens 16kk + 0 / 8, dims 16dn + 0 / 8), transposed on load
        uint32_t b[4];
        const int mrow = 16 * kk + (lane & 7) + 8 * ((lane >> 3) & 1);
        const int mcol = 16 * dn + 8 * (lane >> 4);
        ldmatrix_x4_trans(b, vs_base + (mrow * kRowPad + mcol) * 2);
        mma_bf16_16816(o[2 * dn], pa[kk], b[0], b[1]);
        mma_bf16_16816(o[2 * dn + 1], pa[kk], b[2], b[3]);
      }
    }
  }

  // ---- per-row tails (slots after the shared prefix), scalar path --------
  // Trip counts differ between quads, so the shuffles name only the four lanes
  // of this quad (which share a row and hence a trip count).
  const uint32_t qmask = 0xfu << (lane & ~3);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int beg = p.indptr[qrow[half]] + ls;
    const int end = qlive[half] ? p.indptr[qrow[half] + 1] : beg;
    for (int i = beg; i < end; ++i) {
      int64_t s = p.indices[i];
      s = s < 0 ? 0 : (s >= p.num_slots ? p.num_slots - 1 : s);
      const uint8_t* kp = p.kc + s * p.ck_s + kvh * p.ck_h;
      float dot = 0.f;
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks) {
        const float2 k0 = e4m3x2_to_float2(*reinterpret_cast<const uint16_t*>(kp + ks * 16 + 2 * t));
        const float2 k1 = e4m3x2_to_float2(*reinterpret_cast<const uint16_t*>(kp + ks * 16 + 8 + 2 * t));
        const uint32_t q0 = qa[ks][half], q1 = qa[ks][2 + half];
        dot += bf16lo(q0) * k0.x + bf16hi(q0) * k0.y + bf16lo(q1) * k1.x + bf16hi(q1) * k1.y;
      }
      dot += __shfl_xor_sync(qmask, dot, 1);
      dot += __shfl_xor_sync(qmask, dot, 2);
      const float sc = dot * p.scale_log2;
      const float m_new = fmaxf(m_run[half], sc);
      const float c = exp2f(m_run[half] - m_new);
      const float pr = exp2f(sc - m_new);
      m_run[half] = m_new;
      l_run[half] = l_run[half] * c + (t == 0 ? pr : 0.f);
      const uint8_t* vp = p.vc + s * p.cv_s + kvh * p.cv_h;
#pragma unroll
      for (int dn = 0; dn < kD / 8; ++dn) {
        const float2 vv = e4m3x2_to_float2(*reinterpret_cast<const uint16_t*>(vp + dn * 8 + 2 * t));
        o[dn][2 * half] = o[dn][2 * half] * c + pr * vv.x;
        o[dn][2 * half + 1] = o[dn][2 * half + 1] * c + pr * vv.y;
      }
    }
  }
  // ---- normalise and store -----------------------------------------------
  // l_run holds per-lane partial row sums (each lane saw its own columns of the
  // shared tiles; tail terms were added on lane t == 0 only): add up the quad.
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 1);
    l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 2);
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    if (!qlive[half]) continue;
    const float inv = l_run[half] > 0.f ? 1.0f / l_run[half] : 0.f;
    __nv_bfloat16* op = p.out + qrow[half] * p.o_t + qhead[half] * kD;
#pragma unroll
    for (int dn = 0; dn < kD / 8; ++dn) {
      *reinterpret_cast<uint32_t*>(op + dn * 8 + 2 * t) =
          pack_bf16(o[dn][2 * half] * inv, o[dn][2 * half + 1] * inv);
    }
  }
}

// Longest slot prefix shared by all rows of each group. grid = (row chunks, groups):
// every CTA compares its chunk of rows with the group's first row and lowers
// out[group] with an atomicMin (out is pre-set to the first row's length).
constexpr int kPlanRowsPerCta = 32;

__global__ void plan_init_kernel(const int32_t* __restrict__ indptr, const int32_t* __restrict__ group_rows,
                                 int32_t* __restrict__ out, int n_groups) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n_groups) return;
  const int row0 = group_rows[g], row1 = group_rows[g + 1];
  out[g] = row1 > row0 ? indptr[row0 + 1] - indptr[row0] : 0;
}

__global__ void __launch_bounds__(256) plan_kernel(const int32_t* __restrict__ indptr,
                                                  const int32_t* __restrict__ indices,
                                                  const int32_t* __restrict__ group_rows, int32_t* __restrict__ out) {
  const int grp = blockIdx.y;
  const int row0 = group_rows[grp], row1 = group_rows[grp + 1];
  const int first = row0 + 1 + blockIdx.x * kPlanRowsPerCta;
  if (first >= row1) return;
  const int last = min(first + kPlanRowsPerCta, row1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int32_t* ref = indices + indptr[row0];
  const int ref_len = indptr[row0 + 1] - indptr[row0];
  for (int r = first + warp; r < last; r += 8) {
    const int32_t* cur = indices + indptr[r];
    const int len = min(ref_len, indptr[r + 1] - indptr[r]);
    int lcp = len;
    for (int i = 0; i < len; i += 32) {
      const bool diff = (i + lane < len) && (cur[i + lane] != ref[i + lane]);
      const uint32_t bal = __ballot_sync(0xffffffffu, diff);
      if (bal) { lcp = i + __ffs(bal) - 1; break; }
    }
    if (lane == 0) atomicMin(out + grp, lcp);
  }
}

}  // namespace attn

int decode_attn_tc(const void* q, int64_t q_t, int64_t q_h, const void* k_cache, const void* v_cache, int64_t ck_s,
                   int64_t ck_h, int64_t cv_s, int64_t cv_h, const int32_t* indptr, const int32_t* indices,
                   const int32_t* group_rows, const int32_t* shared_len, void* out, int64_t o_t, int n_rows,
                   int n_groups, int hq, int hkv, int max_group_rows, int num_slots, float sm_scale, void* scratch,
                   int lcap, const int32_t* prepared_len, cudaStream_t stream);  // attn_tc.cu
}  // namespace fr

using namespace fr;

extern "C" int fr_decode_attn_plan(const int32_t* indptr, const int32_t* indices, const int32_t* group_rows,
                                   int n_groups, int max_group_rows, int32_t* shared_len_out, cudaStream_t stream) {
  FR_CHECK_ARG(n_groups >= 0);
  if (n_groups == 0) return FR_OK;
  FR_CHECK_ARG(indptr && indices && group_rows && shared_len_out);
  attn::plan_init_kernel<<<ceil_div(n_groups, 128), 128, 0, stream>>>(indptr, group_rows, shared_len_out, n_groups);
  if (launch_status() != FR_OK) return FR_ERR_CUDA;
  if (max_group_rows <= 1) return FR_OK;
  dim3 grid(ceil_div(max_group_rows - 1, attn::kPlanRowsPerCta), n_groups);
  attn::plan_kernel<<<grid, 256, 0, stream>>>(indptr, indices, group_rows, shared_len_out);
  return launch_status();
}

extern "C" int64_t fr_decode_attn_scratch_bytes(int n_groups, int hkv, int max_shared_len) {
  if (n_groups <= 0 || hkv <= 0 || max_shared_len <= 0) return 0;
  const int64_t lcap = (static_cast<int64_t>(max_shared_len) + 63) / 64 * 64;
  return static_cast<int64_t>(n_groups) * hkv * lcap * attn::kD * 2 /* bf16 */ * 2 /* K and V^T */;
}

static int decode_attn_entry(const void* q, int64_t q_t, int64_t q_h, const void* k_cache, const void* v_cache,
                             int64_t ck_s, int64_t ck_h, int64_t cv_s, int64_t cv_h, const int32_t* indptr,
                             const int32_t* indices, const int32_t* group_rows, const int32_t* shared_len, void* out,
                             int64_t o_t, int n_rows, int n_groups, int hq, int hkv, int head_dim, int max_group_rows,
                             int num_slots, float sm_scale, void* scratch, int64_t scratch_bytes, int max_shared_len,
                             const int32_t* prepared_len, cudaStream_t stream) {
  FR_CHECK_ARG(n_rows >= 0 && n_groups >= 0 && hq > 0 && hkv > 0 && max_group_rows >= 0 && num_slots > 0);
  if (n_rows == 0 || n_groups == 0 || max_group_rows == 0) return FR_OK;
  FR_CHECK_ARG(q && k_cache && v_cache && indptr && indices && group_rows && shared_len && out);
  FR_CHECK_SUPPORTED(head_dim == attn::kD && hq % hkv == 0);
  const int G = hq / hkv;
  FR_CHECK_SUPPORTED(G == 1 || G == 2 || G == 4 || G == 8);
  FR_CHECK_ARG((reinterpret_cast<uintptr_t>(q) & 3u) == 0 && q_t % 2 == 0 && q_h % 2 == 0);
  FR_CHECK_ARG(aligned16(k_cache) && aligned16(v_cache) && ck_s % 16 == 0 && ck_h % 16 == 0 && cv_s % 16 == 0 &&
               cv_h % 16 == 0);
  FR_CHECK_ARG((reinterpret_cast<uintptr_t>(out) & 3u) == 0 && o_t % 2 == 0);
  if (scratch != nullptr && max_shared_len > 0) {
    // tensor-core path: the shared prefix of every group is widened once into the scratch buffer
    const int lcap = (max_shared_len + 63) / 64 * 64;
    FR_CHECK_ARG(scratch_bytes >= fr_decode_attn_scratch_bytes(n_groups, hkv, max_shared_len));
    return decode_attn_tc(q, q_t, q_h, k_cache, v_cache, ck_s, ck_h, cv_s, cv_h, indptr, indices, group_rows,
                          shared_len, out, o_t, n_rows, n_groups, hq, hkv, max_group_rows, num_slots, sm_scale,
                          scratch, lcap, prepared_len, stream);
  }
  attn::Params p{static_cast<const __nv_bfloat16*>(q), q_t, q_h, static_cast<const uint8_t*>(k_cache),
                 static_cast<const uint8_t*>(v_cache), ck_s, ck_h, cv_s, cv_h, indptr, indices, group_rows,
                 shared_len, static_cast<__nv_bfloat16*>(out), o_t, n_rows, n_groups, hq, hkv, num_slots,
                 sm_scale * 1.4426950408889634f};
  const int beams_per_cta = attn::kQPerCta / G;
  dim3 grid(ceil_div(max_group_rows, beams_per_cta), hkv, n_groups);
  switch (G) {
    case 1: attn::decode_attn_kernel<1><<<grid, attn::kThreads, 0, stream>>>(p); break;
    case 2: attn::decode_attn_kernel<2><<<grid, attn::kThreads, 0, stream>>>(p); break;
    case 4: attn::decode_attn_kernel<4><<<grid, attn::kThreads, 0, stream>>>(p); break;
    case 8: attn::decode_attn_kernel<8><<<grid, attn::kThreads, 0, stream>>>(p); break;
    default: return FR_ERR_UNSUPPORTED;
  }
  return launch_status();
}

extern "C" int fr_decode_attn_fp8(const void* q, int64_t q_t, int64_t q_h, const void* k_cache, const void* v_cache,
                                  int64_t ck_s, int64_t ck_h, int64_t cv_s, int64_t cv_h, const int32_t* indptr,
                                  const int32_t* indices, const int32_t* group_rows, const int32_t* shared_len,
                                  void* out, int64_t o_t, int n_rows, int n_groups, int hq, int hkv, int head_dim,
                                  int max_group_rows, int num_slots, float sm_scale, void* scratch,
                                  int64_t scratch_bytes, int max_shared_len, cudaStream_t stream) {
  return decode_attn_entry(q, q_t, q_h, k_cache, v_cache, ck_s, ck_h, cv_s, cv_h, indptr, indices, group_rows,
                           shared_len, out, o_t, n_rows, n_groups, hq, hkv, head_dim, max_group_rows, num_slots,
                           sm_scale, scratch, scratch_bytes, max_shared_len, nullptr, stream);
}

extern "C" int fr_decode_attn_reuse_fp8(const void* q, int64_t q_t, int64_t q_h, const void* k_cache,
                                        const void* v_cache, int64_t ck_s, int64_t ck_h, int64_t cv_s, int64_t cv_h,
                                        const int32_t* indptr, const int32_t* indices, const int32_t* group_rows,
                                        const int32_t* shared_len, void* out, int64_t o_t, int n_rows, int n_groups,
                                        int hq, int hkv, int head_dim, int max_group_rows, int num_slots,
                                        float sm_scale, void* scratch, int64_t scratch_bytes, int max_shared_len,
                                        const int32_t* prepared_len, cudaStream_t stream) {
  FR_CHECK_ARG(scratch != nullptr && max_shared_len > 0 && prepared_len != nullptr);
  return decode_attn_entry(q, q_t, q_h, k_cache, v_cache, ck_s, ck_h, cv_s, cv_h, indptr, indices, group_rows,
                           shared_len, out, o_t, n_rows, n_groups, hq, hkv, head_dim, max_group_rows, num_slots,
                           sm_scale, scratch, scratch_bytes, max_shared_len, prepared_len, stream);
}
