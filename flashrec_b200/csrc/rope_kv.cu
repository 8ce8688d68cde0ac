// Data-movement kernels around the attention of one decode step:
//
//   fr_qk_norm_rope_kv_fp8   per-head RMSNorm of Q and K, NeoX RoPE, Q written
//                            back in place (bf16), K -> bf16 -> e4m3 and V -> e4m3
//                            scattered to their KV-pool slots. Stands in for
//                            fused_qk_norm_rope_store_fp8 (kernel/qk_rope_kv.py:28-250).
//   fr_store_kv_fp8          plain bf16 -> e4m3 scatter of K and V
//                            (TokenToKVPool.store, kvcache/pool.py:121-139).
//   fr_embedding_bf16        token-embedding row gather (models/qwen3.py:266).
//
// All are HBM-bound; a group of D/8 lanes owns one (token, head) pair and moves
// 8 bf16 per lane (4 from each rotary half) with 8-byte accesses.
#include "fr_common.cuh"

namespace fr {

template <int LPH>
__device__ __forceinline__ double group_sum(double v) {
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct RopeArgs {
  __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  int64_t q_t, q_h, k_t, k_h, v_t, v_h;
  const int64_t* pos;
  const int64_t* loc;
  const __nv_bfloat16* qw;
  const __nv_bfloat16* kw;
  float eps;
  const float* cs;
  int max_pos;
  uint8_t* kc;
  uint8_t* vc;
  int64_t ck_s, ck_h, cv_s, cv_h;
  int T, n_q, n_kv, num_slots;
  __nv_bfloat16* k_out;  // NORM == false only: the rotated K is also written back here (bf16, strides k_t / k_h)
};

__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&x)[4]) {
  uint2 u = *reinterpret_cast<const uint2*>(p);
  x[0] = bf16lo(u.x); x[1] = bf16hi(u.x); x[2] = bf16lo(u.y); x[3] = bf16hi(u.y);
}

// ROPE == false: plain conversion of K and V (no norm / rotation), used by fr_store_kv_fp8.
// NORM == false (with ROPE): rotation only, no per-head RMSNorm, K rewritten in place as well as Q
// and the cache writes optional: fr_rope_neox_inplace.
// Each group of D/8 lanes handles HPG consecutive heads of one token; all of their
// loads are issued before any arithmetic. HPG > 1 requires n_q and n_kv to be
// multiples of HPG so that a group never mixes Q, K and V heads.
template <int D, bool ROPE, int HPG, bool NORM = true>
__global__ void __launch_bounds__(256) qk_rope_kv_kernel(RopeArgs a) {
  constexpr int LPH = D / 8;        // lanes per head
  constexpr int GPW = 32 / LPH;     // lane groups per warp
  constexpr int HALF = D / 2;
  const int lane = threadIdx.x & 31;
  const int sub = lane % LPH;
  const int heads_all = a.n_q + 2 * a.n_kv;
  const int groups_per_tok = heads_all / HPG;
  const int64_t item = (static_cast<int64_t>(blockIdx.x) * (256 / 32) + (threadIdx.x >> 5)) * GPW + lane / LPH;
  const bool live = item < static_cast<int64_t>(a.T) * groups_per_tok;
  // dead groups still take part in the shuffles below
  const int t = live ? static_cast<int>(item / groups_per_tok) : 0;
  const int hs0 = live ? static_cast<int>(item % groups_per_tok) * HPG : 0;
  const bool is_q = hs0 < a.n_q;
  const bool is_k = !is_q && hs0 < a.n_q + a.n_kv;
  const int h0 = is_q ? hs0 : (is_k ? hs0 - a.n_q : hs0 - a.n_q - a.n_kv);

  const __nv_bfloat16* src0 = is_q ? (a.q + t * a.q_t + h0 * a.q_h)
                                   : (is_k ? (a.k + t * a.k_t + h0 * a.k_h) : (a.v + t * a.v_t + h0 * a.v_h));
  const int64_t hstride = is_q ? a.q_h : (is_k ? a.k_h : a.v_h);
  const bool rotate = ROPE && (is_q || is_k);
  // The position / slot lookups and the cos / sin row they lead to are independent of the head
  // data: issue them first so that their two dependent round trips overlap the loads of the heads.
  int64_t p = 0, slot = 0;
  if (live && rotate) p = __ldg(a.pos + t);
  if (live && !is_q) slot = __ldg(a.loc + t);
  float lo[HPG][4], hi[HPG][4];
#pragma unroll
  for (int j = 0; j < HPG; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) lo[j][i] = hi[j][i] = 0.f;
    if (live) {
      load4(src0 + j * hstride + 4 * sub, lo[j]);
      load4(src0 + j * hstride + HALF + 4 * sub, hi[j]);
    }
  }
  float cosv[4] = {1.f, 1.f, 1.f, 1.f}, sinv[4] = {0.f, 0.f, 0.f, 0.f};
  float wlo[4] = {0.f, 0.f, 0.f, 0.f}, whi[4] = {0.f, 0.f, 0.f, 0.f};
  if (live && rotate) {
    p = p < 0 ? 0 : (p >= a.max_pos ? a.max_pos - 1 : p);
    const float4 c4 = __ldg(reinterpret_cast<const float4*>(a.cs + p * D + 4 * sub));
    const float4 s4 = __ldg(reinterpret_cast<const float4*>(a.cs + p * D + HALF + 4 * sub));
    cosv[0] = c4.x; cosv[1] = c4.y; cosv[2] = c4.z; cosv[3] = c4.w;
    sinv[0] = s4.x; sinv[1] = s4.y; sinv[2] = s4.z; sinv[3] = s4.w;
    if constexpr (NORM) {
      const __nv_bfloat16* wsrc = is_q ? a.qw : a.kw;
      load4(wsrc + 4 * sub, wlo);
      load4(wsrc + HALF + 4 * sub, whi);
    }
  }
  // sums of squares only where some lane of the warp normalises (Q / K heads); the decision is
  // warp-uniform because all 32 lanes execute the shuffles
  double ss[HPG];
  const bool any_norm = ROPE && NORM && __any_sync(0xffffffffu, live && (is_q || is_k));
#pragma unroll
  for (int j = 0; j < HPG; ++j) {
    ss[j] = 0.0;
    if (any_norm) {
      double acc = 0.0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const double l = static_cast<double>(lo[j][i]), h = static_cast<double>(hi[j][i]);
        acc = fma(l, l, acc);  // the squares are exact (8-bit significands)
        acc = fma(h, h, acc);
      }
      ss[j] = group_sum<LPH>(acc);
    }
  }
  if (!live) return;
  const bool to_cache = a.kc != nullptr && !is_q && slot >= 0 && slot < a.num_slots;  // never write outside the pool
  if (NORM && !is_q && !to_cache) return;
  if (!NORM && !is_q && !is_k && !to_cache) return;  // rotation only: V has work only when it is stored
  if (!ROPE && is_q) return;                         // plain KV store never has Q work
#pragma unroll
  for (int j = 0; j < HPG; ++j) {
    if (rotate) {
      float rstd = 1.f;
      if constexpr (NORM) {
        const float var = static_cast<float>(ss[j] / static_cast<double>(D));
        rstd = rsqrt_rn(__fadd_rn(var, a.eps));
      }
      float y1[4], y2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float x1 = NORM ? __fmul_rn(__fmul_rn(lo[j][i], rstd), wlo[i]) : lo[j][i];
        const float x2 = NORM ? __fmul_rn(__fmul_rn(hi[j][i], rstd), whi[i]) : hi[j][i];
        y1[i] = __fsub_rn(__fmul_rn(x1, cosv[i]), __fmul_rn(x2, sinv[i]));
        y2[i] = __fadd_rn(__fmul_rn(x2, cosv[i]), __fmul_rn(x1, sinv[i]));
      }
      if (is_q) {
        __nv_bfloat16* dst = a.q + t * a.q_t + (h0 + j) * a.q_h;
        uint2 o1, o2;
        o1.x = pack_bf16(y1[0], y1[1]); o1.y = pack_bf16(y1[2], y1[3]);
        o2.x = pack_bf16(y2[0], y2[1]); o2.y = pack_bf16(y2[2], y2[3]);
        *reinterpret_cast<uint2*>(dst + 4 * sub) = o1;
        *reinterpret_cast<uint2*>(dst + HALF + 4 * sub) = o2;
        continue;
      }
      // K: round to bf16 first, as the reference does before the e4m3 cast
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        lo[j][i] = round_bf16(y1[i]);
        hi[j][i] = round_bf16(y2[i]);
      }
      if constexpr (!NORM) {
        if (a.k_out != nullptr) {  // rotation in place: the bf16 K goes back to where it came from
          __nv_bfloat16* dst = a.k_out + t * a.k_t + (h0 + j) * a.k_h;
          uint2 o1, o2;
          o1.x = pack_bf16(lo[j][0], lo[j][1]); o1.y = pack_bf16(lo[j][2], lo[j][3]);
          o2.x = pack_bf16(hi[j][0], hi[j][1]); o2.y = pack_bf16(hi[j][2], hi[j][3]);
          *reinterpret_cast<uint2*>(dst + 4 * sub) = o1;
          *reinterpret_cast<uint2*>(dst + HALF + 4 * sub) = o2;
        }
        if (!to_cache) continue;
      }
    }
    uint8_t* dst = is_k ? (a.kc + slot * a.ck_s + (h0 + j) * a.ck_h) : (a.vc + slot * a.cv_s + (h0 + j) * a.cv_h);
    *reinterpret_cast<uint32_t*>(dst + 4 * sub) = pack_e4m3x4(lo[j][0], lo[j][1], lo[j][2], lo[j][3]);
    *reinterpret_cast<uint32_t*>(dst + HALF + 4 * sub) = pack_e4m3x4(hi[j][0], hi[j][1], hi[j][2], hi[j][3]);
  }
}

template <bool ROPE, bool NORM = true>
static int launch_rope(const RopeArgs& a, int D, cudaStream_t stream) {
  const int heads_all = a.n_q + 2 * a.n_kv;
  if (static_cast<int64_t>(a.T) * heads_all == 0) return FR_OK;
  const bool four = (a.n_q % 4 == 0) && (a.n_kv % 4 == 0);
  const int64_t items = static_cast<int64_t>(a.T) * (four ? heads_all / 4 : heads_all);
  if (D == 128) {
    const int per_cta = 8 * 2;
    if (four) qk_rope_kv_kernel<128, ROPE, 4, NORM><<<ceil_div(items, per_cta), 256, 0, stream>>>(a);
    else qk_rope_kv_kernel<128, ROPE, 1, NORM><<<ceil_div(items, per_cta), 256, 0, stream>>>(a);
  } else if (D == 64) {
    const int per_cta = 8 * 4;
    if (four) qk_rope_kv_kernel<64, ROPE, 4, NORM><<<ceil_div(items, per_cta), 256, 0, stream>>>(a);
    else qk_rope_kv_kernel<64, ROPE, 1, NORM><<<ceil_div(items, per_cta), 256, 0, stream>>>(a);
  } else {
    return FR_ERR_UNSUPPORTED;
  }
  return launch_status();
}

// Scatter of rows that are e4m3 already: cache[loc[t], h, :] = src[t, h, :] as 16-byte pieces.
__global__ void __launch_bounds__(256) kv_scatter_e4m3_kernel(const uint8_t* __restrict__ k, const uint8_t* __restrict__ v,
                                                             int64_t k_t, int64_t k_h, int64_t v_t, int64_t v_h,
                                                             const int64_t* __restrict__ loc, uint8_t* kc, uint8_t* vc,
                                                             int64_t ck_s, int64_t ck_h, int64_t cv_s, int64_t cv_h, int T,
                                                             int n_kv, int D, int num_slots) {
  const int vec = D / 16;
  const int64_t total = static_cast<int64_t>(T) * n_kv * vec * 2;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % vec);
    const int h = static_cast<int>((i / vec) % n_kv);
    const int which = static_cast<int>((i / (static_cast<int64_t>(vec) * n_kv)) & 1);
    const int t = static_cast<int>(i / (static_cast<int64_t>(vec) * n_kv * 2));
    const int64_t slot = loc[t];
    if (slot < 0 || slot >= num_slots) continue;
    if (which == 0)
      *reinterpret_cast<uint4*>(kc + slot * ck_s + h * ck_h + 16 * c) =
          *reinterpret_cast<const uint4*>(k + t * k_t + h * k_h + 16 * c);
    else
      *reinterpret_cast<uint4*>(vc + slot * cv_s + h * cv_h + 16 * c) =
          *reinterpret_cast<const uint4*>(v + t * v_t + h * v_h + 16 * c);
  }
}

__global__ void __launch_bounds__(256) embedding_kernel(const uint4* __restrict__ table, const int64_t* __restrict__ ids,
                                                       uint4* __restrict__ out, int T, int vec_per_row, int vocab) {
  const int64_t total = static_cast<int64_t>(T) * vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / vec_per_row);
    const int c = static_cast<int>(i % vec_per_row);
    int64_t id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    out[i] = __ldg(table + id * vec_per_row + c);
  }
}

}  // namespace fr

using namespace fr;

static bool aligned8(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; }
static bool aligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

extern "C" int fr_qk_norm_rope_kv_fp8(void* q, const void* k, const void* v, int64_t q_t, int64_t q_h, int64_t k_t,
                                      int64_t k_h, int64_t v_t, int64_t v_h, const int64_t* positions,
                                      const int64_t* loc, const void* q_weight, const void* k_weight, float eps,
                                      const float* cos_sin, int max_pos, void* k_cache, void* v_cache, int64_t ck_s,
                                      int64_t ck_h, int64_t cv_s, int64_t cv_h, int T, int n_q, int n_kv, int D,
                                      int num_slots, cudaStream_t stream) {
  FR_CHECK_ARG(T >= 0 && n_q >= 0 && n_kv >= 0 && D > 0 && max_pos > 0 && num_slots > 0);
  if (T == 0) return FR_OK;
  FR_CHECK_ARG(q && k && v && positions && loc && q_weight && k_weight && cos_sin && k_cache && v_cache);
  FR_CHECK_SUPPORTED(D == 128 || D == 64);
  FR_CHECK_ARG(aligned8(q) && aligned8(k) && aligned8(v) && aligned8(q_weight) && aligned8(k_weight));
  FR_CHECK_ARG(q_t % 4 == 0 && q_h % 4 == 0 && k_t % 4 == 0 && k_h % 4 == 0 && v_t % 4 == 0 && v_h % 4 == 0);
  FR_CHECK_ARG(aligned16(cos_sin) && aligned4(k_cache) && aligned4(v_cache));
  FR_CHECK_ARG(ck_s % 4 == 0 && ck_h % 4 == 0 && cv_s % 4 == 0 && cv_h % 4 == 0);
  RopeArgs a{static_cast<__nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
             q_t, q_h, k_t, k_h, v_t, v_h, positions, loc, static_cast<const __nv_bfloat16*>(q_weight),
             static_cast<const __nv_bfloat16*>(k_weight), eps, cos_sin, max_pos, static_cast<uint8_t*>(k_cache),
             static_cast<uint8_t*>(v_cache), ck_s, ck_h, cv_s, cv_h, T, n_q, n_kv, num_slots, nullptr};
  return launch_rope<true>(a, D, stream);
}

extern "C" int fr_rope_neox_inplace(void* q, void* k, const void* v, int64_t q_t, int64_t q_h, int64_t k_t, int64_t k_h,
                                    int64_t v_t, int64_t v_h, const int64_t* positions, const int64_t* loc,
                                    const float* cos_sin, int max_pos, void* k_cache, void* v_cache, int64_t ck_s,
                                    int64_t ck_h, int64_t cv_s, int64_t cv_h, int T, int n_q, int n_kv, int D,
                                    int num_slots, cudaStream_t stream) {
  FR_CHECK_ARG(T >= 0 && n_q >= 0 && n_kv >= 0 && D > 0 && max_pos > 0);
  if (T == 0) return FR_OK;
  FR_CHECK_ARG(q && k && positions && cos_sin && aligned16(cos_sin));
  FR_CHECK_SUPPORTED(D == 128 || D == 64);
  FR_CHECK_ARG(aligned8(q) && aligned8(k) && q_t % 4 == 0 && q_h % 4 == 0 && k_t % 4 == 0 && k_h % 4 == 0);
  const bool store = k_cache != nullptr || v_cache != nullptr;
  if (store) {
    FR_CHECK_ARG(k_cache && v_cache && v && loc && num_slots > 0 && aligned8(v) && v_t % 4 == 0 && v_h % 4 == 0);
    FR_CHECK_ARG(aligned4(k_cache) && aligned4(v_cache) && ck_s % 4 == 0 && ck_h % 4 == 0 && cv_s % 4 == 0 &&
                 cv_h % 4 == 0);
  }
  // without a cache the V heads have no work; loc is then never read for a slot that is used
  RopeArgs a{static_cast<__nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
             static_cast<const __nv_bfloat16*>(store ? v : k), q_t, q_h, k_t, k_h, store ? v_t : k_t,
             store ? v_h : k_h, positions, store ? loc : positions, nullptr, nullptr, 0.f, cos_sin, max_pos,
             static_cast<uint8_t*>(k_cache), static_cast<uint8_t*>(v_cache), ck_s, ck_h, cv_s, cv_h, T, n_q, n_kv,
             store ? num_slots : 1, static_cast<__nv_bfloat16*>(k)};
  return launch_rope<true, false>(a, D, stream);
}

extern "C" int fr_store_kv_fp8(const void* k, const void* v, int64_t k_t, int64_t k_h, int64_t v_t, int64_t v_h,
                               const int64_t* loc, void* k_cache, void* v_cache, int64_t ck_s, int64_t ck_h,
                               int64_t cv_s, int64_t cv_h, int T, int n_kv, int D, int num_slots, int src_is_e4m3,
                               cudaStream_t stream) {
  FR_CHECK_ARG(T >= 0 && n_kv >= 0 && D > 0 && num_slots > 0);
  if (T == 0) return FR_OK;
  FR_CHECK_ARG(k && v && loc && k_cache && v_cache);
  FR_CHECK_SUPPORTED(D == 128 || D == 64);
  if (src_is_e4m3) {
    // rows converted by the caller (TokenToKVPool.store casts before it calls store_kv_cache): byte scatter
    FR_CHECK_ARG(aligned16(k) && aligned16(v) && aligned16(k_cache) && aligned16(v_cache));
    FR_CHECK_ARG(k_t % 16 == 0 && k_h % 16 == 0 && v_t % 16 == 0 && v_h % 16 == 0 && ck_s % 16 == 0 && ck_h % 16 == 0 &&
                 cv_s % 16 == 0 && cv_h % 16 == 0);
    const int64_t total = static_cast<int64_t>(T) * n_kv * (D / 16) * 2;
    int grid = ceil_div(total, 256);
    if (grid > 148 * 16) grid = 148 * 16;
    kv_scatter_e4m3_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(k), static_cast<const uint8_t*>(v), k_t,
                                                    k_h, v_t, v_h, loc, static_cast<uint8_t*>(k_cache),
                                                    static_cast<uint8_t*>(v_cache), ck_s, ck_h, cv_s, cv_h, T, n_kv, D,
                                                    num_slots);
    return launch_status();
  }
  FR_CHECK_ARG(aligned8(k) && aligned8(v) && k_t % 4 == 0 && k_h % 4 == 0 && v_t % 4 == 0 && v_h % 4 == 0);
  FR_CHECK_ARG(aligned4(k_cache) && aligned4(v_cache) && ck_s % 4 == 0 && ck_h % 4 == 0 && cv_s % 4 == 0 && cv_h % 4 == 0);
  RopeArgs a{nullptr, static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), 0, 0, k_t, k_h, v_t,
             v_h, nullptr, loc, nullptr, nullptr, 0.f, nullptr, 1, static_cast<uint8_t*>(k_cache),
             static_cast<uint8_t*>(v_cache), ck_s, ck_h, cv_s, cv_h, T, 0, n_kv, num_slots, nullptr};
  return launch_rope<false>(a, D, stream);
}

extern "C" int fr_embedding_bf16(const void* table, const int64_t* ids, void* out, int T, int hidden, int vocab,
                                 cudaStream_t stream) {
  FR_CHECK_ARG(T >= 0 && hidden > 0 && hidden % 8 == 0 && vocab > 0);
  if (T == 0) return FR_OK;
  FR_CHECK_ARG(table && ids && out && aligned16(table) && aligned16(out));
  const int vec = hidden / 8;
  const int64_t total = static_cast<int64_t>(T) * vec;
  int grid = ceil_div(total, 256);
  if (grid > 148 * 16) grid = 148 * 16;
  embedding_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint4*>(table), ids, static_cast<uint4*>(out), T, vec,
                                            vocab);
  return launch_status();
}
