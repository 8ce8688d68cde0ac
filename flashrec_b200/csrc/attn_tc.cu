// Shared-prefix decode attention on the 5th-generation tensor cores.
//
// The beams of one request (a "group") all attend to the same prompt slots.
// For that shared part, (beams x query heads of one KV head) is the M dimension
// of two tcgen05 contractions per KV tile:
//
//     S = Q . K^T        kind::f16 (bf16 x bf16 -> fp32 in TMEM), M=128, N=64 tokens, K=128 dims
//     O += P . V         P = exp2(S*scale - m) rounded to bf16, written back into TMEM over S
//                        and consumed from there as the A operand (no shared-memory round trip)
//
// Step 1 (shared_kv_prepare_kernel): per layer, the group's shared K rows are
// widened e4m3 -> bf16 into a scratch buffer [group, kv head, token, 128] and V is
// widened and TRANSPOSED into [group, kv head, 128, token], once per group instead
// of once per CTA. Both layouts are K-major for their MMA, so plain TMA tile
// loads (128-byte swizzle, one CTA per tile) feed tcgen05.mma directly.
// Step 2 (decode_attn_tc_kernel): one CTA per (64/G-beam tile... 128 query vectors,
// kv head, group). warp 0 = TMA producer, warp 1 = TMEM allocation + MMA issue,
// warps 2-5 = softmax / correction / tail / epilogue, one query vector per
// thread (TMEM lane == row). The running maximum is only raised when a tile
// exceeds it by more than 8 (log2 units), which keeps the O rescale in TMEM rare.
// The per-row tail (the row's private decode slots after the shared prefix) is
// folded in by the same thread with scalar FMAs, read-modify-writing O in TMEM.
//
// Stands in for the same reference code as attn_decode.cu
// (attention/flashinfer.py:212-238, 380-431).
#include "fr_common.cuh"
#include "sm100_ptx.cuh"

namespace fr {

int* device_status_ptr();  // capi.cu

namespace attn_tc {

constexpr int kD = 128;
constexpr int kM = 128;       // query vectors per CTA (UMMA M)
constexpr int kTileN = 64;    // KV tokens per tile
constexpr int kThreads = 192;
constexpr int kTmemCols = 256;  // S: 2 buffers x 64 columns, O: 128 columns
constexpr int kColS = 0;        // + 64 * (tile & 1)
constexpr int kColO = 128;
constexpr float kRescaleThreshold = 8.0f;

constexpr int kSmemQ = kM * kD * 2;             // 32 KB: two k-blocks of [128 rows x 128 B]
constexpr int kSmemK = kTileN * kD * 2;         // 16 KB per stage: two k-blocks of [64 rows x 128 B]
constexpr int kSmemV = kD * kTileN * 2;         // 16 KB: [128 dims x 128 B (64 tokens)]
constexpr int kSmemBytes = 1024 + kSmemQ + 2 * kSmemK + 2 * kSmemV + 256;  // K and V double buffered

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
  __nv_bfloat16* kb;  // [groups, hkv, lcap, 128]
  __half* vt;         // [groups, hkv, 128, lcap], fp16 (e4m3 values are exact in fp16)
  int lcap;
  int n_rows, n_groups, hq, hkv, num_slots;
  float scale_log2;
  const int32_t* prepared_len;  // per group: tokens of the prefix already widened in scratch (or nullptr)
  // prefill (causal) use: the group's slot list is indices[kv_group_indptr[g] .. kv_group_indptr[g+1])
  // and the group's rows are its last tokens, in order (nullptr for decode)
  const int32_t* kv_group_indptr;
};

// Slot list and number of keys that all rows of group `grp` share (decode: the shared prefix found by the
// plan; prefill: every key of the request).
__device__ __forceinline__ int group_keys(const Params& p, int grp, int row0, const int32_t*& idx) {
  if (p.kv_group_indptr != nullptr) {
    const int b = p.kv_group_indptr[grp];
    idx = p.indices + b;
    return min(max(p.kv_group_indptr[grp + 1] - b, 0), p.lcap);
  }
  idx = p.indices + p.indptr[row0];
  return min(p.shared_len[grp], p.lcap);
}

__device__ __forceinline__ __half2 e4m3x2_to_half2(uint16_t v) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(v), __NV_E4M3);
  return *reinterpret_cast<__half2*>(&h);
}

// exp2 of two fp32 arguments, evaluated as one packed fp16 operation: {2^lo, 2^hi} as an fp16 pair
// (lo in the low half). The arguments are at most the rescale threshold, so 2^x <= 256; arguments
// below -16 lose relative accuracy but their terms are below 2^-16 of the row maximum.
__device__ __forceinline__ uint32_t ex2_f16x2(float lo, float hi) {
  uint32_t packed, r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(r) : "r"(packed));
  return r;
}
__device__ __forceinline__ uint32_t add_f16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ float sum_f16x2(uint32_t v) {
  const __half2 h = *reinterpret_cast<const __half2*>(&v);
  const float2 f = __half22float2(h);
  return f.x + f.y;
}

__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t v) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(v), __NV_E4M3);
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}

// ---------------------------------------------------------------------------
// step 1: widen (and transpose V) the shared prefix of every group
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) shared_kv_prepare_kernel(Params p) {
  const int grp = blockIdx.z, kvh = blockIdx.y;
  const int row0 = p.group_rows[grp];
  const int32_t* idx;
  const int ls = group_keys(p, grp, row0, idx);
  const int padded = (ls + kTileN - 1) / kTileN * kTileN;  // tiles are read whole: zero-fill their tails
  const int tok0 = blockIdx.x * 32;
  if (tok0 >= padded) return;
  // tokens below `done` were widened by an earlier call on the same scratch and are still valid
  const int done = p.prepared_len != nullptr ? min(p.prepared_len[grp], ls) : 0;
  if (tok0 + 32 <= done) return;
  const size_t gh = static_cast<size_t>(grp) * p.hkv + kvh;
  __nv_bfloat16* kb = p.kb + gh * p.lcap * kD;
  __half* vt = p.vt + gh * kD * p.lcap;
  // 32 tokens x 8 chunks of 16 dims; token fastest across lanes so that the
  // transposed V stores of a warp hit consecutive addresses
  const int tok = tok0 + (threadIdx.x & 31);
  const int ch = threadIdx.x >> 5;
  uint4 kraw = make_uint4(0, 0, 0, 0), vraw = make_uint4(0, 0, 0, 0);
  if (tok < ls) {
    int64_t s = idx[tok];
    s = s < 0 ? 0 : (s >= p.num_slots ? p.num_slots - 1 : s);
    kraw = __ldg(reinterpret_cast<const uint4*>(p.kc + s * p.ck_s + kvh * p.ck_h + ch * 16));
    vraw = __ldg(reinterpret_cast<const uint4*>(p.vc + s * p.cv_s + kvh * p.cv_h + ch * 16));
  }
  if (tok >= padded || tok < done) return;
  const uint32_t kw[4] = {kraw.x, kraw.y, kraw.z, kraw.w};
  const uint32_t vw[4] = {vraw.x, vraw.y, vraw.z, vraw.w};
  uint32_t ko[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = e4m3x2_to_float2(static_cast<uint16_t>(kw[i] & 0xffffu));
    const float2 b = e4m3x2_to_float2(static_cast<uint16_t>(kw[i] >> 16));
    ko[2 * i] = pack_bf16(a.x, a.y);
    ko[2 * i + 1] = pack_bf16(b.x, b.y);
  }
  uint4* kdst = reinterpret_cast<uint4*>(kb + static_cast<size_t>(tok) * kD + ch * 16);
  kdst[0] = make_uint4(ko[0], ko[1], ko[2], ko[3]);
  kdst[1] = make_uint4(ko[4], ko[5], ko[6], ko[7]);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 a = e4m3x2_to_half2(static_cast<uint16_t>(vw[i] & 0xffffu));
    const __half2 b = e4m3x2_to_half2(static_cast<uint16_t>(vw[i] >> 16));
    const int d = ch * 16 + 4 * i;
    vt[static_cast<size_t>(d + 0) * p.lcap + tok] = __low2half(a);
    vt[static_cast<size_t>(d + 1) * p.lcap + tok] = __high2half(a);
    vt[static_cast<size_t>(d + 2) * p.lcap + tok] = __low2half(b);
    vt[static_cast<size_t>(d + 3) * p.lcap + tok] = __high2half(b);
  }
}

// ---------------------------------------------------------------------------
// step 2
// ---------------------------------------------------------------------------
// CAUSAL: prefill. The rows of a group are the request's last tokens (its extend tokens), row e sees the
// keys [0, prefix + e] with prefix = keys - rows; tiles past the last row of the CTA are skipped, the
// tiles on the diagonal are masked per row, and there is no per-row tail.
template <int G, bool CAUSAL>
__global__ void __launch_bounds__(kThreads, 2)
decode_attn_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, Params p, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t sm_q = base;
  const uint32_t sm_k = sm_q + kSmemQ;       // 2 stages
  const uint32_t sm_v = sm_k + 2 * kSmemK;   // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemQ + 2 * kSmemK + 2 * kSmemV);
  const uint32_t bar0 = ptx::smem_u32(bars);
  const uint32_t bar_q = bar0;              // Q landed
  const uint32_t bar_kfull = bar0 + 8;      // [2]
  const uint32_t bar_kempty = bar0 + 24;    // [2]
  const uint32_t bar_vfull = bar0 + 40;     // [2]
  const uint32_t bar_vempty = bar0 + 56;    // [2]
  const uint32_t bar_sfull = bar0 + 72;     // [2] S tile complete in TMEM buffer (tile & 1)
  const uint32_t bar_pfull = bar0 + 88;     // P tile written into TMEM (128 arrivals)
  const uint32_t bar_ofull = bar0 + 96;     // P.V accumulated (one phase per tile; waited for by the rare O rescale)
  // Last P.V accumulated. Its own one-phase barrier: the softmax of the last tile can finish while the
  // P.V before the last is still pending (S of tile j + 1 is issued before P.V of tile j), and a parity
  // wait on bar_ofull two phases ahead of the barrier would pass at once.
  const uint32_t bar_done = bar0 + 112;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  constexpr int kBeams = kM / G;
  const int grp = blockIdx.z, kvh = blockIdx.y;
  const int row0 = p.group_rows[grp];
  const int rows_in_group = p.group_rows[grp + 1] - row0;
  const int beam0 = blockIdx.x * kBeams;
  if (beam0 >= rows_in_group) return;
  const int32_t* idx_unused;
  const int ls = group_keys(p, grp, row0, idx_unused);
  const int pfx = CAUSAL ? max(ls - rows_in_group, 0) : 0;
  // keys the last live row of this CTA sees (CTA-uniform: every role derives the same tile count)
  const int vis = CAUSAL ? min(ls, pfx + min(beam0 + kBeams, rows_in_group)) : ls;
  const int n_tiles = (vis + kTileN - 1) / kTileN;
  const int gh = grp * p.hkv + kvh;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    ptx::mbar_init(bar_q, 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(bar_kfull + 8 * i, 1);
      ptx::mbar_init(bar_kempty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(bar_vfull + 8 * i, 1);
      ptx::mbar_init(bar_vempty + 8 * i, 1);
    }
    ptx::mbar_init(bar_sfull, 1);
    ptx::mbar_init(bar_sfull + 8, 1);
    ptx::mbar_init(bar_pfull, 128);
    ptx::mbar_init(bar_ofull, 1);
    ptx::mbar_init(bar_done, 1);
    *abort_flag = 0;
    ptx::mbar_init_fence();
    ptx::prefetch_tmap(&tmap_q);
    ptx::prefetch_tmap(&tmap_k);
    ptx::prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ---------------------------
    if (lane == 0) {
      // Q is needed by the MMAs and, from shared memory, by the per-row tails
      ptx::mbar_expect_tx(bar_q, kSmemQ);
      ptx::tma_load_3d(sm_q, &tmap_q, 0, kvh * G, row0 + beam0, bar_q);
      ptx::tma_load_3d(sm_q + kSmemQ / 2, &tmap_q, 64, kvh * G, row0 + beam0, bar_q);
      bool ok = true;
      auto load_k = [&](int jj) -> bool {
        const uint32_t st = jj & 1, ph = (jj >> 1) & 1;
        if (!ptx::mbar_wait(bar_kempty + 8 * st, ph ^ 1u, abort_flag, status, 11)) return false;
        ptx::mbar_expect_tx(bar_kfull + 8 * st, kSmemK);
        ptx::tma_load_3d(sm_k + st * kSmemK, &tmap_k, 0, jj * kTileN, gh, bar_kfull + 8 * st);
        ptx::tma_load_3d(sm_k + st * kSmemK + kSmemK / 2, &tmap_k, 64, jj * kTileN, gh, bar_kfull + 8 * st);
        return true;
      };
      if (n_tiles > 0) ok = load_k(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        // K runs one tile ahead of V so that S of tile j+1 can be issued during the softmax of tile j
        if (j + 1 < n_tiles) {
          ok = load_k(j + 1);
          if (!ok) break;
        }
        const uint32_t st = j & 1, ph = (j >> 1) & 1;
        ok = ptx::mbar_wait(bar_vempty + 8 * st, ph ^ 1u, abort_flag, status, 12);
        if (!ok) break;
        ptx::mbar_expect_tx(bar_vfull + 8 * st, kSmemV);
        ptx::tma_load_3d(sm_v + st * kSmemV, &tmap_v, j * kTileN, 0, gh, bar_vfull + 8 * st);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer -----------------------------
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = ptx::make_idesc(1u, 1u, kM, kTileN);  // bf16 x bf16, N = 64 tokens
      constexpr uint32_t idesc_o = ptx::make_idesc(0u, 0u, kM, kD);      // fp16 x fp16, N = 128 dims
      bool ok = ptx::mbar_wait(bar_q, 0, abort_flag, status, 13);
      // S = Q K^T for tile jj into TMEM buffer (jj & 1): 2 k-blocks (64 dims) x 4 instructions of K = 16
      auto issue_s = [&](int jj) -> bool {
        const uint32_t st = jj & 1, ph = (jj >> 1) & 1;
        if (!ptx::mbar_wait(bar_kfull + 8 * st, ph, abort_flag, status, 14)) return false;
        ptx::tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t a_desc = ptx::smem_desc_sw128(sm_q + kb * (kSmemQ / 2));
          const uint64_t b_desc = ptx::smem_desc_sw128(sm_k + st * kSmemK + kb * (kSmemK / 2));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            ptx::mma_f16(tmem_base + kColS + st * kTileN, a_desc + 2u * k, b_desc + 2u * k, idesc_s,
                         (kb | k) != 0 ? 1u : 0u);
        }
        ptx::tc_commit(bar_kempty + 8 * st);
        ptx::tc_commit(bar_sfull + 8 * st);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        // S of the next tile runs while the softmax warps work on this one: its TMEM
        // buffer was last read for tile j-1, whose P (written after that read) has
        // already been waited for below in the previous iteration.
        if (j + 1 < n_tiles) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        ok = ptx::mbar_wait(bar_pfull, j & 1, abort_flag, status, 15);
        if (!ok) break;
        ok = ptx::mbar_wait(bar_vfull + 8 * (j & 1), (j >> 1) & 1, abort_flag, status, 16);
        if (!ok) break;
        ptx::tc_fence_after();
        // O (+)= P V: A = P straight from TMEM (bf16 pairs in the first 32 columns of the S
        // buffer of this tile: 16 tokens = 8 columns per instruction), B = V^T tile in shared memory
        {
          const uint32_t a_tmem = tmem_base + kColS + (j & 1) * kTileN;
          const uint64_t b_desc = ptx::smem_desc_sw128(sm_v + (j & 1) * kSmemV);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            ptx::mma_f16_ts(tmem_base + kColO, a_tmem + 8u * k, b_desc + 2u * k, idesc_o, (j | k) != 0 ? 1u : 0u);
        }
        ptx::tc_commit(bar_vempty + 8 * (j & 1));
        ptx::tc_commit(bar_ofull);
        if (j + 1 == n_tiles) ptx::tc_commit(bar_done);
      }
    }
    __syncwarp();
  } else {
    // ------------------- softmax / correction / tail / epilogue -------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // query vector == TMEM lane == P row
    const int beam = beam0 + r / G;
    const bool live = beam < rows_in_group;
    const int row = row0 + (live ? beam : 0);
    const int head = kvh * G + r % G;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      int okw = 0;
      if (lane == 0) okw = ptx::mbar_wait(bar_sfull + 8 * (j & 1), (j >> 1) & 1, abort_flag, status, 17) ? 1 : 0;
      okw = __shfl_sync(0xffffffffu, okw, 0);
      if (!okw) { ok = false; break; }
      ptx::tc_fence_after();
      uint32_t s0[32], s1[32];
      ptx::tmem_ld_32x32(t_lane + kColS + (j & 1) * kTileN, s0);
      ptx::tmem_ld_32x32(t_lane + kColS + (j & 1) * kTileN + 32, s1);
      ptx::tmem_ld_wait();
      // decode: only the last tile of the prefix is short (uniform over the CTA); prefill: row e stops at
      // key prefix + e, so the tiles on the diagonal are short by a different amount per row (never the
      // first tile as a whole: key 0 is visible to every row, the running maximum is finite from tile 0 on)
      const int row_keys = CAUSAL ? min(ls, pfx + (live ? beam : rows_in_group - 1) + 1) : ls;
      const int ntok = min(kTileN, row_keys - j * kTileN);
      if (ntok < kTileN) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          if (c >= ntok) s0[c] = 0xff800000u;       // -inf
          if (c + 32 >= ntok) s1[c] = 0xff800000u;
        }
      }
      // maximum of the raw scores on four independent chains; the softmax scale (> 0) is applied once
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 32; ++c) mx[c & 3] = fmaxf(mx[c & 3], fmaxf(__uint_as_float(s0[c]), __uint_as_float(s1[c])));
      const float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
      // raise the reference maximum only when the tile exceeds it by a margin
      float factor = 1.0f;
      if (tmax > m_used + kRescaleThreshold) {
        factor = exp2f(m_used - tmax);  // 0 on the first tile (m_used = -inf)
        m_used = tmax;
      }
      l_sum *= factor;
      // O may only be rescaled once the previous P.V has completed (rare: the maximum is raised lazily)
      if (j > 0 && __any_sync(0xffffffffu, factor != 1.0f)) {
        if (lane == 0) okw = ptx::mbar_wait(bar_ofull, (j - 1) & 1, abort_flag, status, 18) ? 1 : 0;
        okw = __shfl_sync(0xffffffffu, okw, 0);
        if (!okw) { ok = false; break; }
        ptx::tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < kD / 32; ++c) {
          uint32_t o[32];
          ptx::tmem_ld_32x32(t_lane + kColO + c * 32, o);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
          ptx::tmem_st_32x32(t_lane + kColO + c * 32, o);
        }
        ptx::tmem_st_wait();
      }
      // P is written as fp16 pairs over the first 32 columns of this tile's S buffer
      // (S has just been read into registers; the next S for this buffer is issued after this P.V)
      // P = exp2(s * scale - m) as fp16 pairs: one FMA per score, one conversion and one packed
      // ex2.approx per pair; the row sum runs on four packed fp16 chains of 8 terms each (terms
      // <= 256, relative error of the sum below 2^-10) and is widened to fp32 per tile
      uint32_t ps[4] = {0u, 0u, 0u, 0u};
      uint32_t w[32];
      const float neg_m = -m_used;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int c = 2 * i;  // token index within the tile
        const float a = __fmaf_rn(__uint_as_float(c < 32 ? s0[c & 31] : s1[c & 31]), p.scale_log2, neg_m);
        const float b = __fmaf_rn(__uint_as_float(c + 1 < 32 ? s0[(c + 1) & 31] : s1[(c + 1) & 31]), p.scale_log2, neg_m);
        w[i] = ex2_f16x2(a, b);
        ps[i & 3] = add_f16x2(ps[i & 3], w[i]);
      }
      const float psum = (sum_f16x2(ps[0]) + sum_f16x2(ps[1])) + (sum_f16x2(ps[2]) + sum_f16x2(ps[3]));
      l_sum += psum;
      ptx::tmem_st_32x32(t_lane + kColS + (j & 1) * kTileN, w);
      ptx::tmem_st_wait();
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar_pfull);
    }
    if (ok && n_tiles > 0) {
      int okw = 0;
      if (lane == 0) okw = ptx::mbar_wait(bar_done, 0, abort_flag, status, 19) ? 1 : 0;
      okw = __shfl_sync(0xffffffffu, okw, 0);
      ok = okw != 0;
      ptx::tc_fence_after();
    }
    if (ok) {
      // ---- per-row tail: slots after the shared prefix ------------------------
      const int t_beg = CAUSAL ? 0 : p.indptr[row] + ls;
      const int t_len = (!CAUSAL && live) ? max(p.indptr[row + 1] - t_beg, 0) : 0;
      int max_len = t_len;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) max_len = max(max_len, __shfl_xor_sync(0xffffffffu, max_len, o));
      bool o_valid = n_tiles > 0;
      if (max_len > 0) {  // warp-uniform; Q tile in shared memory (row r, 128-byte swizzle)
        int okq = 0;
        if (lane == 0) okq = ptx::mbar_wait(bar_q, 0, abort_flag, status, 20) ? 1 : 0;
        okq = __shfl_sync(0xffffffffu, okq, 0);
        if (!okq) max_len = 0;
      }
      const uint8_t* q_row = smem + r * 128;  // + k-block * 16 KB + (chunk ^ (r & 7)) * 16
      constexpr int kBatch = 4;
      for (int t0 = 0; t0 < max_len; t0 += kBatch) {
        float sc[kBatch];
        int64_t slot[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
          sc[b] = -INFINITY;
          slot[b] = 0;
          if (t0 + b < t_len) {
            int64_t s = p.indices[t_beg + t0 + b];
            s = s < 0 ? 0 : (s >= p.num_slots ? p.num_slots - 1 : s);
            slot[b] = s;
          }
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
          if (t0 + b < t_len) {
            const uint8_t* kp = p.kc + slot[b] * p.ck_s + kvh * p.ck_h;
            uint4 kk[kD / 16];
#pragma unroll
            for (int c = 0; c < kD / 16; ++c) kk[c] = __ldg(reinterpret_cast<const uint4*>(kp + c * 16));  // all in flight
            float dot = 0.f;
#pragma unroll
            for (int c = 0; c < kD / 16; ++c) {
              const uint8_t* qb = q_row + (c >> 2) * (kSmemQ / 2);
              const int ch = (c & 3) * 2;
              const uint4 q0 = *reinterpret_cast<const uint4*>(qb + (((ch) ^ (r & 7)) << 4));
              const uint4 q1 = *reinterpret_cast<const uint4*>(qb + (((ch + 1) ^ (r & 7)) << 4));
              const uint32_t kw[4] = {kk[c].x, kk[c].y, kk[c].z, kk[c].w};
              const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 ka = e4m3x2_to_float2(static_cast<uint16_t>(kw[i] & 0xffffu));
                const float2 kb2 = e4m3x2_to_float2(static_cast<uint16_t>(kw[i] >> 16));
                dot += bf16lo(qw[2 * i]) * ka.x + bf16hi(qw[2 * i]) * ka.y + bf16lo(qw[2 * i + 1]) * kb2.x +
                       bf16hi(qw[2 * i + 1]) * kb2.y;
              }
            }
            sc[b] = dot * p.scale_log2;
          }
        }
        float bmax = sc[0];
#pragma unroll
        for (int b = 1; b < kBatch; ++b) bmax = fmaxf(bmax, sc[b]);
        const float m_new = fmaxf(m_used, bmax);
        const float c_old = (m_new == -INFINITY) ? 1.0f : exp2f(m_used - m_new);
        float pr[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) pr[b] = (sc[b] == -INFINITY) ? 0.f : exp2f(sc[b] - m_new);
        m_used = m_new;
        l_sum = l_sum * c_old;
#pragma unroll
        for (int b = 0; b < kBatch; ++b) l_sum += pr[b];
        // V rows of the batch, 32 dims at a time; the loads of chunk c + 1 are issued before the
        // arithmetic of chunk c so that their latency is paid once, not once per chunk
        uint4 vnext[kBatch][2];
        auto load_v = [&](int c) {
#pragma unroll
          for (int b = 0; b < kBatch; ++b) {
            vnext[b][0] = vnext[b][1] = make_uint4(0, 0, 0, 0);
            if (pr[b] != 0.f) {
              const uint8_t* vp = p.vc + slot[b] * p.cv_s + kvh * p.cv_h + c * 32;
              vnext[b][0] = __ldg(reinterpret_cast<const uint4*>(vp));
              vnext[b][1] = __ldg(reinterpret_cast<const uint4*>(vp + 16));
            }
          }
        };
        load_v(0);
#pragma unroll 1
        for (int c = 0; c < kD / 32; ++c) {
          uint4 vv[kBatch][2];
#pragma unroll
          for (int b = 0; b < kBatch; ++b) {
            vv[b][0] = vnext[b][0];
            vv[b][1] = vnext[b][1];
          }
          if (c + 1 < kD / 32) load_v(c + 1);
          uint32_t o[32];
          if (o_valid) {
            ptx::tmem_ld_32x32(t_lane + kColO + c * 32, o);
            ptx::tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0u;
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * c_old);
#pragma unroll
          for (int b = 0; b < kBatch; ++b) {
            if (pr[b] != 0.f) {
              const uint32_t vw[8] = {vv[b][0].x, vv[b][0].y, vv[b][0].z, vv[b][0].w,
                                      vv[b][1].x, vv[b][1].y, vv[b][1].z, vv[b][1].w};
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float2 va = e4m3x2_to_float2(static_cast<uint16_t>(vw[i] & 0xffffu));
                const float2 vb = e4m3x2_to_float2(static_cast<uint16_t>(vw[i] >> 16));
                o[4 * i + 0] = __float_as_uint(__uint_as_float(o[4 * i + 0]) + pr[b] * va.x);
                o[4 * i + 1] = __float_as_uint(__uint_as_float(o[4 * i + 1]) + pr[b] * va.y);
                o[4 * i + 2] = __float_as_uint(__uint_as_float(o[4 * i + 2]) + pr[b] * vb.x);
                o[4 * i + 3] = __float_as_uint(__uint_as_float(o[4 * i + 3]) + pr[b] * vb.y);
              }
            }
          }
          ptx::tmem_st_32x32(t_lane + kColO + c * 32, o);
        }
        ptx::tmem_st_wait();
        o_valid = true;
      }
      // ---- normalise and store ----------------------------------------------------
      const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
      __nv_bfloat16* op = p.out + row * p.o_t + head * kD;
      const bool wide_out = (reinterpret_cast<uintptr_t>(p.out) & 31u) == 0 && (p.o_t & 15) == 0;  // CTA-uniform
#pragma unroll 1
      for (int c = 0; c < kD / 32; ++c) {
        uint32_t o[32];
        if (o_valid) {
          ptx::tmem_ld_32x32(t_lane + kColO + c * 32, o);
          ptx::tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (live) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            w[i] = pack_bf16(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
          __nv_bfloat16* dst = op + c * 32;
          if (wide_out) {  // 32-byte stores: one full sector per instruction (rows are 4 KB apart)
            const uint32_t w0[8] = {w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]};
            const uint32_t w1[8] = {w[8], w[9], w[10], w[11], w[12], w[13], w[14], w[15]};
            ptx::st_global_v8(dst, w0);
            ptx::st_global_v8(dst + 16, w1);
          } else {
            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
            for (int i = 0; i < 4; ++i) d4[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
          }
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// bf16 3-D tensor, 128-byte swizzle; dims / box innermost first; strides in bytes for dims 1 and 2.
static int make_tmap_bf16_3d(CUtensorMap* map, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1,
                             uint64_t s2, uint32_t b0, uint32_t b1, uint32_t b2, bool fp16 = false) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return FR_ERR_CUDA;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1, s2};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FR_OK : FR_ERR_CUDA;
}

template <int G, bool CAUSAL>
static int launch(const Params& p, int max_group_rows, cudaStream_t stream) {
  CUtensorMap tq, tk, tv;
  int st = make_tmap_bf16_3d(&tq, p.q, kD, p.hq, p.n_rows, static_cast<uint64_t>(p.q_h) * 2,
                             static_cast<uint64_t>(p.q_t) * 2, 64, G, kM / G);
  if (st != FR_OK) return st;
  const uint64_t gh = static_cast<uint64_t>(p.n_groups) * p.hkv;
  st = make_tmap_bf16_3d(&tk, p.kb, kD, p.lcap, gh, kD * 2, static_cast<uint64_t>(p.lcap) * kD * 2, 64, kTileN, 1);
  if (st != FR_OK) return st;
  st = make_tmap_bf16_3d(&tv, p.vt, p.lcap, kD, gh, static_cast<uint64_t>(p.lcap) * 2,
                         static_cast<uint64_t>(p.lcap) * kD * 2, kTileN, kD, 1, true);
  if (st != FR_OK) return st;
  auto kern = decode_attn_tc_kernel<G, CAUSAL>;
  static PerDeviceFlag attr_done;  // per template instantiation and device
  if (ensure_dyn_smem(attr_done, kern, kSmemBytes) != FR_OK) return FR_ERR_CUDA;
  int* status = device_status_ptr();
  if (!status) return FR_ERR_CUDA;
  dim3 pgrid(ceil_div(p.lcap, 32), p.hkv, p.n_groups);
  shared_kv_prepare_kernel<<<pgrid, 256, 0, stream>>>(p);
  if (launch_status() != FR_OK) return FR_ERR_CUDA;
  dim3 grid(ceil_div(max_group_rows, kM / G), p.hkv, p.n_groups);
  kern<<<grid, kThreads, kSmemBytes, stream>>>(tq, tk, tv, p, status);
  return launch_status();
}

}  // namespace attn_tc

// Called by fr_decode_attn_fp8 when the caller supplies scratch memory.
int decode_attn_tc(const void* q, int64_t q_t, int64_t q_h, const void* k_cache, const void* v_cache, int64_t ck_s,
                   int64_t ck_h, int64_t cv_s, int64_t cv_h, const int32_t* indptr, const int32_t* indices,
                   const int32_t* group_rows, const int32_t* shared_len, void* out, int64_t o_t, int n_rows,
                   int n_groups, int hq, int hkv, int max_group_rows, int num_slots, float sm_scale, void* scratch,
                   int lcap, const int32_t* prepared_len, cudaStream_t stream) {
  const int G = hq / hkv;
  // TMA: 16-byte aligned base and strides for the strided Q view
  FR_CHECK_ARG(aligned16(q) && (q_t * 2) % 16 == 0 && (q_h * 2) % 16 == 0 && aligned16(out) && (o_t * 2) % 16 == 0);
  FR_CHECK_ARG(lcap > 0 && lcap % attn_tc::kTileN == 0 && aligned16(scratch));
  attn_tc::Params p{static_cast<const __nv_bfloat16*>(q), q_t, q_h, static_cast<const uint8_t*>(k_cache),
                    static_cast<const uint8_t*>(v_cache), ck_s, ck_h, cv_s, cv_h, indptr, indices, group_rows,
                    shared_len, static_cast<__nv_bfloat16*>(out), o_t, nullptr, nullptr, lcap, n_rows, n_groups, hq,
                    hkv, num_slots, sm_scale * 1.4426950408889634f, prepared_len};
  const size_t half = static_cast<size_t>(n_groups) * hkv * lcap * attn_tc::kD;
  p.kb = static_cast<__nv_bfloat16*>(scratch);
  p.vt = reinterpret_cast<__half*>(p.kb + half);
  switch (G) {
    case 1: return attn_tc::launch<1, false>(p, max_group_rows, stream);
    case 2: return attn_tc::launch<2, false>(p, max_group_rows, stream);
    case 4: return attn_tc::launch<4, false>(p, max_group_rows, stream);
    case 8: return attn_tc::launch<8, false>(p, max_group_rows, stream);
    default: return FR_ERR_UNSUPPORTED;
  }
}

}  // namespace fr

using namespace fr;

extern "C" int64_t fr_decode_attn_scratch_bytes(int n_groups, int hkv, int max_shared_len);

extern "C" int fr_prefill_attn_fp8(const void* q, int64_t q_t, int64_t q_h, const void* k_cache, const void* v_cache,
                                   int64_t ck_s, int64_t ck_h, int64_t cv_s, int64_t cv_h, const int32_t* qo_indptr,
                                   const int32_t* kv_indptr, const int32_t* kv_indices, void* out, int64_t o_t,
                                   int n_tokens, int n_requests, int hq, int hkv, int head_dim, int max_extend_len,
                                   int max_kv_len, int num_slots, float sm_scale, void* scratch,
                                   int64_t scratch_bytes, cudaStream_t stream) {
  FR_CHECK_ARG(n_tokens >= 0 && n_requests >= 0 && hq > 0 && hkv > 0 && max_extend_len >= 0 && max_kv_len >= 0 &&
               num_slots > 0);
  if (n_tokens == 0 || n_requests == 0 || max_extend_len == 0 || max_kv_len == 0) return FR_OK;
  FR_CHECK_ARG(q && k_cache && v_cache && qo_indptr && kv_indptr && kv_indices && out && scratch);
  FR_CHECK_SUPPORTED(head_dim == attn_tc::kD && hq % hkv == 0);
  const int G = hq / hkv;
  FR_CHECK_SUPPORTED(G == 1 || G == 2 || G == 4 || G == 8);
  FR_CHECK_ARG(aligned16(q) && (q_t * 2) % 16 == 0 && (q_h * 2) % 16 == 0 && aligned16(out) && (o_t * 2) % 16 == 0);
  FR_CHECK_ARG(aligned16(k_cache) && aligned16(v_cache) && ck_s % 16 == 0 && ck_h % 16 == 0 && cv_s % 16 == 0 &&
               cv_h % 16 == 0 && aligned16(scratch));
  FR_CHECK_ARG(scratch_bytes >= fr_decode_attn_scratch_bytes(n_requests, hkv, max_kv_len));
  const int lcap = (max_kv_len + attn_tc::kTileN - 1) / attn_tc::kTileN * attn_tc::kTileN;
  attn_tc::Params p{static_cast<const __nv_bfloat16*>(q), q_t, q_h, static_cast<const uint8_t*>(k_cache),
                    static_cast<const uint8_t*>(v_cache), ck_s, ck_h, cv_s, cv_h, nullptr, kv_indices, qo_indptr,
                    nullptr, static_cast<__nv_bfloat16*>(out), o_t, nullptr, nullptr, lcap, n_tokens, n_requests, hq,
                    hkv, num_slots, sm_scale * 1.4426950408889634f, nullptr, kv_indptr};
  const size_t half = static_cast<size_t>(n_requests) * hkv * lcap * attn_tc::kD;
  p.kb = static_cast<__nv_bfloat16*>(scratch);
  p.vt = reinterpret_cast<__half*>(p.kb + half);
  switch (G) {
    case 1: return attn_tc::launch<1, true>(p, max_extend_len, stream);
    case 2: return attn_tc::launch<2, true>(p, max_extend_len, stream);
    case 4: return attn_tc::launch<4, true>(p, max_extend_len, stream);
    case 8: return attn_tc::launch<8, true>(p, max_extend_len, stream);
    default: return FR_ERR_UNSUPPORTED;
  }
}
