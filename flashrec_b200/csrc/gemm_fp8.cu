// W8A8 FP8 GEMM for the decode-step linear layers (qkv / o / gate_up / down and
// the SID lm_head):
//
//     out[m, n] = cast( (sum_k a[m,k] * b[n,k]) * scale_a[m] * scale_b[n] ) (+ bias[n])
//
// a: e4m3 [M, K] row-major (per-token scales), b: e4m3 [N, K] row-major — the
// reference keeps the weight as the `.t()` view of exactly this buffer
// (layers/linear.py:104-110) — with per-output-channel scales. Stands in for
// Linear.forward_fp8 -> fp8_scaled_mm (layers/linear.py:134-172,
// kernel/sglops.py:99-140).
//
// sm_100a design: a persistent, warp-specialised kernel, one CTA per SM.
//   warp 0      TMA producer: 128x128-byte A tile + BLOCK_N x128-byte B tile per
//               stage, 128-byte swizzle, mbarrier complete_tx
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma
//               (kind::f8f6f4, M=128, N=BLOCK_N, K=32 per instruction, both
//               operands K-major straight from shared memory), accumulating
//               fp32 in TMEM; tcgen05.commit frees the stage / publishes the tile
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp its own lane
//               quadrant), apply per-token x per-channel scales in fp32, round
//               once to bf16 (or keep fp32 for the lm_head logits), store
// Two accumulator buffers in TMEM let the epilogue of tile i overlap the
// main loop of tile i+1.
#include <stdlib.h>

#include "fr_common.cuh"
#include "sid_head.cuh"
#include "sm100_ptx.cuh"

namespace fr {

int* device_status_ptr();  // capi.cu

namespace gemm {

constexpr int kBlockM = 128;
constexpr int kBlockK = 128;  // bytes == e4m3 elements: one 128-byte swizzle span
constexpr int kUmmaK = 32;
// 2 control warps (TMA, MMA) + epilogue warps. The plain epilogue uses one warp per TMEM lane
// quadrant; the SwiGLU epilogue does ~40 instructions per element and gets four warps per quadrant
// (each takes one 32-column chunk) so that it still hides under the main loop.
template <int EPI>
struct EpiCfg {
  static constexpr int kWarps = (EPI == 1 || EPI == 3 || EPI == 4) ? 16 : 4;
  static constexpr int kEpiThreads = kWarps * 32;
  static constexpr int kThreads = 64 + kEpiThreads;
};

template <int BLOCK_N>
struct Cfg {
  static constexpr int kStageA = kBlockM * kBlockK;
  static constexpr int kStageB = BLOCK_N * kBlockK;
  static constexpr int kStageBytes = kStageA + kStageB;
  static constexpr int kStages = BLOCK_N == 256 ? 4 : (BLOCK_N == 128 ? 6 : 8);
  static constexpr int kTmemCols = 2 * BLOCK_N;  // two accumulator buffers (power of two >= 32)
  static constexpr int kScaleBytes = 2 * BLOCK_N * 4 * 2;  // scale_b and bias staging, double buffered
  static constexpr int kBarBytes = (2 * kStages + 4) * 8 + 16;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kScaleBytes + kBarBytes;
};

// `wide`: dst is 32-byte aligned, so a thread's chunk leaves as whole 32-byte sectors (rows are far apart:
// a 16-byte store fills half a sector per instruction).
template <typename OutT>
__device__ __forceinline__ void store_chunk32(OutT* dst, const float (&v)[32], int ncols_valid, bool wide);

template <>
__device__ __forceinline__ void store_chunk32<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[32], int nvalid,
                                                             bool wide) {
  if (nvalid >= 32) {
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) w[i] = pack_bf16(v[2 * i], v[2 * i + 1]);
    if (wide) {
      const uint32_t w0[8] = {w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]};
      const uint32_t w1[8] = {w[8], w[9], w[10], w[11], w[12], w[13], w[14], w[15]};
      ptx::st_global_v8(dst, w0);
      ptx::st_global_v8(dst + 16, w1);
    } else {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int i = 0; i < 4; ++i) d4[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < nvalid) dst[i] = __float2bfloat16_rn(v[i]);
  }
}

template <>
__device__ __forceinline__ void store_chunk32<float>(float* dst, const float (&v)[32], int nvalid, bool wide) {
  if (nvalid >= 32) {
    if (wide) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t w[8] = {__float_as_uint(v[8 * i]),     __float_as_uint(v[8 * i + 1]), __float_as_uint(v[8 * i + 2]),
                               __float_as_uint(v[8 * i + 3]), __float_as_uint(v[8 * i + 4]), __float_as_uint(v[8 * i + 5]),
                               __float_as_uint(v[8 * i + 6]), __float_as_uint(v[8 * i + 7])};
        ptx::st_global_v8(dst + 8 * i, w);
      }
    } else {
      float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
      for (int i = 0; i < 8; ++i) d4[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < nvalid) dst[i] = v[i];
  }
}

// Tile order: groups of kRasterGroup row blocks, column block slowest inside a
// group, so the tiles in flight at any time (one per SM or SM pair) cover a
// roughly square patch: each A row block is streamed from HBM once and the B
// column blocks of the patch stay in L2, also when A alone is larger than L2
// (the long-K down projection).
constexpr int kRasterGroup = 8;
struct TileCoord {
  int mb, nb;
};
__device__ __forceinline__ TileCoord tile_coord(int tile, int m_blocks, int n_blocks) {
  const int per_group = kRasterGroup * n_blocks;
  const int group = tile / per_group;
  const int first = group * kRasterGroup;
  const int rows = min(kRasterGroup, m_blocks - first);
  const int t = tile - group * per_group;
  TileCoord c;
  c.mb = first + t % rows;
  c.nb = t / rows;
  return c;
}

// EPI == 0: plain scaled output. EPI == 1 (BLOCK_N == 256, bf16 out): the weight rows
// are interleaved per tile as [128 gate channels | the 128 matching up channels];
// the epilogue rounds both to bf16 (exactly what the unfused GEMM would have
// stored), applies silu(gate) * up with the bf16 roundings of the unfused SwiGLU
// kernel, stores y [M, N/2] and folds max|y| of every row into row_amax (float
// bits, atomicMax on non-negative values).
template <int BLOCK_N, typename OutT, int EPI>
__global__ void __launch_bounds__(EpiCfg<EPI>::kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                OutT* __restrict__ out, int64_t ldo, const float* __restrict__ scale_a,
                const float* __restrict__ scale_b, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
                unsigned int* __restrict__ row_amax, const uint16_t* __restrict__ silu_table, int* status) {
  using C = Cfg<BLOCK_N>;
  constexpr int kEpiThreads = EpiCfg<EPI>::kEpiThreads;
  constexpr int kSplit = EpiCfg<EPI>::kWarps / 4;  // epilogue warps per lane quadrant
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled operand tiles need a 1024-byte aligned base.
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);

  float* sb_stage = reinterpret_cast<float*>(smem + C::kStages * C::kStageBytes);  // [2][BLOCK_N]
  float* bias_stage = sb_stage + 2 * BLOCK_N;                                      // [2][BLOCK_N]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes + C::kScaleBytes);
  const uint32_t bar_full = ptx::smem_u32(bars);                      // [kStages]
  const uint32_t bar_empty = bar_full + 8 * C::kStages;               // [kStages]
  const uint32_t bar_tfull = bar_empty + 8 * C::kStages;              // [2]
  const uint32_t bar_tempty = bar_tfull + 16;                         // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_blocks = (M + kBlockM - 1) / kBlockM;
  const int n_blocks = (N + BLOCK_N - 1) / BLOCK_N;
  const int num_tiles = m_blocks * n_blocks;
  const int num_kb = (K + kBlockK - 1) / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(bar_tfull + 8 * b, 1);
      ptx::mbar_init(bar_tempty + 8 * b, kEpiThreads / 32);
    }
    *abort_flag = 0;
    ptx::mbar_init_fence();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above touched only this CTA's shared / tensor memory: with a programmatic launch dependency it
  // ran while the previous kernel of the stream was still finishing; global memory is touched from here on
  ptx::griddep_wait();
  ptx::griddep_launch_dependents();

  if (warp == 0) {
    // ------------------------------ TMA producer ---------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, m_blocks, n_blocks);
        const int m0 = tc.mb * kBlockM;
        const int n0 = tc.nb * BLOCK_N;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = ptx::mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, status, 1);
          if (!ok) break;
          const uint32_t sa = base + stage * C::kStageBytes;
          const uint32_t sbm = sa + C::kStageA;
          ptx::mbar_expect_tx(bar_full + 8 * stage, C::kStageBytes);
          ptx::tma_load_2d(sa, &tmap_a, kb * kBlockK, m0, bar_full + 8 * stage);
          ptx::tma_load_2d(sbm, &tmap_b, kb * kBlockK, n0, bar_full + 8 * stage);
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer -----------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc(0u, 0u, kBlockM, BLOCK_N);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const uint32_t buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ok = ptx::mbar_wait(bar_tempty + 8 * buf, acc_phase ^ 1u, abort_flag, status, 2);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BLOCK_N;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = ptx::mbar_wait(bar_full + 8 * stage, phase, abort_flag, status, 3);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint32_t sa = base + stage * C::kStageBytes;
          const uint64_t a_desc = ptx::smem_desc_sw128(sa);
          const uint64_t b_desc = ptx::smem_desc_sw128(sa + C::kStageA);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            // +32 bytes along K inside the swizzled 128-byte row == +2 in the (addr >> 4) field
            ptx::mma_f8f6f4(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          ptx::tc_commit(bar_empty + 8 * stage);  // stage reusable once these MMAs have read it
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) ptx::tc_commit(bar_tfull + 8 * buf);  // accumulator complete
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue -------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    const int epi_tid = threadIdx.x - 64;
    const int part = (warp - 2) >> 2;  // which share of the column chunks this warp takes
    bool ok = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
      const TileCoord tc = tile_coord(tile, m_blocks, n_blocks);
      const int m0 = tc.mb * kBlockM;
      const int n0 = tc.nb * BLOCK_N;
      const uint32_t buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      float* sbs = sb_stage + buf * BLOCK_N;
      float* bss = bias_stage + buf * BLOCK_N;
      for (int i = epi_tid; i < BLOCK_N; i += kEpiThreads) {
        const int n = n0 + i;
        sbs[i] = n < N ? __ldg(scale_b + n) : 0.f;
        bss[i] = (bias != nullptr && n < N) ? __bfloat162float(bias[n]) : 0.f;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      const int row = m0 + quad * 32 + lane;
      const float sa = row < M ? __ldg(scale_a + row) : 0.f;
      int okw = 0;
      if (lane == 0) okw = ptx::mbar_wait(bar_tfull + 8 * buf, acc_phase, abort_flag, status, 4) ? 1 : 0;
      okw = __shfl_sync(0xffffffffu, okw, 0);
      if (!okw) { ok = false; break; }
      ptx::tc_fence_after();
      const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BLOCK_N;
      if constexpr (EPI == 0 || EPI == 2) {
        OutT* out_row = out + static_cast<int64_t>(row) * ldo + n0;
        const bool wide_out = (reinterpret_cast<uintptr_t>(out) & 31u) == 0 && (ldo * sizeof(OutT)) % 32 == 0;
#pragma unroll 1
        for (int c = part; c < BLOCK_N / 32; c += kSplit) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(taddr_row + c * 32, r);
          ptx::tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float t = __fmul_rn(__fmul_rn(__uint_as_float(r[j]), sa), sbs[c * 32 + j]);
            if (bias != nullptr) t = __fadd_rn(round_bf16(t), bss[c * 32 + j]);
            v[j] = t;
          }
          const int nvalid = N - (n0 + c * 32);
          if constexpr (EPI == 2) {
            // out is the residual stream, updated in place: bf16(bf16(x) + residual), as the
            // reference's fused add does on the rounded GEMM output
            if (row < M && nvalid > 0) {
              const __nv_bfloat16* res = reinterpret_cast<const __nv_bfloat16*>(out_row) + c * 32;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < nvalid) v[j] = __fadd_rn(round_bf16(v[j]), __bfloat162float(res[j]));
            }
          }
          if (row < M && nvalid > 0) store_chunk32<OutT>(out_row + c * 32, v, nvalid, wide_out);
        }
      } else {
        __nv_bfloat16* out_row = reinterpret_cast<__nv_bfloat16*>(out) + static_cast<int64_t>(row) * ldo + n0 / 2;
        float amax = 0.f;
#pragma unroll 1
        for (int c = part; c < BLOCK_N / 64; c += kSplit) {
          uint32_t rg[32], ru[32];
          ptx::tmem_ld_32x32(taddr_row + c * 32, rg);                 // gate channels
          ptx::tmem_ld_32x32(taddr_row + BLOCK_N / 2 + c * 32, ru);   // matching up channels
          ptx::tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float g = round_bf16(__fmul_rn(__fmul_rn(__uint_as_float(rg[j]), sa), sbs[c * 32 + j]));
            const float u = round_bf16(__fmul_rn(__fmul_rn(__uint_as_float(ru[j]), sa), sbs[BLOCK_N / 2 + c * 32 + j]));
            const float y = round_bf16(__fmul_rn(silu_bf16(g, silu_table), u));
            v[j] = y;
            amax = fmaxf(amax, fabsf(y));
          }
          if (row < M) store_chunk32<__nv_bfloat16>(out_row + c * 32, v, 32, false);
        }
        if (row < M) atomicMax(row_amax + row, __float_as_uint(amax));
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar_tempty + 8 * buf);
    }
  }

  // common exit: all roles converge, then the allocating warp frees TMEM
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // an aborted pipeline may still have TMA tiles in flight towards this
    // CTA's shared memory: give them (bounded) time to land before exiting
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// SwiGLU on 16 gate / 16 up accumulator columns of one row (one thread): returns max|y| and
// hands back the 16 bf16 results as two 16-byte pieces. Branch-free (inputs whose fast silu
// cannot be trusted take a predicated table load), so the 16 instruction chains interleave.
// sbg / sbu: the 16 per-channel scales of the gate / up columns in global memory (16-byte
// aligned; every thread reads the same addresses, so they come from L1). release_bar: 0, or the
// cluster address of the barrier to arrive on once the accumulator columns are in registers.
__device__ __forceinline__ float swiglu16(uint32_t taddr_g, uint32_t taddr_u, const float* __restrict__ sbg,
                                          const float* __restrict__ sbu, float sa,
                                          const uint16_t* __restrict__ silu_table, uint32_t release_bar, uint4& out0,
                                          uint4& out1) {
  uint32_t rg[16], ru[16];
  ptx::tmem_ld_32x16(taddr_g, rg);
  ptx::tmem_ld_32x16(taddr_u, ru);
  float sg[16], su[16];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(sbg) + q);
    const float4 b = __ldg(reinterpret_cast<const float4*>(sbu) + q);
    sg[4 * q] = a.x, sg[4 * q + 1] = a.y, sg[4 * q + 2] = a.z, sg[4 * q + 3] = a.w;
    su[4 * q] = b.x, su[4 * q + 1] = b.y, su[4 * q + 2] = b.z, su[4 * q + 3] = b.w;
  }
  ptx::tmem_ld_wait();
  if (release_bar != 0u) {  // last read of this accumulator buffer by this warp: hand it back now
    ptx::tc_fence_before();
    __syncwarp();
    if ((threadIdx.x & 31) == 0) ptx::mbar_arrive_cluster(release_bar);
  }
  uint32_t w[8];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float y2[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int jj = 2 * j + e;
      const float g = round_bf16(__fmul_rn(__fmul_rn(__uint_as_float(rg[jj]), sa), sg[jj]));
      const float u = round_bf16(__fmul_rn(__fmul_rn(__uint_as_float(ru[jj]), sa), su[jj]));
      y2[e] = __fmul_rn(silu_bf16(g, silu_table), u);
    }
    w[j] = pack_bf16(y2[0], y2[1]);
    amax = fmaxf(amax, fmaxf(fabsf(bf16lo(w[j])), fabsf(bf16hi(w[j]))));
  }
  out0 = make_uint4(w[0], w[1], w[2], w[3]);
  out1 = make_uint4(w[4], w[5], w[6], w[7]);
  return amax;
}

// Arguments of the qkv epilogue (EPI == 3): per-head RMSNorm + NeoX RoPE of the Q and K heads,
// Q written as bf16, K (rounded to bf16 first) and V written as e4m3 into their KV-pool slots: what
// fr_qk_norm_rope_kv_fp8 does to the qkv GEMM's bf16 output, applied to the accumulator tile.
struct QkvRope {
  const int64_t* pos;        // [M]
  const int64_t* loc;        // [M] KV-pool slot per row
  const __nv_bfloat16* qw;   // [128] q-norm weight
  const __nv_bfloat16* kw;   // [128] k-norm weight
  const float* cs;           // [max_pos, 128] = [cos(64) | sin(64)]
  __nv_bfloat16* q_out;      // [M, n_q * 128], row pitch ldq elements
  uint8_t* kc;               // e4m3 [slots, n_kv, 128], byte strides below
  uint8_t* vc;
  int64_t ldq, ck_s, ck_h, cv_s, cv_h;
  float eps;
  int max_pos, num_slots, n_q, n_kv;
  int wide;  // Q rows and cache rows are 32-byte aligned: 32-byte stores
};

// ---------------------------------------------------------------------------
// CTA-pair variant: cluster of 2 CTAs, pair tile 256 (M) x 256 (N).
// CTA r of the pair owns accumulator rows [m0 + 128 r, +128) and loads, per
// 128-byte k-block, its own 128 rows of A and rows [n0 + 128 r, +128) of B (32 KB
// per stage instead of 48 KB for the same tensor work per SM). The even CTA
// issues tcgen05.mma.cta_group::2 (M = 256, N = 256) for both SMs.
//   full[s]    lives in CTA 0; both CTAs' TMA loads credit their bytes to it
//   empty[s]   one per CTA; CTA 0's MMA thread commits to both
//   tfull[b]   one per CTA (accumulator buffer b complete); committed to both
//   tempty[b]  lives in CTA 0; the epilogue warps of both CTAs arrive on it
// Epilogue: every warp converts its 32 accumulator rows chunk by chunk, writes
// the chunk into a swizzled shared-memory staging tile and hands it to a TMA
// store (full 128-byte lines, clipped at the matrix edge by the hardware), so
// the output leaves the SM as bulk copies instead of per-thread 16-byte stores.
// ---------------------------------------------------------------------------
template <int EPI>
struct PairCfg {
  static constexpr int kBlockN = 256;
  static constexpr int kStageA = kBlockM * kBlockK;           // 16 KB
  static constexpr int kStageB = (kBlockN / 2) * kBlockK;     // 16 KB: this CTA's half of the B rows
  static constexpr int kStageBytes = kStageA + kStageB;
  static constexpr int kStages = 5;
  static constexpr int kTmemCols = 2 * kBlockN;
  // epilogue staging tiles for the TMA stores (EPI 2: three per warp, they also receive the residual)
  static constexpr int kOutStageBytes = (EPI == 2 ? 48 : 32) * 1024;
  static constexpr int kScaleBytes = 2 * kBlockN * 4 * 2;
  static constexpr int kResBars = 12;  // EPI 2: 4 epilogue warps x 3 staging tiles
  static constexpr int kBarBytes = (2 * kStages + 4 + kResBars) * 8 + 16;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kOutStageBytes + kScaleBytes + kBarBytes;
};

template <typename OutT, int EPI>
__global__ void __launch_bounds__(EpiCfg<EPI>::kThreads, 1)
gemm_fp8_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_out, const float* __restrict__ scale_a,
                     const float* __restrict__ scale_b, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
                     unsigned int* __restrict__ row_amax, const uint16_t* __restrict__ silu_table, const QkvRope rp,
                     const HeadEpi hp, int* status) {
  using C = PairCfg<EPI>;
  constexpr int BLOCK_N = C::kBlockN;
  constexpr int kEpiThreads = EpiCfg<EPI>::kEpiThreads;
  constexpr int kEpiWarps = EpiCfg<EPI>::kWarps;
  constexpr int kSplit = kEpiWarps / 4;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);

  uint8_t* out_stage = smem + C::kStages * C::kStageBytes;  // 1024-byte aligned
  float* sb_stage = reinterpret_cast<float*>(out_stage + C::kOutStageBytes);
  float* bias_stage = sb_stage + 2 * BLOCK_N;
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + C::kOutStageBytes + C::kScaleBytes);
  const uint32_t bar_full = ptx::smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * C::kStages;
  const uint32_t bar_tfull = bar_empty + 8 * C::kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  const uint32_t bar_res = bar_tempty + 16;  // [kResBars] residual tile landed (EPI 2)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 4 + C::kResBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  const int m_blocks = (M + 2 * kBlockM - 1) / (2 * kBlockM);  // pair tiles along M
  const int n_blocks = (N + BLOCK_N - 1) / BLOCK_N;
  const int num_tiles = m_blocks * n_blocks;
  const int num_kb = (K + kBlockK - 1) / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(bar_tfull + 8 * b, 1);
      ptx::mbar_init(bar_tempty + 8 * b, 2 * kEpiWarps);  // epilogue warps of both CTAs
    }
    for (int b = 0; b < C::kResBars; ++b) ptx::mbar_init(bar_res + 8 * b, EPI == 3 ? 4 : 1);
    *abort_flag = 0;
    ptx::mbar_init_fence();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
    ptx::prefetch_tmap(&tmap_out);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), C::kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  // neither CTA may signal the other's barriers before they are initialised
  ptx::cluster_arrive();
  ptx::cluster_wait();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  ptx::griddep_wait();  // see gemm_fp8_kernel
  ptx::griddep_launch_dependents();

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ---------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        const TileCoord tc = tile_coord(tile, m_blocks, n_blocks);
        const int m0 = tc.mb * (2 * kBlockM) + static_cast<int>(rank) * kBlockM;
        const int n0 = tc.nb * BLOCK_N + static_cast<int>(rank) * (BLOCK_N / 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = ptx::mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, status, 21);
          if (!ok) break;
          const uint32_t sa = base + stage * C::kStageBytes;
          const uint32_t full0 = ptx::mapa(bar_full + 8 * stage, 0);  // CTA 0 collects both CTAs' bytes
          if (rank == 0) ptx::mbar_expect_tx(bar_full + 8 * stage, 2 * C::kStageBytes);
          ptx::tma_load_2d_pair(sa, &tmap_a, kb * kBlockK, m0, full0);
          ptx::tma_load_2d_pair(sa + C::kStageA, &tmap_b, kb * kBlockK, n0, full0);
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (CTA 0 only) ----------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = ptx::make_idesc(0u, 0u, 2 * kBlockM, BLOCK_N);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++it) {
        const uint32_t buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ok = ptx::mbar_wait(bar_tempty + 8 * buf, acc_phase ^ 1u, abort_flag, status, 22);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BLOCK_N;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = ptx::mbar_wait(bar_full + 8 * stage, phase, abort_flag, status, 23);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint32_t sa = base + stage * C::kStageBytes;
          const uint64_t a_desc = ptx::smem_desc_sw128(sa);
          const uint64_t b_desc = ptx::smem_desc_sw128(sa + C::kStageA);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k)
            ptx::mma_f8f6f4_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          ptx::tc_commit_pair(ptx::mapa(bar_empty + 8 * stage, 0));  // stage reusable in both CTAs
          ptx::tc_commit_pair(ptx::mapa(bar_empty + 8 * stage, 1));
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          ptx::tc_commit_pair(ptx::mapa(bar_tfull + 8 * buf, 0));  // accumulator complete in both CTAs
          ptx::tc_commit_pair(ptx::mapa(bar_tfull + 8 * buf, 1));
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (both CTAs) -------------------
    const int quad = warp & 3;
    const int epi_tid = threadIdx.x - 64;
    const int part = (warp - 2) >> 2;
    bool ok = true;
    int it = 0;
    int xsel = 0;  // EPI 3: which exchange buffer the next sum-of-squares exchange uses
    if constexpr (EPI == 3) {
      // q- / k-norm weights as fp32 in shared memory, once per CTA
      float* wn = reinterpret_cast<float*>(out_stage);
      for (int i = epi_tid; i < 256; i += kEpiThreads)
        wn[i] = __bfloat162float(i < 128 ? rp.qw[i] : rp.kw[i - 128]);
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
    }
    // EPI 3: the values staged per tile (weight scales of the tile's 256 columns, cos / sin row of its first
    // row) are loaded one tile ahead into registers, so the barrier below never waits for global memory.
    float pre_sb = 0.f, pre_cs = 0.f;
    auto prefetch_tile = [&](int t) {
      if (t >= num_tiles) return;
      const TileCoord tn = tile_coord(t, m_blocks, n_blocks);
      if (epi_tid < BLOCK_N) {
        const int n = tn.nb * BLOCK_N + epi_tid;
        pre_sb = n < N ? __ldg(scale_b + n) : 0.f;
      } else if (epi_tid < BLOCK_N + 128) {
        const int mrow = tn.mb * (2 * kBlockM) + static_cast<int>(rank) * kBlockM;
        int64_t p0 = __ldg(rp.pos + min(mrow, M - 1));
        p0 = p0 < 0 ? 0 : (p0 >= rp.max_pos ? rp.max_pos - 1 : p0);
        pre_cs = __ldg(rp.cs + p0 * 128 + (epi_tid - BLOCK_N));
      }
    };
    if constexpr (EPI == 3) prefetch_tile(pair);
    for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++it) {
      const TileCoord tc = tile_coord(tile, m_blocks, n_blocks);
      const int m0 = tc.mb * (2 * kBlockM) + static_cast<int>(rank) * kBlockM;
      const int n0 = tc.nb * BLOCK_N;
      const uint32_t buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      float* sbs = sb_stage + buf * BLOCK_N;
      float* bss = bias_stage + buf * BLOCK_N;
      const int row = m0 + quad * 32 + lane;
      const float sa = row < M ? __ldg(scale_a + row) : 0.f;
      if constexpr (EPI == 3) {
        // The cos / sin row of the tile's first row is staged once per tile: the beams of a request decode at
        // one position, so nearly every row of the tile reads this row (from shared memory instead of sixteen
        // dependent 16-byte global loads per thread); a row at another position reads its own row as before.
        if (epi_tid < BLOCK_N) sbs[epi_tid] = pre_sb;
        else if (epi_tid < BLOCK_N + 128) reinterpret_cast<float*>(out_stage + 16384)[buf * 128 + epi_tid - BLOCK_N] = pre_cs;
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        prefetch_tile(tile + n_pairs);
      } else if constexpr (EPI != 1 && EPI != 4) {  // the SwiGLU and SID-head epilogues read their scales from global memory
        for (int i = epi_tid; i < BLOCK_N; i += kEpiThreads) {
          const int n = n0 + i;
          sbs[i] = n < N ? __ldg(scale_b + n) : 0.f;
          bss[i] = (bias != nullptr && n < N) ? __bfloat162float(bias[n]) : 0.f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      }
      int okw = 0;
      if (lane == 0) okw = ptx::mbar_wait(bar_tfull + 8 * buf, acc_phase, abort_flag, status, 24) ? 1 : 0;
      okw = __shfl_sync(0xffffffffu, okw, 0);
      if (!okw) { ok = false; break; }
      ptx::tc_fence_after();
      const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BLOCK_N;
      const int ewarp = warp - 2;
      const int row_base = m0 + quad * 32;  // first output row of this warp
      // The accumulator buffer goes back to the MMA warp as soon as its last column is in
      // registers, before any store or atomic of this tile is issued: the arrive has release
      // semantics and would otherwise wait for those to complete.
      const uint32_t tempty_remote = ptx::mapa(bar_tempty + 8 * buf, 0);
      if constexpr (EPI == 0) {
        // chunk = 128 bytes of output per row (64 bf16 or 32 f32 columns); two staging tiles per warp
        constexpr int kChunkCols = 128 / static_cast<int>(sizeof(OutT));
        constexpr int kLoads = kChunkCols / 32;
        uint8_t* stage0 = out_stage + ewarp * 8192;
#pragma unroll 1
        for (int c = 0; c < BLOCK_N / kChunkCols; ++c) {
          uint8_t* st = stage0 + (c & 1) * 4096;
          uint32_t w[32];  // 128 bytes of this thread's row
#pragma unroll
          for (int h = 0; h < kLoads; ++h) {
            uint32_t r[32];
            ptx::tmem_ld_32x32(taddr_row + c * kChunkCols + h * 32, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int col = c * kChunkCols + h * 32 + j;
              float t = __fmul_rn(__fmul_rn(__uint_as_float(r[j]), sa), sbs[col]);
              if (bias != nullptr) t = __fadd_rn(round_bf16(t), bss[col]);
              r[j] = __float_as_uint(t);
            }
            if constexpr (sizeof(OutT) == 4) {
#pragma unroll
              for (int j = 0; j < 32; ++j) w[j] = r[j];
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                w[h * 16 + j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            }
          }
          if (c == BLOCK_N / kChunkCols - 1) {
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(tempty_remote);
          }
          if (lane == 0) ptx::bulk_wait_read<1>();  // the store that last used this staging tile has read it
          __syncwarp();
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)  // 128-byte swizzle: 16-byte chunk index ^ (row & 7)
            *reinterpret_cast<uint4*>(st + lane * 128 + ((ch ^ (lane & 7)) << 4)) =
                make_uint4(w[4 * ch], w[4 * ch + 1], w[4 * ch + 2], w[4 * ch + 3]);
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row_base < M && n0 + c * kChunkCols < N) {
            ptx::tma_store_2d(&tmap_out, ptx::smem_u32(st), n0 + c * kChunkCols, row_base);
            ptx::bulk_commit();
          }
        }
      } else if constexpr (EPI == 2) {
        // out += : the output tile is the bf16 residual stream, updated in place. Chunk k of this
        // warp (counted across tiles) uses staging tile k % 3: the residual chunk is brought in
        // by a TMA load issued one chunk ahead, the sum goes back into the same tile and leaves
        // by a TMA store.
        constexpr int kChunkCols = 64;
        constexpr int kChunks = BLOCK_N / kChunkCols;
        uint8_t* stage0 = out_stage + ewarp * 12288;
        const uint32_t bar_w = bar_res + 8 * (ewarp * 3);
        auto issue_res = [&](int tile_i, int c, int kc) {  // lane 0 only
          const TileCoord tcn = tile_coord(tile_i, m_blocks, n_blocks);
          const int rb = tcn.mb * (2 * kBlockM) + static_cast<int>(rank) * kBlockM + quad * 32;
          const int cb = tcn.nb * BLOCK_N + c * kChunkCols;
          const uint32_t b = bar_w + 8 * (kc % 3);
          ptx::mbar_expect_tx(b, 4096);
          ptx::tma_load_2d(ptx::smem_u32(stage0 + (kc % 3) * 4096), &tmap_out, cb, rb, b);
        };
        if (it == 0 && lane == 0) issue_res(tile, 0, 0);
#pragma unroll 1
        for (int c = 0; c < kChunks; ++c) {
          const int kc = it * kChunks + c;
          uint8_t* st = stage0 + (kc % 3) * 4096;
          if (lane == 0) {
            // tile (kc + 1) % 3 was last used by chunk kc - 2: its store must have read it
            ptx::bulk_wait_read<1>();
            if (c + 1 < kChunks) issue_res(tile, c + 1, kc + 1);
            else if (tile + n_pairs < num_tiles) issue_res(tile + n_pairs, 0, kc + 1);
          }
          uint32_t w[32];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            ptx::tmem_ld_32x32(taddr_row + c * kChunkCols + h * 32, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int col = c * kChunkCols + h * 32 + 2 * j;
              w[h * 16 + j] = pack_bf16(__fmul_rn(__fmul_rn(__uint_as_float(r[2 * j]), sa), sbs[col]),
                                        __fmul_rn(__fmul_rn(__uint_as_float(r[2 * j + 1]), sa), sbs[col + 1]));
            }
          }
          if (c == kChunks - 1) {
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(tempty_remote);
          }
          int okr = 0;
          if (lane == 0) okr = ptx::mbar_wait(bar_w + 8 * (kc % 3), (kc / 3) & 1, abort_flag, status, 25) ? 1 : 0;
          okr = __shfl_sync(0xffffffffu, okr, 0);
          if (!okr) { ok = false; break; }
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {  // 128-byte swizzle: 16-byte chunk index ^ (row & 7)
            uint4* cell = reinterpret_cast<uint4*>(st + lane * 128 + ((ch ^ (lane & 7)) << 4));
            const uint4 rv = *cell;
            *cell = make_uint4(add_bf16x2(w[4 * ch], rv.x), add_bf16x2(w[4 * ch + 1], rv.y),
                               add_bf16x2(w[4 * ch + 2], rv.z), add_bf16x2(w[4 * ch + 3], rv.w));
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row_base < M && n0 + c * kChunkCols < N) {
            ptx::tma_store_2d(&tmap_out, ptx::smem_u32(st), n0 + c * kChunkCols, row_base);
            ptx::bulk_commit();
          }
        }
        if (!ok) break;
      } else if constexpr (EPI == 3) {
        // The tile is two whole heads of 128 columns. Warp part p of a lane quadrant takes head
        // p >> 1 of the tile: columns [32 s, 32 s + 32) and their rotary partners [64 + 32 s, +32),
        // s = p & 1; the two warps of a (quadrant, head) add their sums of squares through shared
        // memory (fp64, fixed order) behind a named barrier of their 64 threads. Each thread does
        // one head per tile, so the two heads of a tile are worked on at the same time.
        const float* wn = reinterpret_cast<const float*>(out_stage);  // [q-norm 128 | k-norm 128]
        double* xss = reinterpret_cast<double*>(out_stage + 1024);    // [2][4 quads][4 parts][32]
        const int p = part;
        const int hd = p >> 1, sh = p & 1;
        const bool row_ok = row < M;
        const int hg = n0 / 128 + hd;  // head index among [Q heads | K heads | V heads]
        const bool is_q = hg < rp.n_q;
        const bool is_k = !is_q && hg < rp.n_q + rp.n_kv;
        const int c0 = hd * 128 + 32 * sh;
        uint32_t a1[32], a2[32];
        ptx::tmem_ld_32x32(taddr_row + c0, a1);
        ptx::tmem_ld_32x32(taddr_row + c0 + 64, a2);
        // independent of the accumulators: the row's position / slot (they lead to dependent loads)
        int64_t ps = 0, slot = -1;
        if (row_ok && (is_q || is_k)) ps = __ldg(rp.pos + row);
        if (row_ok && !is_q) slot = __ldg(rp.loc + row);
        ps = ps < 0 ? 0 : (ps >= rp.max_pos ? rp.max_pos - 1 : ps);
        int64_t ps0 = __ldg(rp.pos + min(m0, M - 1));  // the position whose row was staged for this tile
        ps0 = ps0 < 0 ? 0 : (ps0 >= rp.max_pos ? rp.max_pos - 1 : ps0);
        const float* cp = (ps == ps0 ? reinterpret_cast<const float*>(out_stage + 16384) + buf * 128
                                     : rp.cs + ps * 128) + 32 * sh;
        ptx::tmem_ld_wait();
        {  // last read of this accumulator buffer by this warp
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive_cluster_relaxed(tempty_remote);
        }
        // the qkv GEMM's bf16 output values, in place (two values per conversion instruction)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const uint32_t p1 = pack_bf16(__fmul_rn(__fmul_rn(__uint_as_float(a1[i]), sa), sbs[c0 + i]),
                                        __fmul_rn(__fmul_rn(__uint_as_float(a1[i + 1]), sa), sbs[c0 + i + 1]));
          const uint32_t p2 = pack_bf16(__fmul_rn(__fmul_rn(__uint_as_float(a2[i]), sa), sbs[c0 + 64 + i]),
                                        __fmul_rn(__fmul_rn(__uint_as_float(a2[i + 1]), sa), sbs[c0 + 64 + i + 1]));
          a1[i] = p1 << 16; a1[i + 1] = p1 & 0xffff0000u;
          a2[i] = p2 << 16; a2[i + 1] = p2 & 0xffff0000u;
        }
        if (is_q || is_k) {
          // this thread's 64 squares as fp32 pairs (four chains of 16, merged pairwise): see SqSum
          SqSum sq[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            sq_add(sq[i & 3], __uint_as_float(a1[i]));
            sq_add(sq[i & 3], __uint_as_float(a2[i]));
          }
          sq_merge(sq[0], sq[1]);
          sq_merge(sq[2], sq[3]);
          sq_merge(sq[0], sq[2]);
          double* xs = xss + ((xsel * 16 + quad * 4 + hd * 2) * 32);
          xsel ^= 1;  // alternate buffers per exchange: use n + 2 is separated from use n by barrier n + 1
          xs[sh * 32 + lane] = sq_value(sq[0]);
          // the two warps of this (quadrant, head) meet; both take the same path through every tile
          asm volatile("bar.sync %0, 64;" ::"r"(2 + quad * 2 + hd) : "memory");
          double tot = xs[lane] + xs[32 + lane];
          // Both warps hold the same totals lane by lane, so they agree on whether some row needs the fp64 sum
          // (a total whose fp32 rounding the pairs cannot decide: rare) and repeat the exchange together.
          if (__any_sync(0xffffffffu, !sq_rounding_is_safe(tot))) {
            double d4[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const double l = static_cast<double>(__uint_as_float(a1[i])), hh = static_cast<double>(__uint_as_float(a2[i]));
              d4[i & 3] = fma(l, l, d4[i & 3]);
              d4[i & 3] = fma(hh, hh, d4[i & 3]);
            }
            double* xs2 = xss + ((xsel * 16 + quad * 4 + hd * 2) * 32);
            xsel ^= 1;
            xs2[sh * 32 + lane] = (d4[0] + d4[1]) + (d4[2] + d4[3]);
            asm volatile("bar.sync %0, 64;" ::"r"(2 + quad * 2 + hd) : "memory");
            tot = xs2[lane] + xs2[32 + lane];
          }
          const float var = static_cast<float>(tot / 128.0);
          const float rstd = rsqrt_rn(__fadd_rn(var, rp.eps));
          const float* w = wn + (is_q ? 0 : 128) + 32 * sh;
#pragma unroll
          for (int i0 = 0; i0 < 32; i0 += 8) {
            float cv[8], sv[8];
#pragma unroll
            for (int i = 0; i < 8; i += 4) {  // generic loads: cp points into shared or global memory
              const float4 c4 = *reinterpret_cast<const float4*>(cp + i0 + i);
              const float4 s4 = *reinterpret_cast<const float4*>(cp + 64 + i0 + i);
              cv[i] = c4.x; cv[i + 1] = c4.y; cv[i + 2] = c4.z; cv[i + 3] = c4.w;
              sv[i] = s4.x; sv[i + 1] = s4.y; sv[i + 2] = s4.z; sv[i + 3] = s4.w;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float xa = __fmul_rn(__fmul_rn(__uint_as_float(a1[i0 + i]), rstd), w[i0 + i]);
              const float xb = __fmul_rn(__fmul_rn(__uint_as_float(a2[i0 + i]), rstd), w[64 + i0 + i]);
              a1[i0 + i] = __float_as_uint(__fsub_rn(__fmul_rn(xa, cv[i]), __fmul_rn(xb, sv[i])));
              a2[i0 + i] = __float_as_uint(__fadd_rn(__fmul_rn(xb, cv[i]), __fmul_rn(xa, sv[i])));
            }
          }
        }
        if (is_q) {
          if (row_ok) {
            __nv_bfloat16* dst = rp.q_out + static_cast<int64_t>(row) * rp.ldq + hg * 128 + 32 * sh;
#pragma unroll
            for (int i = 0; i < 16; ++i) {  // packed in place: words 0..15 of a1 / a2 hold the 32 bf16 values
              a1[i] = pack_bf16(__uint_as_float(a1[2 * i]), __uint_as_float(a1[2 * i + 1]));
              a2[i] = pack_bf16(__uint_as_float(a2[2 * i]), __uint_as_float(a2[2 * i + 1]));
            }
            if (rp.wide) {
#pragma unroll
              for (int v = 0; v < 2; ++v) {
                const uint32_t w1[8] = {a1[8 * v], a1[8 * v + 1], a1[8 * v + 2], a1[8 * v + 3],
                                        a1[8 * v + 4], a1[8 * v + 5], a1[8 * v + 6], a1[8 * v + 7]};
                const uint32_t w2[8] = {a2[8 * v], a2[8 * v + 1], a2[8 * v + 2], a2[8 * v + 3],
                                        a2[8 * v + 4], a2[8 * v + 5], a2[8 * v + 6], a2[8 * v + 7]};
                ptx::st_global_v8(dst + 16 * v, w1);
                ptx::st_global_v8(dst + 64 + 16 * v, w2);
              }
            } else {
              uint4* d1 = reinterpret_cast<uint4*>(dst);
              uint4* d2 = reinterpret_cast<uint4*>(dst + 64);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                d1[v] = make_uint4(a1[4 * v], a1[4 * v + 1], a1[4 * v + 2], a1[4 * v + 3]);
                d2[v] = make_uint4(a2[4 * v], a2[4 * v + 1], a2[4 * v + 2], a2[4 * v + 3]);
              }
            }
          }
        } else {
          if (is_k) {  // K: round to bf16 first, as the reference does before the e4m3 cast
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const uint32_t p1 = pack_bf16(__uint_as_float(a1[i]), __uint_as_float(a1[i + 1]));
              const uint32_t p2 = pack_bf16(__uint_as_float(a2[i]), __uint_as_float(a2[i + 1]));
              a1[i] = p1 << 16; a1[i + 1] = p1 & 0xffff0000u;
              a2[i] = p2 << 16; a2[i + 1] = p2 & 0xffff0000u;
            }
          }
          if (row_ok && slot >= 0 && slot < rp.num_slots) {  // never write outside the pool
            uint8_t* dst = is_k ? (rp.kc + slot * rp.ck_s + (hg - rp.n_q) * rp.ck_h)
                                : (rp.vc + slot * rp.cv_s + (hg - rp.n_q - rp.n_kv) * rp.cv_h);
            uint32_t w1[8], w2[8];  // 32 e4m3 bytes of each rotary half: one full sector each
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              w1[j] = pack_e4m3x4(__uint_as_float(a1[4 * j]), __uint_as_float(a1[4 * j + 1]), __uint_as_float(a1[4 * j + 2]),
                                  __uint_as_float(a1[4 * j + 3]));
              w2[j] = pack_e4m3x4(__uint_as_float(a2[4 * j]), __uint_as_float(a2[4 * j + 1]), __uint_as_float(a2[4 * j + 2]),
                                  __uint_as_float(a2[4 * j + 3]));
            }
            if (rp.wide) {
              ptx::st_global_v8(dst + 32 * sh, w1);
              ptx::st_global_v8(dst + 64 + 32 * sh, w2);
            } else {
              uint4* d1 = reinterpret_cast<uint4*>(dst + 32 * sh);
              uint4* d2 = reinterpret_cast<uint4*>(dst + 64 + 32 * sh);
              d1[0] = make_uint4(w1[0], w1[1], w1[2], w1[3]);
              d1[1] = make_uint4(w1[4], w1[5], w1[6], w1[7]);
              d2[0] = make_uint4(w2[0], w2[1], w2[2], w2[3]);
              d2[1] = make_uint4(w2[4], w2[5], w2[6], w2[7]);
            }
          }
        }
      } else if constexpr (EPI == 4) {
        // SID head: row statistics + the allowed codes' logits; nothing else leaves the SM. The four warps of
        // a lane quadrant split the tile's 256 codes into four parts of 64 (kHeadParts), each with its own
        // statistics entry and its own share of the candidate records, so no exchange between warps is needed.
        constexpr int kChunks = (BLOCK_N / 32) / kSplit;  // 32-code chunks per warp and tile: 2
        const int cbase = part * kChunks;
        const bool row_ok = row < M;
        const int n_valid = N - n0;  // codes of this tile that exist (the last tile of a level may be short)
        bool live = false;
        int64_t midx = row;
        if (row_ok) {
          live = __ldg(hp.cum + row) != -INFINITY;
          if (hp.mask_index != nullptr) midx = __ldg(hp.mask_index + row);
        }
        bool all_codes = false, no_codes = !live;
        if (live && hp.mask_index != nullptr) {
          if (midx < 0) all_codes = true;
          else if (midx >= hp.mask_rows) no_codes = true;
          else if (hp.level_off != nullptr && __ldg(hp.level_off + midx) != hp.level_off_expected) no_codes = true;
        }
        uint32_t mw[kChunks];
        int cnt = 0;
#pragma unroll
        for (int j = 0; j < kChunks; ++j) {
          uint32_t wv = 0u;
          const int64_t wi = static_cast<int64_t>(hp.mask_word0) + (n0 >> 5) + cbase + j;
          if (all_codes) wv = 0xffffffffu;
          else if (!no_codes && wi < hp.mask_stride) wv = __ldg(hp.mask + midx * hp.mask_stride + wi);
          const int left = n_valid - 32 * (cbase + j);  // valid codes in this word
          if (left <= 0) wv = 0u;
          else if (left < 32) wv &= (1u << left) - 1u;
          mw[j] = wv;
          cnt += __popc(wv);
        }
        // one cursor update per warp: its 32 rows belong to one request (BW is a multiple of 32)
        int incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += y;
        }
        const int total = __shfl_sync(0xffffffffu, incl, 31);
        const int req = row_base / hp.BW;
        int base_pos = 0;
        if (total > 0) {
          if (lane == 0) base_pos = atomicAdd(hp.cand_count + req, total);
          base_pos = __shfl_sync(0xffffffffu, base_pos, 0);
        }
        int pos = base_pos + incl - cnt;
        uint2* cand_req = hp.cand + static_cast<int64_t>(req) * hp.cand_cap;
        const uint32_t flat0 =
            static_cast<uint32_t>(static_cast<int64_t>(row - req * hp.BW) * hp.idx_width + hp.idx_base + n0);
        bool dropped = false;
        float mx = -INFINITY, sum = 0.f;
        constexpr float kLog2e = 1.4426950408889634f;
#pragma unroll
        for (int cc = 0; cc < kChunks; ++cc) {
          const int c = cbase + cc;
          uint32_t r[32];
          ptx::tmem_ld_32x32(taddr_row + c * 32, r);
          ptx::tmem_ld_wait();
          if (cc == kChunks - 1) {  // last read of this accumulator buffer by this warp
            ptx::tc_fence_before();
            __syncwarp();
            // relaxed: the records and statistics of the previous tile are plain global stores still in flight
            if (lane == 0) ptx::mbar_arrive_cluster_relaxed(tempty_remote);
          }
          const int left = n_valid - 32 * c;
          float cm4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // independent chains
          // per-channel scales straight from global memory (every lane reads the same addresses: L1 broadcasts),
          // so that the sixteen epilogue warps need no CTA-wide barrier per tile
          const float* sbp = scale_b + n0 + c * 32;
          if (left >= 32) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float4 s4 = __ldg(reinterpret_cast<const float4*>(sbp + j));
              const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float t = __fmul_rn(__fmul_rn(__uint_as_float(r[j + e]), sa), sv[e]);
                r[j + e] = __float_as_uint(t);
                cm4[e] = fmaxf(cm4[e], t);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float t = -INFINITY;
              if (j < left) t = __fmul_rn(__fmul_rn(__uint_as_float(r[j]), sa), __ldg(sbp + j));
              r[j] = __float_as_uint(t);
              cm4[j & 3] = fmaxf(cm4[j & 3], t);
            }
          }
          const float cm = fmaxf(fmaxf(cm4[0], cm4[1]), fmaxf(cm4[2], cm4[3]));
          if (cm > mx) {  // rescale the running sum to the new maximum
            sum *= ex2_approx((mx - cm) * kLog2e);  // mx == -inf: sum is 0 and stays 0
            mx = cm;
          }
          if (mx != -INFINITY) {
            const float off = mx * kLog2e;
            float p4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 32; ++j) p4[j & 3] += ex2_approx(__fmaf_rn(__uint_as_float(r[j]), kLog2e, -off));
            sum += (p4[0] + p4[1]) + (p4[2] + p4[3]);
          }
          const uint32_t bits = mw[cc];
          if (bits != 0u) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if ((bits >> j) & 1u) {
                if (pos < hp.cand_cap) cand_req[pos] = make_uint2(r[j], flat0 + static_cast<uint32_t>(c * 32 + j));
                else dropped = true;
                ++pos;
              }
            }
          }
        }
        if (row_ok) {
          const int64_t o = (static_cast<int64_t>(tc.nb) * kSplit + part) * M + row;
          hp.tile_max[o] = mx;
          hp.tile_logsum[o] = logf(sum);  // -inf for a part without codes
        }
        if (dropped && atomicCAS(status, 0, FR_ERR_UNSUPPORTED) == 0) status[1] = 51;
      } else {
        // one 32-column chunk of y per warp and tile: 64-byte rows, 64-byte swizzle
        uint8_t* st = out_stage + ewarp * 2048;
        float amax = 0.f;
        const int c = part;
        // two halves of 16 columns (register budget: 18 warps leave 96 registers per thread)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int col = c * 32 + half * 16;
          uint4 o0, o1;
          amax = fmaxf(amax, swiglu16(taddr_row + col, taddr_row + BLOCK_N / 2 + col, scale_b + n0 + col,
                                      scale_b + n0 + BLOCK_N / 2 + col, sa, silu_table,
                                      half == 1 ? tempty_remote : 0u, o0, o1));
          if (half == 0) {  // the previous tile's store must have read the staging tile; by now it has
            if (lane == 0) ptx::bulk_wait_read<0>();
            __syncwarp();
          }
          // 64-byte swizzle: 16-byte chunk index ^ ((row >> 1) & 3)
          *reinterpret_cast<uint4*>(st + lane * 64 + (((half * 2) ^ ((lane >> 1) & 3)) << 4)) = o0;
          *reinterpret_cast<uint4*>(st + lane * 64 + (((half * 2 + 1) ^ ((lane >> 1) & 3)) << 4)) = o1;
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && row_base < M) {
          ptx::tma_store_2d(&tmap_out, ptx::smem_u32(st), n0 / 2 + c * 32, row_base);
          ptx::bulk_commit();
        }
        if (row < M) atomicMax(row_amax + row, __float_as_uint(amax));
      }
    }
  }

  if (warp >= 2 && lane == 0) ptx::bulk_wait_all();  // this warp's output tiles have been written
  // common exit: both CTAs of the pair converge before either frees TMEM or leaves
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// Split-K variant for few rows (a decode step of one request: M = 512). With so few
// row blocks the tiles of the kernels above cannot fill the GPU without re-reading A
// once per column tile from L2, and every CTA runs the whole K loop serially. Here a
// cluster of S CTAs (S in {1, 2, 4, 8}) owns one 128 x 256 output tile: every CTA
// runs the TMA -> tcgen05 pipeline over its own 1/S of the k-blocks, then the partial
// tiles are summed across the cluster through distributed shared memory: CTA q owns
// rows [q 128/S, (q+1) 128/S) of the tile; every CTA stores each of its accumulator
// rows (fp32) straight into the owner's shared memory (remote stores into the
// operand stages, idle by then; slot = sender rank), one cluster barrier, and each
// owner adds its S slots in rank order from local shared memory, scales, converts
// and stores. Deterministic, no workspace, no atomics, nothing remote after the
// barrier.
// EPI 0: out = scaled product (bf16 or f32). EPI 2: bf16 out += (in place, residual).
// ---------------------------------------------------------------------------
// TN = 256 or 128 columns per tile: the narrower tile halves the partial tile a CTA has to exchange, at the
// price of more operand bytes per CTA; the host picks per shape (pick_split_plan).
template <int TN>
struct SplitCfg {
  static constexpr int kTileM = kBlockM;  // 128
  static constexpr int kTileN = TN;
  static constexpr int kStageA = kTileM * kBlockK;  // 16 KB
  static constexpr int kStageB = kTileN * kBlockK;  // 32 / 16 KB
  static constexpr int kStageBytes = kStageA + kStageB;
  static constexpr int kStages = TN == 256 ? 4 : 6;  // 192 KB; the first 128 / 64 KB double as the reduction buffer
  static constexpr int kTmemCols = TN;               // one 128 x TN fp32 accumulator
  static constexpr int kRowBytes = TN * 4;           // one partial row in the reduction buffer
  static constexpr int kBarBytes = (2 * kStages + 1) * 8 + 16;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kBarBytes;
  static constexpr int kThreads = 192;
};

template <typename OutT, int EPI, int S, int TN>
__global__ void __launch_bounds__(SplitCfg<TN>::kThreads, 1)
gemm_fp8_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       OutT* __restrict__ out, int64_t ldo, const float* __restrict__ scale_a,
                       const float* __restrict__ scale_b, int M, int N, int K, int* status) {
  using C = SplitCfg<TN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  const uint32_t bar_full = ptx::smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * C::kStages;
  const uint32_t bar_tfull = bar_empty + 8 * C::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = static_cast<int>(ptx::cluster_ctarank());
  const int tile = blockIdx.x / S;
  const int m_blocks = (M + C::kTileM - 1) / C::kTileM;
  const int m0 = (tile % m_blocks) * C::kTileM;
  const int n0 = (tile / m_blocks) * C::kTileN;
  const int num_kb = (K + kBlockK - 1) / kBlockK;
  const int per = num_kb / S;  // the host picks S that divides the k-blocks
  const int kb0 = rank * per;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, 1);
    }
    ptx::mbar_init(bar_tfull, 1);
    *abort_flag = 0;
    ptx::mbar_init_fence();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  ptx::griddep_wait();  // see gemm_fp8_kernel
  ptx::griddep_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int i = 0; i < per; ++i) {
        if (!ptx::mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, status, 31)) break;
        const uint32_t sa = base + stage * C::kStageBytes;
        const int kx = (kb0 + i) * kBlockK;
        ptx::mbar_expect_tx(bar_full + 8 * stage, C::kStageBytes);
        ptx::tma_load_2d(sa, &tmap_a, kx, m0, bar_full + 8 * stage);
        ptx::tma_load_2d(sa + C::kStageA, &tmap_b, kx, n0, bar_full + 8 * stage);
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc(0u, 0u, kBlockM, C::kTileN);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int i = 0; i < per; ++i) {
        ok = ptx::mbar_wait(bar_full + 8 * stage, phase, abort_flag, status, 32);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t sa = base + stage * C::kStageBytes;
        const uint64_t a_desc = ptx::smem_desc_sw128(sa);
        const uint64_t b_desc = ptx::smem_desc_sw128(sa + C::kStageA);
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k)
          ptx::mma_f8f6f4(tmem_base, a_desc + 2u * k, b_desc + 2u * k, idesc, (i | k) != 0 ? 1u : 0u);
        ptx::tc_commit(bar_empty + 8 * stage);
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
      if (ok) ptx::tc_commit(bar_tfull);
    }
    __syncwarp();
  }

  // ---- cluster-wide reduction. Every thread of every CTA takes part in the cluster barriers;
  // the four epilogue warps do the work.
  // No CTA may receive partial rows before its own pipeline has stopped using the stages:
  // each CTA waits for its accumulator (all its MMAs, hence all its TMA loads, are done), then
  // the first cluster barrier says so to the others.
  const bool epi = warp >= 2;
  const int quad = warp & 3;
  const int epi_tid = threadIdx.x - 64;
  constexpr int rows_per = kBlockM / S;  // rows of the tile this CTA reduces
  if (epi) {
    int okw = 0;
    if (lane == 0) okw = ptx::mbar_wait(bar_tfull, 0, abort_flag, status, 33) ? 1 : 0;
    okw = __shfl_sync(0xffffffffu, okw, 0);
    (void)okw;  // on a time-out the status word is set; the barriers below are still honoured
    ptx::tc_fence_after();
  }
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (epi) {
    // accumulator row r -> owner CTA r / rows_per, slot `rank`, fp32 [rows_per][4 TN bytes] per
    // slot, 16-byte pieces XOR-swizzled by (row & 7) (conflict-free for the stores and the loads)
    const int r = quad * 32 + lane;
    const int owner = r / rows_per;
    const int rl = r % rows_per;
    const uint32_t dst_row = ptx::mapa(base + (rank * rows_per + rl) * C::kRowBytes, owner);
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
    for (int c = 0; c < C::kTileN / 32; ++c) {
      uint32_t v[32];
      ptx::tmem_ld_32x32(taddr + c * 32, v);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 8; ++j)
        ptx::st_cluster_u32x4(dst_row + (((c * 8 + j) ^ (rl & 7)) << 4), v[4 * j], v[4 * j + 1], v[4 * j + 2],
                              v[4 * j + 3]);
    }
  }
  ptx::cluster_arrive();  // release: the remote stores above; acquire: the other CTAs' into this one
  ptx::cluster_wait();
  if (epi) {
    constexpr int kPieces = rows_per * (C::kTileN / 4) / 128;  // 16-byte pieces per thread: 64 / S
    constexpr int kBatch = kPieces < 8 ? kPieces : 8;
#pragma unroll 1
    for (int b0 = 0; b0 < kPieces; b0 += kBatch) {
      float sav[kBatch];
      float4 sbv[kBatch];
      uint2 resv[kBatch];  // EPI 2: the residual piece, fetched with the other loads
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const int idx = (b0 + b) * 128 + epi_tid;
        const int rl = idx / (C::kTileN / 4);
        const int ch = idx % (C::kTileN / 4);
        const int row = m0 + rank * rows_per + rl;
        const int col = n0 + ch * 4;
        sav[b] = row < M ? __ldg(scale_a + row) : 0.f;
        sbv[b].x = col + 0 < N ? __ldg(scale_b + col + 0) : 0.f;
        sbv[b].y = col + 1 < N ? __ldg(scale_b + col + 1) : 0.f;
        sbv[b].z = col + 2 < N ? __ldg(scale_b + col + 2) : 0.f;
        sbv[b].w = col + 3 < N ? __ldg(scale_b + col + 3) : 0.f;
        resv[b] = make_uint2(0u, 0u);
        if constexpr (EPI == 2) {
          if (row < M && col + 4 <= N)
            resv[b] = *reinterpret_cast<const uint2*>(out + static_cast<int64_t>(row) * ldo + col);
        }
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const int idx = (b0 + b) * 128 + epi_tid;
        const int rl = idx / (C::kTileN / 4);
        const int ch = idx % (C::kTileN / 4);
        const uint8_t* src = smem + rl * C::kRowBytes + ((ch ^ (rl & 7)) << 4);
        float4 sum = *reinterpret_cast<const float4*>(src);
#pragma unroll
        for (int pr = 1; pr < S; ++pr) {
          const float4 v = *reinterpret_cast<const float4*>(src + pr * rows_per * C::kRowBytes);
          sum.x = __fadd_rn(sum.x, v.x);
          sum.y = __fadd_rn(sum.y, v.y);
          sum.z = __fadd_rn(sum.z, v.z);
          sum.w = __fadd_rn(sum.w, v.w);
        }
        const int row = m0 + rank * rows_per + rl;
        const int col = n0 + ch * 4;
        if (row < M && col < N) {
          const float sa = sav[b];
          float o[4] = {__fmul_rn(__fmul_rn(sum.x, sa), sbv[b].x), __fmul_rn(__fmul_rn(sum.y, sa), sbv[b].y),
                        __fmul_rn(__fmul_rn(sum.z, sa), sbv[b].z), __fmul_rn(__fmul_rn(sum.w, sa), sbv[b].w)};
          OutT* dst = out + static_cast<int64_t>(row) * ldo + col;
          if constexpr (EPI == 2) {
            if (col + 4 <= N) {
              o[0] = __fadd_rn(round_bf16(o[0]), bf16lo(resv[b].x));
              o[1] = __fadd_rn(round_bf16(o[1]), bf16hi(resv[b].x));
              o[2] = __fadd_rn(round_bf16(o[2]), bf16lo(resv[b].y));
              o[3] = __fadd_rn(round_bf16(o[3]), bf16hi(resv[b].y));
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (col + j < N)
                  o[j] = __fadd_rn(round_bf16(o[j]), __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(dst)[j]));
            }
          }
          if (col + 4 <= N) {
            if constexpr (sizeof(OutT) == 4) {
              *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
            } else {
              *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (col + j < N) {
                if constexpr (sizeof(OutT) == 4) dst[j] = o[j];
                else dst[j] = __float2bfloat16_rn(o[j]);
              }
            }
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
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// e4m3 matrix [rows, cols] with row pitch `ld` bytes; box = 128 bytes x box_rows, 128-byte swizzle.
static int make_tmap_u8(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return FR_ERR_CUDA;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FR_OK : FR_ERR_CUDA;
}

// Output matrix [rows, cols] of 2- or 4-byte elements, row pitch `ld` elements; box = box_cols x 32 rows.
static int make_tmap_out(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t ld, int elem_bytes,
                         int box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return FR_ERR_CUDA;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), 32};
  cuuint32_t estr[2] = {1, 1};
  const int inner = box_cols * elem_bytes;
  const CUtensorMapSwizzle sw = inner == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUresult r = fn(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FR_OK : FR_ERR_CUDA;
}

static int sm_count() { return device_sm_count(); }

// Programmatic dependent launch for the decode step of few rows, where a GEMM's prologue (barrier set-up,
// tensor-memory allocation, descriptor prefetch) and the launch gap are a large share of its few
// microseconds: the kernel may then start while its predecessor in the stream is finishing and waits
// (griddepcontrol.wait) before it touches global memory. FR_GEMM_PDL=0/1 overrides the row threshold.
static bool use_pdl(int M) {
  static int forced = []() {
    const char* e = getenv("FR_GEMM_PDL");
    return e ? (e[0] == '0' ? 0 : 1) : -1;
  }();
  if (forced >= 0) return forced == 1;
  return M <= 2048;
}
static int fill_launch_attrs(cudaLaunchAttribute* attr, int cluster, bool pdl) {
  int n = 0;
  if (cluster > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  return n;
}

// Tile-width choice: whole waves of 128 x BLOCK_N tiles over the SMs, discounted
// by how far a narrower tile falls below the tensor-pipe rate (a 128x64 tile
// needs 192 B/clk of shared-memory operand reads against 128 B/clk available).
static int pick_block_n(int M, int N) {
  const int sms = sm_count();
  const int cand[3] = {256, 128, 64};
  const double rate[3] = {1.0, 0.95, 0.65};
  double best = -1.0;
  int best_n = 128;
  for (int i = 0; i < 3; ++i) {
    const int64_t tiles = static_cast<int64_t>(ceil_div(M, kBlockM)) * ceil_div(N, cand[i]);
    const int64_t waves = (tiles + sms - 1) / sms;
    const double useful = static_cast<double>(N) / (static_cast<double>(ceil_div(N, cand[i])) * cand[i]);
    const double eff = static_cast<double>(tiles) / static_cast<double>(waves * sms) * rate[i] * useful;
    if (eff > best + 1e-9) { best = eff; best_n = cand[i]; }
  }
  return best_n;
}

template <int BLOCK_N, typename OutT, int EPI = 0>
static int launch(const void* a, const void* b, const float* sa, const float* sb, const void* bias, void* out,
                  int64_t ldo, int M, int N, int K, int64_t lda, int64_t ldb, cudaStream_t stream,
                  unsigned int* row_amax = nullptr) {
  using C = Cfg<BLOCK_N>;
  CUtensorMap ta, tb;
  int st = make_tmap_u8(&ta, a, M, K, lda, kBlockM);
  if (st != FR_OK) return st;
  st = make_tmap_u8(&tb, b, N, K, ldb, BLOCK_N);
  if (st != FR_OK) return st;
  auto kern = gemm_fp8_kernel<BLOCK_N, OutT, EPI>;
  static PerDeviceFlag attr_done;  // per template instantiation and device
  if (ensure_dyn_smem(attr_done, kern, C::kSmemBytes) != FR_OK) return FR_ERR_CUDA;
  int* status = device_status_ptr();
  if (!status) return FR_ERR_CUDA;
  const uint16_t* table = EPI == 1 ? silu_table_ptr(stream) : nullptr;
  if (EPI == 1 && !table) return FR_ERR_CUDA;
  const int tiles = ceil_div(M, kBlockM) * ceil_div(N, BLOCK_N);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(EpiCfg<EPI>::kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  cfg.attrs = attr;
  cfg.numAttrs = fill_launch_attrs(attr, 1, use_pdl(M));
  if (cudaLaunchKernelEx(&cfg, kern, ta, tb, static_cast<OutT*>(out), ldo, sa, sb, static_cast<const __nv_bfloat16*>(bias),
                         M, N, K, row_amax, table, status) != cudaSuccess) {
    cudaGetLastError();
    return FR_ERR_CUDA;
  }
  return FR_OK;
}

template <typename OutT, int EPI>
static int launch_pair(const void* a, const void* b, const float* sa, const float* sb, const void* bias, void* out,
                       int64_t ldo, int M, int N, int K, int64_t lda, int64_t ldb, cudaStream_t stream,
                       unsigned int* row_amax = nullptr, const QkvRope& rp = QkvRope{},
                       const HeadEpi& hp = HeadEpi{}) {
  using C = PairCfg<EPI>;
  CUtensorMap ta, tb;
  int st = make_tmap_u8(&ta, a, M, K, lda, kBlockM);
  if (st != FR_OK) return st;
  st = make_tmap_u8(&tb, b, N, K, ldb, C::kBlockN / 2);
  if (st != FR_OK) return st;
  CUtensorMap to;
  if (EPI == 1) st = make_tmap_out(&to, out, M, N / 2, ldo, 2, 32);
  else if (EPI == 4) st = make_tmap_out(&to, hp.tile_max, 32, 32, 32, 4, 32);  // not used by this epilogue; a valid target
  else st = make_tmap_out(&to, out, M, EPI == 3 ? rp.n_q * 128 : N, ldo, static_cast<int>(sizeof(OutT)),
                          128 / static_cast<int>(sizeof(OutT)));
  if (st != FR_OK) return st;
  auto kern = gemm_fp8_pair_kernel<OutT, EPI>;
  static PerDeviceFlag attr_done;  // per template instantiation and device
  if (ensure_dyn_smem(attr_done, kern, C::kSmemBytes) != FR_OK) return FR_ERR_CUDA;
  int* status = device_status_ptr();
  if (!status) return FR_ERR_CUDA;
  const uint16_t* table = EPI == 1 ? silu_table_ptr(stream) : nullptr;
  if (EPI == 1 && !table) return FR_ERR_CUDA;
  const int tiles = ceil_div(M, 2 * kBlockM) * ceil_div(N, C::kBlockN);
  const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(EpiCfg<EPI>::kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  cfg.attrs = attr;
  cfg.numAttrs = fill_launch_attrs(attr, 2, use_pdl(M));
  if (cudaLaunchKernelEx(&cfg, kern, ta, tb, to, sa, sb, static_cast<const __nv_bfloat16*>(bias), M, N, K, row_amax,
                         table, rp, hp, status) != cudaSuccess) {
    cudaGetLastError();
    return FR_ERR_CUDA;
  }
  return FR_OK;
}

// CTA pairs pay off once there are several waves of 256 x 256 tiles; FR_GEMM_PAIR=0/1 overrides.
static bool use_pair(int M, int N) {
  static int forced = []() {
    const char* e = getenv("FR_GEMM_PAIR");
    return e ? (e[0] == '0' ? 0 : 1) : -1;
  }();
  if (forced >= 0) return forced == 1;
  const int64_t tiles = static_cast<int64_t>(ceil_div(M, 2 * kBlockM)) * ceil_div(N, PairCfg<0>::kBlockN);
  // several waves of pair tiles, or — for the few rows of a one-request step — at least one pair tile per SM
  // pair (measured at 512 rows: the gate_up shape, 96 pair tiles, 18.2 us against 20.4 us with 128 x 256 tiles)
  return tiles >= 3 * (sm_count() / 2) || (M <= 1024 && M > kBlockM && tiles >= sm_count() / 2);
}

// Split-K over a cluster. A plan is the number of CTAs S in {8, 4, 2} per tile (it divides the k-blocks,
// leaves each CTA at least two of them, tiles x S fits the SM count) and the tile width (256 or 128
// columns). Among the plans that fit, the cheapest by the two rates measured for a 512-row step wins: a CTA
// pulls its operands at about 48 bytes per clock, and the partial tiles cross the cluster at about 11 bytes
// per clock and SM whichever instruction moves them. splits = 1 (tile 256) when no S fits, 0 when the shape
// has too many rows or tiles for this kernel. `force_tn` (128 / 256) restricts the width.
struct SplitPlan {
  int splits;
  int tile_n;
};
static SplitPlan pick_split_plan(int M, int N, int K, int force_tn = 0) {
  const int num_kb = ceil_div(K, kBlockK);
  SplitPlan best{0, 256};
  double best_cost = 0.0;
  bool any_width = false;
  for (int tn = 256; tn >= 128; tn >>= 1) {
    if (force_tn != 0 && tn != force_tn) continue;
    const int64_t tiles = static_cast<int64_t>(ceil_div(M, kBlockM)) * ceil_div(N, tn);
    if (M > 1024 || tiles > sm_count()) continue;
    any_width = true;
    for (int s = 8; s >= 2; s >>= 1) {
      if (num_kb % s != 0 || num_kb / s < 2 || tiles * s > sm_count()) continue;
      const double feed = static_cast<double>(kBlockM + tn) * kBlockK * (num_kb / s) / 48.0;
      const double exchange = static_cast<double>(kBlockM) * tn * 4.0 * (s - 1) / s / 11.0;
      const double cost = feed + exchange;
      if (best.splits == 0 || cost < best_cost) {
        best = SplitPlan{s, tn};
        best_cost = cost;
      }
    }
  }
  if (best.splits == 0 && any_width) best = SplitPlan{1, force_tn == 128 ? 128 : 256};
  return best;
}

// Chosen by itself only for long reductions (K >= 4096: the down projection of a one-request
// step), where the serial K loop of a lone CTA costs more than the exchange of partial tiles;
// for shorter K the kernels above are faster.
static SplitPlan auto_split_plan(int M, int N, int K) {
  if (ceil_div(K, kBlockK) < 32) return SplitPlan{0, 256};
  const SplitPlan p = pick_split_plan(M, N, K);
  return p.splits >= 2 ? p : SplitPlan{0, 256};
}

// block_n_hint of the GEMM entry points: 1024 = split-K, plan chosen; 1024 + 128 / 1024 + 256 = split-K with
// that tile width; 0 = split-K only where auto_split_plan says so.
static SplitPlan split_plan_for_hint(int block_n_hint, int M, int N, int K) {
  if (block_n_hint == 0) return auto_split_plan(M, N, K);
  SplitPlan p{0, 256};
  if (block_n_hint == 1024) p = pick_split_plan(M, N, K);
  else if (block_n_hint == 1024 + 128) p = pick_split_plan(M, N, K, 128);
  else if (block_n_hint == 1024 + 256) p = pick_split_plan(M, N, K, 256);
  else return p;
  if (p.splits == 0) p.splits = 1;  // asked for by name: run it unsplit rather than refuse
  return p;
}
static bool is_split_hint(int h) { return h == 1024 || h == 1024 + 128 || h == 1024 + 256; }

template <typename OutT, int EPI, int TN>
static int launch_splitk_tn(const void* a, const void* b, const float* sa, const float* sb, void* out, int64_t ldo,
                            int M, int N, int K, int64_t lda, int64_t ldb, int splits, cudaStream_t stream) {
  using C = SplitCfg<TN>;
  CUtensorMap ta, tb;
  int st = make_tmap_u8(&ta, a, M, K, lda, kBlockM);
  if (st != FR_OK) return st;
  st = make_tmap_u8(&tb, b, N, K, ldb, C::kTileN);
  if (st != FR_OK) return st;
  using Kern = void (*)(const CUtensorMap, const CUtensorMap, OutT*, int64_t, const float*, const float*, int, int, int,
                        int*);
  Kern kern = nullptr;
  switch (splits) {
    case 1: kern = gemm_fp8_splitk_kernel<OutT, EPI, 1, TN>; break;
    case 2: kern = gemm_fp8_splitk_kernel<OutT, EPI, 2, TN>; break;
    case 4: kern = gemm_fp8_splitk_kernel<OutT, EPI, 4, TN>; break;
    case 8: kern = gemm_fp8_splitk_kernel<OutT, EPI, 8, TN>; break;
    default: return FR_ERR_UNSUPPORTED;
  }
  static PerDeviceFlag attr_done[9];  // per split count and device (one array per OutT, EPI, TN)
  if (ensure_dyn_smem(attr_done[splits], kern, C::kSmemBytes) != FR_OK) return FR_ERR_CUDA;
  int* status = device_status_ptr();
  if (!status) return FR_ERR_CUDA;
  const int tiles = ceil_div(M, C::kTileM) * ceil_div(N, C::kTileN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * splits);
  cfg.blockDim = dim3(C::kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  cfg.attrs = attr;
  cfg.numAttrs = fill_launch_attrs(attr, splits, use_pdl(M));
  if (cudaLaunchKernelEx(&cfg, kern, ta, tb, static_cast<OutT*>(out), ldo, sa, sb, M, N, K, status) != cudaSuccess) {
    cudaGetLastError();
    return FR_ERR_CUDA;
  }
  return FR_OK;
}

template <typename OutT, int EPI>
static int launch_splitk(const void* a, const void* b, const float* sa, const float* sb, void* out, int64_t ldo, int M,
                         int N, int K, int64_t lda, int64_t ldb, SplitPlan plan, cudaStream_t stream) {
  if (plan.tile_n == 128)
    return launch_splitk_tn<OutT, EPI, 128>(a, b, sa, sb, out, ldo, M, N, K, lda, ldb, plan.splits, stream);
  return launch_splitk_tn<OutT, EPI, 256>(a, b, sa, sb, out, ldo, M, N, K, lda, ldb, plan.splits, stream);
}

}  // namespace gemm

// The head GEMM with the SID-head epilogue (sid_head.cuh); called by fr_sid_head_topk.
int launch_head_gemm(const void* a, const void* b, const float* sa, const float* sb, int M, int N, int K, int64_t lda,
                     int64_t ldb, const HeadEpi& hp, cudaStream_t stream) {
  return gemm::launch_pair<float, 4>(a, b, sa, sb, nullptr, nullptr, 0, M, N, K, lda, ldb, stream, nullptr,
                                     gemm::QkvRope{}, hp);
}

}  // namespace fr

using namespace fr;

extern "C" int fr_gemm_fp8_w8a8(const void* a, const void* b, const float* scale_a, const float* scale_b,
                                const void* bias, void* out, int out_is_f32, int M, int N, int K, int64_t lda,
                                int64_t ldb, int64_t ldo, int block_n_hint, cudaStream_t stream) {
  FR_CHECK_ARG(M >= 0 && N > 0 && K > 0);
  if (M == 0) return FR_OK;
  FR_CHECK_ARG(a && b && scale_a && scale_b && out);
  // TMA: 16-byte aligned base and row pitch; vector stores: 16-byte aligned output rows
  FR_CHECK_ARG(aligned16(a) && aligned16(b) && aligned16(out));
  FR_CHECK_ARG(lda >= K && ldb >= K && ldo >= N && lda % 16 == 0 && ldb % 16 == 0);
  FR_CHECK_ARG(out_is_f32 ? (ldo % 4 == 0) : (ldo % 8 == 0));
  FR_CHECK_ARG(K % 16 == 0);
  FR_CHECK_SUPPORTED(out_is_f32 ? (bias == nullptr) : true);
  if (bias == nullptr && (gemm::is_split_hint(block_n_hint) || block_n_hint == 0)) {
    const gemm::SplitPlan plan = gemm::split_plan_for_hint(block_n_hint, M, N, K);
    if (plan.splits >= 1)
      return out_is_f32 ? gemm::launch_splitk<float, 0>(a, b, scale_a, scale_b, out, ldo, M, N, K, lda, ldb, plan,
                                                        stream)
                        : gemm::launch_splitk<__nv_bfloat16, 0>(a, b, scale_a, scale_b, out, ldo, M, N, K, lda, ldb,
                                                                plan, stream);
  }
  if (block_n_hint == 512 || (block_n_hint == 0 && gemm::use_pair(M, N))) {
    return out_is_f32 ? gemm::launch_pair<float, 0>(a, b, scale_a, scale_b, bias, out, ldo, M, N, K, lda, ldb, stream)
                      : gemm::launch_pair<__nv_bfloat16, 0>(a, b, scale_a, scale_b, bias, out, ldo, M, N, K, lda, ldb,
                                                            stream);
  }
  int bn = block_n_hint;
  if (bn != 64 && bn != 128 && bn != 256) bn = gemm::pick_block_n(M, N);
#define FR_GEMM_CASE(BN)                                                                                          \
  case BN:                                                                                                        \
    return out_is_f32 ? gemm::launch<BN, float>(a, b, scale_a, scale_b, bias, out, ldo, M, N, K, lda, ldb, stream) \
                      : gemm::launch<BN, __nv_bfloat16>(a, b, scale_a, scale_b, bias, out, ldo, M, N, K, lda, ldb, stream)
  switch (bn) {
    FR_GEMM_CASE(256);
    FR_GEMM_CASE(128);
    FR_GEMM_CASE(64);
    default: break;
  }
#undef FR_GEMM_CASE
  return FR_ERR_UNSUPPORTED;
}

extern "C" int fr_gemm_fp8_silu_mul(const void* a, const void* b_interleaved, const float* scale_a,
                                    const float* scale_b_interleaved, void* y_out, float* row_amax, int M, int N,
                                    int K, int64_t lda, int64_t ldb, int64_t ldo, int mode, cudaStream_t stream) {
  FR_CHECK_ARG(M >= 0 && N > 0 && K > 0);
  if (M == 0) return FR_OK;
  FR_CHECK_ARG(a && b_interleaved && scale_a && scale_b_interleaved && y_out && row_amax);
  FR_CHECK_SUPPORTED(N % 256 == 0);
  FR_CHECK_ARG(aligned16(a) && aligned16(b_interleaved) && aligned16(y_out) && aligned16(scale_b_interleaved));
  FR_CHECK_ARG(lda >= K && ldb >= K && ldo >= N / 2 && lda % 16 == 0 && ldb % 16 == 0 && ldo % 8 == 0 && K % 16 == 0);
  if (mode == 2 || (mode == 0 && gemm::use_pair(M, N)))
    return gemm::launch_pair<__nv_bfloat16, 1>(a, b_interleaved, scale_a, scale_b_interleaved, nullptr, y_out, ldo, M,
                                               N, K, lda, ldb, stream, reinterpret_cast<unsigned int*>(row_amax));
  return gemm::launch<256, __nv_bfloat16, 1>(a, b_interleaved, scale_a, scale_b_interleaved, nullptr, y_out, ldo, M, N,
                                             K, lda, ldb, stream, reinterpret_cast<unsigned int*>(row_amax));
}

extern "C" int fr_gemm_fp8_w8a8_add(const void* a, const void* b, const float* scale_a, const float* scale_b,
                                    void* residual_inout, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldr,
                                    int block_n_hint, cudaStream_t stream) {
  FR_CHECK_ARG(M >= 0 && N > 0 && K > 0);
  if (M == 0) return FR_OK;
  FR_CHECK_ARG(a && b && scale_a && scale_b && residual_inout);
  FR_CHECK_ARG(aligned16(a) && aligned16(b) && aligned16(residual_inout));
  FR_CHECK_ARG(lda >= K && ldb >= K && ldr >= N && lda % 16 == 0 && ldb % 16 == 0 && ldr % 8 == 0 && K % 16 == 0);
  if (gemm::is_split_hint(block_n_hint) || block_n_hint == 0) {
    const gemm::SplitPlan plan = gemm::split_plan_for_hint(block_n_hint, M, N, K);
    if (plan.splits >= 1)
      return gemm::launch_splitk<__nv_bfloat16, 2>(a, b, scale_a, scale_b, residual_inout, ldr, M, N, K, lda, ldb, plan,
                                                   stream);
  }
  if (block_n_hint == 512 || (block_n_hint == 0 && gemm::use_pair(M, N)))
    return gemm::launch_pair<__nv_bfloat16, 2>(a, b, scale_a, scale_b, nullptr, residual_inout, ldr, M, N, K, lda, ldb,
                                               stream);
  int bn = block_n_hint;
  if (bn != 64 && bn != 128 && bn != 256) bn = gemm::pick_block_n(M, N);
  switch (bn) {
    case 256:
      return gemm::launch<256, __nv_bfloat16, 2>(a, b, scale_a, scale_b, nullptr, residual_inout, ldr, M, N, K, lda,
                                                 ldb, stream);
    case 128:
      return gemm::launch<128, __nv_bfloat16, 2>(a, b, scale_a, scale_b, nullptr, residual_inout, ldr, M, N, K, lda,
                                                 ldb, stream);
    case 64:
      return gemm::launch<64, __nv_bfloat16, 2>(a, b, scale_a, scale_b, nullptr, residual_inout, ldr, M, N, K, lda,
                                                ldb, stream);
    default: break;
  }
  return FR_ERR_UNSUPPORTED;
}

extern "C" int fr_gemm_fp8_qkv_rope(const void* a, const void* b, const float* scale_a, const float* scale_b, void* q_out,
                                    int64_t ldq, int M, int n_q, int n_kv, int head_dim, int K, int64_t lda, int64_t ldb,
                                    const int64_t* positions, const int64_t* loc, const void* q_weight,
                                    const void* k_weight, float eps, const float* cos_sin, int max_pos, void* k_cache,
                                    void* v_cache, int64_t ck_s, int64_t ck_h, int64_t cv_s, int64_t cv_h, int num_slots,
                                    cudaStream_t stream) {
  FR_CHECK_ARG(M >= 0 && n_q > 0 && n_kv > 0 && K > 0 && max_pos > 0 && num_slots > 0);
  if (M == 0) return FR_OK;
  FR_CHECK_SUPPORTED(head_dim == 128 && n_q % 2 == 0 && n_kv % 2 == 0);  // a 256-column tile is two whole heads
  FR_CHECK_ARG(a && b && scale_a && scale_b && q_out && positions && loc && q_weight && k_weight && cos_sin && k_cache &&
               v_cache);
  FR_CHECK_ARG(aligned16(a) && aligned16(b) && aligned16(q_out) && aligned16(scale_b) && aligned16(cos_sin) &&
               aligned16(k_cache) && aligned16(v_cache));
  const int N = (n_q + 2 * n_kv) * 128;
  FR_CHECK_ARG(lda >= K && ldb >= K && ldq >= n_q * 128 && lda % 16 == 0 && ldb % 16 == 0 && ldq % 8 == 0 && K % 16 == 0);
  FR_CHECK_ARG(ck_s % 16 == 0 && ck_h % 16 == 0 && cv_s % 16 == 0 && cv_h % 16 == 0);
  gemm::QkvRope rp;
  rp.pos = positions;
  rp.loc = loc;
  rp.qw = static_cast<const __nv_bfloat16*>(q_weight);
  rp.kw = static_cast<const __nv_bfloat16*>(k_weight);
  rp.cs = cos_sin;
  rp.q_out = static_cast<__nv_bfloat16*>(q_out);
  rp.kc = static_cast<uint8_t*>(k_cache);
  rp.vc = static_cast<uint8_t*>(v_cache);
  rp.ldq = ldq;
  rp.ck_s = ck_s;
  rp.ck_h = ck_h;
  rp.cv_s = cv_s;
  rp.cv_h = cv_h;
  rp.eps = eps;
  rp.max_pos = max_pos;
  rp.num_slots = num_slots;
  rp.n_q = n_q;
  rp.n_kv = n_kv;
  rp.wide = (reinterpret_cast<uintptr_t>(q_out) % 32 == 0 && (ldq * 2) % 32 == 0 &&
             reinterpret_cast<uintptr_t>(k_cache) % 32 == 0 && reinterpret_cast<uintptr_t>(v_cache) % 32 == 0 &&
             ck_s % 32 == 0 && ck_h % 32 == 0 && cv_s % 32 == 0 && cv_h % 32 == 0) ? 1 : 0;
  // the output tensor map of the launcher is not used by this epilogue; q_out gives it a valid target
  return gemm::launch_pair<__nv_bfloat16, 3>(a, b, scale_a, scale_b, nullptr, q_out, ldq, M, N, K, lda, ldb, stream,
                                             nullptr, rp);
}
