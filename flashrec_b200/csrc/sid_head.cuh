// Shared between the head GEMM's epilogue (gemm_fp8.cu) and the fused SID-head entry (beam_step.cu).
#pragma once

#include "fr_common.cuh"

namespace fr {

// Arguments of the SID-head epilogue (EPI == 4): the fp32 logits tile [rows, 256 codes of one level] is never
// written. Per row and 64 codes the epilogue keeps the pair (max, log-sum-exp) of those codes and appends the
// logits of the codes the row's trie node allows to the candidate list of the row's request.
//   row r = beam r % BW of request r / BW; a row is live when cum[r] is not -inf
//   mask word for codes [32 j, 32 j + 32) of the level shard: mask[idx * mask_stride + mask_word0 + j] with
//   idx = mask_index ? mask_index[r] : r. With mask_index (trie node ids; bitmap tries): idx < 0 allows every
//   code, idx >= mask_rows none, and level_off[idx] must equal level_off_expected (the node belongs to the
//   level being decoded), else none.
//   candidate record = {logit bits, flat index beam * idx_width + idx_base + code}, appended at
//   cand[request * cand_cap + atomicAdd(&cand_count[request], ...)]; records past cand_cap are dropped and the
//   status word is set.
constexpr int kHeadParts = 4;  // statistics entries per 256-code tile (one per epilogue warp of a lane quadrant)
struct HeadEpi {
  float* tile_max;          // [n_tiles_n * kHeadParts, M]
  float* tile_logsum;       // [n_tiles_n * kHeadParts, M]
  const float* cum;         // [M]
  const uint32_t* mask;
  const int64_t* mask_index;   // [M] or null
  const int32_t* level_off;    // per mask row, or null
  int64_t mask_stride;         // words per mask row
  int64_t mask_rows;
  int mask_word0;
  int level_off_expected;
  uint2* cand;              // [n_requests, cand_cap]
  int* cand_count;          // [n_requests]
  int cand_cap;
  int BW;
  int64_t idx_base, idx_width;
};

int launch_head_gemm(const void* a, const void* b, const float* sa, const float* sb, int M, int N, int K, int64_t lda,
                     int64_t ldb, const HeadEpi& hp, cudaStream_t stream);

// Statistics of a row split into S parts, each given as (max, log-sum-exp relative to that max), combined in
// part order: the one formula every path uses (shards of a token range, column tiles of the head GEMM).
__device__ __forceinline__ void lse_combine(const float* __restrict__ pmax, const float* __restrict__ plog, int S,
                                            int64_t stride, float& mx_out, float& ls_out) {
  float mx = -INFINITY;
  for (int s = 0; s < S; ++s) mx = fmaxf(mx, pmax[s * stride]);
  float sum = 0.f;
  for (int s = 0; s < S; ++s) sum += expf(plog[s * stride] + (pmax[s * stride] - mx));  // part sum rescaled to the global max
  mx_out = mx;
  ls_out = logf(sum);
}

}  // namespace fr
