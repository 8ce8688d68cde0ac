// Trie-constrained beam step of the SID decode: masked scores -> sorted top-K
// across all beams of a request -> token-row expand -> trie-node advance.
//
// Stands in for
//   trie_mask_kernel / trie_advance(_batched)_kernel / beam_expand(_batched)_kernel
//   / genrec_mask_topk_expand_kernel          (kernel/csrc/beam_trie.cuh:69-755)
//   and their torch restatements              (kernel/beam_trie.py:82-246, 536-630)
//   BeamValidPathTrie.mask_candidates / advance_node_ids / _csr_lookup
//                                             (search/trie.py:345-368, 445-589)
//   expand_step's no-EOS path                 (search/expand.py:351-372)
//
// Ordering rule (the reference CUDA kernel's, beam_trie.cuh:495-500): score
// descending, ties broken by the smaller flat candidate index b * C + c. With
// masking on, a candidate whose score is -inf is not a candidate at all; when
// fewer than K remain the tail is filled with (-inf, parent 0, token of flat
// index 0), as the reference does (beam_trie.cuh:664-683).
//
// Selection: one CTA per request runs a radix select on the 64-bit composite
// (order-preserving score key << 32 | ~flat index) — 11/11/10-bit digits, each
// pass re-enumerating the candidates and histogramming those that match the
// prefix found so far, stopping as soon as the boundary bin is taken whole —
// then collects the K winners into shared memory and bitonic-sorts them. This
// replaces the reference's K serial block-wide arg-max rounds and has no 512
// limit on beam width.
#include "fr_common.cuh"
#include "sid_head.cuh"
#include "topk_select.cuh"

namespace fr {
namespace beam {

constexpr int kThreads = 1024;
constexpr int kMaxK = 4096;

struct Trie {
  int kind;  // FR_TRIE_NONE / DENSE / CSR / BITMAP
  const uint8_t* allow;
  const void* next;
  int next_is_i32;
  const int64_t* keys;
  const int64_t* child;
  int64_t n_edges;
  const uint32_t* bitmap;
  const int64_t* child_base;
  const int32_t* level_off;
  int words;
  int64_t n_rows;
  int64_t vsz;
  int64_t token_base;
  int64_t invalid_node;
};

__device__ __forceinline__ int64_t clamp64(int64_t x, int64_t lo, int64_t hi) { return x < lo ? lo : (x > hi ? hi : x); }

// first position in keys[0, n) with keys[pos] >= key
__device__ __forceinline__ int64_t lower_bound(const int64_t* __restrict__ keys, int64_t n, int64_t key) {
  int64_t lo = 0, hi = n;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (__ldg(keys + mid) < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// Is `tok` a legal continuation of trie node `node`? node < 0 = unconstrained.
__device__ __forceinline__ bool trie_allowed(const Trie& tr, int64_t node, int64_t tok) {
  if (node < 0 || tr.kind == FR_TRIE_NONE) return true;
  const int64_t rel = tok - tr.token_base;
  if (rel < 0 || rel >= tr.vsz) return false;
  if (tr.kind == FR_TRIE_DENSE) {
    if (tr.n_rows <= 0) return false;
    const int64_t safe = clamp64(node, 0, tr.n_rows - 1);
    return __ldg(tr.allow + safe * tr.vsz + rel) != 0;
  }
  if (tr.kind == FR_TRIE_CSR) {
    if (tr.n_edges <= 0) return false;
    const int64_t key = node * tr.vsz + rel;
    const int64_t pos = lower_bound(tr.keys, tr.n_edges, key);
    return pos < tr.n_edges && __ldg(tr.keys + pos) == key;
  }
  if (tr.kind == FR_TRIE_BITMAP) {
    if (tr.n_rows <= 0) return false;
    const int64_t safe = clamp64(node, 0, tr.n_rows - 1);
    const int64_t c = rel - __ldg(tr.level_off + safe);
    if (c < 0 || c >= static_cast<int64_t>(tr.words) * 32) return false;
    return (__ldg(tr.bitmap + safe * tr.words + (c >> 5)) >> (c & 31)) & 1u;
  }
  return true;
}

// Node reached from `old` by `tok`: old < 0 stays; unknown edge -> invalid_node.
__device__ __forceinline__ int64_t trie_transition(const Trie& tr, int64_t old, int64_t tok) {
  if (old < 0) return old;
  const int64_t rel = tok - tr.token_base;
  if (rel < 0 || rel >= tr.vsz) return tr.invalid_node;
  if (tr.kind == FR_TRIE_DENSE) {
    // a dense trie given for masking only carries no transition table: no edge is known
    if (tr.n_rows <= 0 || tr.next == nullptr) return tr.invalid_node;
    const int64_t safe = clamp64(old, 0, tr.n_rows - 1);
    return tr.next_is_i32 ? static_cast<int64_t>(__ldg(static_cast<const int32_t*>(tr.next) + safe * tr.vsz + rel))
                          : __ldg(static_cast<const int64_t*>(tr.next) + safe * tr.vsz + rel);
  }
  if (tr.kind == FR_TRIE_CSR) {
    if (tr.n_edges <= 0) return tr.invalid_node;
    const int64_t key = old * tr.vsz + rel;
    const int64_t pos = lower_bound(tr.keys, tr.n_edges, key);
    if (pos < tr.n_edges && __ldg(tr.keys + pos) == key) return __ldg(tr.child + pos);
    return tr.invalid_node;
  }
  if (tr.kind == FR_TRIE_BITMAP) {
    if (tr.n_rows <= 0) return tr.invalid_node;
    const int64_t safe = clamp64(old, 0, tr.n_rows - 1);
    const int64_t c = rel - __ldg(tr.level_off + safe);
    if (c < 0 || c >= static_cast<int64_t>(tr.words) * 32) return tr.invalid_node;
    const uint32_t* bm = tr.bitmap + safe * tr.words;
    const uint32_t w = __ldg(bm + (c >> 5));
    if (!((w >> (c & 31)) & 1u)) return tr.invalid_node;
    const int64_t base = __ldg(tr.child_base + safe);
    if (base < 0) return -1;  // children are leaves: unconstrained from here on
    int64_t rank = __popc(w & ((1u << (c & 31)) - 1u));
    for (int i = 0; i < (c >> 5); ++i) rank += __popc(__ldg(bm + i));
    return base + rank;
  }
  return old;
}

// ---------------------------------------------------------------------------
// element-wise entry points
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(512) trie_mask_kernel(float* __restrict__ out, const float* __restrict__ in,
                                                       const int64_t* __restrict__ tok,
                                                       const int64_t* __restrict__ nodes, Trie tr, float neg_inf,
                                                       int64_t rows, int64_t cols) {
  const int64_t total = rows * cols;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / cols;
    out[i] = trie_allowed(tr, nodes[r], tok[i]) ? in[i] : neg_inf;
  }
}

// out[n, k] = transition(node_ids[n, clamp(parents[n, k])], tokens[n, k])
__global__ void __launch_bounds__(512) trie_advance_kernel(int64_t* __restrict__ out,
                                                          const int64_t* __restrict__ nodes,
                                                          const int64_t* __restrict__ parents,
                                                          const int64_t* __restrict__ tok, Trie tr, int N, int BW,
                                                          int K) {
  const int64_t total = static_cast<int64_t>(N) * K;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t n = i / K;
    const int64_t p = clamp64(parents[i], 0, BW - 1);
    out[i] = trie_transition(tr, nodes[n * BW + p], tok[i]);
  }
}

// out[n, b, :] = token_ids[n, clamp(parents[n, b]), :]; out[n, b, col] = new_tokens[n, b]
__global__ void __launch_bounds__(512) beam_expand_kernel(int64_t* __restrict__ out,
                                                         const int64_t* __restrict__ token_ids,
                                                         const int64_t* __restrict__ parents,
                                                         const int64_t* __restrict__ new_tokens, int N, int BW, int L,
                                                         int col) {
  const int64_t total = static_cast<int64_t>(N) * BW * L;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t c = i % L;
    const int64_t nb = i / L;
    const int64_t n = nb / BW;
    if (c == col) {
      out[i] = new_tokens[nb];
    } else {
      const int64_t p = clamp64(parents[nb], 0, BW - 1);
      out[i] = token_ids[(n * BW + p) * L + c];
    }
  }
}

// ---------------------------------------------------------------------------
// fused step
// ---------------------------------------------------------------------------
struct StepParams {
  float* out_vals;         // [N, K]
  int64_t* out_parents;    // [N, K]
  int64_t* out_tokens;     // [N, K]
  int64_t* out_indices;    // [N, K] flat index b * C + c
  int64_t* out_child;      // [N, K] node after the step, or null
  uint4* out_records;      // [N, K] {score bits, flat index, child low, child high} for the shard exchange, or null
  int64_t* token_ids_out;  // [N, max(BW, K), L] or null
  int64_t* node_ids_out;   // [N, max(BW, K)] or null
  const float* cum;        // [N, BW]
  const int64_t* node_in;  // [N, BW] or null
  const int64_t* token_ids_in;
  const uint8_t* do_expand;  // [N] or null (= all)
  const int32_t* col_n;      // [N] or null (= 0)
  // explicit candidates
  const float* lp;     // [N, BW, C]
  const int64_t* tok;  // [N, BW, C]
  float* scratch;      // [N, BW * C] masked scores
  const float* perturb;  // [N, BW, C] or null: added to the score for ranking only (unmasked explicit candidates)
  // full-width candidates straight from the level's logits
  const float* logits;  // [N * BW, ld]
  int64_t ld;
  const float* row_max;     // [N * BW]
  const float* row_logsum;  // [N * BW]
  int64_t level_tok_base;   // token id of code 0 of this level
  int64_t idx_base;         // added to c when forming the flat index (token-range shards)
  int64_t idx_width;        // C used in the flat index (whole level width)
  // compact candidates written by the head GEMM's epilogue: {logit bits, flat index} per record
  const uint2* cand;        // [N, cand_cap]
  const int* cand_count;    // [N]
  int cand_cap;
  Trie trie;
  int N, BW, C, K, L;
  int apply_mask, apply_expand, apply_advance;
  float neg_inf;
};

using topk::compose;
using topk::SelectSmem;

// Candidate enumeration. Calls f(composite) for every live candidate of request n.
// `rng` (FULL + CSR trie): per beam the [first, last) positions of its node's edges in the sorted
// key array, found once per launch; a negative first position means "no range, scan the level".
// MODE 0: explicit candidates (lp / tok); 1: every code of the level, read from the logits matrix;
// 2: the compact candidate records the head GEMM's epilogue emitted (already trie-legal).
template <int MODE, class F>
__device__ __forceinline__ void for_each_candidate(const StepParams& p, int n, bool masked, const int64_t* rng,
                                                   F&& f) {
  constexpr bool FULL = MODE == 1;
  if constexpr (MODE == 2) {
    const uint2* cn = p.cand + static_cast<size_t>(n) * p.cand_cap;
    const int cnt = min(p.cand_count[n], p.cand_cap);
    const size_t row0 = static_cast<size_t>(n) * p.BW;
    for (int i = threadIdx.x; i < cnt; i += kThreads) {
      const uint2 rec = cn[i];
      const uint32_t b = rec.y / static_cast<uint32_t>(p.idx_width);
      const size_t row = row0 + b;
      const float s = __fadd_rn(p.cum[row], __fsub_rn(__fsub_rn(__uint_as_float(rec.x), p.row_max[row]), p.row_logsum[row]));
      if (s != p.neg_inf) f(compose(s, rec.y));
    }
  } else if constexpr (!FULL) {
    const uint32_t M = static_cast<uint32_t>(p.BW) * p.C;
    const float* cum_n = p.cum + static_cast<size_t>(n) * p.BW;
    if (masked) {
      const float* sc = p.scratch + static_cast<size_t>(n) * M;
      for (uint32_t i = threadIdx.x; i < M; i += kThreads) {
        const float s = sc[i];
        if (s != p.neg_inf) f(compose(s, i));
      }
    } else {
      const float* lp_n = p.lp + static_cast<size_t>(n) * M;
      if (p.perturb != nullptr) {
        const float* pt = p.perturb + static_cast<size_t>(n) * M;
        for (uint32_t i = threadIdx.x; i < M; i += kThreads)
          f(compose(__fadd_rn(__fadd_rn(cum_n[i / p.C], lp_n[i]), pt[i]), i));
      } else {
        for (uint32_t i = threadIdx.x; i < M; i += kThreads) f(compose(__fadd_rn(cum_n[i / p.C], lp_n[i]), i));
      }
    }
  } else {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const Trie& tr = p.trie;
    const int64_t first_tok = p.level_tok_base + p.idx_base;  // token of this shard's local code 0
    const int64_t level_off = first_tok - tr.token_base;
    for (int b = warp; b < p.BW; b += kThreads / 32) {
      const size_t row = static_cast<size_t>(n) * p.BW + b;
      const float cumb = p.cum[row];
      if (cumb == p.neg_inf) continue;
      const int64_t node = p.node_in ? p.node_in[row] : -1;
      const float* lg = p.logits + row * p.ld;
      const float mx = p.row_max[row], ls = p.row_logsum[row];
      if (tr.kind == FR_TRIE_CSR && node >= 0) {
        // only the node's own edges can be legal: walk its slice of the sorted key array
        const int64_t k0 = node * tr.vsz + level_off;
        const int64_t e0 = rng[2 * b], e1 = rng[2 * b + 1];
        for (int64_t e = e0 + lane; e < e1; e += 32) {
          const int64_t c = __ldg(tr.keys + e) - k0;
          const float s = __fadd_rn(cumb, __fsub_rn(__fsub_rn(lg[c], mx), ls));
          if (s != p.neg_inf)
            f(compose(s, static_cast<uint32_t>(static_cast<int64_t>(b) * p.idx_width + p.idx_base + c)));
        }
      } else if (tr.kind == FR_TRIE_BITMAP && node >= 0 && node < tr.n_rows) {
        // only the set bits of the node's row can be legal: walk them word by word (a node deep in
        // the trie has a handful of children among thousands of codes)
        const int64_t delta = level_off - __ldg(tr.level_off + node);  // bit index of this shard's code 0
        const uint32_t* bm = tr.bitmap + node * tr.words;
        for (int w = lane; w < tr.words; w += 32) {
          uint32_t bits = __ldg(bm + w);
          while (bits) {
            const int t = __ffs(bits) - 1;
            bits &= bits - 1;
            const int64_t c = static_cast<int64_t>(w) * 32 + t - delta;
            if (c < 0 || c >= p.C) continue;
            const float s = __fadd_rn(cumb, __fsub_rn(__fsub_rn(lg[c], mx), ls));
            if (s != p.neg_inf)
              f(compose(s, static_cast<uint32_t>(static_cast<int64_t>(b) * p.idx_width + p.idx_base + c)));
          }
        }
      } else {
        for (int c = lane; c < p.C; c += 32) {
          if (!trie_allowed(tr, node, first_tok + c)) continue;
          const float s = __fadd_rn(cumb, __fsub_rn(__fsub_rn(lg[c], mx), ls));
          if (s != p.neg_inf)
            f(compose(s, static_cast<uint32_t>(static_cast<int64_t>(b) * p.idx_width + p.idx_base + c)));
        }
      }
    }
  }
}

// Token-row expand and node advance for request n, given the K winners in
// shared memory (sel_parent, sel_token) — same contract as the reference's tail
// of genrec_mask_topk_expand_kernel (beam_trie.cuh:697-754).
__device__ __forceinline__ void apply_winners(const StepParams& p, int n, const int32_t* sel_parent,
                                              const int64_t* sel_token, const int64_t* sel_child) {
  const bool expand_this = p.apply_expand && p.token_ids_in && p.token_ids_out && (!p.do_expand || p.do_expand[n] != 0);
  if (!expand_this) return;
  int64_t col = 0;
  if (p.col_n) col = p.col_n[n] < 0 ? 0 : p.col_n[n];
  // the output planes hold max(BW, K) beams per request: K > BW when a request fans out from fewer
  // input beams than it selects (level 0 from one prefill row)
  const int obw = p.K > p.BW ? p.K : p.BW;
  const int64_t* tin = p.token_ids_in + static_cast<size_t>(n) * p.BW * p.L;
  int64_t* tout = p.token_ids_out + static_cast<size_t>(n) * obw * p.L;
  const int plane = obw * p.L;
  for (int i = threadIdx.x; i < plane; i += kThreads) {
    const int b = i / p.L, c = i - b * p.L;
    if (b >= p.K) { tout[i] = tin[i]; continue; }
    if (c == col) tout[i] = sel_token[b];
    else tout[i] = tin[static_cast<size_t>(sel_parent[b]) * p.L + c];
  }
  if (p.apply_advance && p.node_in && p.node_ids_out) {
    const int64_t* nin = p.node_in + static_cast<size_t>(n) * p.BW;
    int64_t* nout = p.node_ids_out + static_cast<size_t>(n) * obw;
    for (int b = threadIdx.x; b < obw; b += kThreads) nout[b] = b < p.K ? sel_child[b] : nin[b];
  }
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1) beam_step_kernel(StepParams p) {
  constexpr bool FULL = MODE != 0;  // the winners' tokens follow from the flat index over the level
  extern __shared__ __align__(16) uint8_t dyn[];
  __shared__ SelectSmem sm;
  const int n = blockIdx.x;
  int kp2 = 1;
  while (kp2 < p.K) kp2 <<= 1;
  uint64_t* win = reinterpret_cast<uint64_t*>(dyn);                    // [kp2]
  int64_t* sel_token = reinterpret_cast<int64_t*>(win + kp2);          // [K]
  int64_t* sel_child = sel_token + p.K;                                // [K]
  int32_t* sel_parent = reinterpret_cast<int32_t*>(sel_child + p.K);   // [K]
  int64_t* rng = reinterpret_cast<int64_t*>(dyn + ((kp2 * 8 + p.K * 20 + 15) & ~15));  // [2 * BW], FULL + CSR only

  const bool masked = FULL || (p.apply_mask && p.node_in && p.trie.kind != FR_TRIE_NONE);
  const uint32_t M = static_cast<uint32_t>(p.BW) * p.C;

  if constexpr (!FULL) {
    if (masked) {
      // pass 0: masked scores, kept in global scratch for the later passes
      const float* cum_n = p.cum + static_cast<size_t>(n) * p.BW;
      const float* lp_n = p.lp + static_cast<size_t>(n) * M;
      const int64_t* tok_n = p.tok + static_cast<size_t>(n) * M;
      const int64_t* nodes_n = p.node_in + static_cast<size_t>(n) * p.BW;
      float* sc = p.scratch + static_cast<size_t>(n) * M;
      for (uint32_t i = threadIdx.x; i < M; i += kThreads) {
        const uint32_t b = i / p.C;
        float s = __fadd_rn(cum_n[b], lp_n[i]);
        if (!trie_allowed(p.trie, nodes_n[b], tok_n[i])) s = p.neg_inf;
        sc[i] = s;
      }
      __syncthreads();  // same CTA re-reads what it wrote
    }
  }

  if constexpr (MODE == 1) {
    if (p.trie.kind == FR_TRIE_CSR) {
      // every enumeration pass below walks the beams' edge lists: find each list once (one
      // binary-search pair per thread, all beams in parallel) instead of once per pass and warp
      const int64_t level_off = p.level_tok_base + p.idx_base - p.trie.token_base;
      for (int b = threadIdx.x; b < p.BW; b += kThreads) {
        const size_t row = static_cast<size_t>(n) * p.BW + b;
        const int64_t node = p.node_in ? p.node_in[row] : -1;
        int64_t e0 = -1, e1 = -1;
        if (node >= 0 && p.cum[row] != p.neg_inf) {
          const int64_t k0 = node * p.trie.vsz + level_off;
          e0 = lower_bound(p.trie.keys, p.trie.n_edges, k0);
          e1 = lower_bound(p.trie.keys, p.trie.n_edges, k0 + p.C);
        }
        rng[2 * b] = e0;
        rng[2 * b + 1] = e1;
      }
      __syncthreads();
    }
  }

  // ---- select + sort ---------------------------------------------------------
  const int nvalid = topk::radix_select_topk<kThreads>(
      [&](auto&& f) { for_each_candidate<MODE>(p, n, masked, rng, f); }, p.K, win, kp2, sm);

  // ---- outputs ---------------------------------------------------------------
  const int64_t* tok_n = FULL ? nullptr : p.tok + static_cast<size_t>(n) * M;
  const int64_t* nodes_n = p.node_in ? p.node_in + static_cast<size_t>(n) * p.BW : nullptr;
  const int64_t cdiv = FULL ? p.idx_width : p.C;
  for (int k = threadIdx.x; k < p.K; k += kThreads) {
    float v = p.neg_inf;
    uint32_t idx = 0;
    if (k < nvalid) {
      const uint64_t ck = win[k];
      v = topk::composite_score(ck);
      idx = topk::composite_index(ck);
      if constexpr (MODE == 0) {  // ranked with noise: the score that is reported carries none
        if (p.perturb != nullptr && !p.apply_mask)
          v = __fadd_rn(p.cum[static_cast<size_t>(n) * p.BW + idx / p.C], p.lp[static_cast<size_t>(n) * M + idx]);
      }
    }
    const int64_t parent = k < nvalid ? static_cast<int64_t>(idx) / cdiv : 0;
    int64_t token;
    if constexpr (FULL) token = p.level_tok_base + static_cast<int64_t>(idx) % cdiv;
    else token = M > 0 ? tok_n[k < nvalid ? idx : 0] : 0;
    const int64_t pc = clamp64(parent, 0, p.BW - 1);
    int64_t child = 0;
    if (nodes_n) child = trie_transition(p.trie, nodes_n[pc], token);
    const size_t o = static_cast<size_t>(n) * p.K + k;
    p.out_vals[o] = v;
    p.out_parents[o] = parent;
    p.out_tokens[o] = token;
    p.out_indices[o] = k < nvalid ? static_cast<int64_t>(idx) : 0;
    if (p.out_child) p.out_child[o] = child;
    if (p.out_records)
      p.out_records[o] = make_uint4(__float_as_uint(v), k < nvalid ? idx : 0u, static_cast<uint32_t>(child & 0xffffffffll),
                                    static_cast<uint32_t>(static_cast<uint64_t>(child) >> 32));
    sel_parent[k] = static_cast<int32_t>(pc);
    sel_token[k] = token;
    sel_child[k] = child;
  }
  __syncthreads();
  apply_winners(p, n, sel_parent, sel_token, sel_child);
}

// ---------------------------------------------------------------------------
// merge of per-shard winners (token-range sharded lm_head): S sorted lists of K
// records per request -> global sorted top-K, then expand / advance.
// ---------------------------------------------------------------------------
struct MergeParams {
  const float* vals;       // [S, N, K]
  const int64_t* indices;  // [S, N, K] flat index over the whole level
  const int64_t* child;    // [S, N, K]
  const uint4* records;    // [S, N, K] {score bits, flat index, child low, child high}: replaces the three arrays
  int S;
  StepParams step;  // outputs + expand inputs; idx_width / level_tok_base / K / BW / L used
};

// Each shard's list is sorted like the output (score descending, then flat index ascending) and the flat
// indices of different shards are disjoint, so the place of a record in the merged list is its own place
// plus, for every other shard, the number of that shard's records that rank before it: one binary search
// per (record, other shard) over composites held in shared memory. Records that land below K are written
// straight to their place with the child node they carry; no sort, nothing looked up again.
__global__ void __launch_bounds__(kThreads, 1) merge_shards_kernel(MergeParams mp) {
  extern __shared__ __align__(16) uint8_t dyn[];
  __shared__ int live_total;
  const StepParams& p = mp.step;
  const int n = blockIdx.x;
  const int K = p.K;
  const int total = mp.S * K;
  uint64_t* comp = reinterpret_cast<uint64_t*>(dyn);                   // [S * K]
  int64_t* sel_token = reinterpret_cast<int64_t*>(comp + total);       // [K]
  int64_t* sel_child = sel_token + K;                                  // [K]
  int32_t* sel_parent = reinterpret_cast<int32_t*>(sel_child + K);     // [K]
  if (threadIdx.x == 0) live_total = 0;
  __syncthreads();
  int live_mine = 0;
  for (int i = threadIdx.x; i < total; i += kThreads) {
    const int s = i / K, k = i - s * K;
    const size_t o = (static_cast<size_t>(s) * p.N + n) * K + k;
    float v;
    uint32_t idx;
    if (mp.records) {
      const uint4 r = mp.records[o];
      v = __uint_as_float(r.x);
      idx = r.y;
    } else {
      v = mp.vals[o];
      idx = static_cast<uint32_t>(mp.indices[o]);
    }
    const uint64_t ck = v != p.neg_inf ? compose(v, idx) : 0;
    comp[i] = ck;
    live_mine += ck != 0;
  }
  if (live_mine) atomicAdd(&live_total, live_mine);
  __syncthreads();
  const int n_live = min(live_total, K);
  for (int i = threadIdx.x; i < total; i += kThreads) {
    const uint64_t ck = comp[i];
    if (ck == 0) continue;
    const int s = i / K;
    int rank = i - s * K;
    for (int t = 0; t < mp.S && rank < K; ++t) {
      if (t == s) continue;
      const uint64_t* lst = comp + t * K;  // descending; dead entries (0) at the end
      int lo = 0, hi = K;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (lst[mid] > ck) lo = mid + 1; else hi = mid;
      }
      rank += lo;
    }
    if (rank >= K) continue;
    const size_t src = (static_cast<size_t>(s) * p.N + n) * K + (i - s * K);
    int64_t child = 0;
    if (mp.records) {
      const uint4 r = mp.records[src];
      child = static_cast<int64_t>((static_cast<uint64_t>(r.w) << 32) | r.z);
    } else if (mp.child) {
      child = mp.child[src];
    }
    const uint32_t idx = topk::composite_index(ck);
    const int64_t parent = static_cast<int64_t>(idx) / p.idx_width;
    const int64_t token = p.level_tok_base + static_cast<int64_t>(idx) % p.idx_width;
    const size_t o = static_cast<size_t>(n) * K + rank;
    p.out_vals[o] = topk::composite_score(ck);
    p.out_parents[o] = parent;
    p.out_tokens[o] = token;
    p.out_indices[o] = static_cast<int64_t>(idx);
    if (p.out_child) p.out_child[o] = child;
    sel_parent[rank] = static_cast<int32_t>(clamp64(parent, 0, p.BW - 1));
    sel_token[rank] = token;
    sel_child[rank] = child;
  }
  // places past the last live winner (fewer than K live candidates over all shards) are filled as the
  // unsharded step fills them: parent 0, code 0 of the level, and the node that edge leads to
  for (int k = n_live + threadIdx.x; k < K; k += kThreads) {
    int64_t child = 0;
    if (p.node_in && p.trie.kind != FR_TRIE_NONE)
      child = trie_transition(p.trie, p.node_in[static_cast<size_t>(n) * p.BW], p.level_tok_base);
    const size_t o = static_cast<size_t>(n) * K + k;
    p.out_vals[o] = p.neg_inf;
    p.out_parents[o] = 0;
    p.out_tokens[o] = p.level_tok_base;
    p.out_indices[o] = 0;
    if (p.out_child) p.out_child[o] = child;
    sel_parent[k] = 0;
    sel_token[k] = p.level_tok_base;
    sel_child[k] = child;
  }
  __syncthreads();
  apply_winners(p, n, sel_parent, sel_token, sel_child);
}

static int make_trie(const fr_trie* t, Trie* out) {
  Trie tr{};
  if (!t || t->kind == FR_TRIE_NONE) { tr.kind = FR_TRIE_NONE; *out = tr; return FR_OK; }
  tr.kind = t->kind;
  tr.allow = static_cast<const uint8_t*>(t->allow);
  tr.next = t->next;
  tr.next_is_i32 = t->next_is_i32;
  tr.keys = static_cast<const int64_t*>(t->csr_keys);
  tr.child = static_cast<const int64_t*>(t->csr_child);
  tr.n_edges = t->n_edges;
  tr.bitmap = static_cast<const uint32_t*>(t->bitmap);
  tr.child_base = static_cast<const int64_t*>(t->child_base);
  tr.level_off = static_cast<const int32_t*>(t->level_off);
  tr.words = t->words_per_node;
  tr.n_rows = t->n_rows;
  tr.vsz = t->vsz;
  tr.token_base = t->token_base;
  tr.invalid_node = t->invalid_node;
  if (tr.vsz <= 0) return FR_ERR_BAD_ARG;
  switch (tr.kind) {
    case FR_TRIE_DENSE: if (!tr.allow || tr.n_rows <= 0) return FR_ERR_BAD_ARG; break;
    case FR_TRIE_CSR: if (tr.n_edges < 0 || (tr.n_edges > 0 && (!tr.keys || !tr.child))) return FR_ERR_BAD_ARG; break;
    case FR_TRIE_BITMAP:
      if (!tr.bitmap || !tr.child_base || !tr.level_off || tr.words <= 0 || tr.n_rows <= 0) return FR_ERR_BAD_ARG;
      break;
    default: return FR_ERR_BAD_ARG;
  }
  *out = tr;
  return FR_OK;
}

static size_t step_smem(int K, int BW, bool edge_ranges) {
  int kp2 = 1;
  while (kp2 < K) kp2 <<= 1;
  size_t b = (static_cast<size_t>(kp2) * 8 + static_cast<size_t>(K) * (8 + 8 + 4) + 15) & ~static_cast<size_t>(15);
  if (edge_ranges) b += static_cast<size_t>(BW) * 16;
  return b + 16;
}

template <int MODE>
static int launch_step(const StepParams& p, cudaStream_t stream) {
  const size_t smem = step_smem(p.K, p.BW, MODE == 1 && p.trie.kind == FR_TRIE_CSR);
  auto kern = beam_step_kernel<MODE>;
  if (smem > 32 * 1024) {  // static shared memory counts towards the 48 KiB default limit
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return FR_ERR_CUDA;
  }
  kern<<<p.N, kThreads, smem, stream>>>(p);
  return launch_status();
}


// ---------------------------------------------------------------------------
// Stop-token walk over a group's ranked candidates (search/select.py:98-161): candidate i survives when
// it is not a stop token and fewer than K non-stop candidates rank before it; a stop-token candidate is
// finished when fewer than K survivors rank before it. Survivors are compacted into [K] slots in rank
// order, finished candidates into [C] slots; unused slots read zero. One CTA per group.
// ---------------------------------------------------------------------------
struct JointParams {
  const float* vals;        // [G, C] ranked scores (no noise)
  const int64_t* parents;   // [G, C]
  const int64_t* tokens;    // [G, C]
  const int64_t* stop;      // [n_stop]
  int n_stop;
  int64_t* next_tokens;     // [G, K]
  int64_t* parent_idx;      // [G, K]
  float* new_cum;           // [G, K]
  int64_t* num_survivors;   // [G]
  int64_t* fin_tokens;      // [G, C]
  int64_t* fin_parent;      // [G, C]
  float* fin_cum;           // [G, C]
  int64_t* num_finished;    // [G]
  int C, K;
};

constexpr int kScanThreads = 256;

// exclusive prefix of v over the CTA; total returned through `total`
__device__ __forceinline__ int block_exclusive(int v, int* warp_sums, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += y;
  }
  __syncthreads();  // warp_sums may still be read from a previous call
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  int before = 0;
  total = 0;
#pragma unroll
  for (int w = 0; w < kScanThreads / 32; ++w) {
    const int t = warp_sums[w];
    if (w < warp) before += t;
    total += t;
  }
  return before + inc - v;
}

__global__ void __launch_bounds__(kScanThreads) joint_select_scan_kernel(JointParams p) {
  __shared__ int warp_sums[kScanThreads / 32];
  __shared__ int64_t stop_s[64];
  const int g = blockIdx.x, tid = threadIdx.x;
  const int C = p.C, K = p.K;
  const float* vals = p.vals + static_cast<size_t>(g) * C;
  const int64_t* par = p.parents + static_cast<size_t>(g) * C;
  const int64_t* tok = p.tokens + static_cast<size_t>(g) * C;
  for (int i = tid; i < min(p.n_stop, 64); i += kScanThreads) stop_s[i] = p.stop[i];
  for (int i = tid; i < K; i += kScanThreads) {
    p.next_tokens[static_cast<size_t>(g) * K + i] = 0;
    p.parent_idx[static_cast<size_t>(g) * K + i] = 0;
    p.new_cum[static_cast<size_t>(g) * K + i] = 0.f;
  }
  for (int i = tid; i < C; i += kScanThreads) {
    p.fin_tokens[static_cast<size_t>(g) * C + i] = 0;
    p.fin_parent[static_cast<size_t>(g) * C + i] = 0;
    p.fin_cum[static_cast<size_t>(g) * C + i] = 0.f;
  }
  __syncthreads();
  auto is_stop = [&](int64_t t) {
    bool s = false;
    for (int j = 0; j < p.n_stop; ++j) s |= (j < 64 ? stop_s[j] : p.stop[j]) == t;
    return s;
  };
  const int per = (C + kScanThreads - 1) / kScanThreads;  // consecutive candidates per thread (<= 16)
  const int i0 = min(C, tid * per), i1 = min(C, i0 + per);
  uint32_t stop_bits = 0;
  int non_stop = 0;
  for (int i = i0; i < i1; ++i) {
    const bool st = is_stop(tok[i]);
    stop_bits |= (st ? 1u : 0u) << (i - i0);
    non_stop += st ? 0 : 1;
  }
  int total_ns;
  int rank = block_exclusive(non_stop, warp_sums, total_ns);  // non-stop candidates ranked before my first
  int fin = 0;
  {
    int r = rank;
    for (int i = i0; i < i1; ++i) {
      if ((stop_bits >> (i - i0)) & 1u) fin += r < K ? 1 : 0;
      else ++r;
    }
  }
  int total_fin;
  int fin_rank = block_exclusive(fin, warp_sums, total_fin);
  for (int i = i0; i < i1; ++i) {
    if ((stop_bits >> (i - i0)) & 1u) {
      if (rank < K) {
        const size_t o = static_cast<size_t>(g) * C + fin_rank++;
        p.fin_tokens[o] = tok[i];
        p.fin_parent[o] = par[i];
        p.fin_cum[o] = vals[i];
      }
    } else {
      if (rank < K) {
        const size_t o = static_cast<size_t>(g) * K + rank;
        p.next_tokens[o] = tok[i];
        p.parent_idx[o] = par[i];
        p.new_cum[o] = vals[i];
      }
      ++rank;
    }
  }
  if (tid == 0) {
    p.num_survivors[g] = min(total_ns, K);
    p.num_finished[g] = total_fin;
  }
}

static int grid_for(int64_t total, int threads) {
  int64_t g = (total + threads - 1) / threads;
  if (g > 148 * 8) g = 148 * 8;
  return static_cast<int>(g < 1 ? 1 : g);
}

}  // namespace beam
}  // namespace fr

using namespace fr;
using namespace fr::beam;

extern "C" int fr_trie_mask(float* scores_out, const float* scores_in, const int64_t* cand_tokens,
                            const int64_t* node_ids, const fr_trie* trie, float neg_inf, int64_t rows, int64_t cols,
                            cudaStream_t stream) {
  FR_CHECK_ARG(rows >= 0 && cols >= 0);
  if (rows == 0 || cols == 0) return FR_OK;
  FR_CHECK_ARG(scores_out && scores_in && cand_tokens && node_ids && trie);
  Trie tr;
  const int st = make_trie(trie, &tr);
  if (st != FR_OK) return st;
  trie_mask_kernel<<<grid_for(rows * cols, 512), 512, 0, stream>>>(scores_out, scores_in, cand_tokens, node_ids, tr,
                                                                   neg_inf, rows, cols);
  return launch_status();
}

extern "C" int fr_trie_advance(int64_t* out, const int64_t* node_ids, const int64_t* parents, const int64_t* tokens,
                               const fr_trie* trie, int N, int BW, int K, cudaStream_t stream) {
  FR_CHECK_ARG(N >= 0 && BW > 0 && K >= 0);
  if (N == 0 || K == 0) return FR_OK;
  FR_CHECK_ARG(out && node_ids && parents && tokens && trie);
  Trie tr;
  const int st = make_trie(trie, &tr);
  if (st != FR_OK) return st;
  trie_advance_kernel<<<grid_for(static_cast<int64_t>(N) * K, 512), 512, 0, stream>>>(out, node_ids, parents, tokens,
                                                                                      tr, N, BW, K);
  return launch_status();
}

extern "C" int fr_beam_expand(int64_t* out, const int64_t* token_ids, const int64_t* parents,
                              const int64_t* new_tokens, int N, int BW, int L, int col, cudaStream_t stream) {
  FR_CHECK_ARG(N >= 0 && BW > 0 && L > 0);
  if (N == 0) return FR_OK;
  FR_CHECK_ARG(out && token_ids && parents && new_tokens && out != token_ids);
  FR_CHECK_ARG(col >= 0 && col < L);
  beam_expand_kernel<<<grid_for(static_cast<int64_t>(N) * BW * L, 512), 512, 0, stream>>>(out, token_ids, parents,
                                                                                         new_tokens, N, BW, L, col);
  return launch_status();
}

static int check_step_common(const StepParams& p) {
  FR_CHECK_ARG(p.N >= 0 && p.BW > 0 && p.C > 0 && p.K > 0 && p.L >= 0);
  FR_CHECK_SUPPORTED(p.K <= kMaxK && p.K <= p.BW * static_cast<int64_t>(p.C));
  FR_CHECK_SUPPORTED(static_cast<int64_t>(p.BW) * (p.idx_width > 0 ? p.idx_width : p.C) < (1ll << 32));
  FR_CHECK_ARG(p.out_vals && p.out_parents && p.out_tokens && p.out_indices && p.cum);
  if (p.apply_expand) {
    FR_CHECK_ARG(p.token_ids_in && p.token_ids_out && p.token_ids_in != p.token_ids_out && p.L > 0);
  }
  if (p.apply_advance) FR_CHECK_ARG(p.node_in && p.node_ids_out && p.node_in != p.node_ids_out);
  return FR_OK;
}

extern "C" int fr_mask_topk_expand(float* out_vals, int64_t* out_parents, int64_t* out_tokens, int64_t* out_indices,
                                   int64_t* out_child, float* scratch, const float* cum, const float* top_logprobs,
                                   const int64_t* top_tokens, const int64_t* node_in, const int64_t* token_ids_in,
                                   int64_t* token_ids_out, int64_t* node_ids_out, const uint8_t* do_expand,
                                   const int32_t* col_n, const fr_trie* trie, int N, int BW, int C, int K, int L,
                                   int apply_mask, int apply_expand, int apply_advance, cudaStream_t stream) {
  StepParams p{};
  p.out_vals = out_vals; p.out_parents = out_parents; p.out_tokens = out_tokens; p.out_indices = out_indices;
  p.out_child = out_child; p.token_ids_out = token_ids_out; p.node_ids_out = node_ids_out;
  p.cum = cum; p.node_in = node_in; p.token_ids_in = token_ids_in; p.do_expand = do_expand; p.col_n = col_n;
  p.lp = top_logprobs; p.tok = top_tokens; p.scratch = scratch;
  p.N = N; p.BW = BW; p.C = C; p.K = K; p.L = L;
  p.apply_mask = apply_mask; p.apply_expand = apply_expand; p.apply_advance = apply_advance && apply_mask && apply_expand;
  p.neg_inf = -INFINITY;
  p.idx_width = C;
  if (N == 0) return FR_OK;
  int st = make_trie(trie, &p.trie);
  if (st != FR_OK) return st;
  if (!(apply_mask && node_in && p.trie.kind != FR_TRIE_NONE)) { p.apply_mask = 0; p.apply_advance = 0; }
  st = check_step_common(p);
  if (st != FR_OK) return st;
  FR_CHECK_ARG(top_logprobs && top_tokens);
  if (p.apply_mask) FR_CHECK_ARG(scratch);
  return launch_step<0>(p, stream);
}


// joint_select / select_final_topk of the reference (search/select.py:72-179) for G independent groups.
extern "C" int64_t fr_joint_select_workspace_bytes(int G, int C) {
  if (G < 0 || C <= 0) return -1;
  return static_cast<int64_t>(G) * C * (4 + 3 * 8) + 64;
}

extern "C" int fr_joint_select(int64_t* next_tokens, int64_t* parent_idx, float* new_cum, int64_t* num_survivors,
                               int64_t* fin_tokens, int64_t* fin_parent, float* fin_cum, int64_t* num_finished,
                               const float* cum, const float* top_logprobs, const int64_t* top_tokens,
                               const float* perturb, const int64_t* stop_ids, int n_stop, void* workspace,
                               int64_t workspace_bytes, int G, int R, int C, int K, cudaStream_t stream) {
  FR_CHECK_ARG(G >= 0 && R > 0 && C > 0 && K > 0 && n_stop >= 0);
  if (G == 0) return FR_OK;
  FR_CHECK_ARG(next_tokens && parent_idx && new_cum && num_survivors && fin_tokens && fin_parent && fin_cum && num_finished);
  FR_CHECK_ARG(cum && top_logprobs && top_tokens && (n_stop == 0 || stop_ids));
  FR_CHECK_SUPPORTED(C <= kMaxK && C <= kScanThreads * 16);
  FR_CHECK_ARG(workspace && aligned16(workspace) && workspace_bytes >= fr_joint_select_workspace_bytes(G, C));
  const size_t gc = static_cast<size_t>(G) * C;
  uint8_t* w = static_cast<uint8_t*>(workspace);
  int64_t* s_par = reinterpret_cast<int64_t*>(w);
  int64_t* s_tok = s_par + gc;
  int64_t* s_idx = s_tok + gc;
  float* s_val = reinterpret_cast<float*>(s_idx + gc);
  StepParams sp{};
  sp.out_vals = s_val; sp.out_parents = s_par; sp.out_tokens = s_tok; sp.out_indices = s_idx;
  sp.cum = cum; sp.lp = top_logprobs; sp.tok = top_tokens; sp.perturb = perturb;
  sp.N = G; sp.BW = R; sp.C = C; sp.K = C; sp.L = 0;  // the walk looks at the C best of the R * C extensions
  sp.neg_inf = -INFINITY;
  sp.idx_width = C;
  int st = make_trie(nullptr, &sp.trie);
  if (st != FR_OK) return st;
  st = check_step_common(sp);
  if (st != FR_OK) return st;
  st = launch_step<0>(sp, stream);
  if (st != FR_OK) return st;
  JointParams jp{};
  jp.vals = s_val; jp.parents = s_par; jp.tokens = s_tok; jp.stop = stop_ids; jp.n_stop = n_stop;
  jp.next_tokens = next_tokens; jp.parent_idx = parent_idx; jp.new_cum = new_cum; jp.num_survivors = num_survivors;
  jp.fin_tokens = fin_tokens; jp.fin_parent = fin_parent; jp.fin_cum = fin_cum; jp.num_finished = num_finished;
  jp.C = C; jp.K = K;
  joint_select_scan_kernel<<<G, kScanThreads, 0, stream>>>(jp);
  return launch_status();
}

extern "C" int fr_select_final_topk(int64_t* tokens, int64_t* parent_idx, float* cum_out, int64_t* indices_scratch,
                                    const float* cum, const float* top_logprobs, const int64_t* top_tokens,
                                    const float* perturb, int G, int R, int C, int K, cudaStream_t stream) {
  FR_CHECK_ARG(G >= 0 && R > 0 && C > 0 && K > 0);
  if (G == 0) return FR_OK;
  FR_CHECK_ARG(tokens && parent_idx && cum_out && indices_scratch && cum && top_logprobs && top_tokens);
  StepParams sp{};
  sp.out_vals = cum_out; sp.out_parents = parent_idx; sp.out_tokens = tokens; sp.out_indices = indices_scratch;
  sp.cum = cum; sp.lp = top_logprobs; sp.tok = top_tokens; sp.perturb = perturb;
  sp.N = G; sp.BW = R; sp.C = C; sp.K = K; sp.L = 0;
  sp.neg_inf = -INFINITY;
  sp.idx_width = C;
  int st = make_trie(nullptr, &sp.trie);
  if (st != FR_OK) return st;
  st = check_step_common(sp);
  if (st != FR_OK) return st;
  return launch_step<0>(sp, stream);
}

extern "C" int fr_sid_beam_step(float* out_vals, int64_t* out_parents, int64_t* out_tokens, int64_t* out_indices,
                                int64_t* out_child, const float* cum, const float* logits, int64_t ld,
                                const float* row_max, const float* row_logsum, const int64_t* node_in,
                                const int64_t* token_ids_in, int64_t* token_ids_out, int64_t* node_ids_out,
                                const uint8_t* do_expand, const int32_t* col_n, const fr_trie* trie,
                                int64_t level_tok_base, int64_t idx_base, int64_t idx_width, int N, int BW,
                                int level_width, int K, int L, int apply_expand, int apply_advance,
                                cudaStream_t stream) {
  StepParams p{};
  p.out_vals = out_vals; p.out_parents = out_parents; p.out_tokens = out_tokens; p.out_indices = out_indices;
  p.out_child = out_child; p.token_ids_out = token_ids_out; p.node_ids_out = node_ids_out;
  p.cum = cum; p.node_in = node_in; p.token_ids_in = token_ids_in; p.do_expand = do_expand; p.col_n = col_n;
  p.logits = logits; p.ld = ld; p.row_max = row_max; p.row_logsum = row_logsum;
  p.level_tok_base = level_tok_base; p.idx_base = idx_base; p.idx_width = idx_width > 0 ? idx_width : level_width;
  p.N = N; p.BW = BW; p.C = level_width; p.K = K; p.L = L;
  p.apply_mask = 1; p.apply_expand = apply_expand; p.apply_advance = apply_advance && apply_expand;
  p.neg_inf = -INFINITY;
  if (N == 0) return FR_OK;
  int st = make_trie(trie, &p.trie);
  if (st != FR_OK) return st;
  if (p.trie.kind == FR_TRIE_NONE) { p.trie.vsz = 1; p.trie.token_base = 0; }
  st = check_step_common(p);
  if (st != FR_OK) return st;
  FR_CHECK_ARG(logits && row_max && row_logsum && ld >= level_width);
  FR_CHECK_ARG(p.trie.kind == FR_TRIE_NONE || node_in);
  return launch_step<1>(p, stream);
}

extern "C" int fr_topk_merge_shards(float* out_vals, int64_t* out_parents, int64_t* out_tokens, int64_t* out_indices,
                                    int64_t* out_child, const float* shard_vals, const int64_t* shard_indices,
                                    const int64_t* shard_child, const void* shard_records, const int64_t* node_in,
                                    const int64_t* token_ids_in,
                                    int64_t* token_ids_out, int64_t* node_ids_out, const uint8_t* do_expand,
                                    const int32_t* col_n, const fr_trie* trie, int64_t level_tok_base,
                                    int64_t idx_width, int S, int N, int BW, int K, int L, int apply_expand,
                                    int apply_advance, cudaStream_t stream) {
  FR_CHECK_ARG(S > 0 && N >= 0 && BW > 0 && K > 0 && idx_width > 0);
  if (N == 0) return FR_OK;
  FR_CHECK_ARG(out_vals && out_parents && out_tokens && out_indices);
  FR_CHECK_ARG((shard_records && aligned16(shard_records)) || (shard_vals && shard_indices));
  FR_CHECK_SUPPORTED(K <= kMaxK && static_cast<int64_t>(S) * K <= 16384);
  MergeParams mp{};
  mp.vals = shard_vals; mp.indices = shard_indices; mp.child = shard_child; mp.S = S;
  mp.records = static_cast<const uint4*>(shard_records);
  StepParams& p = mp.step;
  {
    const int st = make_trie(trie, &p.trie);
    if (st != FR_OK) return st;
  }
  p.out_vals = out_vals; p.out_parents = out_parents; p.out_tokens = out_tokens; p.out_indices = out_indices;
  p.out_child = out_child; p.token_ids_out = token_ids_out; p.node_ids_out = node_ids_out;
  p.node_in = node_in; p.token_ids_in = token_ids_in; p.do_expand = do_expand; p.col_n = col_n;
  p.level_tok_base = level_tok_base; p.idx_width = idx_width;
  p.N = N; p.BW = BW; p.C = 1; p.K = K; p.L = L;
  p.apply_expand = apply_expand;
  p.apply_advance = apply_advance && apply_expand && (shard_child != nullptr || shard_records != nullptr);
  p.neg_inf = -INFINITY;
  if (apply_expand) {
    FR_CHECK_ARG(token_ids_in && token_ids_out && token_ids_in != token_ids_out && L > 0);
    FR_CHECK_SUPPORTED(K <= BW);
  }
  if (p.apply_advance) FR_CHECK_ARG(node_in && node_ids_out && node_in != node_ids_out);
  const size_t smem = static_cast<size_t>(S) * K * 8 + static_cast<size_t>(K) * 20 + 16;
  if (smem > 32 * 1024) {
    if (cudaFuncSetAttribute(merge_shards_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return FR_ERR_CUDA;
  }
  merge_shards_kernel<<<N, kThreads, smem, stream>>>(mp);
  return launch_status();
}

// ---------------------------------------------------------------------------
// Fused SID head: logits GEMM -> (tile statistics, legal candidates) -> top-K, without the logits matrix.
// ---------------------------------------------------------------------------
namespace fr {
namespace beam {

// Row masks over the codes of the level shard for tries whose layout the GEMM epilogue cannot index by node
// (sorted-key CSR, the reference's dense byte table, a bitmap whose level is not word-aligned with the shard):
// mask[row, c >> 5] bit (c & 31) = code c of the shard is a legal continuation of the row's node. One warp per
// row; `mask` must be zero on entry. Dead rows (cum == -inf) stay zero.
__global__ void __launch_bounds__(256) row_mask_kernel(uint32_t* __restrict__ mask, int words, const float* __restrict__ cum,
                                                      const int64_t* __restrict__ node_in, Trie tr, int64_t first_tok,
                                                      int C, int rows) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  if (cum[row] == -INFINITY) return;
  const int64_t node = node_in ? node_in[row] : -1;
  uint32_t* m = mask + static_cast<size_t>(row) * words;
  if (tr.kind == FR_TRIE_CSR && node >= 0) {
    if (tr.n_edges <= 0) return;
    const int64_t k0 = node * tr.vsz + (first_tok - tr.token_base);
    const int64_t e0 = lower_bound(tr.keys, tr.n_edges, k0);
    const int64_t e1 = lower_bound(tr.keys, tr.n_edges, k0 + C);
    for (int64_t e = e0 + lane; e < e1; e += 32) {
      const int64_t c = __ldg(tr.keys + e) - k0;
      atomicOr(m + (c >> 5), 1u << (c & 31));
    }
    return;
  }
  for (int c0 = 0; c0 < C; c0 += 32) {
    const int c = c0 + lane;
    const bool ok = c < C && trie_allowed(tr, node, first_tok + c);
    const uint32_t w = __ballot_sync(0xffffffffu, ok);
    if (lane == 0) m[c0 >> 5] = w;
  }
}

// Row statistics from the head GEMM's per-part entries ([parts, rows] each): 8 threads per row, each merging
// parts/8 consecutive entries with a running (max, scaled sum), then the eight partial results merged in
// group order through shared memory. 32 rows per CTA; loads are one 128-byte line per warp and part.
__global__ void __launch_bounds__(256) tile_stats_combine_kernel(const float* __restrict__ tmax, const float* __restrict__ tlog,
                                                                float* __restrict__ row_max, float* __restrict__ row_logsum,
                                                                int parts, int rows) {
  __shared__ float sm_m[8][32], sm_s[8][32];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int r = blockIdx.x * 32 + lane;
  const int per = (parts + 7) / 8;
  float m = -INFINITY, s = 0.f;
  if (r < rows) {
    const int p1 = min(parts, (grp + 1) * per);
    for (int p = grp * per; p < p1; ++p) {
      const float pm = __ldg(tmax + static_cast<size_t>(p) * rows + r);
      const float pl = __ldg(tlog + static_cast<size_t>(p) * rows + r);
      if (pm == -INFINITY) continue;  // a part without codes
      const float nm = fmaxf(m, pm);
      s = s * expf(m - nm) + expf(pl + (pm - nm));  // m == -inf: s is 0 and exp(-inf) = 0
      m = nm;
    }
  }
  sm_m[grp][lane] = m;
  sm_s[grp][lane] = s;
  __syncthreads();
  if (grp == 0 && r < rows) {
    float M = -INFINITY;
#pragma unroll
    for (int g = 0; g < 8; ++g) M = fmaxf(M, sm_m[g][lane]);
    float sum = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g)
      if (sm_m[g][lane] != -INFINITY) sum += sm_s[g][lane] * expf(sm_m[g][lane] - M);
    row_max[r] = M;
    row_logsum[r] = logf(sum);
  }
}

struct HeadWorkspace {
  float* tile_max;
  float* tile_logsum;
  float* row_max;
  float* row_logsum;
  int* cand_count;
  uint2* cand;
  uint32_t* row_mask;
  int64_t bytes;
};

static int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

// Carves the workspace; base may be null to compute the size only. needs_row_mask: every trie but an aligned bitmap.
static HeadWorkspace head_workspace(void* base, int N, int BW, int level_width, int cand_cap, bool needs_row_mask) {
  const int64_t rows = static_cast<int64_t>(N) * BW;
  const int64_t tiles = (level_width + 255) / 256 * kHeadParts;  // statistics entries per row
  const int64_t words = (level_width + 31) / 32;
  uint8_t* p = static_cast<uint8_t*>(base);
  int64_t off = 0;
  HeadWorkspace w{};
  auto take = [&](int64_t bytes) { void* q = p ? p + off : nullptr; off += align256(bytes); return q; };
  w.tile_max = static_cast<float*>(take(tiles * rows * 4));
  w.tile_logsum = static_cast<float*>(take(tiles * rows * 4));
  w.row_max = static_cast<float*>(take(rows * 4));
  w.row_logsum = static_cast<float*>(take(rows * 4));
  w.cand_count = static_cast<int*>(take(static_cast<int64_t>(N) * 4));
  w.cand = static_cast<uint2*>(take(static_cast<int64_t>(N) * cand_cap * 8));
  w.row_mask = needs_row_mask ? static_cast<uint32_t*>(take(rows * words * 4)) : nullptr;
  w.bytes = off;
  return w;
}

}  // namespace beam
}  // namespace fr

extern "C" int64_t fr_sid_head_topk_workspace_bytes(int N, int BW, int level_width, int cand_capacity) {
  if (N < 0 || BW <= 0 || level_width <= 0 || cand_capacity < 0) return -1;
  return head_workspace(nullptr, N, BW, level_width, cand_capacity, true).bytes;
}

extern "C" int fr_sid_head_topk(float* out_vals, int64_t* out_parents, int64_t* out_tokens, int64_t* out_indices,
                                int64_t* out_child, void* out_records, const void* a, const float* scale_a, int64_t lda, const void* w,
                                const float* scale_w, int64_t ldw, int K_dim, const float* cum, const int64_t* node_in,
                                const int64_t* token_ids_in, int64_t* token_ids_out, int64_t* node_ids_out,
                                const uint8_t* do_expand, const int32_t* col_n, const fr_trie* trie,
                                int64_t level_tok_base, int64_t idx_base, int64_t idx_width, int N, int BW,
                                int level_width, int K, int L, int apply_expand, int apply_advance, int phase,
                                float* row_max, float* row_logsum, void* workspace, int64_t workspace_bytes,
                                int cand_capacity, cudaStream_t stream) {
  FR_CHECK_ARG(N >= 0 && BW > 0 && level_width > 0 && K > 0 && L >= 0 && K_dim > 0 && cand_capacity > 0);
  FR_CHECK_ARG(phase >= 0 && phase <= 2);
  if (N == 0) return FR_OK;
  FR_CHECK_SUPPORTED(BW % 32 == 0 && idx_base % 32 == 0);
  FR_CHECK_ARG(workspace && aligned16(workspace) && cum);
  StepParams p{};
  p.out_vals = out_vals; p.out_parents = out_parents; p.out_tokens = out_tokens; p.out_indices = out_indices;
  p.out_child = out_child; p.token_ids_out = token_ids_out; p.node_ids_out = node_ids_out;
  p.out_records = static_cast<uint4*>(out_records);
  FR_CHECK_ARG(out_records == nullptr || aligned16(out_records));
  p.cum = cum; p.node_in = node_in; p.token_ids_in = token_ids_in; p.do_expand = do_expand; p.col_n = col_n;
  p.level_tok_base = level_tok_base; p.idx_base = idx_base; p.idx_width = idx_width > 0 ? idx_width : level_width;
  p.N = N; p.BW = BW; p.C = level_width; p.K = K; p.L = L;
  p.apply_mask = 1; p.apply_expand = apply_expand; p.apply_advance = apply_advance && apply_expand;
  p.neg_inf = -INFINITY;
  int st = make_trie(trie, &p.trie);
  if (st != FR_OK) return st;
  FR_CHECK_ARG(p.trie.kind == FR_TRIE_NONE || node_in);
  if (p.trie.kind == FR_TRIE_NONE) { p.trie.vsz = 1; p.trie.token_base = 0; }
  const int64_t first_tok = level_tok_base + idx_base;
  // a bitmap trie is read in place when its rows line up with the shard's 32-code words
  const bool direct_bitmap = p.trie.kind == FR_TRIE_BITMAP && static_cast<int64_t>(p.trie.words) * 32 >= idx_base + level_width;
  const HeadWorkspace ws = head_workspace(workspace, N, BW, level_width, cand_capacity, !direct_bitmap);
  FR_CHECK_ARG(workspace_bytes >= ws.bytes);
  const int rows = N * BW;
  const int tiles = (level_width + 255) / 256 * kHeadParts;
  const int words = (level_width + 31) / 32;
  float* mx = row_max ? row_max : ws.row_max;
  float* ls = row_logsum ? row_logsum : ws.row_logsum;
  if (phase == 0 || phase == 1) {
    FR_CHECK_ARG(a && scale_a && w && scale_w && aligned16(a) && aligned16(w) && aligned16(scale_w));
    FR_CHECK_ARG(lda >= K_dim && ldw >= K_dim && lda % 16 == 0 && ldw % 16 == 0 && K_dim % 16 == 0);
    if (cudaMemsetAsync(ws.cand_count, 0, static_cast<size_t>(N) * 4, stream) != cudaSuccess) return FR_ERR_CUDA;
    HeadEpi hp{};
    hp.tile_max = ws.tile_max; hp.tile_logsum = ws.tile_logsum; hp.cum = cum;
    hp.cand = ws.cand; hp.cand_count = ws.cand_count; hp.cand_cap = cand_capacity; hp.BW = BW;
    hp.idx_base = idx_base; hp.idx_width = p.idx_width;
    if (direct_bitmap) {
      hp.mask = p.trie.bitmap; hp.mask_index = node_in; hp.level_off = p.trie.level_off;
      hp.mask_stride = p.trie.words; hp.mask_rows = p.trie.n_rows; hp.mask_word0 = static_cast<int>(idx_base / 32);
      hp.level_off_expected = static_cast<int>(level_tok_base - p.trie.token_base);
    } else {
      if (cudaMemsetAsync(ws.row_mask, 0, static_cast<size_t>(rows) * words * 4, stream) != cudaSuccess) return FR_ERR_CUDA;
      row_mask_kernel<<<ceil_div(rows, 8), 256, 0, stream>>>(ws.row_mask, words, cum, p.trie.kind == FR_TRIE_NONE ? nullptr : node_in,
                                                            p.trie, first_tok, level_width, rows);
      if (launch_status() != FR_OK) return FR_ERR_CUDA;
      hp.mask = ws.row_mask; hp.mask_index = nullptr; hp.level_off = nullptr;
      hp.mask_stride = words; hp.mask_rows = rows; hp.mask_word0 = 0; hp.level_off_expected = 0;
    }
    st = launch_head_gemm(a, w, scale_a, scale_w, rows, level_width, K_dim, lda, ldw, hp, stream);
    if (st != FR_OK) return st;
    tile_stats_combine_kernel<<<ceil_div(rows, 32), 256, 0, stream>>>(ws.tile_max, ws.tile_logsum, mx, ls, tiles, rows);
    if (launch_status() != FR_OK) return FR_ERR_CUDA;
    if (phase == 1) return FR_OK;
  } else {
    FR_CHECK_ARG(row_max && row_logsum);  // the statistics of the whole row, combined by the caller
  }
  st = check_step_common(p);
  if (st != FR_OK) return st;
  p.row_max = mx; p.row_logsum = ls;
  p.cand = ws.cand; p.cand_count = ws.cand_count; p.cand_cap = cand_capacity;
  return launch_step<2>(p, stream);
}

// ---------------------------------------------------------------------------
// fr_mask_topk_expand without a caller-provided workspace.
//
// Who needs it: a host that binds this C ABI from a decode worker which owns no
// allocator of its own. In the serving engine this library plugs into, device
// memory is carved up once at start-up (weights, then the KV pool takes what is
// left), so by the time a decode tick runs there is nothing to cudaMalloc from,
// and a tick must not stall on the allocator anyway. Such a caller still passes
// its inputs and outputs, but the masked-score workspace comes from the fixed
// array below, which every GPU that loads the library holds until exit.
//
// Limits and rules:
//   * N * BW * C <= FR_STATIC_SCRATCH_FLOATS (2 Mi floats = 8 MiB) whenever the call masks
//     (apply_mask with a trie and node_in: the only case that touches the array); larger
//     requests are refused with FR_ERR_UNSUPPORTED, nothing is launched. Unmasked calls never
//     use the array and have no such limit.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress with that device current) and caches it; make that
//     first call before starting any stream capture. The cache is keyed by device
//     ordinal and filled without a lock (concurrent first calls store the same value);
//     it does not survive cudaDeviceReset: do not reset a device this library has served.
//   * All calls on a device share the one array. The kernel rewrites every
//     workspace entry it later reads, so nothing has to be cleared between
//     calls, but two calls that overlap on the GPU (different streams) race on it.
// ---------------------------------------------------------------------------
#define FR_STATIC_SCRATCH_FLOATS (2u << 20)
static __device__ __align__(256) float g_static_scratch[FR_STATIC_SCRATCH_FLOATS];

extern "C" int fr_mask_topk_expand_static(float* out_vals, int64_t* out_parents, int64_t* out_tokens,
                                          int64_t* out_indices, int64_t* out_child, const float* cum,
                                          const float* top_logprobs, const int64_t* top_tokens, const int64_t* node_in,
                                          const int64_t* token_ids_in, int64_t* token_ids_out, int64_t* node_ids_out,
                                          const uint8_t* do_expand, const int32_t* col_n, const fr_trie* trie, int N,
                                          int BW, int C, int K, int L, int apply_mask, int apply_expand,
                                          int apply_advance, cudaStream_t stream) {
  FR_CHECK_ARG(N >= 0 && BW > 0 && C > 0);
  // the array is only touched when the step masks (same condition as in fr_mask_topk_expand)
  const bool uses_scratch = apply_mask && node_in != nullptr && trie != nullptr && trie->kind != FR_TRIE_NONE;
  if (uses_scratch && static_cast<int64_t>(N) * BW * C > static_cast<int64_t>(FR_STATIC_SCRATCH_FLOATS))
    return FR_ERR_UNSUPPORTED;
  // In host code `g_static_scratch` is only a handle for the symbol, not a device
  // address: resolve it once per device, with that device current.
  constexpr int kMaxDev = 64;
  static float* dev_ptr[kMaxDev] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return FR_ERR_CUDA;
  if (dev_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return FR_ERR_CUDA;
    dev_ptr[dev] = static_cast<float*>(p);
  }
  return fr_mask_topk_expand(out_vals, out_parents, out_tokens, out_indices, out_child, dev_ptr[dev], cum,
                             top_logprobs, top_tokens, node_in, token_ids_in, token_ids_out, node_ids_out, do_expand,
                             col_n, trie, N, BW, C, K, L, apply_mask, apply_expand, apply_advance, stream);
}
