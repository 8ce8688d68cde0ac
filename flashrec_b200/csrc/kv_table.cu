// Bookkeeping on the row -> slot table (`req_to_token`, int32 [pool rows, max_seq]) of the beam
// scheduler: everything one decode tick does to it, without torch index ops.
//
//   fr_gather_kv_indices   ragged copy req_to_token[row, :seq_len] -> flat slot list + indptr
//                          (gather_kv_indices, attention/kv_indices.py:20-132).
//   fr_kv_table_step       the three table operations of a tick in one call: every request's
//                          decode window gathered by last tick's parents (remap_by_parents,
//                          scheduler/kv_remap.py:30-66), the new token's slot written at the end
//                          of each row (scheduler/scheduler.py:1305-1310), and the flat slot list
//                          of the attention call (gather_kv_indices).
//   fr_kv_table_fanout     a prefill row's slots copied to all beam rows of its request
//                          (ModelEngine.copy_prefill_to_beams_many, engine/engine.py:252-274).
//
// The window remap is an in-place gather across rows. It is made race-free without a snapshot
// of the table: the first kernel only READS the table (each row takes its window from its
// parent's row) and writes the flat list; the second kernel only reads the flat list and writes
// the windows and the new column back into the table. Both move 4-byte words, one warp per row.
#include "fr_common.cuh"

namespace fr {

int* device_status_ptr();  // capi.cu

// indptr[0] = 0, indptr[i + 1] = sum of max(seq_lens[..i], 0). One CTA; each thread owns kScanItems
// consecutive rows of a chunk (read with 16-byte loads when the array allows it), so up to 32768 rows take one
// round of the block-wide scan: the kernel is a chain of a few latencies, not bandwidth.
// `status` (optional): the library's sticky status word; it receives {FR_ERR_BAD_ARG, site 41} when the
// list is longer than `capacity`, since the caller cannot see that without a host read.
constexpr int kScanItems = 32;
__global__ void __launch_bounds__(1024) seq_scan_kernel(const int32_t* __restrict__ seq_lens,
                                                       int32_t* __restrict__ indptr, int n, int capacity = 0,
                                                       int* status = nullptr) {
  __shared__ int32_t warp_tot[32];
  __shared__ int32_t carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) { carry_s = 0; indptr[0] = 0; }
  __syncthreads();
  const bool vec_ok = (reinterpret_cast<uintptr_t>(seq_lens) & 15u) == 0;
  for (int base = 0; base < n; base += 1024 * kScanItems) {
    const int i0 = base + threadIdx.x * kScanItems;
    int32_t v[kScanItems];
    if (vec_ok && i0 + kScanItems <= n) {
#pragma unroll
      for (int j = 0; j < kScanItems; j += 4) {
        const int4 q = __ldg(reinterpret_cast<const int4*>(seq_lens + i0 + j));
        v[j] = max(q.x, 0); v[j + 1] = max(q.y, 0); v[j + 2] = max(q.z, 0); v[j + 3] = max(q.w, 0);
      }
    } else {
#pragma unroll
      for (int j = 0; j < kScanItems; ++j) v[j] = i0 + j < n ? max(__ldg(seq_lens + i0 + j), 0) : 0;
    }
    int32_t x = 0;
#pragma unroll
    for (int j = 0; j < kScanItems; ++j) x += v[j];
    const int32_t mine = x;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int32_t y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_tot[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int32_t w = warp_tot[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int32_t y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      warp_tot[lane] = w;  // inclusive
    }
    __syncthreads();
    const int32_t incl = carry_s + x + (warp > 0 ? warp_tot[warp - 1] : 0);
    int32_t run = incl - mine;
#pragma unroll
    for (int j = 0; j < kScanItems; ++j) {
      run += v[j];
      if (i0 + j < n) indptr[i0 + j + 1] = run;
    }
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = incl;
    __syncthreads();
  }
  if (status != nullptr && threadIdx.x == 0 && carry_s > capacity) {
    if (atomicCAS(status, 0, FR_ERR_BAD_ARG) == 0) status[1] = 41;
  }
}

// dst[c] = src[c] for c in [begin, end), c < limit, by one warp: four independent 128-byte rows of
// loads in flight per lane before the stores.
__device__ __forceinline__ void warp_copy_words(const int32_t* __restrict__ src, int32_t* __restrict__ dst, int begin,
                                                int end, int limit, int lane) {
  end = min(end, limit);
  int c = begin + lane;
  for (; c + 96 < end; c += 128) {
    const int32_t v0 = __ldg(src + c), v1 = __ldg(src + c + 32), v2 = __ldg(src + c + 64), v3 = __ldg(src + c + 96);
    dst[c] = v0; dst[c + 32] = v1; dst[c + 64] = v2; dst[c + 96] = v3;
  }
  for (; c < end; c += 32) dst[c] = __ldg(src + c);
}

// The offsets and the copy in one launch: a CTA owns 32 consecutive rows (one warp each) and finds the offset of
// its first row itself, by summing every length before it (the lengths are a few KB that every CTA of an SM
// reads from L1; 512 CTAs reading 8 K values on average is a fraction of the slot ids the copy moves), so there
// is no scan kernel in front and no dependency between CTAs. indptr is written along the way.
// (ROWS = 32 rows per CTA for long lists; 8 for a few hundred rows, where more, smaller CTAs start sooner.)
template <int kFusedRows>
__global__ void __launch_bounds__(kFusedRows * 32) gather_kv_fused_kernel(
    const int32_t* __restrict__ table, int64_t stride, const int64_t* __restrict__ rows,
    const int32_t* __restrict__ seq_lens, int32_t* __restrict__ indptr, int32_t* __restrict__ out, int n, int capacity) {
  __shared__ int32_t warp_part[kFusedRows];
  __shared__ int32_t row_off[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r0 = blockIdx.x * kFusedRows;
  // sum of the lengths before row r0 (r0 is a multiple of 32: whole int4 groups when the array is aligned)
  int32_t acc = 0;
  if ((reinterpret_cast<uintptr_t>(seq_lens) & 15u) == 0) {
    const int4* q = reinterpret_cast<const int4*>(seq_lens);
    for (int i = threadIdx.x; i < r0 / 4; i += blockDim.x) {
      const int4 v = __ldg(q + i);
      acc += max(v.x, 0) + max(v.y, 0) + max(v.z, 0) + max(v.w, 0);
    }
  } else {
    for (int i = threadIdx.x; i < r0; i += blockDim.x) acc += max(__ldg(seq_lens + i), 0);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) warp_part[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    int32_t base = lane < kFusedRows ? warp_part[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) base += __shfl_xor_sync(0xffffffffu, base, o);
    // exclusive offsets of this CTA's rows
    const int r = r0 + lane;
    const int32_t len = (r < n && lane < kFusedRows) ? max(__ldg(seq_lens + r), 0) : 0;
    int32_t incl = len;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    row_off[lane] = base + incl - len;
    if (r < n && lane < kFusedRows) indptr[r + 1] = base + incl;
    if (r0 == 0 && lane == 0) indptr[0] = 0;
  }
  __syncthreads();
  const int r = r0 + warp;
  if (r >= n || capacity == 0) return;
  const int32_t sl = max(seq_lens[r], 0);
  const int32_t off = row_off[warp];
  const int32_t* src = table + rows[r] * stride;
  warp_copy_words(src, out + off, 0, sl, capacity - off, lane);
}

struct StepArgs {
  int32_t* table;
  int64_t stride;
  int n_table_rows, n_cols;
  const int64_t* rows;
  const int32_t* group_indptr;
  int n_groups;
  const int64_t* parents_rel;
  const int32_t* prefix_len;
  const int32_t* seq_lens;
  const int64_t* new_slot;
  const int32_t* indptr;
  int32_t* out;
  int n, capacity;
};

// Length of row i after the tick, and where its window starts and ends.
__device__ __forceinline__ void row_extent(const StepArgs& a, int i, int& sl, int& pre, int& keep) {
  sl = min(max(a.seq_lens[i], 0), a.n_cols);
  keep = max(sl - (a.new_slot ? 1 : 0), 0);
  pre = a.prefix_len ? min(max(a.prefix_len[i], 0), keep) : keep;
}

// Phase 1: out[indptr[i] + c] = slot of column c of row i AFTER the tick, read from the table as it
// was BEFORE the tick: prompt columns from the row itself, window columns from the parent's row,
// the last column from new_slot.
__global__ void __launch_bounds__(256) kv_step_gather_kernel(StepArgs a) {
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= a.n) return;
  const int lane = threadIdx.x & 31;
  int sl, pre, keep;
  row_extent(a, i, sl, pre, keep);
  const int64_t own_row = a.rows[i];
  int64_t par_row = own_row;
  if (a.parents_rel && pre < keep) {
    // request of batch row i: the last g with group_indptr[g] <= i
    int lo = 0, hi = a.n_groups;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (a.group_indptr[mid] <= i) lo = mid; else hi = mid;
    }
    const int g0 = a.group_indptr[lo], k = a.group_indptr[lo + 1] - g0;
    // a malformed group list (empty or reversed group, bounds outside the batch) leaves the row
    // with its own window instead of reading outside `rows`
    if (k > 0 && g0 >= 0 && g0 + k <= a.n) {
      int64_t p = a.parents_rel[i];
      p = p < 0 ? 0 : (p > k - 1 ? k - 1 : p);  // clamp(0, k - 1) as the reference does
      par_row = a.rows[g0 + static_cast<int>(p)];
    }
  }
  const bool own_ok = own_row >= 0 && own_row < a.n_table_rows;
  // a parent whose table row does not exist: the row keeps its own window (identity), so the
  // write-back never copies list entries that no one wrote
  if (par_row < 0 || par_row >= a.n_table_rows) par_row = own_row;
  const bool par_ok = par_row >= 0 && par_row < a.n_table_rows;
  const int32_t off = a.indptr[i];
  int32_t* dst = a.out + off;
  const int limit = a.capacity - off;
  // the table is only read by this kernel, the list only written
  if (own_ok) warp_copy_words(a.table + own_row * a.stride, dst, 0, pre, limit, lane);
  if (par_ok) warp_copy_words(a.table + par_row * a.stride, dst, pre, keep, limit, lane);
  if (a.new_slot && lane == 0 && keep < sl && keep < limit) dst[keep] = static_cast<int32_t>(a.new_slot[i]);
}

// Phase 2: window and new column of every row written back from the flat list.
__global__ void __launch_bounds__(256) kv_step_writeback_kernel(StepArgs a) {
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= a.n) return;
  const int lane = threadIdx.x & 31;
  int sl, pre, keep;
  row_extent(a, i, sl, pre, keep);
  const int64_t own_row = a.rows[i];
  if (own_row < 0 || own_row >= a.n_table_rows) return;
  if (!a.parents_rel) pre = keep;  // no remap: only the new column changes
  int32_t* dst = a.table + own_row * a.stride;
  const int32_t off = a.indptr[i];
  warp_copy_words(a.out + off, dst, pre, sl, a.capacity - off, lane);
}

// table[dst_rows[r * bw + b], :m] = table[src_rows[r], :m]
__global__ void __launch_bounds__(256) kv_fanout_kernel(int32_t* table, int64_t stride, int n_table_rows,
                                                       const int64_t* __restrict__ src_rows,
                                                       const int64_t* __restrict__ dst_rows, int total, int bw, int m) {
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= total) return;
  const int lane = threadIdx.x & 31;
  const int64_t s = src_rows[i / bw], d = dst_rows[i];
  if (s < 0 || s >= n_table_rows || d < 0 || d >= n_table_rows || s == d) return;
  warp_copy_words(table + s * stride, table + d * stride, 0, m, m, lane);
}

}  // namespace fr

using namespace fr;

extern "C" int fr_gather_kv_indices(const int32_t* req_to_token, int64_t row_stride, const int64_t* rows,
                                    const int32_t* seq_lens, int32_t* indptr_out, int32_t* out, int n,
                                    int out_capacity, cudaStream_t stream) {
  FR_CHECK_ARG(n >= 0 && out_capacity >= 0);
  if (n == 0) return FR_OK;
  FR_CHECK_ARG(req_to_token && rows && seq_lens && indptr_out && (out || out_capacity == 0));
  if (n <= 4096)
    gather_kv_fused_kernel<8><<<ceil_div(n, 8), 256, 0, stream>>>(req_to_token, row_stride, rows, seq_lens, indptr_out, out,
                                                                 n, out_capacity);
  else
    gather_kv_fused_kernel<32><<<ceil_div(n, 32), 1024, 0, stream>>>(req_to_token, row_stride, rows, seq_lens, indptr_out,
                                                                    out, n, out_capacity);
  return launch_status();
}

extern "C" int fr_kv_table_step(int32_t* req_to_token, int64_t row_stride, int n_table_rows, int n_cols,
                                const int64_t* rows, const int32_t* group_indptr, int n_groups,
                                const int64_t* parents_rel, const int32_t* prefix_len, const int32_t* seq_lens,
                                const int64_t* new_slot, int32_t* indptr_out, int32_t* out, int n, int out_capacity,
                                cudaStream_t stream) {
  FR_CHECK_ARG(n >= 0 && out_capacity >= 0 && n_table_rows >= 0 && n_cols >= 0 && n_groups >= 0);
  if (n == 0) return FR_OK;
  FR_CHECK_ARG(req_to_token && rows && seq_lens && indptr_out && out && row_stride >= n_cols);
  FR_CHECK_ARG(!parents_rel || (group_indptr && n_groups > 0 && prefix_len));
  seq_scan_kernel<<<1, 1024, 0, stream>>>(seq_lens, indptr_out, n, out_capacity, device_status_ptr());
  if (launch_status() != FR_OK) return FR_ERR_CUDA;
  StepArgs a{req_to_token, row_stride, n_table_rows, n_cols, rows, group_indptr, n_groups, parents_rel, prefix_len,
             seq_lens, new_slot, indptr_out, out, n, out_capacity};
  kv_step_gather_kernel<<<ceil_div(n, 8), 256, 0, stream>>>(a);
  if (launch_status() != FR_OK) return FR_ERR_CUDA;
  if (!parents_rel && !new_slot) return FR_OK;  // nothing to write back: a plain gather
  kv_step_writeback_kernel<<<ceil_div(n, 8), 256, 0, stream>>>(a);
  return launch_status();
}

extern "C" int fr_kv_table_fanout(int32_t* req_to_token, int64_t row_stride, int n_table_rows, const int64_t* src_rows,
                                  const int64_t* dst_rows, int n_requests, int beam_width, int m,
                                  cudaStream_t stream) {
  FR_CHECK_ARG(n_requests >= 0 && beam_width >= 0 && m >= 0 && n_table_rows >= 0);
  const int64_t total = static_cast<int64_t>(n_requests) * beam_width;
  if (total == 0 || m == 0) return FR_OK;
  FR_CHECK_ARG(req_to_token && src_rows && dst_rows && row_stride >= m && total <= INT32_MAX);
  kv_fanout_kernel<<<ceil_div(total, 8), 256, 0, stream>>>(req_to_token, row_stride, n_table_rows, src_rows, dst_rows,
                                                          static_cast<int>(total), beam_width, m);
  return launch_status();
}
