// Catalog trie built on the device from an integer item array [n_items, depth], straight into the
// CSR layout the beam-step kernels read (sorted keys node * vsz + (token - token_base), child ids).
//
// Stands in for BeamValidPathTrie's Python construction: the dict walk of _ensure_gpu_cache and the
// CSR flattening of _build_csr_cache (search/trie.py:222-251, 300-327), with the same node numbering:
// root = 0, internal prefixes numbered by (length, lexicographic prefix), leaves = -1,
// invalid_node = number of internal nodes.
//
// Sort-based, no hashing, no host round trip:
//   1. pack every item into one int64 key (mixed radix over the level sizes),
//   2. radix sort + unique (CUB),
//   3. per depth d = 1..L: the prefix of length d of item i is key / tail[d]; a head flag marks the
//      first item of each distinct prefix, an inclusive scan of the flags numbers the prefixes,
//   4. every head at depth d emits one edge (parent = node of its length d-1 prefix, code = its
//      level d-1 digit, child = its own node or -1 at the last level); edges come out ordered by
//      (depth, prefix), which is ascending key order because deeper nodes have larger ids.
// Counts stay on the device (counts_out) until the caller reads them once.
#include <cub/cub.cuh>

#include "fr_common.cuh"

namespace fr {
namespace trie_build {

constexpr int kMaxDepth = 8;

struct Levels {
  int depth;
  int64_t size[kMaxDepth];      // codebook size per level
  int64_t tail[kMaxDepth + 1];  // tail[d] = prod(size[d:]), tail[depth] = 1
  int64_t off[kMaxDepth + 1];   // token offset of each level, off[depth] = vsz
};

__global__ void __launch_bounds__(256) pack_kernel(const int32_t* __restrict__ items, int64_t n, Levels lv,
                                                   int64_t* __restrict__ keys, int* __restrict__ bad) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int64_t k = 0;
  bool ok = true;
  for (int l = 0; l < lv.depth; ++l) {
    const int64_t c = items[i * lv.depth + l];
    ok = ok && c >= 0 && c < lv.size[l];
    k = k * lv.size[l] + (c < 0 ? 0 : (c >= lv.size[l] ? lv.size[l] - 1 : c));
  }
  keys[i] = k;
  if (!ok) atomicExch(bad, 1);
}

// head[i] = 1 when item i starts a new prefix of length d (d >= 1)
__global__ void __launch_bounds__(256) head_kernel(const int64_t* __restrict__ keys, const int* __restrict__ n_unique,
                                                   int64_t tail_d, int32_t* __restrict__ head) {
  const int64_t n = *n_unique;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  head[i] = (i == 0 || keys[i] / tail_d != keys[i - 1] / tail_d) ? 1 : 0;
}

// counts: [0] = unique items, [1] = internal nodes, [2] = edges, [3 + d] = first node id of depth d
// (d = 0..depth), [3 + depth + 1 + d] = first edge of the edges into depth d + 1 (d = 0..depth).
__global__ void level_counts_kernel(const int* __restrict__ n_unique, const int32_t* __restrict__ rank_d, int d,
                                    int depth, int64_t* __restrict__ counts) {
  // one thread; called after the scan of depth d (1-based); rank_d[n-1] = number of prefixes of length d
  const int64_t n = *n_unique;
  const int64_t cnt = n > 0 ? rank_d[n - 1] : 0;
  int64_t* node_start = counts + 3;
  int64_t* edge_start = counts + 3 + depth + 1;
  if (d == 1) {
    counts[0] = n;
    node_start[0] = 0;
    node_start[1] = 1;  // the root
    edge_start[0] = 0;
  }
  // prefixes of length d are nodes of depth d (internal when d < depth) and the edges into depth d
  if (d < depth) node_start[d + 1] = node_start[d] + cnt;  // node_start has depth + 1 entries
  edge_start[d] = edge_start[d - 1] + cnt;
  if (d == depth) {
    counts[1] = node_start[depth];
    counts[2] = edge_start[depth];
  }
}

// One edge per head of depth d. rank_prev = inclusive ranks of depth d - 1 (nullptr for d == 1: the root).
__global__ void __launch_bounds__(256) edge_kernel(const int64_t* __restrict__ keys, const int* __restrict__ n_unique,
                                                   const int32_t* __restrict__ head, const int32_t* __restrict__ rank_d,
                                                   const int32_t* __restrict__ rank_prev, int d, Levels lv,
                                                   const int64_t* __restrict__ counts, int64_t* __restrict__ out_keys,
                                                   int64_t* __restrict__ out_child, int64_t edge_capacity) {
  const int64_t n = *n_unique;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n || head[i] == 0) return;
  const int64_t* node_start = counts + 3;
  const int64_t* edge_start = counts + 3 + lv.depth + 1;
  const int64_t prefix = keys[i] / lv.tail[d];
  const int64_t code = prefix % lv.size[d - 1];
  const int64_t parent = d == 1 ? 0 : node_start[d - 1] + (rank_prev[i] - 1);
  const int64_t child = d < lv.depth ? node_start[d] + (rank_d[i] - 1) : -1;
  const int64_t e = edge_start[d - 1] + (rank_d[i] - 1);
  if (e < edge_capacity) {
    out_keys[e] = parent * lv.off[lv.depth] + lv.off[d - 1] + code;
    out_child[e] = child;
  }
}

// Bitmap layout from the CSR arrays: one bit per (node, code of the node's own level), the id of the
// node's first child (children are numbered consecutively in code order) and the token offset of the
// node's level. One thread per edge / per node.
struct BitmapArgs {
  const int64_t* keys;
  const int64_t* child;
  int64_t n_edges, n_rows, vsz;
  int depth, words;
  int64_t node_start[kMaxDepth + 1];
  int64_t off[kMaxDepth + 1];
  uint32_t* bitmap;
  int64_t* child_base;
  int32_t* level_off;
};

__global__ void __launch_bounds__(256) bitmap_nodes_kernel(BitmapArgs a) {
  const int64_t node = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (node >= a.n_rows) return;
  int d = 0;
  while (d + 1 < a.depth && node >= a.node_start[d + 1]) ++d;
  if (node >= a.node_start[a.depth]) d = 0;  // the row of the invalid node
  a.level_off[node] = static_cast<int32_t>(a.off[d]);
  a.child_base[node] = -1;
}

__global__ void __launch_bounds__(256) bitmap_edges_kernel(BitmapArgs a) {
  const int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= a.n_edges) return;
  const int64_t key = a.keys[e];
  const int64_t parent = key / a.vsz, rel = key - parent * a.vsz;
  if (parent < 0 || parent >= a.n_rows) return;
  const int64_t code = rel - a.level_off[parent];
  if (code >= 0 && (code >> 5) < a.words)
    atomicOr(a.bitmap + parent * a.words + (code >> 5), 1u << (code & 31));
  if (e == 0 || a.keys[e - 1] / a.vsz != parent) a.child_base[parent] = a.child[e];
}

__global__ void mark_bad_kernel(const int* __restrict__ bad, int64_t* __restrict__ counts) {
  if (*bad) counts[0] = -1;
}

static size_t align_up(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

struct Plan {
  size_t keys_a, keys_b, head, rank0, rank1, scalars, cub, total;
  size_t cub_bytes;
};

static int make_plan(int64_t n_items, Plan* pl) {
  const int n = static_cast<int>(n_items);
  size_t sort_b = 0, uniq_b = 0, scan_b = 0;
  cub::DoubleBuffer<int64_t> db(nullptr, nullptr);
  if (cub::DeviceRadixSort::SortKeys(nullptr, sort_b, db, n, 0, 64) != cudaSuccess) return FR_ERR_CUDA;
  if (cub::DeviceSelect::Unique(nullptr, uniq_b, static_cast<int64_t*>(nullptr), static_cast<int64_t*>(nullptr),
                                static_cast<int*>(nullptr), n) != cudaSuccess)
    return FR_ERR_CUDA;
  if (cub::DeviceScan::InclusiveSum(nullptr, scan_b, static_cast<int32_t*>(nullptr), static_cast<int32_t*>(nullptr),
                                    n) != cudaSuccess)
    return FR_ERR_CUDA;
  pl->cub_bytes = std::max(sort_b, std::max(uniq_b, scan_b));
  size_t o = 0;
  pl->keys_a = o; o += align_up(static_cast<size_t>(n) * 8);
  pl->keys_b = o; o += align_up(static_cast<size_t>(n) * 8);
  pl->head = o; o += align_up(static_cast<size_t>(n) * 4);
  pl->rank0 = o; o += align_up(static_cast<size_t>(n) * 4);
  pl->rank1 = o; o += align_up(static_cast<size_t>(n) * 4);
  pl->scalars = o; o += 256;
  pl->cub = o; o += align_up(pl->cub_bytes);
  pl->total = o;
  return FR_OK;
}

}  // namespace trie_build
}  // namespace fr

using namespace fr;
using namespace fr::trie_build;

extern "C" int64_t fr_trie_build_workspace_bytes(int64_t n_items) {
  if (n_items <= 0) return 256;
  if (n_items > INT32_MAX) return -1;
  Plan pl;
  if (make_plan(n_items, &pl) != FR_OK) return -1;
  return static_cast<int64_t>(pl.total);
}

extern "C" int fr_trie_build_csr(const int32_t* items, int64_t n_items, int depth, const int64_t* sizes,
                                 int64_t* keys_out, int64_t* child_out, int64_t edge_capacity, int64_t* counts_out,
                                 void* workspace, int64_t workspace_bytes, cudaStream_t stream) {
  FR_CHECK_ARG(n_items >= 0 && depth >= 1 && sizes && counts_out && edge_capacity >= 0);
  FR_CHECK_SUPPORTED(depth <= kMaxDepth && n_items <= INT32_MAX);
  Levels lv{};
  lv.depth = depth;
  lv.off[0] = 0;
  for (int l = 0; l < depth; ++l) {
    FR_CHECK_ARG(sizes[l] > 0);
    lv.size[l] = sizes[l];
    lv.off[l + 1] = lv.off[l] + sizes[l];
  }
  lv.tail[depth] = 1;
  int bits = 0;
  for (int l = depth - 1; l >= 0; --l) {
    FR_CHECK_SUPPORTED(lv.tail[l + 1] <= (INT64_MAX >> 1) / lv.size[l]);  // the packed key must fit 62 bits
    lv.tail[l] = lv.tail[l + 1] * lv.size[l];
  }
  while (bits < 63 && (1ll << bits) < lv.tail[0]) ++bits;
  const int n_counts = 3 + 2 * (depth + 1);
  if (cudaMemsetAsync(counts_out, 0, sizeof(int64_t) * n_counts, stream) != cudaSuccess) return FR_ERR_CUDA;
  if (n_items == 0) {
    // an empty catalog: the root alone
    const int64_t one = 1;
    if (cudaMemcpyAsync(counts_out + 1, &one, sizeof(int64_t), cudaMemcpyHostToDevice, stream) != cudaSuccess)
      return FR_ERR_CUDA;
    return FR_OK;
  }
  FR_CHECK_ARG(items && keys_out && child_out && workspace);
  Plan pl;
  int st = make_plan(n_items, &pl);
  if (st != FR_OK) return st;
  FR_CHECK_ARG(workspace_bytes >= static_cast<int64_t>(pl.total) && aligned16(workspace));
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int64_t* keys_a = reinterpret_cast<int64_t*>(ws + pl.keys_a);
  int64_t* keys_b = reinterpret_cast<int64_t*>(ws + pl.keys_b);
  int32_t* head = reinterpret_cast<int32_t*>(ws + pl.head);
  int32_t* rank[2] = {reinterpret_cast<int32_t*>(ws + pl.rank0), reinterpret_cast<int32_t*>(ws + pl.rank1)};
  int* n_unique = reinterpret_cast<int*>(ws + pl.scalars);
  int* bad = n_unique + 1;
  void* cub_ws = ws + pl.cub;
  size_t cub_bytes = pl.cub_bytes;
  const int n = static_cast<int>(n_items);
  const int blocks = ceil_div(n_items, 256);

  if (cudaMemsetAsync(ws + pl.scalars, 0, 256, stream) != cudaSuccess) return FR_ERR_CUDA;
  pack_kernel<<<blocks, 256, 0, stream>>>(items, n_items, lv, keys_a, bad);
  if (launch_status() != FR_OK) return FR_ERR_CUDA;
  cub::DoubleBuffer<int64_t> db(keys_a, keys_b);
  if (cub::DeviceRadixSort::SortKeys(cub_ws, cub_bytes, db, n, 0, bits > 0 ? bits : 1, stream) != cudaSuccess)
    return FR_ERR_CUDA;
  int64_t* sorted = db.Current();
  int64_t* uniq = db.Alternate();
  cub_bytes = pl.cub_bytes;
  if (cub::DeviceSelect::Unique(cub_ws, cub_bytes, sorted, uniq, n_unique, n, stream) != cudaSuccess)
    return FR_ERR_CUDA;
  for (int d = 1; d <= depth; ++d) {
    head_kernel<<<blocks, 256, 0, stream>>>(uniq, n_unique, lv.tail[d], head);
    if (launch_status() != FR_OK) return FR_ERR_CUDA;
    cub_bytes = pl.cub_bytes;
    // scanning all n entries keeps the launch independent of the device-side count; entries past
    // n_unique hold stale flags that nothing reads
    if (cub::DeviceScan::InclusiveSum(cub_ws, cub_bytes, head, rank[d & 1], n, stream) != cudaSuccess)
      return FR_ERR_CUDA;
    level_counts_kernel<<<1, 1, 0, stream>>>(n_unique, rank[d & 1], d, depth, counts_out);
    if (launch_status() != FR_OK) return FR_ERR_CUDA;
    edge_kernel<<<blocks, 256, 0, stream>>>(uniq, n_unique, head, rank[d & 1], d > 1 ? rank[(d - 1) & 1] : nullptr, d,
                                            lv, counts_out, keys_out, child_out, edge_capacity);
    if (launch_status() != FR_OK) return FR_ERR_CUDA;
  }
  // an item code outside its level makes the whole build invalid: reported through the counts
  // (counts[0] = -1) rather than by reading a flag back here
  mark_bad_kernel<<<1, 1, 0, stream>>>(bad, counts_out);
  return launch_status();
}

extern "C" int fr_trie_csr_to_bitmap(const int64_t* keys, const int64_t* child, int64_t n_edges, int depth,
                                     const int64_t* sizes, const int64_t* node_start, uint32_t* bitmap_out,
                                     int64_t* child_base_out, int32_t* level_off_out, int words,
                                     cudaStream_t stream) {
  FR_CHECK_ARG(n_edges >= 0 && depth >= 1 && sizes && node_start && bitmap_out && child_base_out && level_off_out);
  FR_CHECK_SUPPORTED(depth <= kMaxDepth);
  FR_CHECK_ARG(n_edges == 0 || (keys && child));
  BitmapArgs a{};
  a.keys = keys; a.child = child; a.n_edges = n_edges; a.depth = depth; a.words = words;
  a.bitmap = bitmap_out; a.child_base = child_base_out; a.level_off = level_off_out;
  a.off[0] = 0;
  int64_t widest = 0;
  for (int l = 0; l < depth; ++l) {
    FR_CHECK_ARG(sizes[l] > 0);
    a.off[l + 1] = a.off[l] + sizes[l];
    widest = sizes[l] > widest ? sizes[l] : widest;
  }
  for (int d = 0; d <= depth; ++d) a.node_start[d] = node_start[d];
  a.vsz = a.off[depth];
  a.n_rows = node_start[depth] + 1;  // internal nodes + the invalid node's empty row
  FR_CHECK_ARG(words > 0 && static_cast<int64_t>(words) * 32 >= widest && a.n_rows > 0);
  if (cudaMemsetAsync(bitmap_out, 0, static_cast<size_t>(a.n_rows) * words * sizeof(uint32_t), stream) != cudaSuccess)
    return FR_ERR_CUDA;
  bitmap_nodes_kernel<<<ceil_div(a.n_rows, 256), 256, 0, stream>>>(a);
  if (launch_status() != FR_OK) return FR_ERR_CUDA;
  if (n_edges == 0) return FR_OK;
  bitmap_edges_kernel<<<ceil_div(n_edges, 256), 256, 0, stream>>>(a);
  return launch_status();
}
