// Block-wide top-K selection shared by the beam step and the per-row top-k.
//
// Candidates are 64-bit composites (order-preserving fp32 key << 32 | ~index),
// all distinct, so "the K largest composites" is exactly "score descending,
// smaller index first". radix_select_topk() finds the K-th largest composite
// with 11/11/10-bit digit passes over a caller-supplied enumeration (each pass
// histograms the candidates that match the prefix found so far and stops as
// soon as the boundary bin is taken whole), collects the winners into shared
// memory and bitonic-sorts them in descending order.
#pragma once

#include "fr_common.cuh"

namespace fr {
namespace topk {

constexpr int kBins = 2048;

// (-0.0 is folded into +0.0 first: the two compare equal and must tie on the index.)
__device__ __forceinline__ uint64_t compose(float s, uint32_t idx) {
  s = __fadd_rn(s, 0.0f);
  return (static_cast<uint64_t>(float_to_key(s)) << 32) | static_cast<uint64_t>(0xffffffffu - idx);
}
__device__ __forceinline__ float composite_score(uint64_t ck) { return key_to_float(static_cast<uint32_t>(ck >> 32)); }
__device__ __forceinline__ uint32_t composite_index(uint64_t ck) {
  return 0xffffffffu - static_cast<uint32_t>(ck & 0xffffffffu);
}

struct SelectSmem {
  int hist[kBins];
  int res[4];  // bin, count above bin, count in bin, total
  unsigned int wcount;
};

// warp 0: locate the bin that contains the `need`-th largest entry
__device__ __forceinline__ void find_bin(SelectSmem& sm, int nbins, int need) {
  const int lane = threadIdx.x;
  const int per = nbins / 32;
  int s = 0;
  for (int j = 0; j < per; ++j) s += sm.hist[lane * per + j];
  int suffix = s;  // inclusive sum over lanes >= this one
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_down_sync(0xffffffffu, suffix, o);
    if (lane + o < 32) suffix += y;
  }
  const int total = __shfl_sync(0xffffffffu, suffix, 0);
  const int above = suffix - s;
  if (lane == 0) {
    sm.res[3] = total;
    if (total < need) sm.res[0] = -1;
  }
  if (above < need && suffix >= need) {
    int acc = above;
    for (int j = per - 1; j >= 0; --j) {
      const int h = sm.hist[lane * per + j];
      if (acc + h >= need) {
        sm.res[0] = lane * per + j;
        sm.res[1] = acc;
        sm.res[2] = h;
        break;
      }
      acc += h;
    }
  }
}

template <int THREADS>
__device__ __forceinline__ void bitonic_sort_desc(uint64_t* a, int n) {
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n; i += THREADS) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const uint64_t x = a[i], y = a[ixj];
          const bool desc = (i & k) == 0;
          if (desc ? (x < y) : (x > y)) {
            a[i] = y;
            a[ixj] = x;
          }
        }
      }
      __syncthreads();
    }
  }
}

// enumerate(f) must call f(composite) for every live candidate, spread over the
// THREADS threads of the CTA, and produce the same set on every call.
// On return win[0 .. kp2) is sorted descending; the return value is the number
// of live winners (min(K, live candidates)); unused entries are 0.
template <int THREADS, class Enumerate>
__device__ __forceinline__ int radix_select_topk(Enumerate&& enumerate, int K, uint64_t* win, int kp2,
                                                 SelectSmem& sm) {
  uint64_t prefix = 0, pmask = 0;
  int need = K;
  int nvalid = K;
  const int shifts[6] = {53, 42, 32, 21, 10, 0};
  const int widths[6] = {11, 11, 10, 11, 11, 10};
  for (int pass = 0; pass < 6; ++pass) {
    const int nb = 1 << widths[pass];
    for (int i = threadIdx.x; i < kBins; i += THREADS) sm.hist[i] = 0;
    __syncthreads();
    const int sh = shifts[pass];
    enumerate([&](uint64_t ck) {
      if ((ck & pmask) == prefix) atomicAdd(&sm.hist[(ck >> sh) & (nb - 1)], 1);
    });
    __syncthreads();
    if (threadIdx.x < 32) find_bin(sm, nb, need);
    __syncthreads();
    const int bin = sm.res[0];
    if (bin < 0) {  // fewer live candidates than K: take them all
      nvalid = sm.res[3];
      prefix = 0;
      break;
    }
    need -= sm.res[1];
    prefix |= static_cast<uint64_t>(bin) << sh;
    pmask |= static_cast<uint64_t>(nb - 1) << sh;
    if (sm.res[2] == need) break;  // the boundary bin is taken whole
    __syncthreads();
  }
  __syncthreads();
  if (threadIdx.x == 0) sm.wcount = 0;
  for (int i = threadIdx.x; i < kp2; i += THREADS) win[i] = 0;
  __syncthreads();
  enumerate([&](uint64_t ck) {
    if (ck >= prefix) {
      const unsigned int pos = atomicAdd(&sm.wcount, 1u);
      if (pos < static_cast<unsigned int>(kp2)) win[pos] = ck;
    }
  });
  __syncthreads();
  bitonic_sort_desc<THREADS>(win, kp2);
  return nvalid;
}

}  // namespace topk
}  // namespace fr
