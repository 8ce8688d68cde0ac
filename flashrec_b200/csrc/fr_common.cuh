// Shared helpers for the sm_100a kernels of the quantized SID decode step.
//
// Conventions used by every kernel in this directory:
//   * entry points are extern "C", take raw device pointers + sizes + a
//     cudaStream_t, allocate nothing, and return an int status (0 = ok);
//   * floating-point steps whose result is later compared bit-for-bit with
//     the CPU oracle use the explicit round-to-nearest intrinsics
//     (__fmul_rn, __fadd_rn, __fdiv_rn, __fsqrt_rn) so that nvcc can neither
//     contract them into FMAs nor replace them by approximations;
//   * sums of squares are accumulated in fp64 and rounded once to fp32, which
//     makes the result independent of the reduction order.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flashrec_b200.h"

namespace fr {

constexpr float kFp8Max = 448.0f;
constexpr float kAmaxFloor = 1e-12f;  // clamp(min=1e-12) of the per-row amax

#define FR_CHECK_ARG(cond)                \
  do {                                    \
    if (!(cond)) return FR_ERR_BAD_ARG;   \
  } while (0)

#define FR_CHECK_SUPPORTED(cond)            \
  do {                                      \
    if (!(cond)) return FR_ERR_UNSUPPORTED; \
  } while (0)

static inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FR_OK : FR_ERR_CUDA;
}

// Device table silu(bf16) -> bf16 over all 65536 inputs for the current device, built on first use
// (capi.cu). nullptr on a CUDA error.
const uint16_t* silu_table_ptr(cudaStream_t stream);

// Host-side state that belongs to a device, not to the process: a kernel's opt-in dynamic
// shared-memory limit (cudaFuncSetAttribute applies to the device that is current when it is
// called) and the SM count. One process may drive several GPUs through this library, so both are
// kept per device ordinal. Filled without a lock: concurrent first calls store the same values.
constexpr int kMaxDevices = 64;
static inline int current_device() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) return -1;
  return d;
}
struct PerDeviceFlag {
  bool done[kMaxDevices] = {};
};
// Raise `kern`'s dynamic shared-memory limit to `bytes` on the current device, once per device.
template <class Kernel>
static inline int ensure_dyn_smem(PerDeviceFlag& flag, Kernel kern, int bytes) {
  const int d = current_device();
  if (d < 0) return FR_ERR_CUDA;
  if (!flag.done[d]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return FR_ERR_CUDA;
    flag.done[d] = true;
  }
  return FR_OK;
}
// SM count of the current device (148 when it cannot be read).
static inline int device_sm_count() {
  static int cache[kMaxDevices] = {};
  const int d = current_device();
  if (d < 0) return 148;
  if (cache[d] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || v <= 0) v = 148;
    cache[d] = v;
  }
  return cache[d];
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static inline int ceil_div(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------------------
// Sum of squares of bf16 values, exact, without fp64 arithmetic on the common path: for code whose
// warps all square at the same time (the qkv GEMM's epilogue: sixteen warps per SM reach the phase
// together and queue on the fp64 pipe, about 26 cycles per warp instruction). The row kernels keep
// their fp64 FMAs: there the fp64 pipe works beside other warps' fp32 instructions, and the eight
// fp32 instructions per element below were measured slower (RMSNorm -> e4m3 29.1 against 24.6 us).
// The square of a bf16 value is exact in fp32 (8-bit significand); the running sum
// is kept as an unevaluated pair s + e: Knuth's TwoSum makes s + p == t + err exactly, the errs
// are added up in e with plain fp32 adds. For chains of at most 16 squares merged pairwise
// (sq_merge, also across lanes) the pair differs from the exact sum by less than 2^-39 of it,
// for up to 128 squares per thread and 32 threads per row. Callers turn the row total into
// fp64, scale it by a power of two and round to fp32; sq_rounding_is_safe tells whether that
// rounding is certain to equal the rounding of the exact sum (the bits dropped by the rounding
// are further than the error bound from a rounding boundary). When it is not (about one row in
// 8000), the caller recomputes the row in fp64 as before, so results never change.
// ---------------------------------------------------------------------------
struct SqSum {
  float s, e;
};

__device__ __forceinline__ void sq_two_sum(float a, float b, float& t, float& err) {
  t = __fadd_rn(a, b);
  const float bb = __fsub_rn(t, a);
  err = __fadd_rn(__fsub_rn(a, __fsub_rn(t, bb)), __fsub_rn(b, bb));
}

__device__ __forceinline__ void sq_add(SqSum& a, float x) {
  float t, err;
  sq_two_sum(a.s, __fmul_rn(x, x), t, err);
  a.s = t;
  a.e = __fadd_rn(a.e, err);
}

__device__ __forceinline__ void sq_merge(SqSum& a, const SqSum& b) {
  float t, err;
  sq_two_sum(a.s, b.s, t, err);
  a.s = t;
  a.e = __fadd_rn(__fadd_rn(a.e, b.e), err);
}

__device__ __forceinline__ double sq_value(const SqSum& a) { return static_cast<double>(a.s) + static_cast<double>(a.e); }

// v = (row total from SqSum pairs) scaled by a power of two; true when static_cast<float>(v) is the
// fp32 rounding of the exactly summed value as well. fp32 keeps 23 of the 52 fraction bits; the
// error bound 2^-39 |v| is below 2^14 units of the last fp64 place, the window leaves a factor two.
__device__ __forceinline__ bool sq_rounding_is_safe(double v) {
  if (v == 0.0) return true;  // every square was zero
  const int lo = __double2loint(v) & 0x1fffffff;
  const int ex = (__double2hiint(v) >> 20) & 0x7ff;
  const int dist = lo > (1 << 28) ? lo - (1 << 28) : (1 << 28) - lo;
  return dist > (1 << 15) && ex > 1023 - 60 && ex < 1023 + 100;  // squares and the fp32 result stay normal
}

// bf16 <-> fp32 on raw bit patterns (a bf16 is the upper half of an fp32).
__device__ __forceinline__ float bf16lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

// Round-to-nearest-even fp32 -> bf16, result returned as fp32 (lower 16 bits 0).
__device__ __forceinline__ float round_bf16(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// a + b on two packed bf16 pairs, each sum rounded once to bf16. Equal to the fp32 sum rounded to
// bf16: the fp32 sum of two bf16 values is exact unless their exponents differ by more than 16,
// and then either rounding returns the larger operand.
__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// max(acc, |x|) on two packed bf16 lanes (acc >= 0 in both lanes). A NaN lane of x is ignored, as fmaxf does.
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t acc, uint32_t x) {
  uint32_t d;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(acc), "r"(x & 0x7fff7fffu));
  return d;
}

// Two fp32 -> two e4m3 bytes (round to nearest even, saturating). `lo` lands in
// the low byte.
__device__ __forceinline__ uint16_t pack_e4m3x2(float lo, float hi) {
  return static_cast<uint16_t>(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  return static_cast<uint32_t>(pack_e4m3x2(a, b)) | (static_cast<uint32_t>(pack_e4m3x2(c, d)) << 16);
}

// clamp(y / scale, -448, 448): IEEE division, as torch does on fp32 tensors.
__device__ __forceinline__ float quant_div(float y, float scale) {
  float q = __fdiv_rn(y, scale);
  return fminf(fmaxf(q, -kFp8Max), kFp8Max);
}

// The correctly rounded fp32 quotient y / scale without a division and without a branch:
// q0 = y * inv (inv = the correctly rounded 1 / scale), the exact remainder r = y - q0 * scale
// from one FMA, and q0 + r * inv rounded once (Markstein's correction step) equals the IEEE
// quotient. `scale_or_zero` is the scale, or 0 when the scale is not finite (a row that holds an
// infinity): inv is 0 there and the sequence then returns 0 for finite y and NaN for infinite y,
// as the division would. |q| <= 448 (1 + 2^-22) for |y| <= amax: the saturating e4m3 conversion
// does the clamp. The sign is taken from y at the end (the scale is positive): the correction
// step alone would turn the quotient of y = -0 into +0, which is a different e4m3 byte.
__device__ __forceinline__ float finite_or_zero(float s) { return s <= 3.402823466e38f ? s : 0.f; }
__device__ __forceinline__ float quant_div_fast(float y, float scale_or_zero, float inv) {
  const float q0 = __fmul_rn(y, inv);
  const float r = __fmaf_rn(-q0, scale_or_zero, y);
  const float q1 = __fmaf_rn(r, inv, q0);
  return __uint_as_float((__float_as_uint(q1) & 0x7fffffffu) | (__float_as_uint(y) & 0x80000000u));
}

// scale = max(amax, 1e-12) / 448 in fp32.
__device__ __forceinline__ float row_scale(float amax) {
  return __fdiv_rn(fmaxf(amax, kAmaxFloor), kFp8Max);
}

// 1 / sqrt(x) as two correctly rounded fp32 operations (what a vectorised CPU
// rsqrt computes); the hardware rsqrt approximation is deliberately avoided.
__device__ __forceinline__ float rsqrt_rn(float x) { return __fdiv_rn(1.0f, __fsqrt_rn(x)); }

// silu(g) = g / (1 + exp(-g)) correctly rounded to fp32, then to bf16, for a bf16-valued g.
// Fast path: exp(-g) = 2^(th + tl) with th + tl = -g * log2(e) carried in two floats (the
// product's rounding error is recovered with an FMA), ex2.approx on th and a first-order
// correction for tl, then an approximate divide: within ~6 fp32 ulp of the exact value.
// Results that land within 24 ulp of a bf16 rounding midpoint, and tiny / non-finite ones,
// cannot be trusted to round the right way; for those the answer is read from a table of the
// exactly evaluated function over all 65536 bf16 inputs (silu_table_ptr), so the bf16 value
// always equals the one obtained from an exact evaluation and no thread ever runs fp64 code.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Fast path only: returns the approximate silu(g) and sets `hard` when its bf16 rounding cannot
// be trusted. Branch-free.
__device__ __forceinline__ float silu_fast(float g, bool& hard) {
  constexpr float kL2eHi = 1.44269502162933349609375f;  // fp32(log2 e)
  constexpr float kL2eLo = 1.925963033500e-8f;          // log2 e - fp32(log2 e)
  const float th = __fmul_rn(g, -kL2eHi);
  const float tl = __fmaf_rn(g, -kL2eLo, __fmaf_rn(g, -kL2eHi, -th));
  float e = ex2_approx(th);
  e = __fmaf_rn(e, tl * 0.693147182f, e);
  const float s = __fdividef(g, 1.0f + e);
  const uint32_t low = __float_as_uint(s) & 0xffffu;
  // (huge |g|: exp underflows to 0 and s == g exactly, or the quotient collapses to 0 / NaN and
  //  is caught by the magnitude test; silu(+-0) = +-0 is exact)
  hard = (low - (0x8000u - 24u) <= 48u) || (!(fabsf(s) >= 1e-30f) && g != 0.f);
  return s;
}

// fp64 evaluation rounded once to fp32: only the kernel that fills the table runs this.
__device__ __forceinline__ float silu_exact(float g) {
  const double gd = static_cast<double>(g);
  return static_cast<float>(gd / (1.0 + exp(-gd)));
}

// g must be exactly representable in bf16 (its upper 16 bits index the table).
__device__ __forceinline__ float silu_bf16(float g, const uint16_t* __restrict__ table) {
  bool hard;
  const float s = silu_fast(g, hard);
  float r = round_bf16(s);
  if (hard) r = __uint_as_float(static_cast<uint32_t>(__ldg(table + (__float_as_uint(g) >> 16))) << 16);
  return r;
}

__device__ __forceinline__ uint32_t silu_mul_pack(uint32_t g, uint32_t u, const uint16_t* __restrict__ table) {
  float a = __fmul_rn(silu_bf16(bf16lo(g), table), bf16lo(u));
  float b = __fmul_rn(silu_bf16(bf16hi(g), table), bf16hi(u));
  return pack_bf16(a, b);
}

// e4m3 byte -> fp32 (exact).
__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// Order-preserving map fp32 -> uint32 (larger float <=> larger key; -0 < +0).
__device__ __forceinline__ uint32_t float_to_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

}  // namespace fr
