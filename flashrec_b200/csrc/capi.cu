// Library-wide pieces of the C ABI: version string and the sticky device-side
// status word that kernels with bounded waits report into.
#include "fr_common.cuh"

namespace fr {

// {code, site}: written once by the first kernel whose bounded wait gives up.
__device__ int g_device_status[2];

// Device address of the status word for the current device (cached per device).
int* device_status_ptr() {
  constexpr int kMaxDev = 64;
  static int* cache[kMaxDev] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  if (cache[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    cache[dev] = static_cast<int*>(p);
  }
  return cache[dev];
}


// ---------------------------------------------------------------------------
// silu over all bf16 inputs, evaluated in fp64 and rounded fp64 -> fp32 -> bf16 (128 KB, stays in
// L2). The SwiGLU kernels consult it for the few inputs whose fast fp32 evaluation lands too
// close to a bf16 rounding midpoint.
// ---------------------------------------------------------------------------
__device__ uint16_t g_silu_table[65536];

__global__ void silu_table_kernel(uint16_t* __restrict__ table) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  const float g = __uint_as_float(i << 16);
  const __nv_bfloat16 r = __float2bfloat16_rn(silu_exact(g));
  table[i] = *reinterpret_cast<const uint16_t*>(&r);
}

// First use on a device fills the table on `stream` and waits for it, so that later calls on
// any stream may read it. While `stream` is being captured no wait is possible: the fill is
// recorded into the graph instead (it runs, idempotently, on every replay) and the device stays
// marked as not yet filled.
const uint16_t* silu_table_ptr(cudaStream_t stream) {
  constexpr int kMaxDev = 64;
  static uint16_t* cache[kMaxDev] = {nullptr};
  static bool filled[kMaxDev] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  if (cache[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_silu_table) != cudaSuccess) return nullptr;
    cache[dev] = static_cast<uint16_t*>(p);
  }
  if (!filled[dev]) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) return nullptr;
    silu_table_kernel<<<65536 / 256, 256, 0, stream>>>(cache[dev]);
    if (cudaGetLastError() != cudaSuccess) return nullptr;
    if (cap == cudaStreamCaptureStatusNone) {
      if (cudaStreamSynchronize(stream) != cudaSuccess) return nullptr;
      filled[dev] = true;
    }
  }
  return cache[dev];
}

}  // namespace fr

extern "C" const char* fr_version(void) { return "flashrec_b200 0.1 (sm_100a)"; }

extern "C" int fr_device_status(int* status_out, int* site_out) {
  int* p = fr::device_status_ptr();
  if (!p) return FR_ERR_CUDA;
  int host[2] = {0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess) return FR_ERR_CUDA;
  if (cudaMemcpy(host, p, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) return FR_ERR_CUDA;
  if (host[0] != 0) {
    const int zero[2] = {0, 0};
    if (cudaMemcpy(p, zero, sizeof(zero), cudaMemcpyHostToDevice) != cudaSuccess) return FR_ERR_CUDA;
  }
  if (status_out) *status_out = host[0];
  if (site_out) *site_out = host[1];
  return FR_OK;
}
