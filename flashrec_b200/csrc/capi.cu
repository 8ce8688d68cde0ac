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
