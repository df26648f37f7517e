// Per-device runtime state of the kernel library: the status word that kernels use to report a
// bounded wait that ran out (instead of hanging or trapping), and device properties.
#include "common.cuh"
#include "kernels.h"

namespace {
constexpr int kMaxDevices = 16;
int* g_status[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
}  // namespace

int* ogb_status_ptr(int device) { return device >= 0 && device < kMaxDevices ? g_status[device] : nullptr; }

OGB_API int ogb_runtime_init(int device) {
  if (device < 0 || device >= kMaxDevices) return -1;
  if (g_status[device]) return 0;
  int prev = 0;
  if (cudaGetDevice(&prev) != cudaSuccess) return -4;
  if (cudaSetDevice(device) != cudaSuccess) return -4;
  int* p = nullptr;
  int rc = 0;
  if (cudaMalloc(&p, sizeof(int)) != cudaSuccess || cudaMemset(p, 0, sizeof(int)) != cudaSuccess) rc = -2;
  cudaDeviceProp prop;
  if (rc == 0 && cudaGetDeviceProperties(&prop, device) == cudaSuccess) g_sm_count[device] = prop.multiProcessorCount;
  if (rc == 0) g_status[device] = p;
  cudaSetDevice(prev);
  return rc;
}

OGB_API int* ogb_status_device_ptr(int device) { return ogb_status_ptr(device); }

OGB_API int ogb_status_read_and_clear(int device) {
  int* p = ogb_status_ptr(device);
  if (!p) return -1;
  int prev = 0, v = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device);
  cudaError_t e = cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && v != 0) cudaMemset(p, 0, sizeof(int));
  cudaSetDevice(prev);
  return e == cudaSuccess ? v : -4;
}

// Name of the CUDA runtime's last error in this thread (launchers return -4 without the reason; the Python layer appends this).
// Reading does not clear it.
OGB_API const char* ogb_last_cuda_error() { return cudaGetErrorString(cudaPeekAtLastError()); }

OGB_API int ogb_sm_count(int device) { return device >= 0 && device < kMaxDevices ? g_sm_count[device] : 0; }
