// Device binding for threads that reach the library without a current CUDA context.
//
// The library carries its own (static) CUDA runtime.  A thread that PyTorch created (its
// autograd workers, for instance) may have no driver context bound when it first calls in;
// the runtime would then fall back to device 0 and driver entry points such as the tensor-map
// encoder fail with CUDA_ERROR_INVALID_CONTEXT.  The Python wrappers call this once per
// (thread, device) before the first launch.
#include "common.cuh"
#include "api.h"

PF_API int pf_bind_device(int device) {
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return (int)e;
  e = cudaFree(0);  // forces the primary context to be created and made current
  return (int)e;
}

PF_API int pf_device_count() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
  return n;
}
