// Per-thread device binding.  The library links its own copy of the CUDA runtime, whose
// notion of "current device" is per host thread and starts at device 0; PyTorch's autograd
// worker threads also start without a current driver context.  Every Python-side op call
// therefore binds the calling thread to the tensor's device first (cached per thread).
#include "common.cuh"

MLB_API int mlb_set_device(int dev) {
  int cur = -1;
  cudaError_t e = cudaGetDevice(&cur);
  if (e == cudaSuccess && cur == dev) {
    // make sure the primary context is also current at the driver level for this thread
    e = cudaFree(nullptr);
    return (int)e;
  }
  e = cudaSetDevice(dev);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaFree(nullptr);
}

MLB_API int mlb_device_sm_count(int dev) {
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  return n;
}
