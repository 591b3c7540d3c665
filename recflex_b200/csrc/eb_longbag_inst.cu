// Instantiates eb_longbag_kernel (the bags handed over by the fused kernel, pooled by many warps) and its launcher.
#include "eb_launch.h"
#include "eb_longbag.cuh"

namespace ebk {

cudaError_t launch_longbag(const LaunchArgs& a, bool timing, int sm_count, cudaStream_t st) {
  if (a.long_bytes <= 0) return cudaSuccess;
  const unsigned grid = (unsigned)(sm_count * kLongBagCtasPerSm);
  if (timing) eb_longbag_kernel<true><<<grid, kCtaThreads, 0, st>>>(a);
  else eb_longbag_kernel<false><<<grid, kCtaThreads, 0, st>>>(a);
  return cudaGetLastError();
}

}  // namespace ebk
