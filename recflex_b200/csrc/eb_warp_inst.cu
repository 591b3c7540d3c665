// Instantiates eb_warp_kernel (the warp-per-bag schedule's own kernel) and its launcher.
#include "eb_launch.h"
#include "eb_warp.cuh"

namespace ebk {

cudaError_t launch_warp(const LaunchArgs& a, bool timing, int warp_features, cudaStream_t st) {
  // every feature on the warp-per-bag schedule owns ceil(batch / 8) CTAs, whatever the batch holds
  const long long ctas = (long long)warp_features * ((a.batch + kWarpsPerCta - 1) / kWarpsPerCta);
  if (ctas <= 0) return cudaSuccess;
  if (ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
  const unsigned grid = (unsigned)ctas;
  if (timing) eb_warp_kernel<true><<<grid, kCtaThreads, 0, st>>>(a);
  else eb_warp_kernel<false><<<grid, kCtaThreads, 0, st>>>(a);
  return cudaGetLastError();
}

}  // namespace ebk
