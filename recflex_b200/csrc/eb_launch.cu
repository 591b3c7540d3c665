// Launchers: pick the fused-kernel instantiation for an occupancy, launch the
// binding kernel and the table-fill kernel.
#include <mutex>
#include <set>
#include <utility>

#include "eb_bind.cuh"
#include "eb_launch.h"

namespace ebk {

static FusedKernel pick(int occ, bool timing, int kind, int unroll) {
  switch (occ) {
    case 1: return fused_kernel_occ1(timing, kind, unroll);
    case 2: return fused_kernel_occ2(timing, kind, unroll);
    case 3: return fused_kernel_occ3(timing, kind, unroll);
    case 4: return fused_kernel_occ4(timing, kind, unroll);
    case 5: return fused_kernel_occ5(timing, kind, unroll);
    case 6: return fused_kernel_occ6(timing, kind, unroll);
    case 7: return fused_kernel_occ7(timing, kind, unroll);
    default: return fused_kernel_occ8(timing, kind, unroll);
  }
}

cudaError_t launch_bind(const LaunchArgs& a, bool zero_feature_times, cudaStream_t st) {
  eb_bind_kernel<<<1, kBindThreads, 0, st>>>(a, zero_feature_times ? 1 : 0);
  return cudaGetLastError();
}

cudaError_t launch_release(const LaunchArgs& a, cudaStream_t st) {
  ChunkSync* cs = reinterpret_cast<ChunkSync*>(a.ws + ws_layout(a.num_features).chunk_sync);
  eb_release_kernel<<<1, kMaxChunks, 0, st>>>(cs->flag, kMaxChunks, a.epoch);
  return cudaGetLastError();
}

// Dynamic shared memory above 48 KB (static shared memory counts too) must be opted into once per kernel function
// and device.
static cudaError_t allow_smem(FusedKernel k, size_t smem_bytes) {
  static std::mutex mu;
  static std::set<std::pair<int, const void*>> done;
  if (smem_bytes <= 32 * 1024) return cudaSuccess;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const std::pair<int, const void*> key(dev, reinterpret_cast<const void*>(k));
  std::lock_guard<std::mutex> lock(mu);
  if (done.count(key)) return cudaSuccess;
  e = cudaFuncSetAttribute(reinterpret_cast<const void*>(k), cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kPipeMaxCells * kPipeCellBytes * kWarpsPerCta);
  if (e == cudaSuccess) done.insert(key);
  return e;
}

// Grid of the grid-stride helper kernels: a few CTAs per SM of the current device.
static int helper_grid(int64_t wanted, int ctas_per_sm) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 148;
  const int64_t cap = (int64_t)sms * ctas_per_sm;
  return (int)(wanted < 1 ? 1 : (wanted > cap ? cap : wanted));
}

cudaError_t launch_push(const void* send, void* const* peer, long long send_ld_b, long long out_ld_b, long long dest_rows,
                        long long piece_rows, long long piece, int width16, int world, int rank, int first_hop,
                        int sm_count, cudaStream_t st) {
  PushArgs p;
  p.send = static_cast<const char*>(send);
  for (int r = 0; r < kMaxPeers; ++r) p.peer[r] = r < world ? static_cast<char*>(peer[r]) : nullptr;
  p.send_ld_b = send_ld_b;
  p.out_ld_b = out_ld_b;
  p.dest_rows = dest_rows;
  p.piece_rows = piece_rows;
  p.piece = piece;
  p.width16 = width16;
  p.world = world;
  p.rank = rank;
  p.first_hop = first_hop;
  eb_push_kernel<<<sm_count, 128, 0, st>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_fused(const LaunchArgs& a, int occupancy, bool timing, int grid, size_t smem_bytes, cudaStream_t st,
                         int kind, int unroll) {
  if (a.idx64 || timing) kind = unroll = 0;  // the specialised instantiations read 32-bit indices and keep no clocks
  FusedKernel k = pick(occupancy, timing, kind, unroll);
  cudaError_t e = allow_smem(k, smem_bytes);
  if (e != cudaSuccess) return e;
  void* params[] = {const_cast<LaunchArgs*>(&a)};
  return cudaLaunchKernel(reinterpret_cast<const void*>(k), dim3(grid), dim3(kCtaThreads), params, smem_bytes, st);
}

cudaError_t fused_ctas_per_sm(int occupancy, size_t smem_bytes, int* per_sm, int kind, int unroll) {
  FusedKernel k = pick(occupancy, false, kind, unroll);
  cudaError_t e = allow_smem(k, smem_bytes);
  if (e != cudaSuccess) return e;
  return cudaOccupancyMaxActiveBlocksPerMultiprocessor(per_sm, reinterpret_cast<const void*>(k), kCtaThreads,
                                                       smem_bytes);
}

cudaError_t launch_fill(void* table, int64_t elems, int dtype, uint64_t seed, float std, cudaStream_t st) {
  // 65536 * sqrt(4 / 12): standard deviation of the centred sum of four 16-bit fields
  const float scale = std / 37837.227f;
  const int blocks = helper_grid((elems + 255) / 256, 16);
  if (dtype == 1)
    eb_fill_kernel<__half><<<blocks, 256, 0, st>>>(static_cast<__half*>(table), elems, seed, scale);
  else
    eb_fill_kernel<float><<<blocks, 256, 0, st>>>(static_cast<float*>(table), elems, seed, scale);
  return cudaGetLastError();
}

cudaError_t launch_place(const float* src, float* dst, int64_t rows, int64_t dst_ld, int num_segments,
                         const void* segments, int vec_ok, cudaStream_t st) {
  if (rows == 0 || num_segments == 0) return cudaSuccess;
  const int bx = helper_grid((rows * 8 + 255) / 256, 4);  // a few float4 per thread for the narrowest features
  for (int first = 0; first < num_segments; first += 65535) {
    const int n = num_segments - first < 65535 ? num_segments - first : 65535;
    eb_place_kernel<<<dim3((unsigned)bx, (unsigned)n), 256, 0, st>>>(
        src, dst, rows, dst_ld, static_cast<const PlaceSeg*>(segments) + first, vec_ok);
  }
  return cudaGetLastError();
}

cudaError_t launch_lengths(const void* lengths, void* offsets, int num_features, int64_t batch, int idx64,
                           cudaStream_t st) {
  if (num_features == 0) return cudaSuccess;
  if (idx64)
    eb_lengths_kernel<long long><<<num_features, kBindThreads, 0, st>>>(static_cast<const long long*>(lengths),
                                                                        static_cast<long long*>(offsets), batch);
  else
    eb_lengths_kernel<int><<<num_features, kBindThreads, 0, st>>>(static_cast<const int*>(lengths),
                                                                  static_cast<int*>(offsets), batch);
  return cudaGetLastError();
}

}  // namespace ebk
