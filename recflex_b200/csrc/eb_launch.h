// Host-callable launchers of the kernels in eb_fused.cuh.  The fused kernel is
// compiled once per CTAs-per-SM occupancy (its __launch_bounds__ caps the
// registers accordingly), each in its own translation unit so that the
// instantiations build in parallel.
#pragma once
#include "eb_common.cuh"

namespace ebk {

typedef void (*FusedKernel)(LaunchArgs);

// One definition per occupancy, in eb_fused_inst.cu compiled with -DEB_OCC=<n>.  kind / unroll ask for the
// instantiation that holds only that schedule (see eb_fused_kernel); 0 / 0, or a combination that was not
// instantiated, gives the kernel with every schedule.
FusedKernel fused_kernel_occ1(bool timing, int kind, int unroll);
FusedKernel fused_kernel_occ2(bool timing, int kind, int unroll);
FusedKernel fused_kernel_occ3(bool timing, int kind, int unroll);
FusedKernel fused_kernel_occ4(bool timing, int kind, int unroll);
FusedKernel fused_kernel_occ5(bool timing, int kind, int unroll);
FusedKernel fused_kernel_occ6(bool timing, int kind, int unroll);
FusedKernel fused_kernel_occ7(bool timing, int kind, int unroll);
FusedKernel fused_kernel_occ8(bool timing, int kind, int unroll);

cudaError_t launch_bind(const LaunchArgs& a, bool zero_feature_times, cudaStream_t st);
// Chunked ticket order: raises every chunk flag to the call's epoch once the fused kernel is done.
cudaError_t launch_release(const LaunchArgs& a, cudaStream_t st);
cudaError_t launch_fused(const LaunchArgs& a, int occupancy, bool timing, int grid, size_t smem_bytes, cudaStream_t st,
                         int kind = 0, int unroll = 0);
// Chunked order: ships piece `piece` of the send buffer to every other rank with eb_push_kernel (SM copies).
cudaError_t launch_push(const void* send, void* const* peer, long long send_ld_b, long long out_ld_b, long long dest_rows,
                        long long piece_rows, long long piece, int width16, int world, int rank, int first_hop,
                        int sm_count, cudaStream_t st);
cudaError_t launch_longbag(const LaunchArgs& a, bool timing, int sm_count, cudaStream_t st);
// eb_warp_kernel: pools the `warp_features` features on the warp-per-bag schedule (one CTA per 8 bags).
cudaError_t launch_warp(const LaunchArgs& a, bool timing, int warp_features, cudaStream_t st);
cudaError_t fused_ctas_per_sm(int occupancy, size_t smem_bytes, int* per_sm, int kind = 0, int unroll = 0);
cudaError_t launch_place(const float* src, float* dst, int64_t rows, int64_t dst_ld, int num_segments,
                         const void* segments, int vec_ok, cudaStream_t st);

cudaError_t launch_lengths(const void* lengths, void* offsets, int num_features, int64_t batch, int idx64,
                           cudaStream_t st);

// Sets the calling thread's eb_last_error() message (defined beside it).
void set_last_error(const char* msg);

cudaError_t launch_fill(void* table, int64_t elems, int dtype, uint64_t seed, float std, cudaStream_t st);

}  // namespace ebk
