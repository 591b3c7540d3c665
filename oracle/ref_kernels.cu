// ref_kernels.cu — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// A harness around the RecFlex reference's own device templates.  It #includes
// the reference headers from the reference checkout (they are not copied into
// this repository) and wraps each template in a one-feature __global__ kernel,
// so that the GPU parity tests can compare this library's output with what the
// reference's kernels compute on the same inputs:
//   ws::SparseSegmentReduce     examples/csrc/include/warp_per_sample_kernel.cuh:70-82
//   obms::SparseSegmentReduce   examples/csrc/include/one_block_multi_sample_kernel.cuh:110-126
//   onehot::GatherSegments      examples/csrc/include/onehot_kernel.cuh:70-87
// Each wrapper pools ONE feature into a dense [num_segments, EMBED_DIM] fp32
// matrix (EMBED_DIM_SUM == EMBED_DIM, embed_dim_offset == 0); the test places
// the features side by side.  Block-to-task mapping follows the reference's host
// preprocess: ws: one block per 256/X bags (warp_per_sample_preprocess.cu:36-37),
// obms: one block per 256/(X*Y) bags (one_block_multi_sample_preprocess.cu:36-37),
// onehot: min(tiles, blocks) blocks striding over tiles of 256 (onehot_preprocess.cu:17-27).
// Built only where the reference checkout exists (oracle/build_ref.sh); the
// resulting oracle/_ref/libref_kernels.so travels to the GPU box.
#include <cuda_runtime.h>

#include "warp_per_sample_kernel.cuh"
#include "one_block_multi_sample_kernel.cuh"
#include "onehot_kernel.cuh"

namespace {

constexpr int kThreads = 256;

template <int DIM, int VEC, int ITEMS, int X>
__global__ void __launch_bounds__(kThreads) ws_kernel(const float* table, const int* indices, const int* offsets,
                                                      float* out, int num_inputs, int num_segments) {
  ws::SparseSegmentReduce<DIM, DIM, VEC, ITEMS, X, kThreads / X>(
      table, [&](int i) { return indices[i]; }, [&](int i) { return offsets[i]; }, out, num_inputs, num_segments,
      blockIdx.x, 0);
}

template <int DIM, int VEC, int ITEMS, int X, int Y>
__global__ void __launch_bounds__(kThreads) obms_kernel(const float* table, const int* indices, const int* offsets,
                                                        float* out, int num_inputs, int num_segments) {
  constexpr int Z = kThreads / (X * Y);
  __shared__ obms::SparseSegmentReduceTempStorage<VEC, X, Y, Z, float> s;
  obms::SparseSegmentReduce<DIM, DIM, VEC, ITEMS, X, Y, Z>(
      s, table, [&](int i) { return indices[i]; }, [&](int i) { return offsets[i]; }, out, num_inputs, num_segments,
      blockIdx.x, 0);
}

template <int DIM>
__global__ void __launch_bounds__(kThreads) onehot_kernel(const float* table, const int* indices, float* out,
                                                          int num_inputs, int num_tiles) {
  __shared__ onehot::GatherSegmentsTempStorage<kThreads> s;
  onehot::GatherSegments<DIM, DIM, DIM, kThreads>(s, table, [&](int i) { return indices[i]; }, out, num_inputs,
                                                  blockIdx.x, gridDim.x, num_tiles, 0);
}

template <int DIM>
int run_ws(const float* t, const int* idx, const int* off, float* out, int nnz, int nseg, cudaStream_t st) {
  constexpr int VEC = 4;
  constexpr int X = (DIM / VEC) < 32 ? (DIM / VEC) : 32;
  constexpr int Y = kThreads / X;
  const int blocks = (nseg + Y - 1) / Y;
  ws_kernel<DIM, VEC, 4, X><<<blocks, kThreads, 0, st>>>(t, idx, off, out, nnz, nseg);
  return (int)cudaGetLastError();
}

template <int DIM>
int run_obms(const float* t, const int* idx, const int* off, float* out, int nnz, int nseg, cudaStream_t st) {
  constexpr int VEC = 4;
  constexpr int X = (DIM / VEC) < 16 ? (DIM / VEC) : 16;
  constexpr int Y = 4;
  constexpr int Z = kThreads / (X * Y);
  const int blocks = (nseg + Z - 1) / Z;
  obms_kernel<DIM, VEC, 2, X, Y><<<blocks, kThreads, 0, st>>>(t, idx, off, out, nnz, nseg);
  return (int)cudaGetLastError();
}

template <int DIM>
int run_onehot(const float* t, const int* idx, float* out, int n, cudaStream_t st) {
  const int tiles = (n + kThreads - 1) / kThreads;
  const int blocks = tiles < 64 ? tiles : 64;
  onehot_kernel<DIM><<<blocks, kThreads, 0, st>>>(t, idx, out, n, tiles);
  return (int)cudaGetLastError();
}

}  // namespace

#define REF_DIM_SWITCH(CALL)        \
  switch (dim) {                    \
    case 4: return CALL(4);         \
    case 8: return CALL(8);         \
    case 16: return CALL(16);       \
    case 32: return CALL(32);       \
    case 64: return CALL(64);       \
    case 128: return CALL(128);     \
    default: return -1000;          \
  }

extern "C" {

// kind: 0 = ws (warp per sample), 1 = obms (one block multi sample).  All pointers are device pointers.
// Returns 0, a CUDA error code, or -1000 for a dim the harness does not instantiate.
int ref_pool_feature(int kind, int dim, const float* table, const int* indices, const int* offsets, float* out,
                     int num_inputs, int num_segments, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (num_segments == 0) return 0;
  if (kind == 0) {
#define CALL(D) run_ws<D>(table, indices, offsets, out, num_inputs, num_segments, st)
    REF_DIM_SWITCH(CALL)
#undef CALL
  } else {
#define CALL(D) run_obms<D>(table, indices, offsets, out, num_inputs, num_segments, st)
    REF_DIM_SWITCH(CALL)
#undef CALL
  }
}

// The reference's one-hot gather: indices[num_inputs], one row copied per sample.
int ref_onehot_feature(int dim, const float* table, const int* indices, float* out, int num_inputs, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (num_inputs == 0) return 0;
#define CALL(D) run_onehot<D>(table, indices, out, num_inputs, st)
  REF_DIM_SWITCH(CALL)
#undef CALL
}

}  // extern "C"
