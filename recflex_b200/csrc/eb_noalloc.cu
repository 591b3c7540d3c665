// eb_forward_packed_noalloc: the packed fused forward for callers that must
// not allocate device memory.
//
// Who needs it: code that runs where cudaMalloc is off limits — inside a
// serving process whose memory pool hands out every byte up front and treats
// any later driver allocation as a fault, inside a plugin sandbox that forbids
// allocation calls, or on a latency path where an allocation (which may
// synchronise the device) is not acceptable.  Such callers cannot use
// eb_create(), which allocates a descriptor table, nor provide a workspace if
// they have no spare device memory of their own.
//
// How: the descriptor table and the per-call scratch (tile prefix sums, feature
// order, ticket counters, status word) live in ONE file-scope __device__ array
// that is part of the library image.  Every GPU that loads the library holds
// those kNoAllocScratchBytes until the process exits, whether or not this entry
// point is ever called.  The kernels are the same eb_bind_kernel /
// eb_fused_kernel the handle-based entry points launch; only the place of their
// scratch differs.
//
// Rules that follow from the single shared array:
//  - at most EB_NOALLOC_MAX_FEATURES features per call (larger requests are
//    refused with EB_ERR_TOO_LARGE);
//  - all calls on one GPU share the array, which keeps the previous call's
//    contents; everything that must start from zero (ticket counters, status
//    word) is re-initialised by the binding kernel of each call, and the
//    descriptor table is rewritten by each call.  Two calls whose kernels
//    overlap on the GPU (different streams) race on it: issue the calls for
//    one GPU on one stream, or order the streams yourself.  On the host, calls
//    for one GPU are serialised by a lock and each GPU has its own staging
//    buffer, so host threads driving different GPUs do not disturb each other;
//  - the first call on each device looks up the array's device address
//    (cudaGetSymbolAddress) and keeps it; make that first call outside any
//    stream capture;
//  - every call stages its descriptors through host memory that the next call
//    overwrites, so a call is refused while its stream is being captured.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/recflex_b200.h"
#include "eb_common.cuh"
#include "eb_launch.h"

using namespace ebk;

namespace {

constexpr int kMaxFeat = EB_NOALLOC_MAX_FEATURES;
constexpr int kMaxDevices = 16;
constexpr int kNoAllocOccupancy = 4;

// descriptor table first, then a workspace laid out by ws_layout(kMaxFeat)
constexpr size_t kDescBytes = sizeof(FeatStatic) * (size_t)kMaxFeat;
constexpr size_t kWsBytesMax = ws_layout(kMaxFeat).long_list;  // long-bag splitting stays off here
constexpr size_t kNoAllocScratchBytes = kDescBytes + ((kWsBytesMax + 255) / 256) * 256;

// The name below is a host-side stand-in for the device array: host code must
// never pass it to a kernel.  Its device address comes from
// cudaGetSymbolAddress, once per device (scratch_for()).
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

char* g_scratch_ptr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};

// host staging of the descriptor table, one per device (pageable: cudaMemcpyAsync has taken its copy when it
// returns), filled and uploaded under that device's lock
FeatStatic g_host_feats[kMaxDevices][kMaxFeat];
std::mutex g_device_lock[kMaxDevices];

// records the message where eb_last_error() finds it
int fail(int code, const char* fmt, ...) {
  char msg[256];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  set_last_error(msg);
  return code;
}

int pow2_ceil(int x) {
  int p = 1;
  while (p < x) p <<= 1;
  return p;
}

int ilog2(int x) {
  int l = 0;
  while ((1 << l) < x) ++l;
  return l;
}

// Device address of the scratch array on `device` (which must be current).
int scratch_for(int device, char** out) {
  if (!g_scratch_ptr[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return fail(EB_ERR_CUDA, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return fail(EB_ERR_CUDA, "cudaDeviceGetAttribute failed: %s", cudaGetErrorString(e));
    g_sm_count[device] = sms;
    g_scratch_ptr[device] = static_cast<char*>(p);
  }
  *out = g_scratch_ptr[device];
  return EB_OK;
}

}  // namespace

extern "C" {

int eb_forward_packed_noalloc(int device, int num_features, const int64_t* rows, const int32_t* dims,
                              const int32_t* table_dtype, const void* const* table_ptrs, int64_t batch,
                              const void* values, const void* offsets, int index_dtype, float* out, int64_t out_ld,
                              void* stream) {
  if (num_features <= 0) return fail(EB_ERR_INVALID_ARG, "num_features must be positive (got %d)", num_features);
  if (num_features > kMaxFeat)
    return fail(EB_ERR_TOO_LARGE, "%d features exceed the %d the built-in scratch array holds", num_features, kMaxFeat);
  if (!rows || !dims || !table_dtype || !table_ptrs) return fail(EB_ERR_INVALID_ARG, "null argument array");
  if (batch < 0) return fail(EB_ERR_INVALID_ARG, "negative batch");
  if (index_dtype != EB_I32 && index_dtype != EB_I64) return fail(EB_ERR_INVALID_ARG, "bad index_dtype %d", index_dtype);
  if (device < 0 || device >= kMaxDevices) return fail(EB_ERR_INVALID_ARG, "device %d out of range", device);
  if (ws_layout(num_features).long_list + kDescBytes > kNoAllocScratchBytes)
    return fail(EB_ERR_TOO_LARGE, "scratch array too small for %d features", num_features);
  if ((long double)batch * (long double)num_features >= 2147483648.0L)
    return fail(EB_ERR_TOO_LARGE, "batch * num_features must stay below 2^31 tiles");
  if (batch == 0) return EB_OK;
  if (!offsets || !out) return fail(EB_ERR_INVALID_ARG, "null offsets or output pointer");
  if ((reinterpret_cast<uintptr_t>(out) & 3) != 0) return fail(EB_ERR_INVALID_ARG, "output pointer is not 4-byte aligned");

  std::lock_guard<std::mutex> lock(g_device_lock[device]);
  int64_t col = 0;
  for (int f = 0; f < num_features; ++f) {
    if (rows[f] <= 0 || dims[f] <= 0 || (table_dtype[f] != EB_F32 && table_dtype[f] != EB_F16) || !table_ptrs[f])
      return fail(EB_ERR_INVALID_ARG, "feature %d is not a valid table", f);
    FeatStatic& fs = g_host_feats[device][f];
    memset(&fs, 0, sizeof(fs));
    const int esz = table_dtype[f] == EB_F16 ? 2 : 4;
    fs.table = static_cast<const char*>(table_ptrs[f]);
    fs.rows = rows[f];
    fs.dim = dims[f];
    fs.col_off = (int32_t)col;
    fs.row_bytes = dims[f] * esz;
    fs.dtype = table_dtype[f];
    fs.vec = (fs.row_bytes % 16 == 0) && ((reinterpret_cast<uintptr_t>(table_ptrs[f]) & 15) == 0);
    const int lanes = fs.vec ? fs.row_bytes / 16 : dims[f];
    fs.lg_group = ilog2(pow2_ceil(lanes < 32 ? lanes : 32));
    fs.nx = (lanes + 31) / 32;
    fs.kind = EB_SCHED_STREAM;
    fs.unroll = 4;
    fs.bags_per_tile = 0;
    col += dims[f];
    if (col > 0x7fffffff) return fail(EB_ERR_TOO_LARGE, "sum of dims exceeds 2^31");
  }
  if (out_ld < col) return fail(EB_ERR_INVALID_ARG, "out_ld %lld < output units %lld", (long long)out_ld, (long long)col);
  if (out_ld >= (1ll << 30)) return fail(EB_ERR_TOO_LARGE, "out_ld %lld: output rows must stay below 2^30 elements", (long long)out_ld);

  int prev = -1;
  if (cudaGetDevice(&prev) != cudaSuccess) return fail(EB_ERR_CUDA, "cudaGetDevice failed");
  if (prev != device && cudaSetDevice(device) != cudaSuccess) return fail(EB_ERR_CUDA, "cannot select device %d", device);
  int rc = EB_OK;
  do {
    char* scratch = nullptr;
    rc = scratch_for(device, &scratch);
    if (rc != EB_OK) break;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaError_t e = cudaStreamIsCapturing(st, &cap);
    if (e != cudaSuccess) { rc = fail(EB_ERR_CUDA, "cudaStreamIsCapturing failed: %s", cudaGetErrorString(e)); break; }
    if (cap != cudaStreamCaptureStatusNone) {
      rc = fail(EB_ERR_UNSUPPORTED, "the stream is being captured: this call stages descriptors through host memory");
      break;
    }
    e = cudaMemcpyAsync(scratch, g_host_feats[device], sizeof(FeatStatic) * num_features, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) { rc = fail(EB_ERR_CUDA, "descriptor upload failed: %s", cudaGetErrorString(e)); break; }
    LaunchArgs a;
    memset(&a, 0, sizeof(a));
    a.feats = reinterpret_cast<const FeatStatic*>(scratch);
    a.ws = scratch + kDescBytes;
    a.packed_values = static_cast<const char*>(values);
    a.packed_offsets = static_cast<const char*>(offsets);
    a.out = out;
    a.out_ld = out_ld;
    a.batch = batch;
    a.num_features = num_features;
    a.idx64 = index_dtype == EB_I64;
    a.has_end = 1;
    a.packed = 1;
    a.out_vec = ((reinterpret_cast<uintptr_t>(out) & 31) == 0 && out_ld % 8 == 0)
                    ? 2
                    : (((reinterpret_cast<uintptr_t>(out) & 15) == 0 && out_ld % 4 == 0) ? 1 : 0);
    a.warps_total = g_sm_count[device] * kNoAllocOccupancy * kWarpsPerCta;
    e = launch_bind(a, false, st);
    if (e != cudaSuccess) { rc = fail(EB_ERR_CUDA, "bind launch failed: %s", cudaGetErrorString(e)); break; }
    e = launch_fused(a, kNoAllocOccupancy, false, g_sm_count[device] * kNoAllocOccupancy, 0, st);
    if (e != cudaSuccess) { rc = fail(EB_ERR_CUDA, "fused launch failed: %s", cudaGetErrorString(e)); break; }
  } while (0);
  if (prev >= 0 && prev != device) cudaSetDevice(prev);
  return rc;
}

int eb_noalloc_check_status(int device, void* stream) {
  if (device < 0 || device >= kMaxDevices) return fail(EB_ERR_INVALID_ARG, "device %d out of range", device);
  int prev = -1;
  if (cudaGetDevice(&prev) != cudaSuccess) return fail(EB_ERR_CUDA, "cudaGetDevice failed");
  if (prev != device && cudaSetDevice(device) != cudaSuccess) return fail(EB_ERR_CUDA, "cannot select device %d", device);
  int rc = EB_OK;
  do {
    std::lock_guard<std::mutex> lock(g_device_lock[device]);
    char* scratch = nullptr;
    rc = scratch_for(device, &scratch);
    if (rc != EB_OK) break;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    WsHeader hdr;
    cudaError_t e = cudaMemcpyAsync(&hdr, scratch + kDescBytes, sizeof(hdr), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) { rc = fail(EB_ERR_CUDA, "reading the status word failed: %s", cudaGetErrorString(e)); break; }
    if (hdr.status & kStatusBadIndex)
      rc = fail(EB_ERR_BAD_INPUT, "an index outside [0, rows) was met and skipped");
    else if (hdr.status & kStatusBadOffsets)
      rc = fail(EB_ERR_BAD_INPUT, "offsets were not a non-decreasing sequence inside [0, nnz]; they were clamped");
  } while (0);
  if (prev >= 0 && prev != device) cudaSetDevice(prev);
  return rc;
}

}  // extern "C"
