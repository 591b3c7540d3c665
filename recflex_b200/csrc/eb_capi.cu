// C ABI of librecflex_b200.so (declared in include/recflex_b200.h): argument
// checking, the handle, descriptor upload and the launches.  The kernels are
// instantiated once per occupancy in eb_fused_inst.cu.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/recflex_b200.h"
#include "eb_common.cuh"
#include "eb_launch.h"

using namespace ebk;

namespace {

thread_local std::string g_err;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

#define EB_CUDA(expr)                                                                   \
  do {                                                                                  \
    cudaError_t e_ = (expr);                                                            \
    if (e_ != cudaSuccess)                                                              \
      return fail(EB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), \
                  __FILE__, __LINE__);                                                  \
  } while (0)

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() {
    int cur = -1;
    if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
  }
};

constexpr int kRing = 8;  // per-call descriptor uploads that may be in flight at once
constexpr int kTimeRing = 256;  // fused-kernel launches whose event pairs are kept

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

}  // namespace

namespace ebk {
void set_last_error(const char* msg) { g_err = msg ? msg : ""; }
}  // namespace ebk

struct eb_handle {
  int device = 0;
  int num_features = 0;
  int sm_count = 0;
  int clock_khz = 0;
  int occupancy = 4;
  int64_t units = 0;
  std::vector<FeatStatic> feats;
  std::vector<eb_schedule> sched;  // resolved
  FeatStatic* d_feats = nullptr;
  FeatDyn* pinned[kRing] = {};
  cudaEvent_t ev[kRing] = {};
  bool ev_used[kRing] = {};
  int ring_pos = 0;
  // optional event pairs around the fused-kernel launches
  int overlap_ctas = 0;         // > 0: fused kernel on this many CTAs per SM with eb_warp_kernel beside it (see run())
  cudaStream_t side = nullptr;  // stream of the warp-per-bag kernel in overlap mode
  cudaEvent_t fork_ev = nullptr, join_ev = nullptr;
  bool peer_interleave = true;  // eb_forward_peers deals tiles round-robin over the destination ranks
  int warp_features = 0;   // features pooled by eb_warp_kernel (warp-per-bag schedule, vector path)
  size_t smem_bytes = 0;   // dynamic shared memory of the fused kernel (the pipelined schedule's rings)
  bool time_kernels = false;
  std::vector<cudaEvent_t> t0, t1;
  int t_count = 0;
  int out_dtype = EB_OUT_F32;  // element type of the output matrix
  int only_kind = 0, only_unroll = 0;   // the one schedule (and unroll) every fused-kernel feature uses, 0 = mixed
  int64_t long_bag_bytes = 1 << 20;     // bags gathering at least this much are pooled by eb_longbag_kernel (0 = off)
  int exchange_engine = EB_EXCHANGE_COPY_ENGINES;  // who ships the pieces of eb_forward_exchange
  int exchange_direct_hops = 0;  // destinations to the right of this rank whose rows the kernel stores itself
  uint32_t epoch = 0;          // calls in chunked ticket order so far (eb_forward_exchange)
};

namespace {

// AUTO resolution: the blocked stream walk with four rows in flight is the
// robust default; the tuner replaces it per feature.
eb_schedule resolve(const eb_schedule& in) {
  eb_schedule s = in;
  if (s.kind == EB_SCHED_AUTO) s.kind = EB_SCHED_STREAM;
  if (s.unroll == 0) s.unroll = 4;
  if (s.vec_bytes == 0) s.vec_bytes = 16;
  return s;
}

int check_schedule(const eb_schedule& s, int f) {
  if (s.kind < EB_SCHED_AUTO || s.kind > EB_SCHED_PIPE)
    return fail(EB_ERR_INVALID_ARG, "feature %d: unknown schedule kind %d", f, s.kind);
  if (!(s.unroll == 0 || s.unroll == 1 || s.unroll == 2 || s.unroll == 4 || s.unroll == 8 ||
        (s.unroll == 6 && s.kind == EB_SCHED_PIPE)))
    return fail(EB_ERR_INVALID_ARG, "feature %d: unroll must be 0, 1, 2, 4 or 8, or 6 with EB_SCHED_PIPE (got %d)", f,
                s.unroll);
  if (!(s.vec_bytes == 0 || s.vec_bytes == 16))
    return fail(EB_ERR_INVALID_ARG, "feature %d: vec_bytes must be 0 or 16 (got %d)", f, s.vec_bytes);
  if (s.bags_per_tile < 0 || s.bags_per_tile > 1024 || (s.bags_per_tile & (s.bags_per_tile - 1)))
    return fail(EB_ERR_INVALID_ARG, "feature %d: bags_per_tile must be 0 or a power of two <= 1024 (got %d)", f,
                s.bags_per_tile);
  return EB_OK;
}

void apply_schedule(FeatStatic& fs, const eb_schedule& s) {
  fs.kind = s.kind;
  fs.unroll = s.unroll;
  fs.bags_per_tile = s.bags_per_tile;
}

int upload_feats(eb_handle* h) {
  EB_CUDA(cudaMemcpy(h->d_feats, h->feats.data(), sizeof(FeatStatic) * h->feats.size(), cudaMemcpyHostToDevice));
  return EB_OK;
}

size_t out_elem_bytes(const eb_handle* h) { return h->out_dtype == EB_OUT_F32 ? 4 : 2; }

// Widest aligned store the output allows: 2 = eight elements, 1 = four, 0 = one (see store_vals).
int out_vec_of(const void* out, int64_t out_ld, size_t es) {
  const uintptr_t p = reinterpret_cast<uintptr_t>(out);
  if (p % (8 * es) == 0 && out_ld % 8 == 0) return 2;
  if (p % (4 * es) == 0 && out_ld % 4 == 0) return 1;
  return 0;
}

int check_forward_common(const eb_handle* h, int64_t batch, int index_dtype, const float* out, int64_t out_ld,
                         const void* workspace, size_t workspace_bytes) {
  if (!h) return fail(EB_ERR_INVALID_ARG, "null handle");
  if (batch < 0) return fail(EB_ERR_INVALID_ARG, "negative batch %lld", (long long)batch);
  if (index_dtype != EB_I32 && index_dtype != EB_I64)
    return fail(EB_ERR_INVALID_ARG, "index_dtype must be EB_I32 or EB_I64 (got %d)", index_dtype);
  if (batch > 0 && !out) return fail(EB_ERR_INVALID_ARG, "null output pointer");
  if (out_ld < h->units) return fail(EB_ERR_INVALID_ARG, "out_ld %lld < output units %lld", (long long)out_ld, (long long)h->units);
  if (out_ld >= (1ll << 30)) return fail(EB_ERR_TOO_LARGE, "out_ld %lld: output rows must stay below 2^30 elements", (long long)out_ld);
  if ((reinterpret_cast<uintptr_t>(out) & (out_elem_bytes(h) - 1)) != 0)
    return fail(EB_ERR_INVALID_ARG, "output pointer is not aligned to its element size");
  if (!workspace) return fail(EB_ERR_INVALID_ARG, "null workspace");
  if ((reinterpret_cast<uintptr_t>(workspace) & 127) != 0) return fail(EB_ERR_INVALID_ARG, "workspace must be 128-byte aligned");
  const size_t need = ws_layout(h->num_features).total;
  if (workspace_bytes < need)
    return fail(EB_ERR_WORKSPACE_TOO_SMALL, "workspace holds %zu bytes, %zu needed", workspace_bytes, need);
  if ((long double)batch * (long double)h->num_features >= 2147483648.0L)
    return fail(EB_ERR_TOO_LARGE, "batch * num_features must stay below 2^31 tiles");
  return EB_OK;
}

LaunchArgs make_args(const eb_handle* h, int64_t batch, int index_dtype, int has_end, float* out, int64_t out_ld,
                     void* workspace) {
  LaunchArgs a;
  memset(&a, 0, sizeof(a));
  a.feats = h->d_feats;
  a.ws = static_cast<char*>(workspace);
  a.out = out;
  a.out_ld = out_ld;
  a.batch = batch;
  a.num_features = h->num_features;
  a.idx64 = index_dtype == EB_I64;
  a.has_end = has_end != 0;
  a.packed = 0;
  a.out_dtype = h->out_dtype;
  a.out_vec = out_vec_of(out, out_ld, out_elem_bytes(h));
  a.warps_total = h->sm_count * h->occupancy * kWarpsPerCta;
  a.ring_bytes = (int32_t)(h->smem_bytes / kWarpsPerCta);
  a.long_bytes = h->long_bag_bytes;
  return a;
}

int run(eb_handle* h, const LaunchArgs& a_in, bool timing, cudaStream_t st) {
  if (a_in.batch == 0) return EB_OK;
  LaunchArgs a = a_in;
  // Overlap mode: long bags over cache-resident tables keep L1 busy, short bags over large tables keep HBM busy,
  // so the two kernels share the SMs instead of following each other.  The persistent fused kernel goes first on a
  // reduced grid (it holds its CTA slots until its tickets run out); eb_warp_kernel's plain grid fills the rest of
  // every SM from a second stream, forked after the binding kernel and joined before anything the caller enqueues
  // next.  The per-feature timing variant keeps the serial order.
  const bool overlap = h->overlap_ctas > 0 && h->warp_features > 0 && h->warp_features < h->num_features && !timing &&
                       a.chunks == 0;  // chunked order: the warp-per-bag kernel must be done before any chunk is published
  const int ctas_per_sm = overlap && h->overlap_ctas < h->occupancy ? h->overlap_ctas : h->occupancy;
  a.warps_total = h->sm_count * ctas_per_sm * kWarpsPerCta;
  const bool rec = h->time_kernels && h->t_count < kTimeRing;
  if (rec) EB_CUDA(cudaEventRecord(h->t0[h->t_count], st));
  EB_CUDA(launch_bind(a, timing, st));
  if (overlap) {
    EB_CUDA(cudaEventRecord(h->fork_ev, st));
    EB_CUDA(launch_fused(a, h->occupancy, timing, h->sm_count * ctas_per_sm, h->smem_bytes, st, h->only_kind,
                         h->only_unroll));
    EB_CUDA(cudaStreamWaitEvent(h->side, h->fork_ev, 0));
    EB_CUDA(launch_warp(a, timing, h->warp_features, h->side));
    EB_CUDA(cudaEventRecord(h->join_ev, h->side));
    EB_CUDA(cudaStreamWaitEvent(st, h->join_ev, 0));
  } else {
    if (h->warp_features) EB_CUDA(launch_warp(a, timing, h->warp_features, st));
    EB_CUDA(launch_fused(a, h->occupancy, timing, h->sm_count * ctas_per_sm, h->smem_bytes, st, h->only_kind,
                         h->only_unroll));
  }
  if (a.long_bytes > 0) EB_CUDA(launch_longbag(a, timing, h->sm_count, st));
  if (a.chunks > 0) EB_CUDA(launch_release(a, st));
  if (rec) {
    EB_CUDA(cudaEventRecord(h->t1[h->t_count], st));
    ++h->t_count;
  }
  return EB_OK;
}

int upload_dyn(eb_handle* h, int64_t batch, const void* const* values_ptrs, const void* const* offsets_ptrs,
               const int64_t* nnz, int has_end, void* workspace, cudaStream_t st) {
  if (!values_ptrs || !offsets_ptrs) return fail(EB_ERR_INVALID_ARG, "null pointer array");
  if (!has_end && !nnz) return fail(EB_ERR_INVALID_ARG, "nnz array is required when offsets carry no end entry");
  const int F = h->num_features;
  const int slot = h->ring_pos;
  h->ring_pos = (h->ring_pos + 1) % kRing;
  if (h->ev_used[slot]) EB_CUDA(cudaEventSynchronize(h->ev[slot]));
  FeatDyn* p = h->pinned[slot];
  for (int f = 0; f < F; ++f) {
    p[f].values = static_cast<const char*>(values_ptrs[f]);
    p[f].offsets = static_cast<const char*>(offsets_ptrs[f]);
    p[f].nnz = has_end ? 0 : nnz[f];
    p[f].work = 0;
    if (!offsets_ptrs[f] && batch > 0) return fail(EB_ERR_INVALID_ARG, "feature %d: null offsets pointer", f);
    if (!has_end && nnz[f] < 0) return fail(EB_ERR_INVALID_ARG, "feature %d: negative nnz", f);
  }
  const WsLayout L = ws_layout(F);
  EB_CUDA(cudaMemcpyAsync(static_cast<char*>(workspace) + L.dyn, p, sizeof(FeatDyn) * F, cudaMemcpyHostToDevice, st));
  EB_CUDA(cudaEventRecord(h->ev[slot], st));
  h->ev_used[slot] = true;
  return EB_OK;
}

}  // namespace

extern "C" {

const char* eb_last_error(void) { return g_err.c_str(); }

const char* eb_version(void) { return "recflex_b200 0.1 (sm_100a)"; }

int eb_create(eb_handle** out, int device, int num_features, const int64_t* rows, const int32_t* dims,
              const int32_t* table_dtype, const void* const* table_ptrs) {
  if (!out) return fail(EB_ERR_INVALID_ARG, "null output handle pointer");
  *out = nullptr;
  if (num_features <= 0) return fail(EB_ERR_INVALID_ARG, "num_features must be positive (got %d)", num_features);
  if (!rows || !dims || !table_dtype || !table_ptrs) return fail(EB_ERR_INVALID_ARG, "null argument array");
  int ndev = 0;
  EB_CUDA(cudaGetDeviceCount(&ndev));
  if (device < 0 || device >= ndev) return fail(EB_ERR_INVALID_ARG, "device %d out of range (%d visible)", device, ndev);
  DeviceGuard guard(device);
  if (!guard.ok) return fail(EB_ERR_CUDA, "cannot select device %d", device);

  int sm_count = 0, clock_khz = 0;
  EB_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  EB_CUDA(cudaDeviceGetAttribute(&clock_khz, cudaDevAttrClockRate, device));
  eb_handle* h = new eb_handle();
  h->device = device;
  h->num_features = num_features;
  h->sm_count = sm_count;
  h->clock_khz = clock_khz;
  h->feats.resize(num_features);
  h->sched.resize(num_features);
  int64_t col = 0;
  for (int f = 0; f < num_features; ++f) {
    if (rows[f] <= 0 || dims[f] <= 0 || (table_dtype[f] != EB_F32 && table_dtype[f] != EB_F16) || !table_ptrs[f]) {
      const int code = fail(EB_ERR_INVALID_ARG, "feature %d: rows=%lld dim=%d dtype=%d ptr=%p is not a valid table", f,
                            (long long)rows[f], dims[f], table_dtype[f], table_ptrs[f]);
      delete h;
      return code;
    }
    FeatStatic& fs = h->feats[f];
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
    const int g = pow2_ceil(lanes < 32 ? lanes : 32);
    fs.lg_group = ilog2(g);
    fs.nx = (lanes + 31) / 32;
    eb_schedule s = {EB_SCHED_AUTO, 0, 0, 0};
    h->sched[f] = resolve(s);
    apply_schedule(fs, h->sched[f]);
    col += dims[f];
    if (col > 0x7fffffff) {
      delete h;
      return fail(EB_ERR_TOO_LARGE, "sum of dims exceeds 2^31");
    }
  }
  h->units = col;
  cudaError_t e = cudaMalloc(&h->d_feats, sizeof(FeatStatic) * num_features);
  if (e != cudaSuccess) {
    delete h;
    return fail(EB_ERR_CUDA, "cudaMalloc of the descriptor table failed: %s", cudaGetErrorString(e));
  }
  for (int i = 0; i < kRing; ++i) {
    if (cudaMallocHost(&h->pinned[i], sizeof(FeatDyn) * num_features) != cudaSuccess ||
        cudaEventCreateWithFlags(&h->ev[i], cudaEventDisableTiming) != cudaSuccess) {
      eb_destroy(h);
      return fail(EB_ERR_CUDA, "cannot allocate the pinned descriptor ring");
    }
  }
  const int rc = upload_feats(h);
  if (rc != EB_OK) {
    eb_destroy(h);
    return rc;
  }
  *out = h;
  return EB_OK;
}

int eb_destroy(eb_handle* h) {
  if (!h) return EB_OK;
  DeviceGuard guard(h->device);
  for (int i = 0; i < kRing; ++i) {
    if (h->ev[i]) cudaEventDestroy(h->ev[i]);
    if (h->pinned[i]) cudaFreeHost(h->pinned[i]);
  }
  if (h->fork_ev) cudaEventDestroy(h->fork_ev);
  if (h->join_ev) cudaEventDestroy(h->join_ev);
  if (h->side) cudaStreamDestroy(h->side);
  for (cudaEvent_t e : h->t0) cudaEventDestroy(e);
  for (cudaEvent_t e : h->t1) cudaEventDestroy(e);
  if (h->d_feats) cudaFree(h->d_feats);
  delete h;
  return EB_OK;
}

int eb_output_units(const eb_handle* h, int64_t* units) {
  if (!h || !units) return fail(EB_ERR_INVALID_ARG, "null argument");
  *units = h->units;
  return EB_OK;
}

int eb_set_schedules(eb_handle* h, const eb_schedule* per_feature, int occupancy) {
  if (!h) return fail(EB_ERR_INVALID_ARG, "null handle");
  if (occupancy < 0 || occupancy > kMaxOccupancy)
    return fail(EB_ERR_INVALID_ARG, "occupancy must be 0 (keep) or 1..%d (got %d)", kMaxOccupancy, occupancy);
  if (per_feature) {
    for (int f = 0; f < h->num_features; ++f) {
      const int rc = check_schedule(per_feature[f], f);
      if (rc != EB_OK) return rc;
    }
    // deepest ring any pipelined feature needs (pipe_cells: never fewer than the unroll-4 variant's, because batches
    // with 64-bit indices always run that variant whatever was requested)
    int cells = 0;
    for (int f = 0; f < h->num_features; ++f) {
      h->sched[f] = resolve(per_feature[f]);
      // the ring holds 16-byte lane cells: element-wise fallback rows keep the register walk
      if (h->sched[f].kind == EB_SCHED_PIPE && !h->feats[f].vec) {
        h->sched[f].kind = EB_SCHED_STREAM;
        if (h->sched[f].unroll == 6) h->sched[f].unroll = 4;
      }
      apply_schedule(h->feats[f], h->sched[f]);
      if (h->sched[f].kind == EB_SCHED_PIPE) {
        const int need = pipe_cells(h->sched[f].unroll);
        cells = need > cells ? need : cells;
      }
    }
    h->smem_bytes = (size_t)cells * kPipeCellBytes * kWarpsPerCta;
    h->warp_features = 0;
    for (int f = 0; f < h->num_features; ++f)
      h->warp_features += (h->feats[f].kind == EB_SCHED_WARP && h->feats[f].vec) ? 1 : 0;
    // do all features the fused kernel pools by vector rows agree on a stream / pipe schedule (and on its unroll)?
    int kind = -1, unroll = -1;
    for (int f = 0; f < h->num_features; ++f) {
      const FeatStatic& fs = h->feats[f];
      if (!fs.vec || fs.kind == EB_SCHED_WARP) continue;  // element-wise fallback / the warp-per-bag kernel's
      const int u = (fs.kind == EB_SCHED_PIPE && fs.unroll < 2) ? 2 : fs.unroll;
      kind = kind == -1 ? fs.kind : (kind == fs.kind ? kind : 0);
      unroll = unroll == -1 ? u : (unroll == u ? unroll : 0);
    }
    const bool family = kind == EB_SCHED_STREAM || kind == EB_SCHED_PIPE;
    h->only_kind = family ? kind : 0;
    h->only_unroll = (family && (unroll == 2 || unroll == 4 || unroll == 8 || (unroll == 6 && kind == EB_SCHED_PIPE)))
                         ? unroll : 0;
    DeviceGuard guard(h->device);
    const int rc = upload_feats(h);
    if (rc != EB_OK) return rc;
  }
  if (occupancy > 0) h->occupancy = occupancy;
  return EB_OK;
}

int eb_set_output_columns(eb_handle* h, const int32_t* first_column, int64_t units) {
  if (!h) return fail(EB_ERR_INVALID_ARG, "null handle");
  if (!first_column) {  // back to the default: features side by side
    int64_t col = 0;
    for (auto& fs : h->feats) { fs.col_off = (int32_t)col; col += fs.dim; }
    h->units = col;
  } else {
    for (int f = 0; f < h->num_features; ++f)
      if (first_column[f] < 0 || (int64_t)first_column[f] + h->feats[f].dim > units)
        return fail(EB_ERR_INVALID_ARG, "feature %d: columns [%d, %d) fall outside [0, %lld)", f, first_column[f],
                    first_column[f] + h->feats[f].dim, (long long)units);
    for (int f = 0; f < h->num_features; ++f) h->feats[f].col_off = first_column[f];
    h->units = units;
  }
  DeviceGuard guard(h->device);
  return upload_feats(h);
}

int eb_get_schedules(const eb_handle* h, eb_schedule* per_feature, int* occupancy) {
  if (!h) return fail(EB_ERR_INVALID_ARG, "null handle");
  if (per_feature)
    for (int f = 0; f < h->num_features; ++f) per_feature[f] = h->sched[f];
  if (occupancy) *occupancy = h->occupancy;
  return EB_OK;
}

int eb_workspace_bytes(const eb_handle* h, size_t* bytes) {
  if (!h || !bytes) return fail(EB_ERR_INVALID_ARG, "null argument");
  *bytes = ws_layout(h->num_features).total;
  return EB_OK;
}

int eb_max_concurrent_ctas(const eb_handle* h, int occupancy, int* ctas) {
  if (!h || !ctas) return fail(EB_ERR_INVALID_ARG, "null argument");
  if (occupancy < 0 || occupancy > kMaxOccupancy) return fail(EB_ERR_INVALID_ARG, "occupancy out of range");
  const int occ = occupancy ? occupancy : h->occupancy;
  DeviceGuard guard(h->device);
  int per_sm = 0;
  EB_CUDA(fused_ctas_per_sm(occ, h->smem_bytes, &per_sm, h->only_kind, h->only_unroll));
  *ctas = h->sm_count * (per_sm < occ ? per_sm : occ);
  return EB_OK;
}

int eb_forward(eb_handle* h, int64_t batch, const void* const* values_ptrs, const void* const* offsets_ptrs,
               const int64_t* nnz, int index_dtype, int offsets_have_end, float* out, int64_t out_ld, void* workspace,
               size_t workspace_bytes, void* stream) {
  int rc = check_forward_common(h, batch, index_dtype, out, out_ld, workspace, workspace_bytes);
  if (rc != EB_OK) return rc;
  if (batch == 0) return EB_OK;
  DeviceGuard guard(h->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = upload_dyn(h, batch, values_ptrs, offsets_ptrs, nnz, offsets_have_end, workspace, st);
  if (rc != EB_OK) return rc;
  const LaunchArgs a = make_args(h, batch, index_dtype, offsets_have_end, out, out_ld, workspace);
  return run(h, a, false, st);
}

int eb_forward_peers(eb_handle* h, int64_t batch, const void* const* values_ptrs, const void* const* offsets_ptrs,
                     const int64_t* nnz, int index_dtype, int offsets_have_end, float* const* peer_out, int world,
                     int64_t out_ld, void* workspace, size_t workspace_bytes, void* stream) {
  if (world < 1 || world > kMaxPeers) return fail(EB_ERR_INVALID_ARG, "world must be 1..%d (got %d)", kMaxPeers, world);
  if (!peer_out) return fail(EB_ERR_INVALID_ARG, "null peer_out");
  int rc = check_forward_common(h, batch, index_dtype, peer_out[0], out_ld, workspace, workspace_bytes);
  if (rc != EB_OK) return rc;
  if (batch == 0) return EB_OK;
  if (batch % world != 0 || (batch / world) % 32 != 0)
    return fail(EB_ERR_INVALID_ARG, "batch / world must be a whole multiple of 32 (batch %lld, world %d)",
                (long long)batch, world);
  int vec = 2;
  for (int r = 0; r < world; ++r) {
    if (!peer_out[r]) return fail(EB_ERR_INVALID_ARG, "null output pointer for rank %d", r);
    if (reinterpret_cast<uintptr_t>(peer_out[r]) & (out_elem_bytes(h) - 1))
      return fail(EB_ERR_INVALID_ARG, "rank %d: output not aligned to its element size", r);
    const int v = out_vec_of(peer_out[r], out_ld, out_elem_bytes(h));
    vec = v < vec ? v : vec;
  }
  DeviceGuard guard(h->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = upload_dyn(h, batch, values_ptrs, offsets_ptrs, nnz, offsets_have_end, workspace, st);
  if (rc != EB_OK) return rc;
  LaunchArgs a = make_args(h, batch, index_dtype, offsets_have_end, peer_out[0], out_ld, workspace);
  a.out_vec = vec;
  a.rows_per_peer = batch / world;
  a.peer_spread = h->peer_interleave ? world : 0;
  for (int r = 0; r < world; ++r) a.peer_out[r] = peer_out[r];
  return run(h, a, false, st);
}

int eb_set_long_bag_split(eb_handle* h, int64_t min_bytes) {
  if (!h) return fail(EB_ERR_INVALID_ARG, "null handle");
  if (min_bytes < 0) return fail(EB_ERR_INVALID_ARG, "negative size");
  h->long_bag_bytes = min_bytes;
  return EB_OK;
}

int eb_set_exchange_direct(eb_handle* h, int hops) {
  if (!h) return fail(EB_ERR_INVALID_ARG, "null handle");
  if (hops < 0 || hops >= kMaxPeers) return fail(EB_ERR_INVALID_ARG, "hops must be 0..%d (got %d)", kMaxPeers - 1, hops);
  h->exchange_direct_hops = hops;
  return EB_OK;
}

int eb_set_exchange_engine(eb_handle* h, int engine) {
  if (!h) return fail(EB_ERR_INVALID_ARG, "null handle");
  if (engine != EB_EXCHANGE_COPY_ENGINES && engine != EB_EXCHANGE_SM_PUSH)
    return fail(EB_ERR_INVALID_ARG, "engine must be EB_EXCHANGE_COPY_ENGINES or EB_EXCHANGE_SM_PUSH (got %d)", engine);
  h->exchange_engine = engine;
  return EB_OK;
}

int eb_set_output_dtype(eb_handle* h, int out_dtype) {
  if (!h) return fail(EB_ERR_INVALID_ARG, "null handle");
  if (out_dtype != EB_OUT_F32 && out_dtype != EB_OUT_BF16 && out_dtype != EB_OUT_F16)
    return fail(EB_ERR_INVALID_ARG, "out_dtype must be EB_OUT_F32, EB_OUT_BF16 or EB_OUT_F16 (got %d)", out_dtype);
  h->out_dtype = out_dtype;
  return EB_OK;
}

namespace {
// cuStreamWaitValue32 of the driver API, looked up at run time so that the library links against the runtime only.
typedef int (*StreamWaitValue32)(cudaStream_t, unsigned long long, uint32_t, unsigned int);
StreamWaitValue32 stream_wait_value32() {
  static StreamWaitValue32 fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<StreamWaitValue32>(p);
  }();
  return fn;
}
}  // namespace

int eb_forward_exchange(eb_handle* h, int64_t batch, const void* const* values_ptrs, const void* const* offsets_ptrs,
                        const int64_t* nnz, int index_dtype, int offsets_have_end, float* send, int64_t send_ld,
                        float* const* peer_out, int world, int rank, int64_t out_ld, int64_t out_col, int chunks,
                        void* workspace, size_t workspace_bytes, void* stream, void* const* copy_streams,
                        int num_copy_streams) {
  if (world < 1 || world > kMaxPeers) return fail(EB_ERR_INVALID_ARG, "world must be 1..%d (got %d)", kMaxPeers, world);
  if (rank < 0 || rank >= world) return fail(EB_ERR_INVALID_ARG, "rank %d outside [0, %d)", rank, world);
  if (chunks < 1 || chunks > kMaxChunks) return fail(EB_ERR_INVALID_ARG, "chunks must be 1..%d (got %d)", kMaxChunks, chunks);
  if (!peer_out) return fail(EB_ERR_INVALID_ARG, "null peer_out");
  if (!copy_streams || num_copy_streams < 1 || num_copy_streams > kMaxPeers)
    return fail(EB_ERR_INVALID_ARG, "between 1 and %d copy streams are needed", kMaxPeers);
  int rc = check_forward_common(h, batch, index_dtype, send, send_ld, workspace, workspace_bytes);
  if (rc != EB_OK) return rc;
  if (batch == 0) return EB_OK;
  if (batch % ((int64_t)world * chunks) != 0)
    return fail(EB_ERR_INVALID_ARG, "batch %lld must be a whole multiple of world * chunks = %d", (long long)batch, world * chunks);
  if (out_col < 0 || out_col + h->units > out_ld || out_ld >= (1ll << 30))
    return fail(EB_ERR_INVALID_ARG, "columns [%lld, %lld) do not fit rows of %lld elements", (long long)out_col,
                (long long)(out_col + h->units), (long long)out_ld);
  for (int r = 0; r < world; ++r)
    if (!peer_out[r]) return fail(EB_ERR_INVALID_ARG, "null output pointer for rank %d", r);
  StreamWaitValue32 wait32 = stream_wait_value32();
  if (!wait32) return fail(EB_ERR_UNSUPPORTED, "the driver offers no cuStreamWaitValue32 (stream memory operations)");
  DeviceGuard guard(h->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = upload_dyn(h, batch, values_ptrs, offsets_ptrs, nnz, offsets_have_end, workspace, st);
  if (rc != EB_OK) return rc;
  LaunchArgs a = make_args(h, batch, index_dtype, offsets_have_end, send, send_ld, workspace);
  a.chunks = chunks;
  a.dest_rows = batch / world;
  a.chunk_rows = a.dest_rows / chunks;
  if (++h->epoch == 0) h->epoch = 1;  // a fresh workspace holds zeros: epoch 0 is never waited for
  a.epoch = h->epoch;
  const size_t es = out_elem_bytes(h);
  a.own_out = peer_out[rank];  // this rank's own samples skip the send buffer
  a.own_ld = out_ld;
  a.own_col = (int32_t)out_col;
  a.own_rank = rank;
  a.world = world;
  a.direct_hops = h->exchange_direct_hops < world - 1 ? h->exchange_direct_hops : world - 1;
  a.own_vec = 2;
  for (int r = 0; r < world; ++r) {
    a.peer_out[r] = peer_out[r];
    const int v = out_vec_of(peer_out[r], out_ld, es);
    a.own_vec = v < a.own_vec ? v : a.own_vec;
  }
  const int first_copied = a.direct_hops + 1;  // hops first_copied .. world - 1 leave through the send buffer
  rc = run(h, a, false, st);
  if (rc != EB_OK) return rc;
  // copy streams: as soon as chunk k is published, its rows leave for every other rank; destination i hops to the
  // right of this rank uses stream (i - 1) mod n, so several copy engines work at once
  const ChunkSync* cs = reinterpret_cast<const ChunkSync*>(static_cast<char*>(workspace) + ws_layout(h->num_features).chunk_sync);
  const size_t width = (size_t)h->units * es;
  const int copied = world - first_copied;  // destinations served by copies
  const int ns = num_copy_streams < copied ? num_copy_streams : (copied > 0 ? copied : 1);
  // SM copies need 16-byte granularity everywhere; otherwise the copy engines do the work
  const bool push = h->exchange_engine == EB_EXCHANGE_SM_PUSH && width % 16 == 0 && ((size_t)send_ld * es) % 16 == 0 &&
                    ((size_t)out_ld * es) % 16 == 0 && ((size_t)out_col * es) % 16 == 0 &&
                    (reinterpret_cast<uintptr_t>(send) & 15) == 0;
  void* blocks[kMaxPeers] = {};
  bool aligned = push;
  for (int r = 0; r < world; ++r) {
    blocks[r] = reinterpret_cast<char*>(peer_out[r]) + (size_t)out_col * es;
    aligned = aligned && (reinterpret_cast<uintptr_t>(blocks[r]) & 15) == 0;
  }
  if (aligned && first_copied < world) {
    cudaStream_t cst = static_cast<cudaStream_t>(copy_streams[0]);
    for (int k = 0; k < chunks; ++k) {
      const int wrc = wait32(cst, (unsigned long long)reinterpret_cast<uintptr_t>(&cs->flag[k]), a.epoch, 0u /* >= */);
      if (wrc != 0) return fail(EB_ERR_CUDA, "cuStreamWaitValue32 failed with driver error %d", wrc);
      EB_CUDA(launch_push(send, blocks, (long long)send_ld * es, (long long)out_ld * es, a.dest_rows, a.chunk_rows, k,
                          (int)(width / 16), world, rank, first_copied, h->sm_count, cst));
    }
    return EB_OK;
  }
  for (int k = 0; k < chunks; ++k) {
    for (int j = 0; j < ns && first_copied < world; ++j) {
      const int wrc = wait32(static_cast<cudaStream_t>(copy_streams[j]),
                             (unsigned long long)reinterpret_cast<uintptr_t>(&cs->flag[k]), a.epoch, 0u /* >= */);
      if (wrc != 0) return fail(EB_ERR_CUDA, "cuStreamWaitValue32 failed with driver error %d", wrc);
    }
    for (int i = first_copied; i < world; ++i) {
      const int d = (rank + i) % world;
      cudaStream_t cst = static_cast<cudaStream_t>(copy_streams[(i - first_copied) % ns]);
      const char* src = reinterpret_cast<const char*>(send) + ((size_t)d * a.dest_rows + (size_t)k * a.chunk_rows) * send_ld * es;
      char* dst = reinterpret_cast<char*>(peer_out[d]) + ((size_t)k * a.chunk_rows * out_ld + out_col) * es;
      if ((size_t)out_ld * es == width && (size_t)send_ld * es == width)  // rows back to back on both sides: one run
        EB_CUDA(cudaMemcpyAsync(dst, src, width * (size_t)a.chunk_rows, cudaMemcpyDefault, cst));
      else
        EB_CUDA(cudaMemcpy2DAsync(dst, (size_t)out_ld * es, src, (size_t)send_ld * es, width, (size_t)a.chunk_rows,
                                  cudaMemcpyDefault, cst));
    }
  }
  return EB_OK;
}

int eb_set_kernel_overlap(eb_handle* h, int fused_ctas_per_sm) {
  if (!h) return fail(EB_ERR_INVALID_ARG, "null handle");
  if (fused_ctas_per_sm < 0 || fused_ctas_per_sm > kMaxOccupancy)
    return fail(EB_ERR_INVALID_ARG, "fused_ctas_per_sm must be 0 (off) or 1..%d (got %d)", kMaxOccupancy, fused_ctas_per_sm);
  if (fused_ctas_per_sm > 0 && !h->side) {
    DeviceGuard guard(h->device);
    EB_CUDA(cudaStreamCreateWithFlags(&h->side, cudaStreamNonBlocking));
    EB_CUDA(cudaEventCreateWithFlags(&h->fork_ev, cudaEventDisableTiming));
    EB_CUDA(cudaEventCreateWithFlags(&h->join_ev, cudaEventDisableTiming));
  }
  h->overlap_ctas = fused_ctas_per_sm;
  return EB_OK;
}

int eb_set_peer_interleave(eb_handle* h, int enabled) {
  if (!h) return fail(EB_ERR_INVALID_ARG, "null handle");
  h->peer_interleave = enabled != 0;
  return EB_OK;
}

int eb_peer_alloc(int device, size_t bytes, void** ptr, unsigned char* handle64) {
  if (!ptr || !handle64 || bytes == 0) return fail(EB_ERR_INVALID_ARG, "invalid argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
  DeviceGuard guard(device);
  if (!guard.ok) return fail(EB_ERR_CUDA, "cannot select device %d", device);
  void* p = nullptr;
  EB_CUDA(cudaMalloc(&p, bytes));
  cudaIpcMemHandle_t hd;
  cudaError_t e = cudaIpcGetMemHandle(&hd, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(EB_ERR_CUDA, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
  }
  memcpy(handle64, &hd, 64);
  *ptr = p;
  return EB_OK;
}

int eb_peer_open(int device, const unsigned char* handle64, void** ptr) {
  if (!ptr || !handle64) return fail(EB_ERR_INVALID_ARG, "invalid argument");
  DeviceGuard guard(device);
  if (!guard.ok) return fail(EB_ERR_CUDA, "cannot select device %d", device);
  cudaIpcMemHandle_t hd;
  memcpy(&hd, handle64, 64);
  EB_CUDA(cudaIpcOpenMemHandle(ptr, hd, cudaIpcMemLazyEnablePeerAccess));
  return EB_OK;
}

int eb_peer_close(int device, void* ptr) {
  if (!ptr) return EB_OK;
  DeviceGuard guard(device);
  EB_CUDA(cudaIpcCloseMemHandle(ptr));
  return EB_OK;
}

int eb_peer_free(int device, void* ptr) {
  if (!ptr) return EB_OK;
  DeviceGuard guard(device);
  EB_CUDA(cudaFree(ptr));
  return EB_OK;
}

int eb_forward_packed(eb_handle* h, int64_t batch, const void* values, const void* offsets, int index_dtype,
                      float* out, int64_t out_ld, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_forward_common(h, batch, index_dtype, out, out_ld, workspace, workspace_bytes);
  if (rc != EB_OK) return rc;
  if (batch == 0) return EB_OK;
  if (!offsets) return fail(EB_ERR_INVALID_ARG, "null offsets pointer");
  DeviceGuard guard(h->device);
  LaunchArgs a = make_args(h, batch, index_dtype, 1, out, out_ld, workspace);
  a.packed = 1;
  a.packed_values = static_cast<const char*>(values);
  a.packed_offsets = static_cast<const char*>(offsets);
  return run(h, a, false, static_cast<cudaStream_t>(stream));
}

int eb_host_staging_bytes(const eb_handle* h, int64_t batch, int64_t total_nnz, int index_dtype, size_t* bytes) {
  if (!h || !bytes) return fail(EB_ERR_INVALID_ARG, "null argument");
  if (batch < 0 || total_nnz < 0) return fail(EB_ERR_INVALID_ARG, "negative size");
  const size_t isz = index_dtype == EB_I64 ? 8 : 4;
  size_t o = align_up((size_t)total_nnz * isz, 256);
  o = align_up(o + (size_t)h->num_features * (size_t)(batch + 1) * isz, 256);
  o = align_up(o + (size_t)batch * (size_t)h->units * out_elem_bytes(h), 256);
  *bytes = o;
  return EB_OK;
}

int eb_forward_host(eb_handle* h, int64_t batch, const void* host_values, int64_t total_nnz, const void* host_offsets,
                    int index_dtype, float* host_out, void* staging, size_t staging_bytes, void* workspace,
                    size_t workspace_bytes, void* stream) {
  if (!h) return fail(EB_ERR_INVALID_ARG, "null handle");
  if (!staging || (reinterpret_cast<uintptr_t>(staging) & 255) != 0)
    return fail(EB_ERR_INVALID_ARG, "staging must be a 256-byte aligned device buffer");
  size_t need = 0;
  int rc = eb_host_staging_bytes(h, batch, total_nnz, index_dtype, &need);
  if (rc != EB_OK) return rc;
  if (staging_bytes < need) return fail(EB_ERR_WORKSPACE_TOO_SMALL, "staging holds %zu bytes, %zu needed", staging_bytes, need);
  if (batch == 0) return EB_OK;
  if (!host_offsets || !host_out || (total_nnz > 0 && !host_values)) return fail(EB_ERR_INVALID_ARG, "null host buffer");
  const size_t isz = index_dtype == EB_I64 ? 8 : 4;
  char* d_values = static_cast<char*>(staging);
  char* d_offsets = d_values + align_up((size_t)total_nnz * isz, 256);
  const size_t off_bytes = (size_t)h->num_features * (size_t)(batch + 1) * isz;
  float* d_out = reinterpret_cast<float*>(d_offsets + align_up(off_bytes, 256));
  DeviceGuard guard(h->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (total_nnz > 0) EB_CUDA(cudaMemcpyAsync(d_values, host_values, (size_t)total_nnz * isz, cudaMemcpyHostToDevice, st));
  EB_CUDA(cudaMemcpyAsync(d_offsets, host_offsets, off_bytes, cudaMemcpyHostToDevice, st));
  rc = eb_forward_packed(h, batch, d_values, d_offsets, index_dtype, d_out, h->units, workspace, workspace_bytes, stream);
  if (rc != EB_OK) return rc;
  EB_CUDA(cudaMemcpyAsync(host_out, d_out, (size_t)batch * (size_t)h->units * out_elem_bytes(h), cudaMemcpyDeviceToHost, st));
  return EB_OK;
}

int eb_forward_timed(eb_handle* h, int64_t batch, const void* const* values_ptrs, const void* const* offsets_ptrs,
                     const int64_t* nnz, int index_dtype, int offsets_have_end, float* out, int64_t out_ld,
                     void* workspace, size_t workspace_bytes, void* stream, double* per_feature_ns) {
  int rc = check_forward_common(h, batch, index_dtype, out, out_ld, workspace, workspace_bytes);
  if (rc != EB_OK) return rc;
  if (!per_feature_ns) return fail(EB_ERR_INVALID_ARG, "null per_feature_ns");
  const int F = h->num_features;
  for (int f = 0; f < F; ++f) per_feature_ns[f] = 0.0;
  if (batch == 0) return EB_OK;
  DeviceGuard guard(h->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = upload_dyn(h, batch, values_ptrs, offsets_ptrs, nnz, offsets_have_end, workspace, st);
  if (rc != EB_OK) return rc;
  const LaunchArgs a = make_args(h, batch, index_dtype, offsets_have_end, out, out_ld, workspace);
  rc = run(h, a, true, st);
  if (rc != EB_OK) return rc;
  std::vector<unsigned long long> cycles(F);
  const WsLayout L = ws_layout(F);
  EB_CUDA(cudaMemcpyAsync(cycles.data(), static_cast<char*>(workspace) + L.feat_ns, sizeof(unsigned long long) * F,
                          cudaMemcpyDeviceToHost, st));
  EB_CUDA(cudaStreamSynchronize(st));
  const double ns_per_cycle = 1.0e6 / (double)h->clock_khz;
  for (int f = 0; f < F; ++f) per_feature_ns[f] = (double)cycles[f] * ns_per_cycle;
  return EB_OK;
}

int eb_kernel_timing(eb_handle* h, int enable) {
  if (!h) return fail(EB_ERR_INVALID_ARG, "null handle");
  DeviceGuard guard(h->device);
  if (enable && h->t0.empty()) {
    h->t0.resize(kTimeRing);
    h->t1.resize(kTimeRing);
    for (int i = 0; i < kTimeRing; ++i) {
      EB_CUDA(cudaEventCreate(&h->t0[i]));
      EB_CUDA(cudaEventCreate(&h->t1[i]));
    }
  }
  h->time_kernels = enable != 0;
  h->t_count = 0;
  return EB_OK;
}

int eb_kernel_times(eb_handle* h, float* ms, int cap, int* count) {
  if (!h || !count || (cap > 0 && !ms)) return fail(EB_ERR_INVALID_ARG, "null argument");
  DeviceGuard guard(h->device);
  int n = 0;
  for (int i = 0; i < h->t_count && n < cap; ++i) {
    EB_CUDA(cudaEventSynchronize(h->t1[i]));
    EB_CUDA(cudaEventElapsedTime(&ms[n], h->t0[i], h->t1[i]));
    ++n;
  }
  h->t_count = 0;
  *count = n;
  return EB_OK;
}

int eb_check_status(eb_handle* h, void* workspace, void* stream) {
  if (!h || !workspace) return fail(EB_ERR_INVALID_ARG, "null argument");
  DeviceGuard guard(h->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  WsHeader hdr;
  EB_CUDA(cudaMemcpyAsync(&hdr, workspace, sizeof(hdr), cudaMemcpyDeviceToHost, st));
  EB_CUDA(cudaStreamSynchronize(st));
  if (hdr.status & kStatusBadIndex)
    return fail(EB_ERR_BAD_INPUT, "an index outside [0, rows) was met and skipped%s",
                (hdr.status & kStatusBadOffsets) ? "; offsets were not a non-decreasing sequence inside [0, nnz]" : "");
  if (hdr.status & kStatusBadOffsets)
    return fail(EB_ERR_BAD_INPUT, "offsets were not a non-decreasing sequence inside [0, nnz]; they were clamped");
  return EB_OK;
}

int eb_last_binding(eb_handle* h, void* workspace, void* stream, int32_t* bags_per_tile) {
  if (!h || !workspace || !bags_per_tile) return fail(EB_ERR_INVALID_ARG, "null argument");
  DeviceGuard guard(h->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const WsLayout L = ws_layout(h->num_features);
  EB_CUDA(cudaMemcpyAsync(bags_per_tile, static_cast<char*>(workspace) + L.bags_per_tile,
                          sizeof(int32_t) * h->num_features, cudaMemcpyDeviceToHost, st));
  EB_CUDA(cudaStreamSynchronize(st));
  return EB_OK;
}

int eb_fill_table(void* table, int64_t rows, int32_t dim, int32_t table_dtype, uint64_t seed, float std, int device,
                  void* stream) {
  if (!table || rows <= 0 || dim <= 0) return fail(EB_ERR_INVALID_ARG, "invalid table");
  if (table_dtype != EB_F32 && table_dtype != EB_F16) return fail(EB_ERR_INVALID_ARG, "invalid dtype %d", table_dtype);
  DeviceGuard guard(device);
  if (!guard.ok) return fail(EB_ERR_CUDA, "cannot select device %d", device);
  EB_CUDA(launch_fill(table, rows * (int64_t)dim, table_dtype, seed, std, static_cast<cudaStream_t>(stream)));
  return EB_OK;
}

int eb_place_columns(const float* src, float* dst, int64_t rows, int64_t dst_ld, int32_t num_segments,
                     const void* segments, int device, void* stream) {
  if (rows < 0 || num_segments < 0) return fail(EB_ERR_INVALID_ARG, "negative size");
  if (rows == 0 || num_segments == 0) return EB_OK;
  if (!src || !dst || !segments) return fail(EB_ERR_INVALID_ARG, "null pointer");
  DeviceGuard guard(device);
  if (!guard.ok) return fail(EB_ERR_CUDA, "cannot select device %d", device);
  const int vec_ok = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0 && dst_ld % 4 == 0;
  EB_CUDA(launch_place(src, dst, rows, dst_ld, num_segments, segments, vec_ok, static_cast<cudaStream_t>(stream)));
  return EB_OK;
}

int eb_offsets_from_lengths(const void* lengths, void* offsets, int32_t num_features, int64_t batch, int index_dtype,
                            int device, void* stream) {
  if (num_features < 0 || batch < 0) return fail(EB_ERR_INVALID_ARG, "negative size");
  if (index_dtype != EB_I32 && index_dtype != EB_I64) return fail(EB_ERR_INVALID_ARG, "bad index_dtype %d", index_dtype);
  if (num_features == 0) return EB_OK;
  if (!offsets || (batch > 0 && !lengths)) return fail(EB_ERR_INVALID_ARG, "null pointer");
  if (num_features > 65535 * 32768) return fail(EB_ERR_TOO_LARGE, "too many features");
  DeviceGuard guard(device);
  if (!guard.ok) return fail(EB_ERR_CUDA, "cannot select device %d", device);
  EB_CUDA(launch_lengths(lengths, offsets, num_features, batch, index_dtype == EB_I64, static_cast<cudaStream_t>(stream)));
  return EB_OK;
}

int eb_parse_bags(const char* text, size_t text_len, int64_t batch, int32_t* values_out, int64_t values_cap,
                  int32_t* offsets_out, int64_t* nnz_out) {
  if ((!text && text_len) || batch < 0 || !offsets_out || !nnz_out || (values_cap > 0 && !values_out))
    return fail(EB_ERR_INVALID_ARG, "invalid argument");
  // One bag per '\n'-separated line.  Inside a line every non-digit byte ends a
  // number (so "3,,5" holds 3, 0, 5) and a non-empty line's tail is a number
  // too; an empty line is an empty bag.
  int64_t n = 0, line = 0;
  size_t pos = 0;
  offsets_out[0] = 0;
  while (line < batch) {
    int64_t cur = 0;
    bool any = false;
    while (pos < text_len && text[pos] != '\n') {
      const unsigned char ch = (unsigned char)text[pos++];
      any = true;
      if (ch >= '0' && ch <= '9') {
        cur = cur * 10 + (ch - '0');
      } else {
        if (n >= values_cap) return fail(EB_ERR_WORKSPACE_TOO_SMALL, "values_out holds %lld entries, more needed", (long long)values_cap);
        values_out[n++] = (int32_t)cur;
        cur = 0;
      }
    }
    if (any) {
      if (n >= values_cap) return fail(EB_ERR_WORKSPACE_TOO_SMALL, "values_out holds %lld entries, more needed", (long long)values_cap);
      values_out[n++] = (int32_t)cur;
    }
    if (pos < text_len) ++pos;  // skip '\n'
    ++line;
    if (n > 0x7fffffff) return fail(EB_ERR_TOO_LARGE, "more than 2^31 indices in one feature");
    offsets_out[line] = (int32_t)n;
  }
  *nnz_out = n;
  return EB_OK;
}

}  // extern "C"
