// eb_warp_kernel: the warp-per-bag schedule (EB_SCHED_WARP) as a kernel of its own.
//
// Long, evenly sized bags over tables whose hot rows sit in L1/L2 are bound by instruction count and by L1
// throughput, and register spills travel through that same L1.  The loop below is therefore as lean as the
// reference's ws::SparseSegmentReduceCore (examples/csrc/include/warp_per_sample_kernel.cuh:48-60: about 11
// instructions per 512-byte row at 32 registers): scalars only, no votes, no zero-filled buffers.  It lives in its
// own kernel, built for 8 CTAs per SM, because inside the fused kernel it degraded the register allocation of
// every other schedule (and theirs degraded its own), and as a plain grid (one CTA per 8 consecutive bags of a
// feature, found through the second prefix sum the binding kernel writes) because tickets, chunks and tile
// state cost registers that the row buffers need.  Input sanitising (per bag) and output addressing (single
// matrix or peers) follow eb_fused_kernel.
#pragma once
#include "eb_common.cuh"
#include "eb_schedules.cuh"

namespace ebk {

template <int V>
struct AccPack {
  float v[V];
};

// U consecutive indices with one load (vp is aligned to U indices).
template <int U, bool IDX64>
__device__ __forceinline__ void load_index_vector(const typename IdxOf<IDX64>::type* vp, typename IdxOf<IDX64>::type (&idx)[U]) {
  if constexpr (!IDX64 && U == 4) {
    const int4 q = __ldg(reinterpret_cast<const int4*>(vp));
    idx[0] = q.x; idx[1] = q.y; idx[2] = q.z; idx[3] = q.w;
  } else if constexpr (!IDX64 && U == 2) {
    const int2 q = __ldg(reinterpret_cast<const int2*>(vp));
    idx[0] = q.x; idx[1] = q.y;
  } else if constexpr (IDX64 && U == 2) {
    const longlong2 q = __ldg(reinterpret_cast<const longlong2*>(vp));
    idx[0] = q.x; idx[1] = q.y;
  } else {
#pragma unroll
    for (int u = 0; u < U; ++u) idx[u] = __ldg(vp + u);
  }
}

// Sum of the rows vp[0 .. n): a slot's own contiguous run of the bag's entries.  Entries up to the first position
// aligned to U indices and the ragged end go one at a time; in between every macro-step fetches its U indices with one
// vector load.  A lane whose indices are all valid loads unconditionally; a lane that meets a bad index takes the
// careful branch on its own (no warp-wide vote, so slots may run different numbers of steps).
template <typename T, int V, int U, bool IDX64>
__device__ __forceinline__ AccPack<V> bag_sum(const typename IdxOf<IDX64>::type* vp, const char* tcol,
                                              unsigned row_bytes, unsigned long long rows, int n, uint32_t* status) {
  using Ops = RowOps<T, V>;
  using IdxT = typename IdxOf<IDX64>::type;
  AccPack<V> a;
  zero_vals<V>(a.v);
  const unsigned rows32 = rows > 0x80000000ull ? 0x80000000u : (unsigned)rows;
  auto one = [&](IdxT ix) {
    bool ok;
    if constexpr (IDX64) ok = (unsigned long long)ix < rows;
    else ok = (unsigned)ix < rows32;
    if (ok) {
      if constexpr (IDX64) Ops::add(a.v, Ops::load(tcol + ix * (long long)row_bytes));
      else Ops::add(a.v, Ops::load(tcol + (unsigned long long)(unsigned)ix * row_bytes));
    } else {
      flag(status, kStatusBadIndex);
    }
  };
  int head = (int)((U - (reinterpret_cast<uintptr_t>(vp) / sizeof(IdxT)) % U) % U);
  head = head < n ? head : n;
  for (int u = 0; u < head; ++u) one(__ldg(vp + u));
  vp += head;
  n -= head;
  const int n_full = n / U;
  for (int i = 0; i < n_full; ++i) {
    IdxT idx[U];
    load_index_vector<U, IDX64>(vp, idx);
    vp += U;
    bool valid = true;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if constexpr (IDX64) valid = valid && (unsigned long long)idx[u] < rows;
      else valid = valid && (unsigned)idx[u] < rows32;
    }
    if (valid) {
      typename Ops::Raw rows_[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if constexpr (IDX64) rows_[u] = Ops::load(tcol + idx[u] * (long long)row_bytes);
        else rows_[u] = Ops::load(tcol + (unsigned long long)(unsigned)idx[u] * row_bytes);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) Ops::add(a.v, rows_[u]);
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) one(idx[u]);
    }
  }
  const int tail = n - n_full * U;
  for (int u = 0; u < tail; ++u) one(__ldg(vp + u));  // ragged end, one entry at a time
  return a;
}

// One bag, one warp: the warp's R slots each take a contiguous run of ceil(len / R) entries.
template <typename T, int V, int U, bool IDX64>
__device__ __forceinline__ void bag_warp(const FeatStatic& fs, const char* values, int64_t s, int64_t e, char* orow,
                                         int out_vec, int out_dt, uint32_t* status, int lane) {
  const int lgG = fs.lg_group, G = 1 << lgG, lgR = 5 - lgG;
  const int r = lane >> lgG, cl = lane & (G - 1);
  const int len = (int)(e - s);
  const int run = (len + (1 << lgR) - 1) >> lgR;
  const int first = min(r * run, len);
  const int n = min(run, len - first);
  const typename IdxOf<IDX64>::type* vp = reinterpret_cast<const typename IdxOf<IDX64>::type*>(values) + s + first;
  for (int xc = 0; xc < fs.nx; ++xc) {
    const int cs = (xc * G + cl) * V;
    const bool col_ok = cs < fs.dim;
    AccPack<V> a;
    if (col_ok) {
      a = bag_sum<T, V, U, IDX64>(vp, fs.table + (size_t)cs * sizeof(T), (unsigned)fs.row_bytes,
                                  (unsigned long long)fs.rows, n, status);
    } else {
      zero_vals<V>(a.v);
    }
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      if (d >= G) {
#pragma unroll
        for (int k = 0; k < V; ++k) a.v[k] += __shfl_xor_sync(kFull, a.v[k], d);
      }
    }
    if (r == 0 && col_ok) store_vals<V>(orow + ((size_t)cs << (out_dt ? 1 : 2)), a.v, out_vec, out_dt);  // an empty bag stores zeros
  }
}

constexpr int kWarpKernelOccupancy = 8;

// Plain grid: CTA t pools 8 consecutive bags (one per warp) of the feature that the binding kernel's second
// prefix sum maps t to.  Nothing else is alive in a warp besides its bag: no tickets, no chunks.
template <bool TIMING>
__global__ void __launch_bounds__(kCtaThreads, kWarpKernelOccupancy) eb_warp_kernel(LaunchArgs a) {
  const int lane = threadIdx.x & 31;
  const int F = a.num_features;
  const WsLayout L = ws_layout(F);
  WsHeader* hdr = reinterpret_cast<WsHeader*>(a.ws + L.header);
  const int32_t* prefix = reinterpret_cast<const int32_t*>(a.ws + L.cta_prefix);
  const uint32_t t = blockIdx.x;
  if (t >= hdr->cta_tiles) return;
  int lo = 0, hi = F;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if ((uint32_t)__ldg(prefix + mid) <= t) lo = mid; else hi = mid;
  }
  const int f = __ldg(reinterpret_cast<const int32_t*>(a.ws + L.order) + lo);
  int64_t tile = (int64_t)(t - (uint32_t)__ldg(prefix + lo));
  if (a.peer_spread) tile = spread_tile(tile, kWarpsPerCta, a.peer_spread, a.rows_per_peer);
  const int64_t bag = tile * kWarpsPerCta + (threadIdx.x >> 5);
  if (bag >= a.batch) return;
  const FeatStatic fs = a.feats[f];
  const FeatDyn fd = reinterpret_cast<const FeatDyn*>(a.ws + L.dyn)[f];
  long long c0 = 0;
  if (TIMING) c0 = clock64();

  // this bag's entries, forced inside [0, nnz] and non-negative in length
  const bool idx64 = a.idx64 != 0;
  int64_t s = load_index(fd.offsets, bag, idx64);
  int64_t e = (!a.has_end && bag + 1 >= a.batch) ? fd.nnz : load_index(fd.offsets, bag + 1, idx64);
  const int64_t s0 = s, e0 = e;
  s = clamp_off(s, fd.nnz);
  e = clamp_off(e, fd.nnz);
  if (e < s) e = s;
  if (e - s > 0x3fffffff) e = s + 0x3fffffff;
  if ((s != s0 || e != e0) && lane == 0) flag(&hdr->status, kStatusBadOffsets);

  const int es_shift = a.out_dtype ? 1 : 2;
  char* orow;
  if (a.rows_per_peer == 0) {
    orow = reinterpret_cast<char*>(a.out) + ((bag * a.out_ld + fs.col_off) << es_shift);
  } else {
    const int64_t d = bag / a.rows_per_peer;
    orow = reinterpret_cast<char*>(hdr->peer_out[d]) + (((bag - d * a.rows_per_peer) * a.out_ld + fs.col_off) << es_shift);
  }
  int out_vec = (a.out_vec == 2 && (fs.col_off & 7) == 0) ? 2 : ((a.out_vec != 0 && (fs.col_off & 3) == 0) ? 1 : 0);
  if (a.chunks > 0 && a.own_out != nullptr) {
    // chunked order: rows for this rank and its direct destinations go straight to the destination's block (see
    // LaunchArgs::own_out)
    const int64_t d = bag / a.dest_rows;
    int hop = (int)d - a.own_rank;
    hop = hop < 0 ? hop + a.world : hop;
    if (hop <= a.direct_hops) {
      const int col = a.own_col + fs.col_off;
      orow = reinterpret_cast<char*>(hdr->peer_out[d]) + (((bag - d * a.dest_rows) * a.own_ld + col) << es_shift);
      out_vec = (a.own_vec == 2 && (col & 7) == 0) ? 2 : ((a.own_vec != 0 && (col & 3) == 0) ? 1 : 0);
    }
  }
  uint32_t* status = &hdr->status;
  const bool u2 = fs.unroll <= 2;  // two or four rows per lane in flight
  if (idx64) {
    if (fs.dtype == 1) bag_warp<__half, 8, 2, true>(fs, fd.values, s, e, orow, out_vec, a.out_dtype, status, lane);
    else bag_warp<float, 4, 2, true>(fs, fd.values, s, e, orow, out_vec, a.out_dtype, status, lane);
  } else if (fs.dtype == 1) {
    if (u2) bag_warp<__half, 8, 2, false>(fs, fd.values, s, e, orow, out_vec, a.out_dtype, status, lane);
    else bag_warp<__half, 8, 4, false>(fs, fd.values, s, e, orow, out_vec, a.out_dtype, status, lane);
  } else {
    if (u2) bag_warp<float, 4, 2, false>(fs, fd.values, s, e, orow, out_vec, a.out_dtype, status, lane);
    else bag_warp<float, 4, 4, false>(fs, fd.values, s, e, orow, out_vec, a.out_dtype, status, lane);
  }
  if (TIMING) {
    __syncwarp();
    const long long c1 = clock64();
    if (lane == 0) atomicAdd(reinterpret_cast<unsigned long long*>(a.ws + L.feat_ns) + f, (unsigned long long)(c1 - c0));
  }
}

}  // namespace ebk
