// eb_longbag_kernel: pools the bags the fused kernel handed over because one warp would take too long over them
// (LaunchArgs::long_bytes; the list lives in the workspace, see LongBagList in eb_common.cuh).
//
// It is this library's block-per-bag schedule, and more: the counterpart of the reference's mbs::
// SparseSegmentReduceCore (examples/csrc/include/multi_block_per_sample_kernel.cuh:17-112), which splits long
// bags into tiles over many blocks and combines them with atomicAdd into an output nobody zeroed.  Here a bag is
// cut into segments of about 128 KB of rows, every warp of a small persistent grid draws segments by ticket and
// pools one with the lean loop of eb_warp_kernel, writes the segment's partial sum to the workspace, and the warp
// that completes a bag's LAST segment adds the bag's partials in segment order and stores the row: no atomics on
// the data, the same bits on every run, nothing to zero beforehand.  The only cross-warp communication is one
// counter per bag (threadfence + atomicAdd, the "last block" pattern); nobody waits for anybody.
#pragma once
#include "eb_common.cuh"
#include "eb_schedules.cuh"
#include "eb_warp.cuh"

namespace ebk {

constexpr int kLongSegBytes = 128 * 1024;  // rows a segment gathers, about
constexpr int kLongBagCtasPerSm = 2;

// Segments of a listed bag: as many as its length asks for, capped per bag and by what is left of the pool.
struct LongPlan {
  int seg_len;    // entries per segment
  int nseg;
  int pool_off;   // first float of the bag's partials in the pool (nseg x dim floats); unused when nseg == 1
};

template <bool TIMING>
__global__ void __launch_bounds__(kCtaThreads, kLongBagCtasPerSm) eb_longbag_kernel(LaunchArgs a) {
  const int lane = threadIdx.x & 31;
  const int F = a.num_features;
  const WsLayout L = ws_layout(F);
  WsHeader* hdr = reinterpret_cast<WsHeader*>(a.ws + L.header);
  LongBagList* ll = reinterpret_cast<LongBagList*>(a.ws + L.long_list);
  float* pool = reinterpret_cast<float*>(a.ws + L.long_pool);
  const int nbags = (int)min(ll->count, (uint32_t)kMaxLongBags);
  if (nbags == 0) return;

  // every CTA derives the same plan from the list: thread i plans bag i, one thread turns counts into prefix sums
  __shared__ LongPlan plan[kMaxLongBags];
  __shared__ int seg_prefix[kMaxLongBags + 1];
  for (int i = threadIdx.x; i < nbags; i += kCtaThreads) {
    const LongBag lb = ll->item[i];
    const FeatStatic fs = a.feats[lb.feat];
    const long long len = lb.end - lb.begin;
    long long seg_len = kLongSegBytes / fs.row_bytes;
    seg_len = seg_len < 64 ? 64 : seg_len;
    long long nseg = (len + seg_len - 1) / seg_len;
    if (nseg > kMaxLongSegments) {
      nseg = kMaxLongSegments;
      seg_len = (len + nseg - 1) / nseg;
      nseg = (len + seg_len - 1) / seg_len;
    }
    plan[i].seg_len = (int)seg_len;
    plan[i].nseg = (int)(nseg < 1 ? 1 : nseg);
    plan[i].pool_off = 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int segs = 0, used = 0;
    for (int i = 0; i < nbags; ++i) {
      const int dim = a.feats[ll->item[i].feat].dim;
      int nseg = plan[i].nseg;
      if (nseg > 1 && (long long)used + (long long)nseg * dim > kLongPoolFloats) {
        // the pool is nearly full: fewer, longer segments (one segment needs no partial at all)
        const long long len = ll->item[i].end - ll->item[i].begin;
        nseg = (kLongPoolFloats - used) / dim;
        nseg = nseg < 2 ? 1 : nseg;
        const long long seg_len = (len + nseg - 1) / nseg;
        plan[i].seg_len = (int)(seg_len > 0x3fffffff ? 0x3fffffff : seg_len);
        nseg = (int)((len + plan[i].seg_len - 1) / plan[i].seg_len);
        plan[i].nseg = nseg < 1 ? 1 : nseg;
      }
      plan[i].pool_off = used;
      if (plan[i].nseg > 1) used += plan[i].nseg * dim;
      seg_prefix[i] = segs;
      segs += plan[i].nseg;
    }
    seg_prefix[nbags] = segs;
  }
  __syncthreads();
  const uint32_t total = (uint32_t)seg_prefix[nbags];
  const bool idx64 = a.idx64 != 0;

  uint32_t t = 0;
  if (lane == 0) t = atomicAdd(&ll->seg_ticket, 1u);
  t = __shfl_sync(kFull, t, 0);
  while (t < total) {
    int lo = 0, hi = nbags;  // seg_prefix[lo] <= t < seg_prefix[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if ((uint32_t)seg_prefix[mid] <= t) lo = mid; else hi = mid;
    }
    const int bag_i = lo, k = (int)(t - (uint32_t)seg_prefix[lo]);
    const LongBag lb = ll->item[bag_i];
    const LongPlan pl = plan[bag_i];
    const FeatStatic fs = a.feats[lb.feat];
    const FeatDyn fd = reinterpret_cast<const FeatDyn*>(a.ws + L.dyn)[lb.feat];
    long long c0 = 0;
    if (TIMING) c0 = clock64();
    const int64_t s = lb.begin + (int64_t)k * pl.seg_len;
    const int64_t e = (s + pl.seg_len < lb.end) ? s + pl.seg_len : lb.end;

    // where the bag's row goes (as in eb_warp_kernel)
    const int es_shift = a.out_dtype ? 1 : 2;
    char* orow;
    if (a.rows_per_peer == 0) {
      orow = reinterpret_cast<char*>(a.out) + ((lb.bag * a.out_ld + fs.col_off) << es_shift);
    } else {
      const int64_t d = lb.bag / a.rows_per_peer;
      orow = reinterpret_cast<char*>(hdr->peer_out[d]) + (((lb.bag - d * a.rows_per_peer) * a.out_ld + fs.col_off) << es_shift);
    }
    const int out_vec = (a.out_vec == 2 && (fs.col_off & 7) == 0) ? 2 : ((a.out_vec != 0 && (fs.col_off & 3) == 0) ? 1 : 0);
    // one segment: the row itself; several: this segment's partial, fp32, 16-byte aligned whenever dim allows
    float* part = pool + pl.pool_off + (size_t)k * fs.dim;
    const bool direct = pl.nseg == 1;
    char* dst = direct ? orow : reinterpret_cast<char*>(part);
    const int dst_vec = direct ? out_vec : (((pl.pool_off + k * fs.dim) & 7) == 0 ? 2 : (((pl.pool_off + k * fs.dim) & 3) == 0 ? 1 : 0));
    const int dst_dt = direct ? a.out_dtype : 0;
    uint32_t* status = &hdr->status;
    if (idx64) {
      if (fs.dtype == 1) bag_warp<__half, 8, 4, true>(fs, fd.values, s, e, dst, dst_vec, dst_dt, status, lane);
      else bag_warp<float, 4, 4, true>(fs, fd.values, s, e, dst, dst_vec, dst_dt, status, lane);
    } else if (fs.dtype == 1) {
      bag_warp<__half, 8, 4, false>(fs, fd.values, s, e, dst, dst_vec, dst_dt, status, lane);
    } else {
      bag_warp<float, 4, 4, false>(fs, fd.values, s, e, dst, dst_vec, dst_dt, status, lane);
    }
    if (!direct) {
      // publish the partial; whoever completes the bag adds the partials in segment order and stores the row
      __threadfence();
      __syncwarp();
      uint32_t done = 0;
      if (lane == 0) done = atomicAdd(&ll->done[bag_i], 1u) + 1u;
      done = __shfl_sync(kFull, done, 0);
      if (done == (uint32_t)pl.nseg) {
        __threadfence();
        const float* p0 = pool + pl.pool_off;
        for (int c = lane; c < fs.dim; c += 32) {
          float sum = 0.f;
          for (int q = 0; q < pl.nseg; ++q) sum += __ldcg(p0 + (size_t)q * fs.dim + c);
          float one[1] = {sum};
          store_vals<1>(orow + ((size_t)c << es_shift), one, 0, a.out_dtype);
        }
      }
    }
    if (TIMING) {
      __syncwarp();
      const long long c1 = clock64();
      if (lane == 0) atomicAdd(reinterpret_cast<unsigned long long*>(a.ws + L.feat_ns) + lb.feat, (unsigned long long)(c1 - c0));
    }
    uint32_t tn = 0;
    if (lane == 0) tn = atomicAdd(&ll->seg_ticket, 1u);
    t = __shfl_sync(kFull, tn, 0);
  }
}

}  // namespace ebk
