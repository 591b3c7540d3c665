// eb_fused_kernel: persistent CTAs; every warp draws tile tickets, finds the
// ticket's feature with a 32-way search in the prefix sum that eb_bind_kernel
// (eb_bind.cuh) left in the workspace and runs that feature's schedule.
// Replaces the generated FusedKnl dispatcher
// (RecFlex/code_emitter/codegen.py:318-383).
// (Features on the warp-per-bag schedule get no tiles here: eb_warp_kernel, eb_warp.cuh, pools them.)
#pragma once
#include "eb_common.cuh"
#include "eb_schedules.cuh"

namespace ebk {

// ---------------------------------------------------------------------------
// schedule dispatch
// ---------------------------------------------------------------------------
#define EB_DISPATCH_UNROLL(FN, T, V, I64)                          \
  switch (fs.unroll) {                                             \
    case 1: FN<T, V, 1, I64>(ctx, b0, b1, lane); break;            \
    case 2: FN<T, V, 2, I64>(ctx, b0, b1, lane); break;            \
    case 4: FN<T, V, 4, I64>(ctx, b0, b1, lane); break;            \
    default: FN<T, V, 8, I64>(ctx, b0, b1, lane); break;           \
  }

#define EB_DISPATCH_DTYPE(FN, I64)                                 \
  if (fs.dtype == 1) {                                             \
    EB_DISPATCH_UNROLL(FN, __half, 8, I64)                         \
  } else {                                                         \
    EB_DISPATCH_UNROLL(FN, float, 4, I64)                          \
  }

// EB_SCHED_STREAM: the register walk.  FS: fp32 output aligned for the widest store (see walk_store).
#define EB_DISPATCH_STREAM_T(T, V, I64, FS)                                           \
  switch (fs.unroll) {                                                                \
    case 1: tile_stream<T, V, 1, I64, 0, FS>(a, ctx, b0, b1, lane, items); break;        \
    case 2: tile_stream<T, V, 2, I64, 0, FS>(a, ctx, b0, b1, lane, items); break;        \
    case 4: tile_stream<T, V, 4, I64, 0, FS>(a, ctx, b0, b1, lane, items); break;        \
    default: tile_stream<T, V, 8, I64, 0, FS>(a, ctx, b0, b1, lane, items); break;       \
  }

#define EB_DISPATCH_STREAM(I64)                                    \
  if (fs.dtype == 1) {                                             \
    if (ctx.out_dt == 0 && ctx.out_vec == 2) { EB_DISPATCH_STREAM_T(__half, 8, I64, true) } \
    else { EB_DISPATCH_STREAM_T(__half, 8, I64, false) }           \
  } else {                                                         \
    if (ctx.out_dt == 0 && ctx.out_vec >= 1) { EB_DISPATCH_STREAM_T(float, 4, I64, true) } \
    else { EB_DISPATCH_STREAM_T(float, 4, I64, false) }            \
  }

// EB_SCHED_PIPE: ring depth is tied to the unroll (pipe_depth, eb_common.cuh).
#define EB_DISPATCH_PIPE_T(T, V, I64, FS)                                                              \
  switch (fs.unroll) {                                                                                 \
    case 1:                                                                                            \
    case 2: tile_stream<T, V, 2, I64, pipe_depth(2), FS>(a, ctx, b0, b1, lane, items, ring); break;       \
    case 4: tile_stream<T, V, 4, I64, pipe_depth(4), FS>(a, ctx, b0, b1, lane, items, ring); break;       \
    case 6: tile_stream<T, V, 6, I64, pipe_depth(6), FS>(a, ctx, b0, b1, lane, items, ring); break;       \
    default: tile_stream<T, V, 8, I64, pipe_depth(8), FS>(a, ctx, b0, b1, lane, items, ring); break;      \
  }

#define EB_DISPATCH_PIPE(I64)                                      \
  if (fs.dtype == 1) {                                             \
    if (ctx.out_dt == 0 && ctx.out_vec == 2) { EB_DISPATCH_PIPE_T(__half, 8, I64, true) } \
    else { EB_DISPATCH_PIPE_T(__half, 8, I64, false) }             \
  } else {                                                         \
    if (ctx.out_dt == 0 && ctx.out_vec >= 1) { EB_DISPATCH_PIPE_T(float, 4, I64, true) } \
    else { EB_DISPATCH_PIPE_T(float, 4, I64, false) }              \
  }

// 64-bit indices are the uncommon case: every schedule kind is instantiated for
// them, but only at unroll 4 (the requested unroll is ignored).
#define EB_DISPATCH_DTYPE_U4(FN, I64)                              \
  if (fs.dtype == 1) FN<__half, 8, 4, I64>(ctx, b0, b1, lane);     \
  else FN<float, 4, 4, I64>(ctx, b0, b1, lane);

#define EB_DISPATCH_KIND64()                                       \
  if (!fs.vec) {                                                   \
    if (fs.dtype == 1) tile_warp<__half, 1, 4, true>(ctx, b0, b1, lane); \
    else tile_warp<float, 1, 4, true>(ctx, b0, b1, lane);          \
  } else if (fs.kind == 1) {                                       \
    EB_DISPATCH_DTYPE_U4(tile_group, true)                         \
  } else if (fs.kind == 3) {                                       \
    EB_DISPATCH_DTYPE_U4(tile_flat, true)                          \
  } else if (fs.kind == 4) {                                       \
    if (fs.dtype == 1) tile_stream<__half, 8, 4, true>(a, ctx, b0, b1, lane, items); \
    else tile_stream<float, 4, 4, true>(a, ctx, b0, b1, lane, items); \
  } else {                                                         \
    if (fs.dtype == 1) tile_stream<__half, 8, 4, true, pipe_depth(4)>(a, ctx, b0, b1, lane, items, ring); \
    else tile_stream<float, 4, 4, true, pipe_depth(4)>(a, ctx, b0, b1, lane, items, ring); \
  }

#define EB_DISPATCH_KIND(I64)                                      \
  if (!fs.vec) {                                                   \
    if (fs.dtype == 1) tile_warp<__half, 1, 4, I64>(ctx, b0, b1, lane); \
    else tile_warp<float, 1, 4, I64>(ctx, b0, b1, lane);           \
  } else if (fs.kind == 1) {                                       \
    EB_DISPATCH_DTYPE(tile_group, I64)                             \
  } else if (fs.kind == 3) {                                       \
    EB_DISPATCH_DTYPE(tile_flat, I64)                              \
  } else if (fs.kind == 4) {                                       \
    EB_DISPATCH_STREAM(I64)                                        \
  } else {                                                         \
    EB_DISPATCH_PIPE(I64)                                          \
  }

// One schedule at one unroll, both table dtypes, with and without the fast store.
#define EB_ONE_WALK(U, D)                                                                              \
  if (fs.dtype == 1) {                                                                                 \
    if (ctx.out_dt == 0 && ctx.out_vec == 2) tile_stream<__half, 8, U, false, D, true>(a, ctx, b0, b1, lane, items, ring);  \
    else tile_stream<__half, 8, U, false, D, false>(a, ctx, b0, b1, lane, items, ring);                   \
  } else {                                                                                             \
    if (ctx.out_dt == 0 && ctx.out_vec >= 1) tile_stream<float, 4, U, false, D, true>(a, ctx, b0, b1, lane, items, ring);   \
    else tile_stream<float, 4, U, false, D, false>(a, ctx, b0, b1, lane, items, ring);                    \
  }

// KIND / UNROLL select what the kernel holds.  0 / 0: every schedule at every unroll (any assignment, any index
// width).  KIND = EB_SCHED_STREAM (4) or EB_SCHED_PIPE (5): only that schedule (plus the element-wise fallback), at
// every unroll (UNROLL = 0) or at one; for batches with 32-bit indices whose features all agree on it.  What the
// reference reaches by generating and compiling one kernel per schedule assignment
// (RecFlex/code_emitter/codegen.py:233-262: only the schedules in use are emitted), these instantiations reach for
// the assignments that matter most: the register allocation and the instruction-cache footprint are those of the
// schedule in use, not of the largest one in the library.
template <int OCC, bool TIMING, int KIND = 0, int UNROLL = 0>
__global__ void __launch_bounds__(kCtaThreads, OCC) eb_fused_kernel(LaunchArgs a) {
  const int lane = threadIdx.x & 31;
  const int F = a.num_features;
  const WsLayout L = ws_layout(F);
  WsHeader* hdr = reinterpret_cast<WsHeader*>(a.ws + L.header);
  const int32_t* tile_prefix = reinterpret_cast<const int32_t*>(a.ws + L.tile_prefix);
  const int32_t* order = reinterpret_cast<const int32_t*>(a.ws + L.order);
  const int32_t* bpt = reinterpret_cast<const int32_t*>(a.ws + L.bags_per_tile);
  const FeatDyn* dyn = reinterpret_cast<const FeatDyn*>(a.ws + L.dyn);
  unsigned long long* feat_ns = reinterpret_cast<unsigned long long*>(a.ws + L.feat_ns);
  const uint32_t total = hdr->total_tiles;
  // chunked order (a.chunks > 0): the tickets walk the batch chunk by chunk, every feature's tiles of chunk 0
  // first, and the warp that completes a chunk's last tile publishes the chunk (see LaunchArgs)
  const uint32_t per_chunk = a.chunks > 0 ? (uint32_t)__ldg(tile_prefix + F) : total;
  // per-warp ring of the pipelined schedule (a.ring_bytes per warp when any feature uses it, else none)
  extern __shared__ __align__(16) unsigned char eb_smem[];
  unsigned char* ring = eb_smem + (threadIdx.x >> 5) * a.ring_bytes;
  // per-warp list of a chunk's non-empty bags (stream and pipe schedules)
  __shared__ int2 eb_items[kWarpsPerCta][kBagItems];
  int2* items = eb_items[threadIdx.x >> 5];

  uint32_t t = 0;
  if (lane == 0) t = atomicAdd(&hdr->ticket, 1u);
  t = __shfl_sync(kFull, t, 0);
  while (t < total) {
    // draw the next ticket now; its latency hides behind this tile
    uint32_t tn = 0;
    if (lane == 0) tn = atomicAdd(&hdr->ticket, 1u);

    uint32_t chunk = 0, tt = t;
    if (a.chunks > 0) {
      chunk = t / per_chunk;
      tt = t - chunk * per_chunk;
    }
    // The ticket's feature: the last position of the prefix sum that is <= tt.  The warp probes 32 evenly spaced
    // positions of the remaining range per round (two dependent loads for up to 1024 features, where a binary
    // search makes ten); the last round, at spacing 1, fetches the feature ids along with the prefix values.
    int lo = 0, span = F, f, k;
    uint32_t pv;
    while (true) {
      const int step = (span + 31) >> 5;
      const bool in = lane * step < span;
      const int i = lo + lane * step;
      pv = in ? (uint32_t)__ldg(tile_prefix + i) : 0xffffffffu;
      f = (in && step == 1) ? __ldg(order + i) : 0;
      k = __popc(__ballot_sync(kFull, in && pv <= tt)) - 1;  // tile_prefix[lo] <= tt, so lane 0 always votes
      lo += k * step;
      if (step == 1) break;
      span = min(step, span - k * step);
    }
    f = __shfl_sync(kFull, f, k);
    int64_t tile = (int64_t)(tt - __shfl_sync(kFull, pv, k));
    const FeatStatic fs = a.feats[f];
    const FeatDyn fd = dyn[f];
    const int n = __ldg(bpt + f);
    if (a.peer_spread) tile = spread_tile(tile, n, a.peer_spread, a.rows_per_peer);
    int64_t b0 = tile * n;
    bool own = false;  // chunked order: this tile's rows are stored straight into their destination's block
    int64_t own_d = 0;
    if (a.chunks > 0) {
      // tile of the chunk's own bag numbering [0, world * chunk_rows): destination d's run of chunk_rows bags
      // starts at batch position d * dest_rows + chunk * chunk_rows; n divides chunk_rows
      const int64_t d = b0 / a.chunk_rows;
      b0 = d * a.dest_rows + (int64_t)chunk * a.chunk_rows + (b0 - d * a.chunk_rows);
      int hop = (int)d - a.own_rank;
      hop = hop < 0 ? hop + a.world : hop;
      own = a.own_out != nullptr && hop <= a.direct_hops;
      own_d = d;
    }
    const int64_t b1 = (b0 + n) < a.batch ? (b0 + n) : a.batch;

    TileCtx ctx;
    ctx.table = fs.table;
    ctx.values = fd.values;
    ctx.offsets = fd.offsets;
    ctx.rows = fs.rows;
    ctx.nnz = fd.nnz;
    ctx.batch = a.batch;
    ctx.out = reinterpret_cast<char*>(a.out);
    ctx.out_ld = a.out_ld;
    ctx.out_dt = a.out_dtype;
    ctx.es_shift = a.out_dtype ? 1 : 2;
    ctx.peer_out = hdr->peer_out;
    ctx.rows_per_peer = a.rows_per_peer;
    ctx.col_off = fs.col_off;
    ctx.status = &hdr->status;
    if (lane == 0) items[kBagItems - 1].x = f;  // for the rare hand-over of a long bag (tile_stream)
    ctx.dim = fs.dim;
    ctx.row_bytes = fs.row_bytes;
    ctx.lg_group = fs.lg_group;
    ctx.nx = fs.nx;
    ctx.idx64 = a.idx64 != 0;
    ctx.has_end = a.has_end != 0;
    ctx.out_vec = (a.out_vec == 2 && (fs.col_off & 7) == 0) ? 2 : ((a.out_vec != 0 && (fs.col_off & 3) == 0) ? 1 : 0);
    if (own) {
      // row b of the batch is row b - d * dest_rows of destination d's block
      ctx.out = reinterpret_cast<char*>(hdr->peer_out[own_d]) - ((own_d * a.dest_rows * a.own_ld) << ctx.es_shift);
      ctx.out_ld = a.own_ld;
      ctx.col_off = a.own_col + fs.col_off;
      ctx.out_vec = (a.own_vec == 2 && (ctx.col_off & 7) == 0) ? 2 : ((a.own_vec != 0 && (ctx.col_off & 3) == 0) ? 1 : 0);
    }

    long long c0 = 0;
    if (TIMING) c0 = clock64();

    if constexpr (KIND == 0) {
      if (a.idx64) {
        EB_DISPATCH_KIND64()
      } else {
        EB_DISPATCH_KIND(false)
      }
    } else {
      if (!fs.vec) {
        if (fs.dtype == 1) tile_warp<__half, 1, 4, false>(ctx, b0, b1, lane);
        else tile_warp<float, 1, 4, false>(ctx, b0, b1, lane);
      } else if constexpr (KIND == 5 && UNROLL == 0) {
        EB_DISPATCH_PIPE(false)
      } else if constexpr (KIND == 5) {
        EB_ONE_WALK(UNROLL, pipe_depth(UNROLL))
      } else if constexpr (UNROLL == 0) {
        EB_DISPATCH_STREAM(false)
      } else {
        EB_ONE_WALK(UNROLL, 0)
      }
    }

    if (TIMING) {
      __syncwarp();
      const long long c1 = clock64();
      if (lane == 0) atomicAdd(feat_ns + f, (unsigned long long)(c1 - c0));
    }
    if (a.chunks > 0) {
      // publish: every lane's stores first, then one count per tile; the last tile of a chunk raises its flag
      __threadfence();
      __syncwarp();
      if (lane == 0) {
        ChunkSync* cs = reinterpret_cast<ChunkSync*>(a.ws + L.chunk_sync);
        const uint32_t done = atomicAdd(&cs->done[chunk], 1u) + 1u;
        if (done == per_chunk) {
          __threadfence();
          *reinterpret_cast<volatile uint32_t*>(&cs->flag[chunk]) = a.epoch;
        }
      }
    }
    t = __shfl_sync(kFull, tn, 0);
  }
}

#undef EB_ONE_WALK
#undef EB_DISPATCH_UNROLL
#undef EB_DISPATCH_DTYPE
#undef EB_DISPATCH_KIND
#undef EB_DISPATCH_KIND64
#undef EB_DISPATCH_PIPE
#undef EB_DISPATCH_PIPE_T
#undef EB_DISPATCH_STREAM
#undef EB_DISPATCH_STREAM_T
#undef EB_DISPATCH_DTYPE_U4

}  // namespace ebk
