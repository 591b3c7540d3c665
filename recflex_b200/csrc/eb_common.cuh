// Shared declarations of the fused embedding-bag library: the device-side
// feature descriptors, the per-call scratch ("workspace") layout and the
// launch argument block.  Host and device code both include this file.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ebk {

constexpr int kCtaThreads = 256;        // one value for every feature, as in the reference (codegen.py:24-26)
constexpr int kWarpsPerCta = kCtaThreads / 32;
constexpr int kMaxOccupancy = 8;        // 2048 threads per SM / 256
constexpr int kBindThreads = 1024;
constexpr int kPipeCellBytes = 512;      // one ring cell: 32 lanes x 16 bytes
constexpr int kPipeMaxCells = 16;        // unroll x stages of the deepest pipelined variant
// Macro-steps the pipelined schedule keeps in flight, by unroll (rows per macro-step); the ring holds unroll x depth
// cells of 512 bytes per warp.  Batches with 64-bit indices always run the unroll-4 variant.
__host__ __device__ constexpr inline int pipe_depth(int unroll) {
  return unroll <= 2 ? 4 : (unroll == 4 ? 3 : 2);  // 6 and 8: two macro-steps
}
__host__ __device__ constexpr inline int pipe_cells(int unroll) {
  const int u = unroll <= 2 ? 2 : (unroll == 4 ? 4 : (unroll == 6 ? 6 : 8));
  const int own = u * pipe_depth(u), i64 = 4 * pipe_depth(4);
  return own > i64 ? own : i64;
}
constexpr int kMaxLptFeatures = 2048;   // features beyond this keep their input order

// status bits written by the kernels (never a trap)
constexpr uint32_t kStatusBadIndex = 1u;    // an index outside [0, rows) was skipped
constexpr uint32_t kStatusBadOffsets = 2u;  // offsets were clamped to a non-decreasing sequence inside [0, nnz]

// Static per-feature descriptor; lives in device memory owned by the handle.
struct __align__(16) FeatStatic {
  const char* table;     // row-major [rows, dim]
  int64_t rows;
  int32_t dim;
  int32_t col_off;       // first output column of this feature
  int32_t row_bytes;     // dim * sizeof(element)
  int32_t dtype;         // 0 = f32, 1 = f16
  int32_t kind;          // EB_SCHED_* after AUTO resolution
  int32_t unroll;        // 1, 2, 4, 8
  int32_t lg_group;      // log2(lanes that share one row)
  int32_t nx;            // column passes (rows wider than 32 lanes' worth)
  int32_t vec;           // 1 = 16-byte lane loads; 0 = element-wise fallback
  int32_t bags_per_tile; // 0 = decided per batch on the device
  int32_t pad_[2];
};
static_assert(sizeof(FeatStatic) == 64, "FeatStatic must stay 64 bytes");

// Per-call, per-feature inputs.
struct __align__(8) FeatDyn {
  const char* values;
  const char* offsets;
  int64_t nnz;      // end of the feature's index list (the last boundary; offsets are clamped to [0, nnz])
  int64_t work;     // indices this call pools: nnz minus the first boundary (written by the binding kernel)
};
static_assert(sizeof(FeatDyn) == 32, "FeatDyn must stay 32 bytes");

constexpr int kMaxPeers = 16;            // ranks whose output matrices one launch can store into

// First 256 bytes of the workspace.
struct __align__(128) WsHeader {
  uint32_t ticket;        // next warp tile
  uint32_t total_tiles;
  uint32_t cta_ticket;    // reserved (eb_warp_kernel runs a plain grid and draws no tickets); kept zero
  uint32_t cta_tiles;     // CTAs of eb_warp_kernel that have work (features on the warp-per-bag schedule)
  uint32_t status;
  uint32_t pad_[27];
  float* peer_out[kMaxPeers];  // peer mode: output matrix of every rank (this GPU's view of their memory)
};
static_assert(sizeof(WsHeader) == 256, "WsHeader must stay 256 bytes");

constexpr int kMaxChunks = 64;           // batch chunks of the chunked ticket order

// Chunked order: done[k] counts the finished tiles of chunk k (zeroed by the binding kernel of every call);
// flag[k] receives the call's epoch when the chunk's last tile is done.  Epochs only grow, so the flags are never
// reset and a waiter compares with "at least this call's epoch".
struct __align__(128) ChunkSync {
  uint32_t done[kMaxChunks];
  uint32_t flag[kMaxChunks];
};
static_assert(sizeof(ChunkSync) == 512, "ChunkSync must stay 512 bytes");

// Long bags: a bag whose rows add up to LaunchArgs::long_bytes or more is not pooled by the warp that meets it
// (it would be that warp's, and the kernel's, tail); the warp appends it to this list and eb_longbag_kernel, launched
// after the fused kernel, pools every listed bag with many warps: the bag is cut into segments, every segment's
// partial sum goes to `long_pool`, and the warp that finishes a bag's last segment adds the partials in segment
// order (no atomics on the data, same result on every run).  A full list simply stops accepting bags.
constexpr int kMaxLongBags = 256;
constexpr int kMaxLongSegments = 128;          // per bag
constexpr int kLongPoolFloats = 256 * 1024;    // 1 MB of partial sums

struct __align__(16) LongBag {
  int32_t feat;
  int32_t pad_;
  int64_t bag;     // position in the batch
  int64_t begin;   // entries [begin, end) of the feature's index list, already validated
  int64_t end;
};

struct __align__(128) LongBagList {
  uint32_t count;        // bags appended (may exceed kMaxLongBags: the excess was pooled in place)
  uint32_t seg_ticket;   // next segment to pool
  uint32_t pad_[30];
  uint32_t done[kMaxLongBags];  // finished segments per bag
  LongBag item[kMaxLongBags];
};

// Host/device view of where each array sits inside the workspace.  The long-bag sections come last: a caller that
// keeps long-bag splitting off (long_bytes == 0) may pass a workspace that ends at `long_list`.
struct WsLayout {
  size_t header, tile_prefix, cta_prefix, order, bags_per_tile, dyn, feat_ns, chunk_sync, long_list, long_pool, total;
};

__host__ __device__ constexpr inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

__host__ __device__ constexpr inline WsLayout ws_layout(int F) {
  WsLayout l{};
  size_t o = 0;
  l.header = o;        o += sizeof(WsHeader);
  l.tile_prefix = o;   o = align_up(o + sizeof(int32_t) * (size_t)(F + 1), 128);
  l.cta_prefix = o;    o = align_up(o + sizeof(int32_t) * (size_t)(F + 1), 128);
  l.order = o;         o = align_up(o + sizeof(int32_t) * (size_t)F, 128);
  l.bags_per_tile = o; o = align_up(o + sizeof(int32_t) * (size_t)F, 128);
  l.dyn = o;           o = align_up(o + sizeof(FeatDyn) * (size_t)F, 128);
  l.feat_ns = o;       o = align_up(o + sizeof(unsigned long long) * (size_t)F, 128);
  l.chunk_sync = o;    o += sizeof(ChunkSync);
  l.long_list = o;     o += sizeof(LongBagList);
  l.long_pool = o;     o += sizeof(float) * (size_t)kLongPoolFloats;
  l.total = o;
  return l;
}

// Everything a launch needs, passed by value as the kernel parameter.
struct LaunchArgs {
  const FeatStatic* feats;
  char* ws;               // workspace base
  const char* packed_values;   // packed mode only
  const char* packed_offsets;  // packed mode only: [F, batch + 1]
  float* out;
  int64_t out_ld;
  int64_t batch;
  int32_t num_features;
  int32_t idx64;          // values/offsets are int64 (else int32)
  int32_t has_end;        // offsets carry batch + 1 entries
  int32_t packed;
  int32_t out_vec;        // out base and out_ld allow stores of four (1) or eight (2) aligned elements
  int32_t out_dtype;      // output element type: 0 = fp32, 1 = bfloat16, 2 = binary16 (out_ld counts elements)
  int32_t warps_total;    // persistent warps of the fused kernel (for tile sizing)
  int32_t ring_bytes;     // shared memory per warp for the pipelined schedule's ring (0 when no feature uses it)
  int32_t peer_spread;    // peer mode: number of ranks to deal a feature's consecutive tiles over (0 = batch order)
  int64_t long_bytes;     // bags that gather at least this many bytes go to eb_longbag_kernel (0 = pooled in place)
  // chunked ticket order (chunks > 0; for exchanges that ship finished chunks while later ones are pooled): the
  // batch is seen as `world` runs of dest_rows bags (one per destination rank), each cut into `chunks` pieces of
  // chunk_rows bags; the tickets cover piece 0 of every run for every feature, then piece 1, ...  A tile never
  // straddles two pieces (the binding kernel makes bags_per_tile divide chunk_rows).
  int32_t chunks;
  uint32_t epoch;         // value written to a chunk's flag when its last tile is done
  int64_t chunk_rows;
  int64_t dest_rows;
  // chunked order: rows for this rank itself (destination own_rank) and for the direct_hops ranks to its right skip
  // the send buffer: the kernel stores them straight into the destination's result block, peer_out[d] ([dest_rows,
  // own_ld] elements, the same geometry on every rank) at columns own_col + the feature's column; own_out null = no
  // such shortcut.  The other destinations' rows go to the send buffer and leave by copy.
  float* own_out;
  int64_t own_ld;
  int32_t own_col;
  int32_t own_rank;
  int32_t own_vec;        // like out_vec, for the direct destinations' blocks
  int32_t direct_hops;
  int32_t world;
  int32_t pad2_;
  // peer mode (rows_per_peer > 0): sample b is stored to peer_out[b / rows_per_peer], row b % rows_per_peer
  int64_t rows_per_peer;
  float* peer_out[kMaxPeers];
};

// Peer mode: which slice of the batch the i-th tile (of `n` bags) of a feature pools.  In batch order every
// GPU of the node would store to rank 0's rows first, then rank 1's, ...: the receivers' links take turns being
// oversubscribed.  Dealing consecutive tiles round-robin over the destination ranks keeps all links busy at once.
// The mapping is a bijection on [0, batch / n); it needs tiles that do not straddle two ranks' rows.
__host__ __device__ inline int64_t spread_tile(int64_t tile, int n, int world, int64_t rows_per_peer) {
  if (world <= 1 || rows_per_peer <= 0 || rows_per_peer > 0x7fffffff) return tile;
  const uint32_t rpp = (uint32_t)rows_per_peer, per_peer = rpp / (uint32_t)n;
  if (per_peer * (uint32_t)n != rpp) return tile;
  const uint32_t i = (uint32_t)tile, w = (uint32_t)world;
  return (int64_t)(i % w) * per_peer + i / w;
}

}  // namespace ebk
