// eb_bind_kernel: one CTA; turns the batch's per-feature index counts into
// tile sizes of equal estimated time, a longest-first feature order and an exclusive prefix sum of
// tile counts: the run-time block-to-feature binding.  Replaces the host
// GetTaskMapping (RecFlex/sched_basic_csrc/task_mapping.cu:6-18) and the
// per-schedule num_tiles / num_blocks arithmetic of the host preprocess
// (examples/csrc/*_preprocess.cu).
// eb_fill_kernel: counter-based synthetic table weights.
// eb_place_kernel: receive-side column placement of the sharded path.
// Included by exactly one translation unit (eb_launch.cu).
#pragma once
#include "eb_common.cuh"
#include "eb_schedules.cuh"

namespace ebk {

constexpr int kTilesPerWarp = 16;  // tiles a persistent warp should get (cfg3: 8 and 12 are 2.5 % slower, 24 is 4 % slower)

// ---------------------------------------------------------------------------
// block-wide exclusive scan of one int64 per thread (kBindThreads threads)
// ---------------------------------------------------------------------------
__device__ __forceinline__ long long block_excl_scan(long long v, long long* s_warp, long long& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  long long inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const long long t = __shfl_up_sync(kFull, inc, d);
    if (lane >= d) inc += t;
  }
  __syncthreads();  // s_warp may still be read from a previous call
  if (lane == 31) s_warp[warp] = inc;
  __syncthreads();
  long long w = s_warp[lane];  // kBindThreads / 32 == 32 warps
  long long winc = w;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const long long t = __shfl_up_sync(kFull, winc, d);
    if (lane >= d) winc += t;
  }
  total = __shfl_sync(kFull, winc, 31);
  const long long warp_excl = __shfl_sync(kFull, winc - w, warp);
  return warp_excl + inc - v;
}

__device__ __forceinline__ int pow2_floor(long long x) {
  if (x < 1) return 1;
  if (x > (1 << 20)) x = 1 << 20;
  return 1 << (31 - __clz((int)x));
}

// What pooling one bag of a feature costs a warp, in bytes of gathered rows: measured per-tile times of the
// pipelined walk fit (rows x (row bytes + 24) + 600) x 0.43 cycles, the 24 being a row's instructions and the 600 a
// bag's share of its chunk's start-up (offsets, indices and rows each wait for memory once per chunk of 32 bags).
// Tiles sized and ordered by gathered bytes alone made the tiles of 16-byte rows take three times as long as those
// of 512-byte rows, and come last.
constexpr long long kRowOverheadBytes = 24;
constexpr long long kBagOverheadBytes = 600;
__device__ __forceinline__ long long bag_cost(long long work, long long batch, long long row_bytes) {
  return (batch > 0 ? work * (row_bytes + kRowOverheadBytes) / batch : 0) + kBagOverheadBytes;
}

__device__ __forceinline__ int tiles_of(int64_t batch, int bpt) { return (int)((batch + bpt - 1) / bpt); }

__global__ void __launch_bounds__(kBindThreads) eb_bind_kernel(LaunchArgs a, int zero_ns) {
  static_assert(kBindThreads == 1024, "block scan assumes 32 warps");
  __shared__ long long s_warp[32];
  __shared__ float s_cost[kMaxLptFeatures];
  const int tid = threadIdx.x;
  const int F = a.num_features;
  const WsLayout L = ws_layout(F);
  WsHeader* hdr = reinterpret_cast<WsHeader*>(a.ws + L.header);
  int32_t* tile_prefix = reinterpret_cast<int32_t*>(a.ws + L.tile_prefix);
  int32_t* order = reinterpret_cast<int32_t*>(a.ws + L.order);
  int32_t* bpt = reinterpret_cast<int32_t*>(a.ws + L.bags_per_tile);
  FeatDyn* dyn = reinterpret_cast<FeatDyn*>(a.ws + L.dyn);
  unsigned long long* feat_ns = reinterpret_cast<unsigned long long*>(a.ws + L.feat_ns);
  const int isz = a.idx64 ? 8 : 4;
  const int64_t B = a.batch;
  uint32_t status = 0;

  // pass 1: index counts, packed-mode pointers, estimated cost of the batch (bag_cost).  The first boundary need not be 0
  // (a caller may pass a window of a longer offsets array): the work estimate counts the indices between the
  // first and the last boundary, while clamping uses the absolute end.
  long long carry = 0, my_cost = 0;
  for (int base = 0; base < F; base += kBindThreads) {
    const int f = base + tid;
    long long nnz = 0, work = 0;
    const char* offp = nullptr;
    if (f < F) {
      if (a.packed) {
        offp = a.packed_offsets + (int64_t)f * (B + 1) * isz;
        nnz = load_index(offp, B, a.idx64);
      } else {
        const FeatDyn d = dyn[f];
        offp = d.offsets;
        nnz = a.has_end ? load_index(d.offsets, B, a.idx64) : d.nnz;
      }
      if (nnz < 0) { nnz = 0; status |= kStatusBadOffsets; }
      long long first = (B > 0 || a.has_end) ? load_index(offp, 0, a.idx64) : 0;
      first = first < 0 ? 0 : (first > nnz ? nnz : first);
      work = nnz - first;
    }
    long long total;
    // packed mode: a feature's indices start where the previous feature's end (rows of the offsets matrix start at 0)
    const long long excl = block_excl_scan(nnz, s_warp, total) + carry;
    carry += total;
    if (f < F) {
      if (a.packed) {
        dyn[f].values = a.packed_values + excl * isz;
        dyn[f].offsets = offp;
      }
      dyn[f].nnz = nnz;
      dyn[f].work = work;
      my_cost += bag_cost(work, B, a.feats[f].row_bytes) * B;
      if (zero_ns) feat_ns[f] = 0ull;
    }
  }
  long long total_cost;
  block_excl_scan(my_cost, s_warp, total_cost);

  // pass 2: bags per tile.  Tiles aim at the same estimated cost so that a
  // ticket takes about the same time whatever the feature; about 16 tiles per warp.
  // In chunked order a tile must stay inside one piece of chunk_rows bags.
  const long long piece_cap = a.chunks > 0 ? (a.chunk_rows & -a.chunk_rows) : (1ll << 30);
  long long target = total_cost / ((long long)a.warps_total * kTilesPerWarp);
  // a tile below 64 KB of cost spends more on its own start-up than it gains in balance (measured on batches of
  // 2048 to 16384 bags)
  target = target < (64 << 10) ? (64 << 10) : (target > (256 << 10) ? (256 << 10) : target);
  for (int f = tid; f < F; f += kBindThreads) {
    const FeatStatic fs = a.feats[f];
    const long long per_bag = bag_cost(dyn[f].work, B, fs.row_bytes);
    int n = fs.bags_per_tile > 0 ? fs.bags_per_tile : pow2_floor(target / per_bag);
    const int lo = fs.bags_per_tile > 0 ? 1 : (fs.kind == 1 /*GROUP*/ ? 32 : 1);
    n = n < lo ? lo : (n > 1024 ? 1024 : n);
    if (n > piece_cap) n = (int)piece_cap;
    bpt[f] = n;
    if (F <= kMaxLptFeatures) s_cost[f] = (float)n * (float)per_bag;
  }
  __syncthreads();

  // pass 3: longest tiles first (longest-processing-time order) to shorten the tail
  for (int f = tid; f < F; f += kBindThreads) {
    int rank = f;
    if (F <= kMaxLptFeatures) {
      const float c = s_cost[f];
      rank = 0;
      for (int g = 0; g < F; ++g) {
        const float cg = s_cost[g];
        rank += (cg > c || (cg == c && g < f)) ? 1 : 0;
      }
    }
    order[rank] = f;
  }
  __syncthreads();

  // pass 4: exclusive prefix sums of tile counts in that order, one per kernel: features on the warp-per-bag
  // schedule (kind 2, vector path) are pooled by eb_warp_kernel, all others by eb_fused_kernel.  In chunked
  // order the fused kernel's prefix sum covers ONE chunk (batch / chunks bags); its tickets repeat it per chunk.
  int32_t* warp_prefix = reinterpret_cast<int32_t*>(a.ws + L.cta_prefix);
  const int64_t tile_bags = a.chunks > 0 ? B / a.chunks : B;
  carry = 0;
  long long carry_w = 0;
  for (int base = 0; base < F; base += kBindThreads) {
    const int k = base + tid;
    long long t = 0, tw = 0;
    if (k < F) {
      const int f = order[k];
      const bool lean = a.feats[f].kind == 2 && a.feats[f].vec != 0;
      t = lean ? 0 : tiles_of(tile_bags, bpt[f]);
      tw = lean ? (B + kWarpsPerCta - 1) / kWarpsPerCta : 0;  // eb_warp_kernel: one CTA per 8 bags
    }
    long long total;
    const long long excl = block_excl_scan(t, s_warp, total) + carry;
    carry += total;
    const long long excl_w = block_excl_scan(tw, s_warp, total) + carry_w;
    carry_w += total;
    if (k < F) {
      tile_prefix[k] = (int32_t)excl;
      warp_prefix[k] = (int32_t)excl_w;
    }
  }
  status = __syncthreads_or((int)status);
  if (tid == 0) {
    tile_prefix[F] = (int32_t)carry;
    warp_prefix[F] = (int32_t)carry_w;
    hdr->ticket = 0;
    hdr->total_tiles = (uint32_t)(carry * (a.chunks > 0 ? a.chunks : 1));
    hdr->cta_ticket = 0;
    hdr->cta_tiles = (uint32_t)carry_w;
    hdr->status = status;
  }
  if (tid < kMaxPeers) hdr->peer_out[tid] = a.peer_out[tid];
  if (tid < kMaxChunks) reinterpret_cast<ChunkSync*>(a.ws + L.chunk_sync)->done[tid] = 0u;
  if (a.long_bytes > 0) {
    LongBagList* ll = reinterpret_cast<LongBagList*>(a.ws + L.long_list);
    if (tid < kMaxLongBags) ll->done[tid] = 0u;
    if (tid == 0) { ll->count = 0u; ll->seg_ticket = 0u; }
  }
}

// Sets every chunk flag to the call's epoch.  Launched right after the fused kernel in chunked order, so that a
// stream waiting for a flag can never wait longer than that kernel runs, whatever the counts did.
__global__ void eb_release_kernel(uint32_t* flags, int n, uint32_t epoch) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) *reinterpret_cast<volatile uint32_t*>(flags + i) = epoch;
}

// ---------------------------------------------------------------------------
// eb_push_kernel: ships one finished piece of the send buffer to the other ranks with the SMs instead of the copy
// engines.  Small CTAs (128 threads, few registers) that fit beside the persistent pooling CTAs; every warp moves
// whole 512-byte runs (32 lanes x 16 bytes, loaded from local memory, stored to the peer), so what crosses NVLink is
// full lines, unlike the 64 to 512-byte pieces the pooling kernel itself would store.  Needs rows, leading dimensions
// and column offsets that are multiples of 16 bytes.
// ---------------------------------------------------------------------------
struct PushArgs {
  const char* send;        // first row of destination 0's piece is send + (0 * dest_rows + piece * piece_rows) * send_ld_b
  char* peer[kMaxPeers];   // result matrices (already advanced to this rank's column block)
  long long send_ld_b, out_ld_b;
  long long dest_rows, piece_rows, piece;
  int width16;             // 16-byte units per row
  int world, rank;
  int first_hop;           // destinations first_hop .. world - 1 hops to the right are served
};

__global__ void __launch_bounds__(128) eb_push_kernel(PushArgs p) {
  const long long per_dest = p.piece_rows * p.width16;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int i = p.first_hop; i < p.world; ++i) {
    const int d = (p.rank + i) % p.world;
    const char* src0 = p.send + (d * p.dest_rows + p.piece * p.piece_rows) * p.send_ld_b;
    char* dst0 = p.peer[d] + p.piece * p.piece_rows * p.out_ld_b;
    long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; u + 3 * stride < per_dest; u += 4 * stride) {  // four loads in flight per thread, then four stores
      uint4 v[4];
      long long row[4];
      int c[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const long long uu = u + k * stride;
        row[k] = uu / p.width16;
        c[k] = (int)(uu - row[k] * p.width16);
        v[k] = __ldcs(reinterpret_cast<const uint4*>(src0 + row[k] * p.send_ld_b) + c[k]);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) *(reinterpret_cast<uint4*>(dst0 + row[k] * p.out_ld_b) + c[k]) = v[k];
    }
    for (; u < per_dest; u += stride) {
      const long long row = u / p.width16;
      const int c = (int)(u - row * p.width16);
      *(reinterpret_cast<uint4*>(dst0 + row * p.out_ld_b) + c) = __ldcs(reinterpret_cast<const uint4*>(src0 + row * p.send_ld_b) + c);
    }
  }
}

// ---------------------------------------------------------------------------
// table fill: counter-based synthetic weights (bit-reproducible on the CPU)
// ---------------------------------------------------------------------------
__host__ __device__ inline uint64_t mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// Sum of four 16-bit fields, centred: integer in [-131070, 131070] with
// standard deviation 65536 * sqrt(4 / 12); one fp32 multiply maps it to the
// requested scale, so the CPU and the GPU agree to the bit.
__host__ __device__ inline float synth_weight(uint64_t seed, uint64_t elem, float scale) {
  const uint64_t h = mix64(seed * 0xD1342543DE82EF95ull + elem);
  const int s = (int)(h & 0xffff) + (int)((h >> 16) & 0xffff) + (int)((h >> 32) & 0xffff) +
                (int)((h >> 48) & 0xffff) - 131070;
  return (float)s * scale;
}

template <typename T>
__global__ void __launch_bounds__(256) eb_fill_kernel(T* table, int64_t elems, uint64_t seed, float scale) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < elems; i += stride) {
    const float w = synth_weight(seed, (uint64_t)i, scale);
    if constexpr (sizeof(T) == 2) table[i] = __float2half_rn(w);
    else table[i] = w;
  }
}

// ---------------------------------------------------------------------------
// column placement: after the all-to-all of pooled outputs, rank-major blocks
// [rows, sum(dim of the sender's features)] are scattered to each feature's
// canonical columns of the [rows, dst_ld] result.  One descriptor per feature:
// {element offset of the feature's first column in row 0 of its block, the
// block's row length, destination column, width}.
// ---------------------------------------------------------------------------
struct PlaceSeg {
  long long src_off;
  int src_ld, dst_col, width, pad_;
};

__global__ void __launch_bounds__(256) eb_place_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                       long long rows, long long dst_ld,
                                                       const PlaceSeg* __restrict__ segs, int vec_ok) {
  const PlaceSeg sg = segs[blockIdx.y];
  const float* s0 = src + sg.src_off;
  float* d0 = dst + sg.dst_col;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const bool v4 = vec_ok && (sg.width & 3) == 0 && (sg.src_ld & 3) == 0 && (sg.src_off & 3) == 0 && (sg.dst_col & 3) == 0;
  if (v4) {
    const int w4 = sg.width >> 2;
    const long long items = rows * w4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < items; i += stride) {
      const long long row = i / w4;
      const int c = (int)(i - row * w4) << 2;
      const float4 v = __ldcs(reinterpret_cast<const float4*>(s0 + row * sg.src_ld + c));
      __stcs(reinterpret_cast<float4*>(d0 + row * dst_ld + c), v);
    }
  } else {
    const long long items = rows * sg.width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < items; i += stride) {
      const long long row = i / sg.width;
      const int c = (int)(i - row * sg.width);
      d0[row * dst_ld + c] = s0[row * sg.src_ld + c];
    }
  }
}

// ---------------------------------------------------------------------------
// lengths -> offsets: one CTA per feature scans that feature's batch of bag
// lengths into batch + 1 exclusive offsets (offsets[f][0] = 0, offsets[f][B] =
// nnz_f).  Negative lengths count as 0.
// ---------------------------------------------------------------------------
template <typename IdxT>
__global__ void __launch_bounds__(kBindThreads) eb_lengths_kernel(const IdxT* __restrict__ lengths,
                                                                  IdxT* __restrict__ offsets, long long batch) {
  __shared__ long long s_warp[32];
  const IdxT* len = lengths + (long long)blockIdx.x * batch;
  IdxT* off = offsets + (long long)blockIdx.x * (batch + 1);
  long long carry = 0;
  for (long long base = 0; base < batch; base += kBindThreads) {
    const long long i = base + threadIdx.x;
    long long v = 0;
    if (i < batch) {
      v = (long long)len[i];
      if (v < 0) v = 0;
    }
    long long total;
    const long long excl = block_excl_scan(v, s_warp, total) + carry;
    if (i < batch) off[i] = (IdxT)excl;
    carry += total;
  }
  if (threadIdx.x == 0) off[batch] = (IdxT)carry;
}

}  // namespace ebk
