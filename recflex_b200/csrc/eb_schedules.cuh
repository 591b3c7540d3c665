// Per-feature schedule templates of the fused embedding-bag kernel (sm_100a).
//
// Every schedule works on one *tile* = a run of consecutive bags of one feature,
// bound to one warp.  A row of the table is read by a *group* of G = 2^lg_group
// lanes, each lane owning V consecutive elements (one 16-byte load), so a warp
// holds R = 32 / G row *slots*.  Accumulation is always fp32.
//
//   tile_group  (EB_SCHED_GROUP)  slot-per-bag, serial walk, no reduction
//   tile_warp   (element-wise)    warp-per-bag for rows that are not a whole number of 16-byte lane loads
//                                 (V = 1); EB_SCHED_WARP on vector rows is eb_warp_kernel (eb_warp.cuh)
//   tile_flat   (EB_SCHED_FLAT)   flattened entry stream dealt round-robin to the slots,
//                                 segmented reduce at bag boundaries
//   tile_stream (EB_SCHED_STREAM) flattened entry stream cut into one contiguous piece per
//                                 slot; each slot walks its piece serially, bags that
//                                 straddle pieces are patched once per 32 bags; with D > 0
//                                 (EB_SCHED_PIPE) the rows in flight sit in a cp.async ring in
//                                 shared memory instead of registers
//
// They cover the same ground as the reference's ws:: / onehot:: / obms:: / rbk::
// device templates (examples/csrc/include/*_kernel.cuh) but share one load/store
// core, 64-bit row addressing, and write every bag of the tile (empty bags -> 0).
#pragma once
#include <cuda_bf16.h>

#include "eb_common.cuh"

namespace ebk {

constexpr unsigned kFull = 0xffffffffu;

struct TileCtx {
  const char* table;
  const char* values;
  const char* offsets;
  int64_t rows;
  int64_t nnz;
  int64_t batch;
  char* out;         // output matrix (unused in peer mode); elements are fp32, or 2 bytes wide when out_dt != 0
  int64_t out_ld;    // row length in elements
  float* const* peer_out;  // peer mode: every rank's output matrix
  int64_t rows_per_peer;   // 0 = single output matrix
  int32_t col_off;   // the feature's first column
  int32_t out_dt;    // element type of the output: 0 = fp32, 1 = bfloat16, 2 = binary16
  int32_t es_shift;  // log2 of the output element size: 2 or 1
  uint32_t* status;
  int32_t dim;
  int32_t row_bytes;
  int32_t lg_group;
  int32_t nx;
  bool idx64;
  bool has_end;
  int out_vec;       // widest aligned store the output allows: 0 = one element, 1 = four elements, 2 = eight elements
};

__device__ __forceinline__ int64_t load_index(const char* base, int64_t i, bool idx64) {
  return idx64 ? (int64_t)__ldg(reinterpret_cast<const long long*>(base) + i)
               : (int64_t)__ldg(reinterpret_cast<const int*>(base) + i);
}

// Address of this feature's first column in the row of bag `bb`.  In peer mode the bag's row lives in the
// output matrix of rank bb / rows_per_peer; chunks of 32 bags never straddle two ranks because rows_per_peer is a
// multiple of 32.
__device__ __forceinline__ char* chunk_out(const TileCtx& c, int64_t bb) {
  if (c.rows_per_peer == 0) return c.out + ((bb * c.out_ld + c.col_off) << c.es_shift);
  const int64_t d = bb / c.rows_per_peer;
  return reinterpret_cast<char*>(c.peer_out[d]) + (((bb - d * c.rows_per_peer) * c.out_ld + c.col_off) << c.es_shift);
}

__device__ __forceinline__ void flag(uint32_t* status, uint32_t bit) {
  if ((*reinterpret_cast<volatile uint32_t*>(status) & bit) == 0) atomicOr(status, bit);
}

// ---------------------------------------------------------------------------
// Row element access: V elements per lane.
// ---------------------------------------------------------------------------
template <typename T, int V>
struct RowOps;

template <>
struct RowOps<float, 4> {
  using Raw = uint4;
  __device__ __forceinline__ static Raw zero() { return make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ static Raw load(const char* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ static void add(float (&a)[4], const Raw& r) {
    a[0] += __uint_as_float(r.x);
    a[1] += __uint_as_float(r.y);
    a[2] += __uint_as_float(r.z);
    a[3] += __uint_as_float(r.w);
  }
};

template <>
struct RowOps<__half, 8> {
  using Raw = uint4;
  __device__ __forceinline__ static Raw zero() { return make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ static Raw load(const char* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
  // sm_100 mixed-precision add: fp32 accumulator += binary16 operand, one
  // instruction per element instead of convert + add; same rounding (the
  // binary16 value is exact in fp32, the sum is rounded to nearest even).
  __device__ __forceinline__ static void add2(float& x, float& y, unsigned w) {
    asm("{\n\t"
        ".reg .b16 lo, hi;\n\t"
        "mov.b32 {lo, hi}, %2;\n\t"
        "add.f32.f16 %0, lo, %0;\n\t"
        "add.f32.f16 %1, hi, %1;\n\t"
        "}"
        : "+f"(x), "+f"(y)
        : "r"(w));
  }
  __device__ __forceinline__ static void add(float (&a)[8], const Raw& r) {
    add2(a[0], a[1], r.x);
    add2(a[2], a[3], r.y);
    add2(a[4], a[5], r.z);
    add2(a[6], a[7], r.w);
  }
};

template <>
struct RowOps<float, 1> {
  using Raw = float;
  __device__ __forceinline__ static Raw zero() { return 0.f; }
  __device__ __forceinline__ static Raw load(const char* p) { return __ldg(reinterpret_cast<const float*>(p)); }
  __device__ __forceinline__ static void add(float (&a)[1], const Raw& r) { a[0] += r; }
};

template <>
struct RowOps<__half, 1> {
  using Raw = unsigned short;
  __device__ __forceinline__ static Raw zero() { return 0; }
  __device__ __forceinline__ static Raw load(const char* p) { return __ldg(reinterpret_cast<const unsigned short*>(p)); }
  __device__ __forceinline__ static void add(float (&a)[1], const Raw& r) { a[0] += __half2float(__ushort_as_half(r)); }
};

// Streaming (evict-first) stores: the output is written once and never re-read
// by this kernel, so it should not displace table rows from L2.
// A lane that owns 8 floats writes them with ONE 32-byte store when alignment
// allows: two 16-byte stores would each cover only half of every 32-byte
// sector, which L2 merges for local memory but which crosses NVLink as
// half-filled packets when the destination is a peer's memory.
// `dt` != 0 narrows the output: the fp32 sums are rounded to nearest even into bfloat16 (1) or binary16 (2)
// elements, a lane's V values leaving as one 2 * V byte store when alignment allows (`ov` as for fp32).
__device__ __forceinline__ unsigned pack_narrow(float lo, float hi, int dt) {
  if (dt == 1) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
  }
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}

__device__ __forceinline__ float unpack_narrow(unsigned short bits, int dt) {
  if (dt == 1) return __uint_as_float((unsigned)bits << 16);
  return __half2float(__ushort_as_half(bits));
}

template <int V>
__device__ __forceinline__ void store_vals(char* dstb, const float (&a)[V], int vec_ok, int dt = 0) {
  if (dt != 0) {
    if constexpr (V == 1) {
      const unsigned w = pack_narrow(a[0], 0.f, dt);
      __stcs(reinterpret_cast<unsigned short*>(dstb), (unsigned short)(w & 0xffffu));
    } else {
      unsigned w[V / 2];
#pragma unroll
      for (int k = 0; k < V / 2; ++k) w[k] = pack_narrow(a[2 * k], a[2 * k + 1], dt);
      if constexpr (V == 8) {
        if (vec_ok == 2) {
          __stcs(reinterpret_cast<uint4*>(dstb), make_uint4(w[0], w[1], w[2], w[3]));
          return;
        }
      }
      if (vec_ok) {
#pragma unroll
        for (int k = 0; k < V / 2; k += 2) __stcs(reinterpret_cast<uint2*>(dstb + 4 * k), make_uint2(w[k], w[k + 1]));
      } else {
#pragma unroll
        for (int k = 0; k < V / 2; ++k) {
          __stcs(reinterpret_cast<unsigned short*>(dstb + 4 * k), (unsigned short)(w[k] & 0xffffu));
          __stcs(reinterpret_cast<unsigned short*>(dstb + 4 * k + 2), (unsigned short)(w[k] >> 16));
        }
      }
    }
    return;
  }
  float* dst = reinterpret_cast<float*>(dstb);
  if constexpr (V == 1) {
    __stcs(dst, a[0]);
  } else {
    if constexpr (V == 8) {
      if (vec_ok == 2) {
        // no "memory" clobber: the walk's reads of the ring may move across this store; the one place that reads an
        // output row back (the patch pass) sits behind a compiler barrier of its own
        asm volatile("st.global.cs.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "f"(a[0]), "f"(a[1]),
                     "f"(a[2]), "f"(a[3]), "f"(a[4]), "f"(a[5]), "f"(a[6]), "f"(a[7]));
        return;
      }
    }
    if (vec_ok) {
#pragma unroll
      for (int k = 0; k < V; k += 4)
        __stcs(reinterpret_cast<float4*>(dst + k), make_float4(a[k], a[k + 1], a[k + 2], a[k + 3]));
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) __stcs(dst + k, a[k]);
    }
  }
}

// Read back what store_vals wrote (the head partial of a bag cut by a piece boundary) and add `add` to it.
template <int V>
__device__ __forceinline__ void reload_add(const char* srcb, const float (&add)[V], float (&res)[V], int vec_ok, int dt) {
  if (dt != 0) {
    const unsigned short* src = reinterpret_cast<const unsigned short*>(srcb);
#pragma unroll
    for (int k = 0; k < V; ++k) res[k] = unpack_narrow(src[k], dt) + add[k];
    return;
  }
  const float* src = reinterpret_cast<const float*>(srcb);
  if constexpr (V == 1) {
    res[0] = src[0] + add[0];
  } else {
    if (vec_ok) {
#pragma unroll
      for (int k = 0; k < V; k += 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(src + k);
        res[k] = q4.x + add[k];
        res[k + 1] = q4.y + add[k + 1];
        res[k + 2] = q4.z + add[k + 2];
        res[k + 3] = q4.w + add[k + 3];
      }
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) res[k] = src[k] + add[k];
    }
  }
}

template <int V>
__device__ __forceinline__ void zero_vals(float (&a)[V]) {
#pragma unroll
  for (int k = 0; k < V; ++k) a[k] = 0.f;
}

// ---------------------------------------------------------------------------
// Bag boundaries of up to 32 consecutive bags, one per lane, relative to the
// first one.  The sequence is forced to be non-decreasing and inside [0, nnz]
// (status bit set when that changed anything), so no later step can index
// outside the feature's index list.
// ---------------------------------------------------------------------------
__device__ __forceinline__ int64_t raw_offset(const TileCtx& c, int64_t b) {
  if (!c.has_end && b >= c.batch) return c.nnz;
  return load_index(c.offsets, b, c.idx64);
}

__device__ __forceinline__ int64_t clamp_off(int64_t v, int64_t nnz) {
  return v < 0 ? 0 : (v > nnz ? nnz : v);
}

struct Chunk {
  int64_t e0;  // absolute position of the chunk's first entry
  int lo, hi;  // this lane's bag: entries [lo, hi) relative to e0 (lo == hi == n for lanes past the chunk)
  int n;       // entries in the chunk
};

// Slow path of load_chunk: force the sequence into shape and say so.
static __device__ __noinline__ Chunk repair_chunk(const TileCtx& c, int64_t a_raw, int64_t end_raw, int lane) {
  int64_t m = clamp_off(a_raw, c.nnz);
  int64_t endm = clamp_off(end_raw, c.nnz);
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int64_t t = __shfl_up_sync(kFull, m, d);
    if (lane >= d && t > m) m = t;
  }
  const int64_t m31 = __shfl_sync(kFull, m, 31);
  if (m31 > endm) endm = m31;
  Chunk ch;
  ch.e0 = __shfl_sync(kFull, m, 0);
  int64_t nxt = __shfl_down_sync(kFull, m, 1);
  if (lane == 31) nxt = endm;
  int64_t total = endm - ch.e0;
  if (total > 0x3fffffff) total = 0x3fffffff;  // more than 2^30 indices in 32 bags: refuse the excess
  int64_t lo = m - ch.e0, hi = nxt - ch.e0;
  if (lo > total) lo = total;
  if (hi > total) hi = total;
  ch.lo = (int)lo;
  ch.hi = (int)hi;
  ch.n = (int)total;
  if (lane == 0) flag(c.status, kStatusBadOffsets);
  return ch;
}

// One warp vote decides whether the 33 boundaries are already a non-decreasing sequence inside [0, nnz] spanning at
// most 2^30 entries (the normal case: a handful of instructions, 32-bit when the batch's integers are); only
// otherwise is the sequence repaired.  Must be called by all 32 lanes.
// 32-bit boundaries: this lane's boundary `a` and the boundary `end` after the chunk's last bag -> Chunk.
__device__ __forceinline__ Chunk chunk_from32(const TileCtx& c, int a, int end, int lane) {
  const int nnz = c.nnz > 0x7fffffff ? 0x7fffffff : (int)c.nnz;
  int nxt = __shfl_down_sync(kFull, a, 1);
  if (lane == 31) nxt = end;
  const int a0 = __shfl_sync(kFull, a, 0);
  const bool good = a >= 0 && a <= nxt && nxt <= nnz && (unsigned)(end - a0) <= 0x3fffffffu;
  if (__all_sync(kFull, good)) {
    Chunk ch;
    ch.e0 = a0;
    ch.lo = a - a0;
    ch.hi = nxt - a0;
    ch.n = end - a0;
    return ch;
  }
  return repair_chunk(c, (int64_t)a, (int64_t)end, lane);
}

// Boundary number `pos` of a feature with 32-bit offsets (an offsets array without end entry lacks the last one).
__device__ __forceinline__ int boundary32(const TileCtx& c, int64_t pos) {
  if (!c.has_end && pos >= c.batch) return c.nnz > 0x7fffffff ? 0x7fffffff : (int)c.nnz;
  return __ldg(reinterpret_cast<const int*>(c.offsets) + pos);
}

template <bool IDX64>
__device__ __forceinline__ Chunk load_chunk(const TileCtx& c, int64_t bb, int nb, int lane) {
  const int li = lane <= nb ? lane : nb;
  Chunk ch;
  if constexpr (!IDX64) {
    const int a = boundary32(c, bb + li);
    int end = __shfl_sync(kFull, a, 31);
    if (nb == 32) end = boundary32(c, bb + 32);
    return chunk_from32(c, a, end, lane);
  } else {
    const int64_t a = raw_offset(c, bb + li);
    int64_t end = __shfl_sync(kFull, a, 31);
    if (nb == 32) end = raw_offset(c, bb + 32);
    int64_t nxt = __shfl_down_sync(kFull, a, 1);
    if (lane == 31) nxt = end;
    const int64_t a0 = __shfl_sync(kFull, a, 0);
    const bool good = a >= 0 && a <= nxt && nxt <= c.nnz && end - a0 <= 0x3fffffff;
    if (__all_sync(kFull, good)) {
      ch.e0 = a0;
      ch.lo = (int)(a - a0);
      ch.hi = (int)(nxt - a0);
      ch.n = (int)(end - a0);
      return ch;
    }
    return repair_chunk(c, a, end, lane);
  }
}

// Index element type of a batch.
template <bool IDX64>
struct IdxOf { using type = int; };
template <>
struct IdxOf<true> { using type = long long; };

// Fetch U rows: indices vp[p[u]] -> rows.  With 32-bit indices the bounds check
// is one unsigned compare and the row address one 32x32+64 multiply-add.
// CHECK = false means every entry is in range (`ok` is not read).
// When every lane's entries are in range and every index is valid (one warp
// vote), the row loads are issued unconditionally: no predicates and no
// zero-initialised buffers on the path that carries almost all the traffic.
// Must be called by all 32 lanes.
template <typename T, int V, int U, bool IDX64, bool CHECK>
__device__ __forceinline__ void fetch_rows(const TileCtx& c, const typename IdxOf<IDX64>::type* vp,
                                           const char* tcol, bool col_ok, const int (&p)[U], const bool (&ok)[U],
                                           typename RowOps<T, V>::Raw (&rows)[U]) {
  using Ops = RowOps<T, V>;
  typename IdxOf<IDX64>::type idx[U];
  bool all_ok = true;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const bool want = col_ok && (!CHECK || ok[u]);
    idx[u] = want ? __ldg(vp + p[u]) : 0;
    if (CHECK) all_ok = all_ok && (ok[u] || !col_ok);
  }
  const unsigned rows32 = c.rows > 0x80000000ll ? 0x80000000u : (unsigned)c.rows;
  bool valid = true;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if constexpr (IDX64) valid = valid && (uint64_t)idx[u] < (uint64_t)c.rows;
    else valid = valid && (unsigned)idx[u] < rows32;
  }
  if (__all_sync(kFull, all_ok && valid)) {
    // lanes whose columns lie past the row's end (col_ok false) load nothing; all others load unconditionally
    if (col_ok) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if constexpr (IDX64) rows[u] = Ops::load(tcol + idx[u] * (int64_t)c.row_bytes);
        else rows[u] = Ops::load(tcol + (uint64_t)(unsigned)idx[u] * (unsigned)c.row_bytes);
      }
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) rows[u] = Ops::zero();
    }
    return;
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    rows[u] = Ops::zero();
    if (col_ok && (!CHECK || ok[u])) {
      if constexpr (IDX64) {
        if ((uint64_t)idx[u] < (uint64_t)c.rows)
          rows[u] = Ops::load(tcol + idx[u] * (int64_t)c.row_bytes);
        else
          flag(c.status, kStatusBadIndex);
      } else {
        if ((unsigned)idx[u] < rows32)
          rows[u] = Ops::load(tcol + (uint64_t)(unsigned)idx[u] * (unsigned)c.row_bytes);
        else
          flag(c.status, kStatusBadIndex);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// EB_SCHED_GROUP: each slot owns one bag at a time and walks it serially.
// ---------------------------------------------------------------------------
template <typename T, int V, int U, bool IDX64>
__device__ __forceinline__ void tile_group(const TileCtx& c, int64_t b0, int64_t b1, int lane) {
  using Ops = RowOps<T, V>;
  const int lgG = c.lg_group, G = 1 << lgG, R = 32 >> lgG;
  const int r = lane >> lgG, cl = lane & (G - 1);
  for (int xc = 0; xc < c.nx; ++xc) {
    const int cs = (xc * G + cl) * V;
    const bool col_ok = cs < c.dim;
    const char* tcol = c.table + (size_t)cs * sizeof(T);
    for (int64_t bb = b0; bb < b1; bb += 32) {
      const int nb = (int)((b1 - bb) < 32 ? (b1 - bb) : 32);
      const Chunk ch = load_chunk<IDX64>(c, bb, nb, lane);
      char* orow = chunk_out(c, bb) + ((size_t)cs << c.es_shift);
      const size_t row_b = (size_t)c.out_ld << c.es_shift;
      const typename IdxOf<IDX64>::type* vals = reinterpret_cast<const typename IdxOf<IDX64>::type*>(c.values) + ch.e0;
      for (int i0 = 0; i0 < nb; i0 += R) {
        const int bi = i0 + r;
        const int s = __shfl_sync(kFull, ch.lo, bi & 31);
        const int e = __shfl_sync(kFull, ch.hi, bi & 31);
        const int len = bi < nb ? e - s : 0;
        const int maxlen = __reduce_max_sync(kFull, len);
        float acc[V];
        zero_vals<V>(acc);
        for (int q = 0; q < maxlen; q += U) {
          int p[U];
          bool ok[U];
          typename Ops::Raw rows[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            p[u] = s + q + u;
            ok[u] = q + u < len;
          }
          fetch_rows<T, V, U, IDX64, true>(c, vals, tcol, col_ok, p, ok, rows);
#pragma unroll
          for (int u = 0; u < U; ++u) Ops::add(acc, rows[u]);
        }
        if (bi < nb && col_ok) store_vals<V>(orow + (size_t)bi * row_b, acc, c.out_vec, c.out_dt);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Warp-per-bag inside the fused kernel: the warp owns one bag at a time; its R slots
// split the bag.  Used for the element-wise fallback only (V = 1).
// ---------------------------------------------------------------------------
template <typename T, int V, int U, bool IDX64>
__device__ __forceinline__ void tile_warp(const TileCtx& c, int64_t b0, int64_t b1, int lane) {
  using Ops = RowOps<T, V>;
  const int lgG = c.lg_group, G = 1 << lgG, R = 32 >> lgG;
  const int r = lane >> lgG, cl = lane & (G - 1);
  for (int xc = 0; xc < c.nx; ++xc) {
    const int cs = (xc * G + cl) * V;
    const bool col_ok = cs < c.dim;
    const char* tcol = c.table + (size_t)cs * sizeof(T);
    for (int64_t bb = b0; bb < b1; bb += 32) {
      const int nb = (int)((b1 - bb) < 32 ? (b1 - bb) : 32);
      const Chunk ch = load_chunk<IDX64>(c, bb, nb, lane);
      char* orow = chunk_out(c, bb) + ((size_t)cs << c.es_shift);
      const size_t row_b = (size_t)c.out_ld << c.es_shift;
      const typename IdxOf<IDX64>::type* vals = reinterpret_cast<const typename IdxOf<IDX64>::type*>(c.values) + ch.e0;
      for (int i = 0; i < nb; ++i) {
        const int s = __shfl_sync(kFull, ch.lo, i);
        const int e = __shfl_sync(kFull, ch.hi, i);
        float acc[V];
        zero_vals<V>(acc);
        for (int q = s; q < e; q += R * U) {
          int p[U];
          bool ok[U];
          typename Ops::Raw rows[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            p[u] = q + u * R + r;
            ok[u] = p[u] < e;
          }
          fetch_rows<T, V, U, IDX64, true>(c, vals, tcol, col_ok, p, ok, rows);
#pragma unroll
          for (int u = 0; u < U; ++u) Ops::add(acc, rows[u]);
        }
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          if (d >= G) {
#pragma unroll
            for (int k = 0; k < V; ++k) acc[k] += __shfl_xor_sync(kFull, acc[k], d);
          }
        }
        if (r == 0 && col_ok) store_vals<V>(orow + (size_t)i * row_b, acc, c.out_vec, c.out_dt);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// EB_SCHED_FLAT: the warp streams the chunk's entries R at a time ("steps"),
// U steps in flight, whatever the bag lengths.  Slot r of step j holds entry
// j + r.  While a step lies strictly inside the open bag W every slot just
// accumulates.  A step that touches a boundary closes W (butterfly over the
// slots' partial sums), reduces the bags that start inside the step with a
// segmented shuffle reduction, stores the ones that also end there, and keeps
// the last one as the new open bag.
// ---------------------------------------------------------------------------
template <typename T, int V, int U, bool IDX64>
__device__ __forceinline__ void tile_flat(const TileCtx& c, int64_t b0, int64_t b1, int lane) {
  using Ops = RowOps<T, V>;
  const int lgG = c.lg_group, G = 1 << lgG, R = 32 >> lgG;
  const int r = lane >> lgG, cl = lane & (G - 1);
  for (int xc = 0; xc < c.nx; ++xc) {
    const int cs = (xc * G + cl) * V;
    const bool col_ok = cs < c.dim;
    const char* tcol = c.table + (size_t)cs * sizeof(T);
    for (int64_t bb = b0; bb < b1; bb += 32) {
      const int nb = (int)((b1 - bb) < 32 ? (b1 - bb) : 32);
      const Chunk ch = load_chunk<IDX64>(c, bb, nb, lane);
      char* orow = chunk_out(c, bb) + ((size_t)cs << c.es_shift);
      const size_t row_b = (size_t)c.out_ld << c.es_shift;
      const typename IdxOf<IDX64>::type* vals = reinterpret_cast<const typename IdxOf<IDX64>::type*>(c.values) + ch.e0;
      const int n = ch.n;
      const bool nonempty = ch.hi > ch.lo;

      // empty bags pool to zero
      {
        const unsigned valid = nb == 32 ? kFull : ((1u << nb) - 1u);
        unsigned em = ~__ballot_sync(kFull, nonempty) & valid;
        float z[V];
        zero_vals<V>(z);
        while (em) {
          // slot r takes the r-th remaining empty bag
          const int i = (int)__fns(em, 0, r + 1);  // -1 when fewer than r + 1 remain
          if (i >= 0 && col_ok) store_vals<V>(orow + (size_t)i * row_b, z, c.out_vec, c.out_dt);
          // drop the R lowest set bits
          for (int k = 0; k < R && em; ++k) em &= em - 1;
        }
      }

      int wbag = -1;  // open bag (chunk-local), -1 = none
      int endw = 0;   // its end; when none, a position <= the next step so that the step takes the boundary path
      float acc[V];
      zero_vals<V>(acc);

      for (int base = 0; base < n; base += R * U) {
        int p[U];
        bool ok[U];
        typename Ops::Raw rows[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          p[u] = base + u * R + r;
          ok[u] = p[u] < n;
        }
        fetch_rows<T, V, U, IDX64, true>(c, vals, tcol, col_ok, p, ok, rows);

#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = base + u * R;
          if (j < n) {
            if (j + R < endw) {
              Ops::add(acc, rows[u]);
            } else {
              const int pj = j + r;
              const bool inw = pj < endw;  // false everywhere when no bag is open
              float x[V];
              zero_vals<V>(x);
              if (wbag >= 0) {
                if (inw) Ops::add(acc, rows[u]);
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                  if (d >= G) {
#pragma unroll
                    for (int k = 0; k < V; ++k) acc[k] += __shfl_xor_sync(kFull, acc[k], d);
                  }
                }
                if (r == 0 && col_ok) store_vals<V>(orow + (size_t)wbag * row_b, acc, c.out_vec, c.out_dt);
              }
              if (!inw) Ops::add(x, rows[u]);

              // bags that start inside [j, j + R): one head bit per slot
              const bool head_here = nonempty && ch.lo >= j && ch.lo < j + R;
              const unsigned head_mask = __reduce_or_sync(kFull, head_here ? (1u << (ch.lo - j)) : 0u);
              if (head_mask == 0u) {
                wbag = -1;
                endw = j + R;
                zero_vals<V>(acc);
              } else {
                const unsigned m_before = __ballot_sync(kFull, nonempty && ch.lo < j);
                const unsigned m_upto = __ballot_sync(kFull, nonempty && ch.lo < j + R);
                const unsigned head_bags = m_upto & ~m_before;
                const int lastbag = 31 - __clz(m_upto);
                const int last_end = __shfl_sync(kFull, ch.hi, lastbag);
                const bool last_cont = last_end > j + R;
                const int last_head = 31 - __clz(head_mask);

                const unsigned below = head_mask & ((2u << r) - 1u);
                const bool has_seg = below != 0u;
                const int seg_start = 31 - __clz(below);
                const unsigned above = r == 31 ? 0u : (head_mask >> (r + 1));
                const int seg_end = above ? (r + __ffs(above) - 1) : (R - 1);
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                  if (d < R) {
                    const bool take = has_seg && (r + d <= seg_end);
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                      const float y = __shfl_down_sync(kFull, x[k], d << lgG);
                      if (take) x[k] += y;
                    }
                  }
                }
                const bool is_head = has_seg && r == seg_start;
                const bool keeps = is_head && seg_start == last_head && last_cont;
                if (is_head && !keeps && col_ok) {
                  const int q = __popc(head_mask & ((1u << r) - 1u));
                  const int mybag = __fns(head_bags, 0, q + 1);
                  store_vals<V>(orow + (size_t)mybag * row_b, x, c.out_vec, c.out_dt);
                }
#pragma unroll
                for (int k = 0; k < V; ++k) acc[k] = keeps ? x[k] : 0.f;
                if (last_cont) {
                  wbag = lastbag;
                  endw = last_end;
                } else {
                  wbag = -1;
                  endw = j + R;
                }
              }
            }
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// cp.async primitives of the pipelined stream walk: each lane copies 16 bytes
// global -> shared without passing through registers and later reads back only
// its own cells, so no barrier is needed, only the per-thread group wait.
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned smem_addr(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src, unsigned src_bytes) {
  // src_bytes = 0 reads nothing and fills the 16 destination bytes with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint4 lds16(unsigned addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// Indices of the U entries starting at `first` (0 for entries at or past `limit`).
template <int U, bool IDX64>
__device__ __forceinline__ void load_indices(const typename IdxOf<IDX64>::type* vp, int first, int limit, bool col_ok,
                                             typename IdxOf<IDX64>::type (&idx)[U]) {
#pragma unroll
  for (int u = 0; u < U; ++u) idx[u] = (col_ok && first + u < limit) ? __ldg(vp + first + u) : 0;
}

// Issue the copies of one macro-step (U entries starting at `first`) into ring cells dst + u * 512.
// Entries at or past `limit` carry index 0 (see load_indices), so every source address is inside the table;
// they and out-of-range indices copy zero bytes (the cell is zero-filled).  Returns whether a bad index was met.
template <typename T, int U, bool IDX64>
__device__ __forceinline__ bool issue_rows(const TileCtx& c, const char* tcol, bool col_ok,
                                           const typename IdxOf<IDX64>::type (&idx)[U], int first, int limit,
                                           unsigned dst) {
  const unsigned rows32 = c.rows > 0x80000000ll ? 0x80000000u : (unsigned)c.rows;
  bool bad = false;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const bool ok = col_ok && first + u < limit;
    if constexpr (IDX64) {
      const bool valid = (uint64_t)idx[u] < (uint64_t)c.rows;
      bad |= ok && !valid;
      cp_async16(dst + u * 512, tcol + (valid ? idx[u] : 0) * (int64_t)c.row_bytes, ok && valid ? 16u : 0u);
    } else {
      const unsigned i = (unsigned)idx[u];
      const bool valid = i < rows32;
      bad |= ok && !valid;
      cp_async16(dst + u * 512, tcol + (uint64_t)min(i, rows32 - 1u) * (unsigned)c.row_bytes, ok && valid ? 16u : 0u);
    }
  }
  return bad;
}

// ---------------------------------------------------------------------------
// EB_SCHED_STREAM: the chunk's n entries are cut into R contiguous pieces, one
// per slot, of floor(n / R) or one more entries.  Every slot walks its piece
// serially with U rows in flight, whatever the bag lengths: a bag that ends
// inside the piece is stored at once.  While a whole macro-step of U entries
// stays inside the current bag for every slot (one warp vote), the walk is a
// pure load + accumulate loop.  A bag cut by a piece boundary leaves a tail
// partial in the slot's accumulator and a head partial in the output row; after
// the walk a segmented shuffle scan over the slots' tails patches each head
// (once per 32 bags).
//
// What a slot needs at a bag end is the next non-empty bag and where it ends.
// The chunk's non-empty bags are therefore listed once per chunk in shared
// memory ({end, bag}, closed by a sentinel): non-empty bags are contiguous in
// the entry stream, so the next list item starts where the current one ends,
// and a bag end costs one store, one 8-byte shared load and no warp-wide
// operation: slots that are not at a bag end simply skip the block.  An end
// that lies beyond the slot's piece is replaced by a value no position reaches,
// so entries past the piece's end (fetched as zeros) need no guard either.
//
// D > 0 selects the pipelined form (EB_SCHED_PIPE): the rows in flight live in a
// per-warp shared-memory ring of D macro-steps (D * U * 512 bytes) filled by
// per-lane cp.async copies instead of in registers, so D * U rows per lane are
// in flight (against U) and the row registers are free; the walk, the stores
// and the patch pass are the same.  Macro-steps in which every slot has U real
// entries with valid indices (two uniform tests) issue their copies without any
// predicate; only the ragged end of a piece and bad input take the checked path.
// ---------------------------------------------------------------------------
constexpr int kBagItems = 34;        // per-warp list of a chunk's non-empty bags: 32 + sentinel; the last entry is
                                     // never part of the list (the kernel keeps the tile's feature number there)
constexpr int kNoEnd = 0x7fffffff;   // "this bag does not end inside my piece"


// A slot's cursor in the chunk's list of non-empty bags.  The item after the current bag is fetched one bag ahead, so
// that the shared-memory latency is not in the chain bag end -> next end -> next comparison.
struct BagCursor {
  const int2* p;  // the prefetched item (shared memory)
  int2 nxt;       // the item after the current bag
  __device__ __forceinline__ void init(const int2* current_item) {
    p = current_item + 1;
    nxt = *p;
  }
  // Make the next list item the current bag; an end beyond the piece never matches a position.
  __device__ __forceinline__ void advance(int e_end, int& kb, int& kend) {
    kb = nxt.y;
    kend = nxt.x > e_end ? kNoEnd : nxt.x;
    nxt = *++p;
  }
};

// Stores of the stream walk.  FS (fast store) = fp32 output whose alignment allows the widest store: no run-time
// choice is left in the walk's hot block.
template <int V, bool FS>
__device__ __forceinline__ void walk_store(char* dst, const float (&a)[V], int ov, int dt) {
  if constexpr (FS) store_vals<V>(dst, a, V == 8 ? 2 : 1, 0);
  else store_vals<V>(dst, a, ov, dt);
}

template <typename T, int V, int U, bool IDX64, int D = 0, bool FS = false>
__device__ __forceinline__ void tile_stream(const LaunchArgs& ka, const TileCtx& c, int64_t b0, int64_t b1, int lane,
                                            int2* items, unsigned char* ring = nullptr) {
  static_assert(D == 0 || V * sizeof(T) == 16, "the ring holds 16-byte lane cells");
  using Ops = RowOps<T, V>;
  using IdxT = typename IdxOf<IDX64>::type;
  const int lgG = c.lg_group, lgR = 5 - lgG, G = 1 << lgG, R = 1 << lgR;
  const int r = lane >> lgG, cl = lane & (G - 1);
  const unsigned ld_bytes = FS ? (unsigned)c.out_ld * 4u : (unsigned)c.out_ld << c.es_shift;  // rows stay below 4 GB
  const int dt = FS ? 0 : c.out_dt;
  const unsigned rows32 = c.rows > 0x80000000ll ? 0x80000000u : (unsigned)c.rows;
  const int ov = FS ? (V == 8 ? 2 : 1) : c.out_vec;
  for (int xc = 0; xc < c.nx; ++xc) {
    const int cs = (xc * G + cl) * V;
    const bool col_ok = cs < c.dim;
    const char* tcol = c.table + (size_t)cs * sizeof(T);
    // Chunks end at multiples of 32 bags (of the batch), so none straddles two ranks' rows in peer mode; a tile
    // starts at a multiple of its own size, so only a tile narrower than 32 bags starts elsewhere.
    // 32-bit offsets: the boundaries of the next two chunks are fetched while this one is walked, so that a chunk
    // starts without waiting for its offsets (lane i holds boundary pos0 + min(i, bags of the chunk at pos0)).
    auto bounds_at = [&](int64_t pos0) -> int {
      if (pos0 > b1) return 0;
      int64_t cnt = 32 - (pos0 & 31);
      if (b1 - pos0 < cnt) cnt = b1 - pos0;
      return boundary32(c, pos0 + (lane < cnt ? lane : cnt));
    };
    int a_cur = 0, a_nxt = 0;
    // Can a bag of this tile be long enough for eb_longbag_kernel?  Only if the whole tile is: one test per tile,
    // kept as a predicate; everything else about long bags is looked up again in the rare branch that needs it.
    bool maybe_long = false;
    if constexpr (!IDX64) {
      a_cur = bounds_at(b0);
      a_nxt = bounds_at(b0 + (32 - (b0 & 31)));
      if (ka.long_bytes > 0 && ka.chunks == 0 && c.nx == 1) {
        const int64_t tile_entries = (int64_t)boundary32(c, b1) - (int64_t)boundary32(c, b0);
        maybe_long = tile_entries * c.row_bytes >= ka.long_bytes;
      }
    }
    int nb = 0;
    for (int64_t bb = b0; bb < b1; bb += nb) {
      nb = 32 - (int)(bb & 31);
      if (b1 - bb < nb) nb = (int)(b1 - bb);
      Chunk ch;
      if constexpr (!IDX64) {
        if (!maybe_long) {
          const int a_fut = bounds_at(bb + nb + 32);  // the chunk after the next one (which starts at a multiple of 32)
          ch = chunk_from32(c, a_cur, nb == 32 ? __shfl_sync(kFull, a_nxt, 0) : __shfl_sync(kFull, a_cur, nb), lane);
          a_cur = a_nxt;
          a_nxt = a_fut;
        } else {
          // rare: a tile heavy enough to hold a long bag.  A chunk with such a bag is taken one bag at a time; the
          // long ones go to eb_longbag_kernel's list (a full list takes no more: the bag is then walked here, alone)
          ch = load_chunk<false>(c, bb, nb, lane);
          const int64_t long_len = (ka.long_bytes + c.row_bytes - 1) / c.row_bytes;
          if (__any_sync(kFull, (int64_t)(ch.hi - ch.lo) >= long_len)) {
            nb = 1;
            ch = load_chunk<false>(c, bb, 1, lane);
            if ((int64_t)ch.n >= long_len) {
              LongBagList* ll = reinterpret_cast<LongBagList*>(ka.ws + ws_layout(ka.num_features).long_list);
              unsigned slot = 0;
              if (lane == 0) slot = atomicAdd(&ll->count, 1u);
              slot = __shfl_sync(kFull, slot, 0);
              if (slot < (unsigned)kMaxLongBags) {
                if (lane == 0) {
                  LongBag lb;
                  lb.feat = items[kBagItems - 1].x;  // the tile's feature, left there by the kernel
                  lb.pad_ = 0;
                  lb.bag = bb;
                  lb.begin = ch.e0;
                  lb.end = ch.e0 + ch.n;
                  ll->item[slot] = lb;
                }
                continue;  // skipped here: eb_longbag_kernel pools it
              }
            }
          }
        }
      } else {
        ch = load_chunk<IDX64>(c, bb, nb, lane);
      }
      const int n = ch.n;
      // my piece [s, e_end): the first n % R slots hold one entry more
      const int q = n >> lgR, rem = n & (R - 1);
      const int s = r * q + min(r, rem);
      const int e_end = s + q + (r < rem ? 1 : 0);
      const int ls = q + (rem ? 1 : 0);  // longest piece; the shortest has q entries
      const IdxT* vp = reinterpret_cast<const IdxT*>(c.values) + ch.e0;
      // pipelined walk: the indices of macro-step 0 are asked for now, so that they travel while the chunk's
      // bookkeeping below runs; `full`: every slot has U real entries there, so they are fetched without guards
      IdxT idx[U];
      bool full = U <= q;
      if constexpr (D > 0) {
        if (full) {
#pragma unroll
          for (int u = 0; u < U; ++u) idx[u] = __ldg(vp + s + u);
        } else {
          load_indices<U, IDX64>(vp, s, e_end, col_ok, idx);
        }
      }
      char* const orow = chunk_out(c, bb) + ((size_t)cs << (FS ? 2 : c.es_shift));
      const bool nonempty = ch.hi > ch.lo;
      const unsigned nz = __ballot_sync(kFull, nonempty);

      // empty bags pool to zero: slot r takes the r-th remaining one
      {
        const unsigned valid = nb == 32 ? kFull : ((1u << nb) - 1u);
        unsigned em = ~nz & valid;
        float z[V];
        zero_vals<V>(z);
        while (em) {
          const int i = (int)__fns(em, 0, r + 1);
          if (i >= 0 && col_ok) walk_store<V, FS>(orow + (size_t)i * ld_bytes, z, ov, dt);
          for (int k = 0; k < R && em; ++k) em &= em - 1;
        }
      }
      if (n == 0) continue;

      // the chunk's non-empty bags, in order
      __syncwarp();  // nobody still reads the previous chunk's list
      if (nonempty) items[__popc(nz & ((1u << lane) - 1u))] = make_int2(ch.hi, lane);
      if (lane == 0) items[__popc(nz)] = make_int2(kNoEnd, 0);
      __syncwarp();

      // the bag that holds my first entry
      int kb = 0;
#pragma unroll
      for (int step = 16; step >= 1; step >>= 1) {
        const int t = __shfl_sync(kFull, ch.hi, kb + step - 1);
        if (t <= s) kb += step;
      }
      int kend = __shfl_sync(kFull, ch.hi, kb);
      const int klo = __shfl_sync(kFull, ch.lo, kb);
      BagCursor cur;
      cur.init(items + __popc(nz & ((1u << kb) - 1u)));  // its place in the list
      const bool began_earlier = klo < s && e_end > s;
      const bool had_head = began_earlier && kend <= e_end;  // it ends inside my piece: its first part lies in earlier pieces
      const bool inside_one = began_earlier && kend > e_end;  // my whole piece lies inside one bag
      const int head_bag = kb;
      if (kend > e_end) kend = kNoEnd;
      int e = s;
      float acc[V];
      zero_vals<V>(acc);

      if constexpr (D == 0) {
        for (int k = 0; k < ls; k += U) {
          int p[U];
          bool ok[U];
          typename Ops::Raw rows[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            p[u] = e + u;
            ok[u] = p[u] < e_end;
          }
          if (k + U <= q) fetch_rows<T, V, U, IDX64, false>(c, vp, tcol, col_ok, p, ok, rows);
          else fetch_rows<T, V, U, IDX64, true>(c, vp, tcol, col_ok, p, ok, rows);
          if (__all_sync(kFull, e + U < kend)) {
#pragma unroll
            for (int u = 0; u < U; ++u) Ops::add(acc, rows[u]);
            e += U;
          } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
              Ops::add(acc, rows[u]);
              if (++e == kend) {
                if (col_ok) walk_store<V, FS>(orow + (size_t)((unsigned)kb * (uint64_t)ld_bytes), acc, ov, dt);
                zero_vals<V>(acc);
                cur.advance(e_end, kb, kend);
              }
            }
          }
        }
      } else {
        const unsigned cell = smem_addr(ring) + lane * 16;  // my 16-byte cell of ring slot 0, entry 0
        const int nsteps = (ls + U - 1) / U;
        bool bad = false;
        unsigned cell_in = cell;  // ring cursors: copies go in by shared-memory address, rows come out by pointer
        const unsigned cell_end = cell + D * U * 512;
        const unsigned char* const ring_lane = ring + lane * 16;
        int out_off = 0;
        // iteration m issues the copies of macro-step m + D - 1, fetches the indices of macro-step m + D and, from
        // m = 0 on, consumes macro-step m.  The indices fetched in one iteration are first looked at in the next
        // one (validity test and copies), a whole macro-step of work later.
#pragma unroll 1
        for (int m = 1 - D; m < nsteps; ++m) {
          const int first = s + (m + D - 1) * U;
          if (m + D - 1 >= nsteps) {
            // past every piece's end: an empty copy group keeps the group count in step
          } else {
            bool plain = false;
            if (full) {
              bool valid = true;
#pragma unroll
              for (int u = 0; u < U; ++u) {
                if constexpr (IDX64) valid = valid && (uint64_t)idx[u] < (uint64_t)c.rows;
                else valid = valid && (unsigned)idx[u] < rows32;
              }
              plain = __all_sync(kFull, valid);
            }
            if (plain) {
              // every slot has U real entries with valid indices: no predicate on the copies
              if (col_ok) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                  if constexpr (IDX64) cp_async16(cell_in + u * 512, tcol + idx[u] * (int64_t)c.row_bytes, 16u);
                  else cp_async16(cell_in + u * 512, tcol + (uint64_t)(unsigned)idx[u] * (unsigned)c.row_bytes, 16u);
                }
              }
            } else {
              bad |= issue_rows<T, U, IDX64>(c, tcol, col_ok, idx, first, e_end, cell_in);
            }
          }
          cp_async_commit();
          full = (m + D + 1) * U <= q;
          if (full) {
#pragma unroll
            for (int u = 0; u < U; ++u) idx[u] = __ldg(vp + first + U + u);
          } else if (m + D < nsteps) {
            load_indices<U, IDX64>(vp, first + U, e_end, col_ok, idx);
          }
          cell_in += U * 512;
          if (cell_in == cell_end) cell_in = cell;
          if (m < 0) continue;
          cp_async_wait<D - 1>();
          // rows are read out of the ring where they are added: holding all U of them in registers across the
          // branch below costs more (spills at 3 CTAs per SM) than it saves
#define EB_ROW(u) (*reinterpret_cast<const uint4*>(ring_lane + out_off + (u) * 512))
          if (__all_sync(kFull, e + U < kend)) {
#pragma unroll
            for (int u = 0; u < U; ++u) Ops::add(acc, EB_ROW(u));
            e += U;
          } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
              Ops::add(acc, EB_ROW(u));
              if (++e == kend) {
                if (col_ok) walk_store<V, FS>(orow + (size_t)((unsigned)kb * (uint64_t)ld_bytes), acc, ov, dt);
                zero_vals<V>(acc);
                cur.advance(e_end, kb, kend);
              }
            }
          }
          out_off += U * 512;
          if (out_off == D * U * 512) out_off = 0;
        }
#undef EB_ROW
        cp_async_wait<0>();  // the ring is reused by the next chunk
        if (bad) flag(c.status, kStatusBadIndex);
      }

      // patch the bags cut by piece boundaries
      asm volatile("" ::: "memory");  // the head partials are read back below: keep those loads after the walk's stores
      if (R > 1 && __any_sync(kFull, had_head)) {
        bool f = !inside_one;  // my tail starts a new run unless my whole piece lies inside one bag
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          if (d < R) {
            const bool take = (r >= d) && !f;
            const int fv = __shfl_up_sync(kFull, (int)f, d << lgG);
#pragma unroll
            for (int k = 0; k < V; ++k) {
              const float y = __shfl_up_sync(kFull, acc[k], d << lgG);
              if (take) acc[k] += y;
            }
            if (take) f = fv != 0;
          }
        }
        float prev[V];
#pragma unroll
        for (int k = 0; k < V; ++k) prev[k] = __shfl_up_sync(kFull, acc[k], G);
        if (had_head && col_ok) {
          char* dst = orow + (size_t)((unsigned)head_bag * (uint64_t)ld_bytes);
          float hv[V];
          reload_add<V>(dst, prev, hv, ov, dt);
          walk_store<V, FS>(dst, hv, ov, dt);
        }
      }
    }
  }
}

}  // namespace ebk
