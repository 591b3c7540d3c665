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
  float* out;        // already advanced to the feature's first column (unused in peer mode)
  int64_t out_ld;
  float* const* peer_out;  // peer mode: every rank's output matrix
  int64_t rows_per_peer;   // 0 = single output matrix
  int32_t col_off;
  uint32_t* status;
  int32_t dim;
  int32_t row_bytes;
  int32_t lg_group;
  int32_t nx;
  bool idx64;
  bool has_end;
  int out_vec;       // widest aligned store the output allows: 0 = scalar, 1 = 16 bytes, 2 = 32 bytes
};

__device__ __forceinline__ int64_t load_index(const char* base, int64_t i, bool idx64) {
  return idx64 ? (int64_t)__ldg(reinterpret_cast<const long long*>(base) + i)
               : (int64_t)__ldg(reinterpret_cast<const int*>(base) + i);
}

// First output element (this feature's first column) of bag `bb`.  In peer mode
// the bag's row lives in the output matrix of rank bb / rows_per_peer; chunks of
// 32 bags never straddle two ranks because rows_per_peer is a multiple of 32.
__device__ __forceinline__ float* chunk_out(const TileCtx& c, int64_t bb) {
  if (c.rows_per_peer == 0) return c.out + bb * c.out_ld;
  const int64_t d = bb / c.rows_per_peer;
  return c.peer_out[d] + c.col_off + (bb - d * c.rows_per_peer) * c.out_ld;
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
template <int V>
__device__ __forceinline__ void store_vals(float* dst, const float (&a)[V], int vec_ok) {
  if constexpr (V == 1) {
    __stcs(dst, a[0]);
  } else {
    if constexpr (V == 8) {
      if (vec_ok == 2) {
        asm volatile("st.global.cs.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "f"(a[0]), "f"(a[1]),
                     "f"(a[2]), "f"(a[3]), "f"(a[4]), "f"(a[5]), "f"(a[6]), "f"(a[7])
                     : "memory");
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

__device__ __forceinline__ Chunk load_chunk(const TileCtx& c, int64_t bb, int nb, int lane) {
  const int li = lane <= nb ? lane : nb;
  const int64_t a_raw = raw_offset(c, bb + li);
  int64_t end_raw = __shfl_sync(kFull, a_raw, 31);
  if (nb == 32) end_raw = raw_offset(c, bb + 32);
  int64_t m = clamp_off(a_raw, c.nnz);
  int64_t endm = clamp_off(end_raw, c.nnz);
  bool bad = (m != a_raw) || (endm != end_raw);
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int64_t t = __shfl_up_sync(kFull, m, d);
    if (lane >= d && t > m) { m = t; bad = true; }
  }
  const int64_t m31 = __shfl_sync(kFull, m, 31);
  if (m31 > endm) { endm = m31; bad = true; }
  Chunk ch;
  ch.e0 = __shfl_sync(kFull, m, 0);
  int64_t nxt = __shfl_down_sync(kFull, m, 1);
  if (lane == 31) nxt = endm;
  int64_t total = endm - ch.e0;
  if (total > 0x3fffffff) { total = 0x3fffffff; bad = true; }  // more than 2^30 indices in 32 bags: refuse the excess
  int64_t lo = m - ch.e0, hi = nxt - ch.e0;
  if (lo > total) lo = total;
  if (hi > total) hi = total;
  ch.lo = (int)lo;
  ch.hi = (int)hi;
  ch.n = (int)total;
  if (__any_sync(kFull, bad) && lane == 0) flag(c.status, kStatusBadOffsets);
  return ch;
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
      const Chunk ch = load_chunk(c, bb, nb, lane);
      float* orow = chunk_out(c, bb) + cs;
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
        if (bi < nb && col_ok) store_vals<V>(orow + (int64_t)bi * c.out_ld, acc, c.out_vec);
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
      const Chunk ch = load_chunk(c, bb, nb, lane);
      float* orow = chunk_out(c, bb) + cs;
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
        if (r == 0 && col_ok) store_vals<V>(orow + (int64_t)i * c.out_ld, acc, c.out_vec);
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
      const Chunk ch = load_chunk(c, bb, nb, lane);
      float* orow = chunk_out(c, bb) + cs;
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
          if (i >= 0 && col_ok) store_vals<V>(orow + (int64_t)i * c.out_ld, z, c.out_vec);
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
                if (r == 0 && col_ok) store_vals<V>(orow + (int64_t)wbag * c.out_ld, acc, c.out_vec);
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
                  store_vals<V>(orow + (int64_t)mybag * c.out_ld, x, c.out_vec);
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
// EB_SCHED_STREAM: the chunk's n entries are cut into R contiguous pieces of
// ceil(n / R) entries, one per slot.  Every slot walks its piece serially with
// U rows in flight, whatever the bag lengths: a bag that ends inside the piece
// is stored at once (a warp vote guards the store path, so steps without a
// boundary pay one vote).  While a whole macro-step of U entries stays inside
// the current bag for every slot, the walk is a pure load + accumulate loop.
// A bag cut by a piece boundary leaves a tail partial in the slot's
// accumulator and a head partial in the output row; after the walk a segmented
// shuffle scan over the slots' tails patches each head (once per 32 bags).
// ---------------------------------------------------------------------------
//
// D > 0 selects the pipelined form (EB_SCHED_PIPE): the rows in flight live in a
// per-warp shared-memory ring of D macro-steps (D * U * 512 bytes) filled by
// per-lane cp.async copies instead of in registers, so D * U rows per lane are
// in flight (against U) and the row registers are free; the walk, the stores
// and the patch pass are the same.
template <typename T, int V, int U, bool IDX64, int D = 0>
__device__ __forceinline__ void tile_stream(const TileCtx& c, int64_t b0, int64_t b1, int lane,
                                            unsigned char* ring = nullptr) {
  static_assert(D == 0 || V * sizeof(T) == 16, "the ring holds 16-byte lane cells");
  using Ops = RowOps<T, V>;
  using IdxT = typename IdxOf<IDX64>::type;
  const int lgG = c.lg_group, lgR = 5 - lgG, G = 1 << lgG, R = 1 << lgR;
  const int r = lane >> lgG, cl = lane & (G - 1);
  for (int xc = 0; xc < c.nx; ++xc) {
    const int cs = (xc * G + cl) * V;
    const bool col_ok = cs < c.dim;
    const char* tcol = c.table + (size_t)cs * sizeof(T);
    for (int64_t bb = b0; bb < b1; bb += 32) {
      const int nb = (int)((b1 - bb) < 32 ? (b1 - bb) : 32);
      const Chunk ch = load_chunk(c, bb, nb, lane);
      const int n = ch.n;
      float* orow = chunk_out(c, bb) + cs;
      const unsigned nz = __ballot_sync(kFull, ch.hi > ch.lo);

      // empty bags pool to zero: slot r takes the r-th remaining one
      {
        const unsigned valid = nb == 32 ? kFull : ((1u << nb) - 1u);
        unsigned em = ~nz & valid;
        float z[V];
        zero_vals<V>(z);
        while (em) {
          const int i = (int)__fns(em, 0, r + 1);
          if (i >= 0 && col_ok) store_vals<V>(orow + (int64_t)i * c.out_ld, z, c.out_vec);
          for (int k = 0; k < R && em; ++k) em &= em - 1;
        }
      }
      if (n == 0) continue;

      // my piece [s, e_end) and the bag that holds its first entry
      const int ls = (n + R - 1) >> lgR;
      const int s = min(r * ls, n);
      const int e_end = min(s + ls, n);
      int kb = 0;
#pragma unroll
      for (int step = 16; step >= 1; step >>= 1) {
        const int t = __shfl_sync(kFull, ch.hi, kb + step - 1);
        if (t <= s) kb += step;
      }
      int kend = __shfl_sync(kFull, ch.hi, kb);
      bool head_pending = __shfl_sync(kFull, ch.lo, kb) < s;  // my first bag began in an earlier piece
      bool had_head = false;
      int head_bag = 0;
      int e = s;
      const IdxT* vp = reinterpret_cast<const IdxT*>(c.values) + ch.e0;
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
          const bool inner = (e + U < kend) && (e + U <= e_end);
          if (__all_sync(kFull, inner)) {
            fetch_rows<T, V, U, IDX64, false>(c, vp, tcol, col_ok, p, ok, rows);
  #pragma unroll
            for (int u = 0; u < U; ++u) Ops::add(acc, rows[u]);
            e += U;
          } else {
            fetch_rows<T, V, U, IDX64, true>(c, vp, tcol, col_ok, p, ok, rows);
  #pragma unroll
            for (int u = 0; u < U; ++u) {
              Ops::add(acc, rows[u]);
              const bool at_end = ok[u] && (e + 1 == kend);
              if (__any_sync(kFull, at_end)) {
                const unsigned rest = kb >= 31 ? 0u : (nz & (0xfffffffeu << kb));
                const int nkb = rest ? (__ffs(rest) - 1) : 31;
                int nend = __shfl_sync(kFull, ch.hi, nkb);
                if (!rest) nend = 0x7fffffff;
                if (at_end) {
                  if (col_ok) store_vals<V>(orow + (int64_t)kb * c.out_ld, acc, c.out_vec);
                  if (head_pending) {
                    had_head = true;
                    head_bag = kb;
                    head_pending = false;
                  }
                  zero_vals<V>(acc);
                  kb = nkb;
                  kend = nend;
                }
              }
              e += ok[u] ? 1 : 0;
            }
          }
        }
      } else {
        const unsigned cell = smem_addr(ring) + lane * 16;  // my 16-byte cell of ring slot 0, entry 0
        const int nsteps = (ls + U - 1) / U;
        IdxT idx[U];
        bool bad = false;
        load_indices<U, IDX64>(vp, s, e_end, col_ok, idx);
#pragma unroll
        for (int pm = 0; pm < D - 1; ++pm) {  // fill the pipeline
          bad |= issue_rows<T, U, IDX64>(c, tcol, col_ok, idx, s + pm * U, e_end, cell + pm * U * 512);
          cp_async_commit();
          load_indices<U, IDX64>(vp, s + (pm + 1) * U, e_end, col_ok, idx);
        }
        unsigned cell_in = cell + (D - 1) * U * 512, cell_out = cell;  // ring cursors
        const unsigned cell_end = cell + D * U * 512;
        for (int m = 0; m < nsteps; ++m) {
          bad |= issue_rows<T, U, IDX64>(c, tcol, col_ok, idx, s + (m + D - 1) * U, e_end, cell_in);
          cp_async_commit();
          load_indices<U, IDX64>(vp, s + (m + D) * U, e_end, col_ok, idx);  // indices one macro-step ahead of their copies
          cp_async_wait<D - 1>();
          bool ok[U];
          typename Ops::Raw rows[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            ok[u] = e + u < e_end;
            rows[u] = lds16(cell_out + u * 512);
          }
          const bool inner = (e + U < kend) && (e + U <= e_end);
          if (__all_sync(kFull, inner)) {
#pragma unroll
            for (int u = 0; u < U; ++u) Ops::add(acc, rows[u]);
            e += U;
          } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
              Ops::add(acc, rows[u]);
              const bool at_end = ok[u] && (e + 1 == kend);
              if (__any_sync(kFull, at_end)) {
                const unsigned rest = kb >= 31 ? 0u : (nz & (0xfffffffeu << kb));
                const int nkb = rest ? (__ffs(rest) - 1) : 31;
                int nend = __shfl_sync(kFull, ch.hi, nkb);
                if (!rest) nend = 0x7fffffff;
                if (at_end) {
                  if (col_ok) store_vals<V>(orow + (int64_t)kb * c.out_ld, acc, c.out_vec);
                  if (head_pending) {
                    had_head = true;
                    head_bag = kb;
                    head_pending = false;
                  }
                  zero_vals<V>(acc);
                  kb = nkb;
                  kend = nend;
                }
              }
              e += ok[u] ? 1 : 0;
            }
          }
          cell_in += U * 512;
          if (cell_in == cell_end) cell_in = cell;
          cell_out += U * 512;
          if (cell_out == cell_end) cell_out = cell;
        }
        cp_async_wait<0>();  // the ring is reused by the next chunk
        if (bad) flag(c.status, kStatusBadIndex);
      }

      // patch the bags cut by piece boundaries
      if (R > 1 && __any_sync(kFull, had_head)) {
        bool f = !(head_pending && e_end > s);  // my tail starts a new run unless my whole piece lies inside one bag
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
          float* dst = orow + (int64_t)head_bag * c.out_ld;
          float hv[V];
          if constexpr (V == 1) {
            hv[0] = dst[0] + prev[0];
          } else {
            if (c.out_vec) {
#pragma unroll
              for (int k = 0; k < V; k += 4) {
                const float4 q = *reinterpret_cast<const float4*>(dst + k);
                hv[k] = q.x + prev[k];
                hv[k + 1] = q.y + prev[k + 1];
                hv[k + 2] = q.z + prev[k + 2];
                hv[k + 3] = q.w + prev[k + 3];
              }
            } else {
#pragma unroll
              for (int k = 0; k < V; ++k) hv[k] = dst[k] + prev[k];
            }
          }
          store_vals<V>(dst, hv, c.out_vec);
        }
      }
    }
  }
}

}  // namespace ebk
