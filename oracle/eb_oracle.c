/*
 * eb_oracle.c — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement of what RecFlex's fused embedding-bag forward computes, used
 * only by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline and
 * reference arms as the checker / the reported CPU baseline.  Nothing in the
 * recflex_b200 package may call it.
 *
 * What it restates (paths relative to the RecFlex repository):
 *   oracle_pool_*      the expected result of the fused kernel as defined by the
 *                      reference's own checker, examples/test.py:68-86: for
 *                      every feature and sample, look up the sample's indices
 *                      in the feature's table and sum the rows
 *                      (F.embedding(indices, table).sum(0)); an empty line gives
 *                      zeros; results are laid out [batch, sum(dim)] with the
 *                      features side by side (examples/test.py:73,
 *                      RecFlex/rec_modules.py:177).  The device kernels that
 *                      produce it are ws::SparseSegmentReduceCore
 *                      (examples/csrc/include/warp_per_sample_kernel.cuh:10-68),
 *                      obms:: (one_block_multi_sample_kernel.cuh:16-108) and
 *                      onehot::GatherSegmentsCore (onehot_kernel.cuh:14-47).
 *   oracle_parse_bags  the text -> CSR step, ws::StringSplitToInt
 *                      (examples/csrc/warp_per_sample_preprocess.cu:6-38).
 *   oracle_synth_rows  the synthetic table weights of this repository's
 *                      benchmarks (no counterpart in the reference, which uses
 *                      torch.randn / torch.ones tables).
 *
 * Parity pin: tests/golden/ holds inputs and outputs produced in this
 * repository's build container by the reference's Python checker formula and by
 * the reference's host parser compiled from its own sources (see
 * tests/golden/make_golden.py and oracle/build_ref.sh); tests/test_oracle.py
 * checks this file against them.
 */
#include <stdint.h>
#include <string.h>

/* IEEE binary16 -> binary32, all cases (subnormals, inf, nan). */
static float half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while ((man & 0x400u) == 0);
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp - 15 + 127) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, sizeof(f));
  return f;
}

/*
 * Pool one feature.  table: [rows, dim] (fp32 when table_f16 == 0, binary16
 * otherwise); values: nnz indices; offsets: batch + 1 bag boundaries; out:
 * [batch, out_ld] fp32, this feature's columns start at col_off.
 * acc64 != 0 accumulates in double (used to bound both sides' rounding error),
 * else in float in index order.
 * Returns 0, or -1 when an index or an offset is out of range (nothing is read
 * out of bounds; the offending entry is skipped).
 */
int oracle_pool_feature(const void* table, int table_f16, int64_t rows, int32_t dim, const int64_t* values,
                        const int64_t* offsets, int64_t batch, float* out, int64_t out_ld, int64_t col_off,
                        int acc64) {
  int rc = 0;
  const float* tf = (const float*)table;
  const uint16_t* th = (const uint16_t*)table;
  for (int64_t b = 0; b < batch; ++b) {
    float* dst = out + b * out_ld + col_off;
    int64_t s = offsets[b], e = offsets[b + 1];
    if (s < 0 || e < s) {
      rc = -1;
      e = s;
    }
    for (int32_t c = 0; c < dim; ++c) {
      double a64 = 0.0;
      float a32 = 0.0f;
      for (int64_t p = s; p < e; ++p) {
        const int64_t idx = values[p];
        if (idx < 0 || idx >= rows) {
          rc = -1;
          continue;
        }
        const float w = table_f16 ? half_to_float(th[idx * dim + c]) : tf[idx * dim + c];
        if (acc64) a64 += (double)w; else a32 += w;
      }
      dst[c] = acc64 ? (float)a64 : a32;
    }
  }
  return rc;
}

/*
 * Text -> CSR for one feature: `text` holds `batch` lines separated by '\n'.
 * Inside a line every byte outside '0'..'9' ends the current number (which is 0
 * when no digit preceded it) and, when the line is not empty, what remains at
 * its end is a number as well.  Returns the number of indices written, or -1 if
 * `cap` is too small.
 */
int64_t oracle_parse_bags(const char* text, int64_t len, int64_t batch, int32_t* values, int64_t cap,
                          int32_t* offsets) {
  int64_t n = 0, pos = 0;
  offsets[0] = 0;
  for (int64_t line = 0; line < batch; ++line) {
    int64_t start = pos;
    int32_t cur = 0;
    while (pos < len && text[pos] != '\n') {
      const char ch = text[pos++];
      if (ch < '0' || ch > '9') {
        if (n >= cap) return -1;
        values[n++] = cur;
        cur = 0;
      } else {
        cur = cur * 10 + (ch - '0');
      }
    }
    if (pos > start) {
      if (n >= cap) return -1;
      values[n++] = cur;
    }
    if (pos < len) ++pos;
    offsets[line + 1] = (int32_t)n;
  }
  return n;
}

static uint64_t mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

/* Rows `row_ids[0..n)` of the synthetic table `seed`, as fp32 (before any cast to binary16). */
void oracle_synth_rows(uint64_t seed, const int64_t* row_ids, int64_t n, int32_t dim, float std, float* out) {
  const float scale = std / 37837.227f;
  for (int64_t i = 0; i < n; ++i) {
    for (int32_t c = 0; c < dim; ++c) {
      const uint64_t elem = (uint64_t)row_ids[i] * (uint64_t)dim + (uint64_t)c;
      const uint64_t h = mix64(seed * 0xD1342543DE82EF95ull + elem);
      const int s = (int)(h & 0xffff) + (int)((h >> 16) & 0xffff) + (int)((h >> 32) & 0xffff) +
                    (int)((h >> 48) & 0xffff) - 131070;
      out[i * dim + c] = (float)s * scale;
    }
  }
}
