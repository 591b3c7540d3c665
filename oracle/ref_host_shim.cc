// ref_host_shim.cc — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// C entry points around the RecFlex reference's host-side text parsers, which
// are compiled from the reference checkout (examples/csrc/warp_per_sample_preprocess.cu,
// examples/csrc/onehot_preprocess.cu) and linked with this shim into
// oracle/_ref/libref_host.so.  tests/golden/make_golden.py runs them to produce
// the parser fixtures; nothing else uses them.
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "onehot_preprocess.cuh"
#include "warp_per_sample_preprocess.cuh"

static std::vector<std::string> split_lines(const char* text, int64_t len, int64_t batch) {
  std::vector<std::string> lines;
  lines.reserve(batch);
  int64_t pos = 0;
  for (int64_t i = 0; i < batch; ++i) {
    int64_t start = pos;
    while (pos < len && text[pos] != '\n') ++pos;
    lines.emplace_back(text + start, text + pos);
    if (pos < len) ++pos;
  }
  return lines;
}

extern "C" {

// ws::StringSplitToInt on `batch` '\n'-separated lines.  Returns the number of indices (or -1 if cap is too
// small); writes batch + 1 offsets, and the reference's tile/block counts for `tile_size` bags per block.
int64_t ref_ws_parse(const char* text, int64_t len, int64_t batch, int tile_size, int32_t* values, int64_t cap,
                     int32_t* offsets, int32_t* num_tiles, int32_t* num_blocks) {
  std::vector<std::string> lines = split_lines(text, len, batch);
  std::vector<int> indices, segment_offsets;
  int tiles = 0, blocks = 0, num_inputs = 0, num_segments = 0;
  ws::StringSplitToInt(lines, tile_size, indices, segment_offsets, tiles, blocks, num_inputs, num_segments);
  if ((int64_t)indices.size() > cap) return -1;
  std::memcpy(values, indices.data(), indices.size() * sizeof(int));
  std::memcpy(offsets, segment_offsets.data(), segment_offsets.size() * sizeof(int));
  *num_tiles = tiles;
  *num_blocks = blocks;
  return (int64_t)indices.size();
}

// onehot::OneHotMultiBlock: one index per (non-empty) line.
int64_t ref_onehot_parse(const char* text, int64_t len, int64_t batch, int max_concurrent_blocks, int tile_size,
                         int32_t* values, int32_t* num_tiles, int32_t* num_blocks) {
  std::vector<std::string> lines = split_lines(text, len, batch);
  std::vector<int> indices;
  int tiles = 0, blocks = 0, num_inputs = 0;
  onehot::OneHotMultiBlock(lines, max_concurrent_blocks, tile_size, indices, tiles, blocks, num_inputs);
  std::memcpy(values, indices.data(), indices.size() * sizeof(int));
  *num_tiles = tiles;
  *num_blocks = blocks;
  return (int64_t)indices.size();
}

}  // extern "C"
