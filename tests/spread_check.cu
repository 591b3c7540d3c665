// Host-side check of ebk::spread_tile (recflex_b200/csrc/eb_common.cuh): for every (bags per tile, ranks, rows per
// rank) it must be a bijection on the feature's tiles, keep every tile inside one rank's rows, and send consecutive
// tiles to consecutive ranks.  Prints "ok <cases>" or the first failing case.
#include <cstdio>
#include <vector>

#include "eb_common.cuh"

int main() {
  long cases = 0;
  const int ns[] = {1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024};
  const int worlds[] = {1, 2, 3, 4, 8, 16};
  const long long rpps[] = {32, 64, 96, 160, 512, 1024, 8192};
  for (int n : ns)
    for (int world : worlds)
      for (long long rpp : rpps) {
        const long long batch = rpp * world;
        const long long tiles = (batch + n - 1) / n;
        std::vector<char> seen(tiles, 0);
        const bool spreads = world > 1 && rpp % n == 0;
        for (long long i = 0; i < tiles; ++i) {
          const long long t = ebk::spread_tile(i, n, world, rpp);
          if (t < 0 || t >= tiles || seen[t]) {
            printf("not a bijection: n=%d world=%d rpp=%lld tile %lld -> %lld\n", n, world, rpp, i, t);
            return 1;
          }
          seen[t] = 1;
          if (!spreads) {
            if (t != i) {
              printf("batch order expected: n=%d world=%d rpp=%lld tile %lld -> %lld\n", n, world, rpp, i, t);
              return 1;
            }
            continue;
          }
          const long long first = t * n, last = first + n - 1;
          if (first / rpp != last / rpp || first / rpp != i % world) {
            printf("wrong rank: n=%d world=%d rpp=%lld tile %lld -> bags [%lld, %lld]\n", n, world, rpp, i, first, last);
            return 1;
          }
        }
        ++cases;
      }
  printf("ok %ld\n", cases);
  return 0;
}
