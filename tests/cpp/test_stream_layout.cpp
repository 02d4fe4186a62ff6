// Host-side check of the decode kernel's weight-stream bookkeeping (csrc/kernels.h): the tile order of the packed
// stream is a permutation in which every CTA's tiles are consecutive, and cutting a CTA's units into ring stages
// covers every unit exactly once, in order, with the two tiles of a stage adjacent in memory. No GPU involved.
#include <cstdio>
#include <vector>

#include "kernels.h"

using namespace vkl;

static int check(uint32_t tiles, uint32_t grid, uint32_t blocks) {
  std::vector<int> seen(tiles, 0);
  for (uint32_t t = 0; t < tiles; ++t) {
    const uint32_t pos = mega_stream_tile(t, tiles, grid);
    if (pos >= tiles || seen[pos]++) return 1;  // a permutation
  }
  for (uint32_t tile0 = 0; tile0 < grid && tile0 < tiles; ++tile0) {
    const uint32_t tl = (tiles - tile0 + grid - 1) / grid;
    for (uint32_t lt = 1; lt < tl; ++lt)  // a CTA's tiles follow each other
      if (mega_stream_tile(tile0 + lt * grid, tiles, grid) != mega_stream_tile(tile0, tiles, grid) + lt) return 2;
    // stage cutting: every unit once, in order
    uint32_t tm = 0, kg = 0;
    uint64_t next_unit = 0;  // position in the CTA's own unit sequence
    uint32_t stages = 0;
    while (tm < tl) {
      const MegaCut cut = mega_stage_cut(kg, blocks, tm + 1 < tl);
      if (cut.n0 == 0 || cut.n0 + cut.n1 > MEGA_SU) return 3;
      if ((uint64_t)tm * blocks + kg != next_unit) return 4;
      if (cut.n1 && kg + cut.n0 != blocks) return 5;  // the second tile's units start where the first tile ends
      next_unit += cut.n0 + cut.n1;
      mega_stage_advance(cut, blocks, tm, kg);
      if (++stages > 1000000) return 6;
    }
    if (next_unit != (uint64_t)tl * blocks) return 7;
  }
  return 0;
}

int main() {
  const uint32_t grids[] = {1, 2, 7, 132, 148};
  const uint32_t tile_counts[] = {1, 3, 128, 147, 148, 149, 160, 384, 480, 688, 864, 1000};
  const uint32_t block_counts[] = {1, 2, 29, 30, 31, 40, 128, 160, 344, 432};
  for (uint32_t g : grids)
    for (uint32_t t : tile_counts)
      for (uint32_t b : block_counts)
        if (int rc = check(t, g, b)) {
          std::printf("FAIL tiles=%u grid=%u blocks=%u code=%d\n", t, g, b, rc);
          return 1;
        }
  // attention split helpers: the splits of a KV length cover it exactly
  for (uint32_t L = 1; L <= 4096; L += (L < 700 ? 1 : 97))
    for (uint32_t splits : {1u, 3u, 4u, 8u, 29u})
      for (uint32_t split_rows : {0u, 128u, 384u}) {
        const uint32_t S = mega_splits(L, splits, split_rows);
        if (S < 1 || S > splits) {
          std::printf("FAIL splits L=%u\n", L);
          return 1;
        }
        uint32_t at = 0;
        for (uint32_t s = 0; s < S; ++s) {
          uint32_t c0, c1;
          mega_kv_range(L, S, s, c0, c1);
          if (c0 != at || c1 < c0) {
            std::printf("FAIL kv range L=%u S=%u s=%u\n", L, S, s);
            return 1;
          }
          at = c1;
        }
        if (at != L) {
          std::printf("FAIL kv cover L=%u S=%u\n", L, S);
          return 1;
        }
      }
  std::printf("OK\n");
  return 0;
}
