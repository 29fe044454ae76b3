// Host check of the tile partition shared by the tiled decode kernel and its merge kernel:
// the 32-bit tile-range functions against a 64-bit restatement; the ranges must tile the flat list.
// Built and run by tests/test_host.py::test_tile_partition_matches_bruteforce.
#include <cstdio>
#include <vector>
#include "../muzero_b200/csrc/mz_decode.cuh"
int check(int pairs, int packed, int dense_tiles, int cq, int cd, long long W) {
  MzTilesPlan t{};
  t.packed_tiles = packed; t.cost_q = cq; t.cost_d = cd; t.tiles_per_pair = packed + dense_tiles;
  t.total_tiles = (long long)pairs * t.tiles_per_pair;
  t.pair_cost = (long long)packed * cq + (long long)dense_tiles * cd; if (t.pair_cost < 1) t.pair_cost = 1;
  t.total_cost = pairs * t.pair_cost; t.total_warps = (int)W;
  t.cost_quot = (unsigned)(t.total_cost / W); t.cost_rem = (unsigned)(t.total_cost % W);
  long long prev = 0; int bad = 0;
  for (long long g = 0; g < W; ++g) {
    long long f0, f1; mz_warp_tiles(t, g, &f0, &f1);
    // reference: 64-bit formulas
    auto before = [&](long long c) { long long pair = c / t.pair_cost, r = c % t.pair_cost, qc = (long long)packed * cq;
      long long in = r <= qc ? (r + cq - 1) / cq : packed + (r - qc + cd - 1) / cd; return pair * t.tiles_per_pair + in; };
    long long r0 = before(g * t.total_cost / W), r1 = before((g + 1) * t.total_cost / W);
    if (f0 != r0 || f1 != r1 || f0 != prev || f1 < f0) { if (bad < 3) printf("  g=%lld got [%lld,%lld) ref [%lld,%lld) prev %lld\n", g, f0, f1, r0, r1, prev); ++bad; }
    prev = f1;
  }
  if (prev != t.total_tiles) { printf("  end %lld != %lld\n", prev, t.total_tiles); ++bad; }
  printf("pairs %d packed %d dense %d W %lld: %s\n", pairs, packed, dense_tiles, W, bad ? "BAD" : "ok");
  return bad;
}
int main() {
  int bad = 0;
  bad += check(8, 62, 8, 74, 32, 8); bad += check(8, 62, 8, 74, 32, 16); bad += check(8, 62, 8, 74, 32, 40); bad += check(8, 62, 8, 74, 32, 512);
  bad += check(512, 64, 8, 74, 32, 1776); bad += check(4, 2, 5, 74, 32, 256); bad += check(3, 0, 8, 74, 32, 7); bad += check(16, 9, 8, 42, 32, 16 * 5);
  bad += check(2, 9, 8, 74, 32, 128); bad += check(64, 2048, 8, 74, 32, 1776); bad += check(1, 1, 0, 138, 48, 1); bad += check(512, 512, 8, 74, 32, 70000);
  return bad != 0;
}
