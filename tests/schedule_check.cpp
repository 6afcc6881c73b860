// CPU check of the tile schedule of the persistent GEMM kernels (int4linear_b200/csrc/schedule.cuh):
// for many (tiles, K blocks, workers) combinations every K block of every tile must be computed
// exactly once; a tile that is cut along K must have exactly one segment that starts at K block 0
// (the one that brings the bias) and all of its segments must add; whole tiles and half-width items
// must store; the half-width items of a tile must cover its two halves; no worker may get more than
// two partial segments.  Prints "SCHEDULE_OK <cases>".
#include <cstdio>
#include <vector>

#include "../int4linear_b200/csrc/schedule.cuh"

using namespace i4l;

static int check(int tiles_m, int tiles_n, int kb, int workers, bool can_add, bool can_halve)
{
    const int bn = 256;
    double cost = 0.0;
    const Schedule s = plan_schedule(tiles_m, tiles_n, kb, workers, can_add, can_halve, &cost);
    const int tiles = tiles_m * tiles_n;
    if (s.whole + s.half_tiles + s.sk_tiles != tiles) return 1;
    if (s.half_tiles && s.sk_tiles) return 2;
    if (s.workers < 1 || s.workers > workers) return 3;
    if ((!can_add && s.sk_tiles) || (!can_halve && s.half_tiles)) return 4;
    std::vector<int> cover(static_cast<size_t>(tiles) * kb * 2, 0);  // [tile][kb][half]
    std::vector<int> firsts(tiles, 0), adds(tiles, 0), stores(tiles, 0);
    for (int w = 0; w < s.workers; ++w) {
        Segment g;
        int partial = 0;
        for (int i = 0; segment_of(s, w, bn, i, &g); ++i) {
            if (g.tile < 0 || g.tile >= tiles || g.kb0 < 0 || g.kb1 > kb || g.kb0 >= g.kb1) return 5;
            if (g.width != bn && g.width != bn / 2) return 6;
            if (g.mode == kSegStore) {
                ++stores[g.tile];
                if (g.kb0 != 0 || g.kb1 != kb || g.tile >= s.whole + s.half_tiles) return 7;
            } else {
                ++partial;
                ++adds[g.tile];
                if (g.tile < s.whole || g.width != bn || g.col_off != 0) return 8;
                if ((g.mode == kSegAddFirst) != (g.kb0 == 0)) return 9;
                if (g.mode == kSegAddFirst) ++firsts[g.tile];
            }
            for (int b = g.kb0; b < g.kb1; ++b)
                for (int h = 0; h < 2; ++h)
                    if (g.width == bn || g.col_off == h * (bn / 2)) ++cover[(static_cast<size_t>(g.tile) * kb + b) * 2 + h];
            if (i > 1000000) return 10;
        }
        if (partial > 2) return 11;
    }
    for (int v : cover) if (v != 1) return 12;
    for (int t = 0; t < tiles; ++t) {
        if (adds[t] > 0 && (firsts[t] != 1 || stores[t] != 0)) return 13;
        if (adds[t] == 0 && firsts[t] != 0) return 14;
    }
    if (cost <= 0.0) return 15;
    // the raster must be a bijection between tile indices and (row block, column block)
    std::vector<int> seen(tiles, 0);
    for (int t = 0; t < tiles; ++t) {
        int tm, tn;
        tile_coord(s, t, &tm, &tn);
        if (tm < 0 || tm >= tiles_m || tn < 0 || tn >= tiles_n) return 16;
        ++seen[tm * tiles_n + tn];
    }
    for (int v : seen) if (v != 1) return 17;
    return 0;
}

int main()
{
    long cases = 0;
    const int worker_counts[] = {1, 2, 3, 7, 64, 66, 74, 132, 148};
    const int kbs[] = {1, 2, 3, 4, 5, 8, 13, 32, 64, 127, 1023};
    for (int workers : worker_counts)
        for (int kb : kbs)
            for (int tm = 1; tm <= 40; tm += (tm < 6 ? 1 : 7))
                for (int tn = 1; tn <= 120; tn += (tn < 9 ? 1 : 13))
                    for (int mode = 0; mode < 4; ++mode) {
                        const int rc = check(tm, tn, kb, workers, mode & 1, mode & 2);
                        if (rc) {
                            std::printf("SCHEDULE_BAD rc=%d tiles=%dx%d kb=%d workers=%d mode=%d\n", rc, tm, tn, kb, workers, mode);
                            return 1;
                        }
                        ++cases;
                    }
    // the shapes the design notes quote
    Schedule s = plan_schedule(32, 4, 64, 74, true, true);   // 8192 x 1024 x 8192 on 74 CTA pairs: 128 = 74 + 54, the cut does not pay
    if (s.sk_tiles != 0 || s.half_tiles != 0 || s.whole != 128) { std::printf("SCHEDULE_BAD m8 shard\n"); return 1; }
    s = plan_schedule(32, 4, 64, 74, true, true, nullptr, true);   // ... unless it is forced
    if (s.sk_tiles != 54 || s.whole != 74 || s.sk_workers != 74) { std::printf("SCHEDULE_BAD m8 shard, forced\n"); return 1; }
    s = plan_schedule(32, 14, 64, 74, true, true);            // 8192 x 3584 x 8192: 448 = 6 * 74 + 4
    if (s.sk_tiles != 4 || s.whole != 444 || s.sk_workers != 64) { std::printf("SCHEDULE_BAD c5 shard\n"); return 1; }
    s = plan_schedule(32, 14, 64, 74, false, true);
    if (s.half_tiles != 4 || s.sk_tiles != 0) { std::printf("SCHEDULE_BAD c5 shard, half\n"); return 1; }
    s = plan_schedule(16, 16, 32, 74, true, true);            // 4096^3: the half-width tail is cheaper than the cut
    if (s.half_tiles != 34 || s.sk_tiles != 0) { std::printf("SCHEDULE_BAD c2\n"); return 1; }
    s = plan_schedule(16, 16, 64, 74, true, true);            // 4096 x 4096 x 8192: the cut is (just) cheaper
    if (s.sk_tiles != 34 || s.half_tiles != 0) { std::printf("SCHEDULE_BAD c3\n"); return 1; }
    std::printf("SCHEDULE_OK %ld\n", cases);
    return 0;
}
