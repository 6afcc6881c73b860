// CPU check of the tile schedule of the persistent GEMM kernels (int4linear_b200/csrc/schedule.cuh):
// for many (tiles, workers) combinations every tile must be covered exactly once -- whole, or by
// its two half-width items -- and no worker may be handed more than its share.
// Prints "SCHEDULE_OK <cases>".
#include <cstdio>
#include <vector>

#include "../int4linear_b200/csrc/schedule.cuh"

using namespace i4l;

static int check(int tiles_m, int tiles_n, int workers, bool can_halve)
{
    const int bn = 256;
    double cost = 0.0;
    const Schedule s = plan_schedule(tiles_m, tiles_n, workers, can_halve, &cost);
    const int tiles = tiles_m * tiles_n;
    if (s.whole + s.half_tiles != tiles) return 1;
    if (s.workers < 1 || s.workers > workers) return 2;
    if (!can_halve && s.half_tiles) return 3;
    std::vector<int> cover(static_cast<size_t>(tiles) * 2, 0);  // [tile][half]
    int busiest = 0;
    for (int w = 0; w < s.workers; ++w) {
        Segment g;
        int i = 0;
        for (; segment_of(s, w, bn, i, &g); ++i) {
            if (g.tile < 0 || g.tile >= tiles) return 4;
            if (g.width == bn) { if (g.col_off != 0) return 5; ++cover[g.tile * 2]; ++cover[g.tile * 2 + 1]; }
            else if (g.width == bn / 2 && (g.col_off == 0 || g.col_off == bn / 2)) ++cover[g.tile * 2 + (g.col_off ? 1 : 0)];
            else return 6;
            if (i > 1000000) return 7;
        }
        if (i > busiest) busiest = i;
    }
    for (int v : cover) if (v != 1) return 8;
    if (busiest > (tiles + workers - 1) / workers + 1) return 9;
    if (cost <= 0.0 || cost > busiest + 1e-9) return 10;
    return 0;
}

int main()
{
    long cases = 0;
    const int worker_counts[] = {1, 2, 3, 7, 64, 66, 74, 132, 148};
    for (int workers : worker_counts)
        for (int tm = 1; tm <= 40; ++tm)
            for (int tn = 1; tn <= 120; tn += (tn < 9 ? 1 : 5))
                for (int halve = 0; halve < 2; ++halve) {
                    const int rc = check(tm, tn, workers, halve != 0);
                    if (rc) {
                        std::printf("SCHEDULE_BAD rc=%d tiles=%dx%d workers=%d halve=%d\n", rc, tm, tn, workers, halve);
                        return 1;
                    }
                    ++cases;
                }
    Schedule s = plan_schedule(32, 14, 74, true);   // 8192 x 3584 outputs on 74 CTA pairs: 448 = 6 * 74 + 4
    if (s.half_tiles != 4 || s.whole != 444 || s.workers != 74) { std::printf("SCHEDULE_BAD c5 shard\n"); return 1; }
    s = plan_schedule(32, 4, 74, true);             // 8192 x 1024: 128 = 74 + 54, too many for halving
    if (s.half_tiles != 0 || s.whole != 128) { std::printf("SCHEDULE_BAD m8 shard\n"); return 1; }
    std::printf("SCHEDULE_OK %ld\n", cases);
    return 0;
}
