// CPU check of the tile schedule of the persistent GEMM kernels (int4linear_b200/csrc/schedule.cuh):
// for many (tiles, K blocks, workers) combinations every K block of every tile must be computed
// exactly once, a tile that is cut along K must have exactly one owning segment and the number of
// adding segments every segment of it reports, an adding segment must be its worker's last, and the
// half-width items of a tile must cover its two halves.  Prints "SCHEDULE_OK <cases>".
#include <cstdio>
#include <vector>

#include "../int4linear_b200/csrc/schedule.cuh"

using namespace i4l;

static int check(int tiles_m, int tiles_n, int kb, int workers, bool can_add, bool can_halve)
{
    const int bn = 256;
    const Schedule s = plan_schedule(tiles_m, tiles_n, kb, workers, can_add, can_halve);
    const int tiles = tiles_m * tiles_n;
    if (s.whole + s.half_tiles + s.sk_tiles != tiles) return 1;
    if (s.half_tiles && s.sk_tiles) return 2;
    if (s.workers < 1 || s.workers > workers) return 3;
    std::vector<int> cover(static_cast<size_t>(tiles) * kb * 2, 0);  // [tile][kb][half]
    std::vector<int> owners(tiles, 0), adds(tiles, 0), claimed(tiles, -1);
    for (int w = 0; w < s.workers; ++w) {
        Segment g;
        bool seen_add = false;
        for (int i = 0; segment_of(s, w, bn, i, &g); ++i) {
            if (seen_add) return 4;  // something after an adding segment
            if (g.tile < 0 || g.tile >= tiles || g.kb0 < 0 || g.kb1 > kb || g.kb0 >= g.kb1) return 5;
            if (g.width != bn && g.width != bn / 2) return 6;
            if (g.mode == kSegAdd) { seen_add = true; ++adds[g.tile]; }
            if (g.mode == kSegOwner) ++owners[g.tile];
            if (g.mode != kSegStore) {
                if (g.tile < s.whole || g.sk_index != g.tile - s.whole || g.sk_index >= kSkMaxTiles) return 7;
                if (claimed[g.tile] >= 0 && claimed[g.tile] != g.adders) return 8;
                claimed[g.tile] = g.adders;
            }
            if (g.mode == kSegStore && (g.kb0 != 0 || g.kb1 != kb)) return 9;
            if ((g.mode == kSegOwner) != (g.kb0 == 0 && g.kb1 < kb)) return 10;
            if ((g.mode == kSegAdd) != (g.kb0 > 0)) return 11;
            for (int b = g.kb0; b < g.kb1; ++b)
                for (int h = 0; h < 2; ++h)
                    if (g.width == bn || g.col_off == h * (bn / 2)) ++cover[(static_cast<size_t>(g.tile) * kb + b) * 2 + h];
            if (i > 1000000) return 12;
        }
    }
    for (int v : cover) if (v != 1) return 13;
    for (int t = 0; t < tiles; ++t) {
        if (adds[t] > 0 && owners[t] != 1) return 14;
        if (adds[t] == 0 && owners[t] != 0) return 15;
        if (adds[t] > 0 && claimed[t] != adds[t]) return 16;
    }
    return 0;
}

int main()
{
    long cases = 0;
    const int worker_counts[] = {1, 2, 3, 7, 64, 66, 74, 132, 148};
    const int kbs[] = {1, 2, 3, 4, 5, 8, 13, 32, 64, 127};
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
    Schedule s = plan_schedule(32, 4, 64, 74, true, true);   // 8192 x 1024 x 8192 on 74 CTA pairs
    if (s.sk_tiles != 54 || s.whole != 74 || s.sk_workers != 74) { std::printf("SCHEDULE_BAD m8 shard\n"); return 1; }
    s = plan_schedule(32, 14, 64, 74, true, true);            // 8192 x 3584 x 8192
    if (s.sk_tiles != 4 || s.whole != 444 || s.sk_workers != 64) { std::printf("SCHEDULE_BAD c5 shard\n"); return 1; }
    s = plan_schedule(32, 14, 64, 74, false, true);
    if (s.half_tiles != 4 || s.sk_tiles != 0) { std::printf("SCHEDULE_BAD c5 shard, half\n"); return 1; }
    std::printf("SCHEDULE_OK %ld\n", cases);
    return 0;
}
