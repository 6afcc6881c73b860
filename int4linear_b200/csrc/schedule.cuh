// Work schedule of the persistent tensor-memory GEMM kernels (host + device).
//
// The reference launches one CTA per 256 x 128 output tile and lets the hardware scheduler fill
// the machine (kernels/linear_v21.cu:20-37).  A persistent kernel with W workers (CTAs, or CTA
// pairs) walks T output tiles itself, and T is rarely a multiple of W:
//
//   whole tiles   tiles [0, whole) go round-robin to the workers and are computed start to end;
//   K cut         the last `sk_tiles` tiles (fewer than W) are laid end to end along K --
//                 sk_tiles * kb_count K blocks -- and that line is cut into `sk_workers`
//                 contiguous, near-equal ranges, one per worker.  A range covers the end of one
//                 tile and/or the start of the next, so a worker computes at most two partial
//                 tiles ("segments").  Every segment ADDS its partial sums into Y (integer adds
//                 commute: the result is bit-exact and does not depend on arrival order); the
//                 segment that holds K block 0 also brings the bias.  The tiles are cleared by a
//                 small kernel launched in front of the GEMM on the same stream, so inside the
//                 GEMM no CTA ever waits for another;
//   half tiles    where partial sums cannot be added into the output (rounded 16-bit output, a
//                 result that is stored into several GPUs), a last wave that would keep at most half
//                 of the workers busy is cut into half-width items instead (about three quarters of
//                 a tile time instead of a whole one).
//
// Every role of the kernel (TMA producer, unpack, UMMA issuer, epilogue) enumerates the same list
// with segment_of(), so the roles agree without talking to each other.
#pragma once

#include <stdint.h>

#ifndef __CUDACC__
#define I4L_HD inline
#else
#define I4L_HD __host__ __device__ __forceinline__
#endif

namespace i4l {

constexpr int kSkMinBlocks = 4;         // shortest K range worth a segment of its own
// What the cut costs beyond its K blocks, in K blocks of main-loop time (0.39 us each for a CTA pair):
// two more epilogues per worker, the last one exposed, plus clearing and read-modify-write traffic
// that grows with the number of cut tiles.  Measured on B200 with the clearing kernel overlapped
// (programmatic dependent launch): 11 K blocks with 34 cut tiles of 74 workers (4096 x 4096 x 8192),
// 18 (4096^3, 34 tiles), 24 (8192^3, 62 tiles).
constexpr double kSkSplitCostBase = 8.0, kSkSplitCostPerFullWave = 20.0;

struct Schedule {
    int tiles_m = 0, tiles_n = 0, kb_count = 0;
    int workers = 0;     // grid size in workers
    int whole = 0;       // tiles computed as they are
    int half_tiles = 0;  // tiles (after the whole ones) cut into two half-width items
    int sk_tiles = 0;    // tiles (after the whole ones) cut along K; never together with half_tiles
    int sk_workers = 0;
};

enum SegMode { kSegStore = 0, kSegAddFirst = 1, kSegAdd = 2 };

struct Segment {
    int tile;            // linear tile index (raster order)
    int kb0, kb1;        // K blocks [kb0, kb1)
    int col_off, width;  // columns of the tile this item covers (half-width items)
    int mode;            // SegMode: stored; added, with the bias; added
};

// Raster order: groups of 16 consecutive M blocks share their W panel in L2.
I4L_HD void tile_coord(const Schedule& s, int tile, int* tm, int* tn)
{
    constexpr int kGroupM = 16;
    const int group_size = kGroupM * s.tiles_n;
    const int group = tile / group_size;
    const int first_m = group * kGroupM;
    const int gm = s.tiles_m - first_m < kGroupM ? s.tiles_m - first_m : kGroupM;
    const int in_group = tile - group * group_size;
    *tm = first_m + in_group % gm;
    *tn = in_group / gm;
}

// First K block (in the line of cut tiles) of worker w.
I4L_HD long long sk_begin(const Schedule& s, int w)
{
    return static_cast<long long>(w) * s.sk_tiles * s.kb_count / s.sk_workers;
}

// The i-th segment of `worker` (i = 0, 1, ...); false when the worker has no more work.
I4L_HD bool segment_of(const Schedule& s, int worker, int bn, int i, Segment* out)
{
    const int items = s.whole + 2 * s.half_tiles;
    Segment g;
    const int item = worker + i * s.workers;  // (no division on this path: it runs before a kernel's first load)
    if (item < items) {
        g.kb0 = 0;
        g.kb1 = s.kb_count;
        g.mode = kSegStore;
        if (item < s.whole) {
            g.tile = item;
            g.col_off = 0;
            g.width = bn;
        } else {
            const int h = item - s.whole;
            g.tile = s.whole + (h >> 1);
            g.col_off = (h & 1) * (bn / 2);
            g.width = bn / 2;
        }
        *out = g;
        return true;
    }
    if (s.sk_tiles == 0 || worker >= s.sk_workers) return false;
    const long long u0 = sk_begin(s, worker), u1 = sk_begin(s, worker + 1);
    if (u1 <= u0) return false;
    const int ta = static_cast<int>(u0 / s.kb_count), tb = static_cast<int>((u1 - 1) / s.kb_count);
    const int mine = worker < items ? (items - worker + s.workers - 1) / s.workers : 0;
    const int j = i - mine;
    int t;
    if (ta == tb) {
        if (j != 0) return false;
        t = ta;
        g.kb0 = static_cast<int>(u0 - static_cast<long long>(ta) * s.kb_count);
        g.kb1 = static_cast<int>(u1 - static_cast<long long>(ta) * s.kb_count);
    } else if (j == 0) {  // the shorter piece first, so that its epilogue hides behind the longer one
        const int len_a = static_cast<int>(static_cast<long long>(tb) * s.kb_count - u0);
        const int len_b = static_cast<int>(u1 - static_cast<long long>(tb) * s.kb_count);
        const bool a_first = len_a <= len_b;
        t = a_first ? ta : tb;
        g.kb0 = a_first ? s.kb_count - len_a : 0;
        g.kb1 = a_first ? s.kb_count : len_b;
    } else if (j == 1) {
        const int len_a = static_cast<int>(static_cast<long long>(tb) * s.kb_count - u0);
        const int len_b = static_cast<int>(u1 - static_cast<long long>(tb) * s.kb_count);
        const bool a_first = len_a <= len_b;
        t = a_first ? tb : ta;
        g.kb0 = a_first ? 0 : s.kb_count - len_a;
        g.kb1 = a_first ? len_b : s.kb_count;
    } else {
        return false;
    }
    g.tile = s.whole + t;
    g.col_off = 0;
    g.width = bn;
    g.mode = g.kb0 == 0 ? kSegAddFirst : kSegAdd;
    *out = g;
    return true;
}

// Chooses the schedule for tiles_m x tiles_n output tiles of `kb_count` K blocks on at most
// `max_workers` workers.  can_add: partial sums may be added into the output (int32 Y of one GPU);
// can_halve: half-width items are available; force_add: cut whenever it is possible, whatever the
// estimate says (tests, experiments); block_time: time of this tile shape's K block relative to the
// CTA pair's (the cut's overhead is a time, and counts for fewer of the longer K blocks);
// cut_overhead >= 0: the cut's overhead in K blocks of the calling kernel, measured for that kernel,
// instead of the estimate for 256 x 256 pair tiles.  *cost receives the time of the busiest worker in
// tile times, for the dispatcher's choice between tile shapes.
inline Schedule plan_schedule(int tiles_m, int tiles_n, int kb_count, int max_workers, bool can_add, bool can_halve,
                              double* cost = nullptr, bool force_add = false, double block_time = 1.0,
                              double cut_overhead = -1.0)
{
    Schedule s;
    s.tiles_m = tiles_m;
    s.tiles_n = tiles_n;
    s.kb_count = kb_count;
    const int tiles = tiles_m * tiles_n;
    const int rem = tiles % max_workers;
    s.whole = tiles;
    s.workers = tiles < max_workers ? tiles : max_workers;
    double c = static_cast<double>((tiles + max_workers - 1) / max_workers);
    if (rem > 0) {
        const long long units = static_cast<long long>(rem) * kb_count;
        long long skw = units / kSkMinBlocks;
        if (skw > max_workers) skw = max_workers;
        const long long longest = skw > 0 ? (units + skw - 1) / skw : kb_count;
        const double overhead = cut_overhead >= 0.0 ? cut_overhead
                                                    : (kSkSplitCostBase + kSkSplitCostPerFullWave * rem / max_workers) / block_time;
        const double cut_cost = (static_cast<double>(longest) + overhead) / kb_count;
        // A half-width item still expands the whole X tile: about 0.75 of a tile time; a launch that
        // consists of nothing else is dominated by filling the pipeline (measured).
        const bool halvable = can_halve && 2 * rem <= max_workers;
        const double half_cost = halvable ? (tiles > rem ? 0.75 : 1.0) : 1.0;
        if (can_add && kb_count >= kSkMinBlocks && skw >= rem && (cut_cost < half_cost || force_add)) {
            s.whole = tiles - rem;
            s.sk_tiles = rem;
            s.sk_workers = static_cast<int>(skw);
            s.workers = s.whole > 0 ? max_workers : s.sk_workers;
            c = s.whole / max_workers + cut_cost;
        } else if (halvable) {
            s.whole = tiles - rem;
            s.half_tiles = rem;
            s.workers = s.whole > 0 ? max_workers : 2 * rem;
            c = s.whole / max_workers + half_cost;
        }
    }
    if (cost) *cost = c;
    return s;
}

}  // namespace i4l
