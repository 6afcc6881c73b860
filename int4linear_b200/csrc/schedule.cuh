// Work schedule of the persistent tensor-memory GEMM kernels (host + device).
//
// The reference launches one CTA per 256 x 128 output tile and lets the hardware scheduler fill
// the machine (kernels/linear_v21.cu:20-37).  A persistent kernel with W workers (CTAs, or CTA
// pairs) has to cut T output tiles into W equal shares itself, and T is rarely a multiple of W:
//
//   whole tiles   tiles [0, whole) go round-robin to the workers and are computed start to end;
//   stream-K      the last `sk_tiles` tiles (fewer than W) are laid end to end along K --
//                 sk_tiles * kb_count K blocks -- and that line is cut into `sk_workers`
//                 contiguous, near-equal ranges, one per worker.  A range covers the end of one
//                 tile and/or the start of the next, so a worker computes at most two partial
//                 tiles ("segments").  Every segment ADDS its partial sums into Y (integer adds
//                 commute, so the result is bit-exact and does not depend on arrival order).  The
//                 worker whose range contains K block 0 of a tile OWNS it: at the very start of
//                 the kernel it clears the tile in Y and raises the tile's flag, its segment also
//                 brings the bias; every segment checks the flag before it adds;
//   half tiles    where partial sums cannot be added into the output (rounded 16-bit output, a
//                 result that is stored into several GPUs), a last wave that fills at most half
//                 of the workers is cut into half-width items instead.
//
// A worker runs its whole tiles first, then the segment of the tile it owns, then the other one.
// The flags are raised in the first microsecond of the kernel by epilogue warps that have nothing
// else to do yet, so no segment ever waits for another segment's work.
#pragma once

#include <stdint.h>

#ifndef __CUDACC__
#define I4L_HD inline
#else
#define I4L_HD __host__ __device__ __forceinline__
#endif

namespace i4l {

constexpr int kSkMinBlocks = 4;       // shortest K range worth a segment of its own
constexpr int kSkSplitCostBlocks = 6;  // what one more epilogue costs, in K blocks of main-loop time
constexpr int kSkMaxTiles = 160;       // upper bound of sk_tiles (workers never exceed the SM count)
constexpr int kSkRegions = 32;         // flag sets handed to consecutive launches in turn

struct Schedule {
    int tiles_m = 0, tiles_n = 0, kb_count = 0;
    int workers = 0;     // grid size in workers
    int whole = 0;       // tiles computed whole
    int half_tiles = 0;  // tiles cut into two half-width items (after the whole ones)
    int sk_tiles = 0;    // tiles cut along K (after the whole ones); never together with half_tiles
    int sk_workers = 0;
    unsigned* flags = nullptr;  // [kSkMaxTiles][ctas][4 warps][2] words of this launch's region
};

enum SegMode { kSegStore = 0, kSegOwner = 1, kSegAdd = 2 };

struct Segment {
    int tile;            // linear tile index (raster order)
    int kb0, kb1;        // K blocks [kb0, kb1)
    int col_off, width;  // columns of the tile this item covers (half-width items)
    int mode;            // SegMode
    int sk_index;        // tile - whole, for the flag slot (stream-K segments)
    int adders;          // segments of this tile besides the owner's (stream-K)
};

// First K block (in the stream-K line) of worker w.
I4L_HD long long sk_begin(const Schedule& s, int w)
{
    return static_cast<long long>(w) * s.sk_tiles * s.kb_count / s.sk_workers;
}
// Worker whose range contains unit u.
I4L_HD int sk_worker_of(const Schedule& s, long long u)
{
    const long long total = static_cast<long long>(s.sk_tiles) * s.kb_count;
    return static_cast<int>(((u + 1) * s.sk_workers - 1) / total);
}

// The i-th segment of `worker` (i = 0, 1, ...); false when the worker has no more work.
I4L_HD bool segment_of(const Schedule& s, int worker, int bn, int i, Segment* out)
{
    const int items = s.whole + 2 * s.half_tiles;
    const int mine = worker < items ? (items - worker + s.workers - 1) / s.workers : 0;
    Segment g;
    g.sk_index = 0;
    g.adders = 0;
    if (i < mine) {
        const int item = worker + i * s.workers;
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
    const int j = i - mine;
    int t;
    if (ta == tb) {
        if (j != 0) return false;
        t = ta;
        g.kb0 = static_cast<int>(u0 - static_cast<long long>(ta) * s.kb_count);
        g.kb1 = static_cast<int>(u1 - static_cast<long long>(ta) * s.kb_count);
    } else if (j == 0) {  // the start of the later tile first: this worker owns it
        t = tb;
        g.kb0 = 0;
        g.kb1 = static_cast<int>(u1 - static_cast<long long>(tb) * s.kb_count);
    } else if (j == 1) {
        t = ta;
        g.kb0 = static_cast<int>(u0 - static_cast<long long>(ta) * s.kb_count);
        g.kb1 = s.kb_count;
    } else {
        return false;
    }
    g.tile = s.whole + t;
    g.sk_index = t;
    g.col_off = 0;
    g.width = bn;
    const long long first = static_cast<long long>(t) * s.kb_count;
    g.adders = sk_worker_of(s, first + s.kb_count - 1) - sk_worker_of(s, first);
    g.mode = g.kb0 != 0 ? kSegAdd : (g.adders > 0 ? kSegOwner : kSegStore);
    *out = g;
    return true;
}

// Chooses the schedule for `tiles` output tiles of `kb_count` K blocks on at most `max_workers`
// workers.  can_add: partial sums may be added into the output (int32 Y of one GPU);
// can_halve: half-width items are available.  Returns the schedule and, in *cost, the time of the
// busiest worker in tile times (for the dispatcher's choice between tile shapes).
inline Schedule plan_schedule(int tiles_m, int tiles_n, int kb_count, int max_workers, bool can_add, bool can_halve,
                              double* cost = nullptr)
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
        if (can_add && rem <= kSkMaxTiles && kb_count >= kSkMinBlocks && skw >= rem &&
            kb_count - longest >= kSkSplitCostBlocks) {
            s.whole = tiles - rem;
            s.sk_tiles = rem;
            s.sk_workers = static_cast<int>(skw);
            s.workers = s.whole > 0 ? max_workers : s.sk_workers;
            c = s.whole / max_workers + static_cast<double>(longest + kSkSplitCostBlocks) / kb_count;
        } else if (can_halve && 2 * rem <= max_workers) {
            s.whole = tiles - rem;
            s.half_tiles = rem;
            s.workers = s.whole > 0 ? max_workers : 2 * rem;
            // A half-width item still expands the whole X tile: about 0.75 of a tile time; a
            // launch that consists of nothing else is dominated by filling the pipeline (measured).
            c = s.whole > 0 ? s.whole / max_workers + 0.75 : 1.0;
        }
    }
    if (cost) *cost = c;
    return s;
}

}  // namespace i4l
