// Work schedule of the persistent tensor-memory GEMM kernels (host + device).
//
// The reference launches one CTA per 256 x 128 output tile and lets the hardware scheduler fill
// the machine (kernels/linear_v21.cu:20-37).  A persistent kernel with W workers (CTAs, or CTA
// pairs) walks T output tiles itself, and T is rarely a multiple of W:
//
//   whole tiles   tiles [0, whole) go round-robin to the workers;
//   half tiles    a last wave that would keep at most half of the workers busy is issued as
//                 half-width items (two per tile), which costs about three quarters of a tile time
//                 instead of a whole one (the X half of the work is not halved).
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

struct Schedule {
    int tiles_m = 0, tiles_n = 0;
    int workers = 0;     // grid size in workers
    int whole = 0;       // tiles computed as they are
    int half_tiles = 0;  // tiles (after the whole ones) cut into two half-width items
};

struct Segment {
    int tile;            // linear tile index (raster order)
    int col_off, width;  // columns of the tile this item covers
};

// The i-th item of `worker` (i = 0, 1, ...); false when the worker has no more work.
I4L_HD bool segment_of(const Schedule& s, int worker, int bn, int i, Segment* out)
{
    const int items = s.whole + 2 * s.half_tiles;
    const int item = worker + i * s.workers;
    if (item >= items) return false;
    if (item < s.whole) {
        out->tile = item;
        out->col_off = 0;
        out->width = bn;
    } else {
        const int h = item - s.whole;
        out->tile = s.whole + (h >> 1);
        out->col_off = (h & 1) * (bn / 2);
        out->width = bn / 2;
    }
    return true;
}

// Chooses the schedule for tiles_m x tiles_n output tiles on at most `max_workers` workers;
// can_halve: half-width items are available (CTA pairs, packed weights).  *cost receives the time
// of the busiest worker in tile times, for the dispatcher's choice between tile shapes.
inline Schedule plan_schedule(int tiles_m, int tiles_n, int max_workers, bool can_halve, double* cost = nullptr)
{
    Schedule s;
    s.tiles_m = tiles_m;
    s.tiles_n = tiles_n;
    const int tiles = tiles_m * tiles_n;
    const int rem = tiles % max_workers;
    s.whole = tiles;
    s.workers = tiles < max_workers ? tiles : max_workers;
    double c = static_cast<double>((tiles + max_workers - 1) / max_workers);
    if (can_halve && rem > 0 && 2 * rem <= max_workers) {
        s.whole = tiles - rem;
        s.half_tiles = rem;
        s.workers = s.whole > 0 ? max_workers : 2 * rem;
        // A half-width item still expands the whole X tile: about 0.75 of a tile time; a launch
        // that consists of nothing else is dominated by filling the pipeline (measured).
        c = s.whole > 0 ? s.whole / max_workers + 0.75 : 1.0;
    }
    if (cost) *cost = c;
    return s;
}

}  // namespace i4l
