// GEMM kernel for a few rows of X (M <= 128): the operands change places and W goes through tensor
// memory instead of shared memory.
//
// With so few rows every byte of W is used once, so the operator is a stream of W from HBM, and in the
// main kernel (gemm_tcgen05.cu) such a stream is held back twice: by the rate at which one SM's TMA
// unit turns out requests (a box of 64-byte rows is one request per row, and with only those loads
// left in the kernel a CTA still needs a quarter of a microsecond per 8 KB of W), and by the
// shared-memory data path (per 128-element K block a tile of 128 W rows costs 8 KB of TMA writes,
// 8 KB of packed reads, 16 KB of expanded writes and 16 KB of operand reads by the tensor core, plus
// the same again for a 128-row X tile that is mostly padding).  Here
//   * K advances in steps of 256 elements, so that every TMA request is a whole 128-byte line;
//   * the 128-row (M) side of the UMMA holds rows of W and the N side the rows of X, rounded up to
//     16 (tcgen05.mma 128 x N x 32, N = 16 .. 64), so the accumulator is a tile of Y transposed and
//     the epilogue writes it back transposed;
//   * the threads that expand W own one row each (the lane of tensor memory that row lives in),
//     read its 128 packed bytes from the TMA-written stage (128-byte swizzle: those row-strided
//     16-byte reads are conflict-free), expand them in registers and write the 256 bytes straight
//     into tensor memory (tcgen05.st); the UMMA takes its A operand from there.  W costs shared
//     memory its packed bytes only, written once and read once;
//   * X is expanded into shared memory per K step as in the main kernel;
//   * the ring of packed stages holds 6 x 16 KB of W (4 x 16 KB in the two-half form), because with
//     every byte coming from HBM once a CTA needs bandwidth x latency bytes in flight.
// Two forms (template parameter XH, the number of 64-row halves of X).  XH = 1, M <= 64: the two
// UMMA-issuing threads take alternate K steps, each into an accumulator of its own, and the epilogue
// adds the two.  XH = 2, 65 <= M <= 128: every stage of W in tensor memory is multiplied with both
// halves of X, issuing thread h taking half h in every step, so W is still loaded and expanded once
// and accumulator h is rows 64h .. of Y.
// Replaces, for these shapes, kernels/linear_v21.h:471-753 run on a 256 x 128 tile of padding.
//
// Tensor memory (512 columns): two accumulator buffers of two accumulators (one per issuing thread)
// of 64 columns, then the stages of 64 columns for W (lane = W row; 32-bit column c of a stage holds bytes 4c .. 4c+3 of the expanded row; UMMA j of
// a K step reads columns 8j .. 8j+7).  The expanded row is [even elements of packed chunk j | odd
// elements of packed chunk j] for j = 0 .. 7 -- the order the X rows have in shared memory, so both
// operands carry the same permutation of K.
//
// Work is handed out by the same schedule as in the main kernel (schedule.cuh) over tiles of Y
// transposed: whole tiles round-robin, the last wave cut along K with the shares added into Y
// (bulk reductions, or atomic adds where Y's row pitch forbids TMA; a clearing kernel runs in front,
// see gemm_tcgen05.cu).
#include "common.h"
#include "ptx.cuh"
#include "epilogue.cuh"
#include "schedule.cuh"

namespace i4l {

namespace {

constexpr int kRowsW = 128;        // W rows per tile = UMMA M = lanes of tensor memory
constexpr int kHalfRowsX = 64;     // X rows per UMMA (its N) at most
constexpr int kBKBytes = 128;      // packed bytes per row per K step (256 elements)
constexpr int kGroups = 2;         // groups of four unpack warps; group g converts K steps g, g + kGroups, ...
constexpr int kIssuers = 2;        // threads that issue UMMAs, an accumulator each
constexpr int kXTile = kHalfRowsX * 128;           // expanded X: one 64-row half, one 128-element half of a K step
constexpr int kAccCols = kHalfRowsX;
constexpr int kStageCols = kBKBytes / 2;           // tensor-memory columns of one expanded W stage
constexpr int kTmemCols = 512;
constexpr int kTmemWCol = 2 * kIssuers * kAccCols;  // first column of the W stages
constexpr int kStoreStageBytes = 4 * 4096;          // one 32 x 32 int32 staging tile per epilogue warp
constexpr int kThreads = 32 * (7 + 4 * kGroups);
// Measured with three groups: slower (14.0 against 13.7 us at 64 x 14336 x 4096); only two are tested.
static_assert(kGroups == 2, "tested with two unpack groups");

// Ring geometry for XH halves of X.
template <int XH>
struct Geo {
    static constexpr int kP = XH == 1 ? 6 : 4;       // packed stages
    static constexpr int kU = XH == 1 ? 4 : 2;       // expanded stages: W in tensor memory, X in shared memory
    static constexpr int kRowsX = XH * kHalfRowsX;
    static constexpr int kPkStage = (kRowsW + kRowsX) * kBKBytes;
    static constexpr int kUpStage = XH * 2 * kXTile;  // [half of X][half of the K step][64 rows x 128 B]
    static constexpr int kNumBarriers = 2 * kP + 2 * kU + 4;
    static constexpr int kSmemBytes = 1024 + kU * kUpStage + kP * kPkStage + kStoreStageBytes + kNumBarriers * 8 + 16;
    // Every use of a packed stage must be consumed by the same unpack group.  A wait names a phase
    // by its parity only, and TMA loads do not land in the order they were issued: a group that runs
    // ahead could otherwise ask for a stage's next use while the use before it -- the other group's
    // -- is still in flight, find the parity it wants (left by the use before that) and read a stage
    // that has not arrived.  (The expanded stages are released by tcgen05.commit in issue order, so
    // for them it is enough that the ring is at least as deep as there are groups.)
    static_assert(kP % kGroups == 0 && kU >= kGroups, "ring depths and unpack groups");
    static_assert(kTmemWCol + kStageCols * kU <= kTmemCols, "tensor memory budget");
    static_assert(kUpStage % 1024 == 0 && kPkStage % 1024 == 0, "stage bases must keep the swizzle alignment");
    static_assert(kSmemBytes <= 232448, "shared memory budget");
};

template <int XH>
__global__ void __launch_bounds__(kThreads, 1)
gemm_s4_fewrows_kernel(const __grid_constant__ CUtensorMap tm_w,
                       const __grid_constant__ CUtensorMap tm_x,
                       const __grid_constant__ CUtensorMap tm_y, int tma_store,
                       int* __restrict__ y, int w_rows, int x_rows, int x_pad,
                       const Schedule sched, int* status, const int* __restrict__ bias)
{
    using G = Geo<XH>;
    constexpr int kP = G::kP, kU = G::kU, kPkStage = G::kPkStage, kUpStage = G::kUpStage, kNumBarriers = G::kNumBarriers;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - raw);

    const uint32_t up_base = base;
    const uint32_t pk_base = up_base + kU * kUpStage;
    const uint32_t st_base = pk_base + kP * kPkStage;
    const uint32_t bar_base = st_base + kStoreStageBytes;
    auto pk_full  = [&](int i) { return bar_base + 8u * i; };
    auto pk_empty = [&](int i) { return bar_base + 8u * (kP + i); };
    auto up_full  = [&](int i) { return bar_base + 8u * (2 * kP + i); };
    auto up_empty = [&](int i) { return bar_base + 8u * (2 * kP + kU + i); };
    auto tm_full  = [&](int i) { return bar_base + 8u * (2 * kP + 2 * kU + i); };
    auto tm_empty = [&](int i) { return bar_base + 8u * (2 * kP + 2 * kU + 2 + i); };
    const uint32_t misc_off = (bar_base - base) + 8u * kNumBarriers;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + misc_off + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int worker = static_cast<int>(blockIdx.x);

    if (warp == 2) {
        for (int b = lane; b < kNumBarriers; b += 32) {
            // pk_full | pk_empty | up_full | up_empty | tm_full | tm_empty
            uint32_t count = 1;
            if (b >= kP && b < 2 * kP + kU) count = 4;                 // the four warps of a group
            else if (b >= 2 * kP + kU && b < 2 * kP + 2 * kU) count = XH;  // the issuer(s) that read the stage
            else if (b >= 2 * kP + 2 * kU && b < 2 * kP + 2 * kU + 2) count = kIssuers;  // every issuer commits
            else if (b >= 2 * kP + 2 * kU + 2) count = 4;              // the four epilogue warps
            mbar_init(bar_base + 8u * b, count);
        }
        if (lane == 0) *abort_flag = 0;
        mbar_init_fence();
    } else if (tid == 0) {
        tma_prefetch_desc(&tm_w);
        tma_prefetch_desc(&tm_x);
        if (tma_store) tma_prefetch_desc(&tm_y);
    }
    __syncthreads();
    // The TMA producer needs the barriers only; every other warp also needs the tensor-memory base.
    uint32_t tmem_base = 0;
    if (warp != 0) {
        if (warp == 1) {
            tmem_alloc<1>(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
            tmem_relinquish<1>();
            tc_fence_before_sync();
        }
        named_barrier_sync(1, kThreads - 32);
        tc_fence_after_sync();
        tmem_base = *tmem_slot;
    }

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool alive = true;
            Segment sg;
            const uint32_t tx = static_cast<uint32_t>(kRowsW + x_pad) * kBKBytes;
            for (int si = 0; alive && segment_of(sched, worker, x_pad, si, &sg); ++si) {
                const int tm = sg.tile;  // one column of tiles (tiles_n == 1): the tile's index is its row block of W
                for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                    const uint32_t s = it % kP, r = it / kP;
                    if (!mbar_wait(pk_empty(s), (r & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                    mbar_expect_tx(pk_full(s), tx);
                    const uint32_t dst = pk_base + s * kPkStage;
                    tma_load_2d(dst, &tm_w, pk_full(s), kb * kBKBytes, tm * kRowsW);
                    tma_load_2d(dst + kRowsW * kBKBytes, &tm_x, pk_full(s), kb * kBKBytes, 0);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 6 + 4 * kGroups) {
        // ------------------------------------------------------ UMMA issuers
        // Issuing one tcgen05.mma with its A operand in tensor memory keeps the issuing thread busy
        // for about a hundred cycles whatever N is, and a commit for two hundred (measured: 440 ns for
        // the eight UMMAs of a step, 540 with the commit), while the tensor pipe needs 32 cycles per
        // UMMA at N = 64.  Two threads in different warps therefore share the work, each with an
        // accumulator of its own (UMMAs of different threads are not ordered against one another):
        // alternate K steps, the epilogue adding the two (XH = 1), or one half of X each (XH = 2).
        const uint32_t which = warp == 1 ? 0u : 1u;
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_s8(kRowsW, XH == 1 ? x_pad : (which == 0 ? kHalfRowsX : x_pad - kHalfRowsX));
            uint32_t it = 0, local_tile = 0;
            bool alive = true;
            Segment sg;
            for (int si = 0; alive && segment_of(sched, worker, x_pad, si, &sg); ++si, ++local_tile) {
                const uint32_t buf = local_tile & 1u, br = local_tile >> 1;
                if (!mbar_wait(tm_empty(buf), (br & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (buf * kIssuers + which) * kAccCols;
                bool first = true;
                for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                    if (XH == 1 && (it & 1u) != which) continue;
                    const uint32_t s = it % kU, r = it / kU;
                    if (!mbar_wait(up_full(s), r & 1u, abort_flag)) { alive = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a_tmem = tmem_base + kTmemWCol + kStageCols * s;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        // 32 bytes of K per instruction: 8 columns of tensor memory, 32 bytes of an X row
                        const uint64_t b_desc = umma_desc_sw128(up_base + s * kUpStage + (XH == 2 ? which * 2 * kXTile : 0) + (j >> 2) * kXTile) + 2u * (j & 3);
                        umma_i8_a_tmem(d_tmem, a_tmem + 8u * j, b_desc, idesc, (first && j == 0) ? 0u : 1u);
                    }
                    first = false;
                    umma_commit(up_empty(s));
                }
                if (alive) umma_commit(tm_full(buf));  // with nothing issued in this segment it arrives at once
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // ---------------------------------------------------------- epilogue
        const int sp = warp & 3;  // quarter of the tensor-memory lanes this warp may read
        uint32_t local_tile = 0, it = 0;
        bool alive = true;
        Segment sg;
        // Behind a clearing kernel this grid starts early; nothing is added into Y before that
        // kernel has completed.
        if (sched.sk_tiles > 0) asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int si = 0; alive && segment_of(sched, worker, x_pad, si, &sg); ++si, ++local_tile) {
            const int tm = sg.tile;
            const uint32_t buf = local_tile & 1u, br = local_tile >> 1;
            if (!mbar_wait_warp(tm_full(buf), br & 1u, abort_flag)) { alive = false; break; }
            tc_fence_after_sync();
            const int row0 = tm * kRowsW + sp * 32;
            // XH = 1: which issuers hold a part of this segment (both unless it is a single step); their
            // accumulators are added.  XH = 2: accumulator h is rows 64 h .. of Y.
            const uint32_t steps = static_cast<uint32_t>(sg.kb1 - sg.kb0);
            const uint32_t first_acc = (XH == 2 || steps >= 2) ? 0u : (it & 1u);
            const int second_acc = (XH == 1 && steps >= 2) ? kAccCols : -1;
            it += steps;
            const int* seg_bias = (sg.mode == kSegStore || sg.mode == kSegAddFirst) ? bias : nullptr;
#pragma unroll
            for (int h = 0; h < XH; ++h) {
                const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(sp * 32) << 16) + (buf * kIssuers + first_acc + h) * kAccCols;
                const int col0 = h * kHalfRowsX;     // first row of Y (= row of X) of this accumulator
                // whole 32-column loads; columns beyond x_rows are not written
                const int width = XH == 1 ? ((x_pad + 31) & ~31) : (h == 0 ? kHalfRowsX : ((x_pad - kHalfRowsX + 31) & ~31));
                if (tma_store) {
                    const uint32_t stg = st_base + (warp - 2) * 4096;
                    if (sg.mode != kSegStore)
                        drain_accumulator_transposed_tma<true>(t_addr, width, row0, col0, w_rows, x_rows, seg_bias, &tm_y, stg, lane, second_acc);
                    else
                        drain_accumulator_transposed_tma<false>(t_addr, width, row0, col0, w_rows, x_rows, seg_bias, &tm_y, stg, lane, second_acc);
                } else if (sg.mode != kSegStore) {
                    drain_accumulator_transposed<true>(t_addr, width, row0, col0, w_rows, x_rows, y, seg_bias, lane, second_acc);
                } else {
                    drain_accumulator_transposed<false>(t_addr, width, row0, col0, w_rows, x_rows, y, seg_bias, lane, second_acc);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(tm_empty(buf));
        }
        if (tma_store && lane == 0) tma_store_wait_all<0>();
        __syncwarp();
    } else {
        // ------------------------------------------------------------ unpack (warps 6 .. 6 + 4 * kGroups - 1)
        const int uw = warp - 6;
        const int group = uw >> 2;
        const int sp = warp & 3;             // the lanes of tensor memory this warp may write
        const int wrow = sp * 32 + lane;     // this thread's W row of the tile
        const uint32_t wsw = wrow & 7;       // 128-byte swizzle of the packed W stage
        const int gtid = (uw & 3) * 32 + lane;
        const int x_chunks = x_pad * 8;       // 16-byte packed chunks of the X stage (at most 512 per half of X)
        uint32_t it = 0;
        bool alive = true;
        Segment sg;
        for (int si = 0; alive && segment_of(sched, worker, x_pad, si, &sg); ++si) {
            for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                if (static_cast<int>(it % kGroups) != group) continue;
                const uint32_t ps = it % kP, pr = it / kP;
                const uint32_t us = it % kU, ur = it / kU;
                if (!mbar_wait(pk_full(ps), pr & 1u, abort_flag)) { alive = false; break; }
                const uint32_t src = pk_base + ps * kPkStage;
                uint4 wq[8], xq[4 * XH];
#pragma unroll
                for (int c = 0; c < 8; ++c) wq[c] = lds128(src + wrow * kBKBytes + ((c ^ wsw) << 4));
#pragma unroll
                for (int i = 0; i < 4 * XH; ++i)
                    if (i * 128 + gtid < x_chunks) xq[i] = lds128(src + kRowsW * kBKBytes + (i * 128 + gtid) * 16);
                // Hand the packed stage back to the producer as soon as it is in registers -- which is
                // when the loads have returned their data, not when they were issued: the arrive is
                // made to depend on one destination register of every load (a warp's load instruction
                // completes for all its lanes together, so lane 0's registers stand for the warp's).
                uint32_t landed = 0;
#pragma unroll
                for (int c = 0; c < 8; ++c) landed ^= wq[c].x;
#pragma unroll
                for (int i = 0; i < 4 * XH; ++i)
                    if (i * 128 + gtid < x_chunks) landed ^= xq[i].x;
                __syncwarp();
                if (lane == 0) mbar_arrive_after(pk_empty(ps), landed);
                if (!mbar_wait_warp(up_empty(us), (ur & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t v[32];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint32_t w4[4] = {wq[4 * h + c].x, wq[4 * h + c].y, wq[4 * h + c].z, wq[4 * h + c].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            v[8 * c + e] = (w4[e] << 4) & 0xF0F0F0F0u;
                            v[8 * c + 4 + e] = w4[e] & 0xF0F0F0F0u;
                        }
                    }
                    tmem_st_32x32(tmem_base + (static_cast<uint32_t>(sp * 32) << 16) + kTmemWCol + kStageCols * us + 32u * h, v);
                }
#pragma unroll
                for (int i = 0; i < 4 * XH; ++i) {
                    const int q = i * 128 + gtid;
                    if (q >= x_chunks) break;
                    const int r = (q >> 3) & (kHalfRowsX - 1), c = q & 3;   // row within its half of X
                    const uint32_t dst = up_base + us * kUpStage + (q >> 9) * 2 * kXTile + ((q >> 2) & 1) * kXTile;
                    uint4 lo, hi;
                    lo.x = (xq[i].x << 4) & 0xF0F0F0F0u; hi.x = xq[i].x & 0xF0F0F0F0u;
                    lo.y = (xq[i].y << 4) & 0xF0F0F0F0u; hi.y = xq[i].y & 0xF0F0F0F0u;
                    lo.z = (xq[i].z << 4) & 0xF0F0F0F0u; hi.z = xq[i].z & 0xF0F0F0F0u;
                    lo.w = (xq[i].w << 4) & 0xF0F0F0F0u; hi.w = xq[i].w & 0xF0F0F0F0u;
                    const uint32_t rowaddr = dst + r * 128;
                    const uint32_t sw = r & 7;
                    sts128(rowaddr + (((2 * c) ^ sw) << 4), lo);
                    sts128(rowaddr + (((2 * c + 1) ^ sw) << 4), hi);
                }
                fence_proxy_async_smem();
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(up_full(us));
            }
        }
    }

    // ------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // Something never arrived.  Report, give copies in flight time to land, then release tensor
        // memory so the SM stays usable.
        if (tid == 0) atomicExch(status, INT4L_ERR_DEVICE_TIMEOUT);
        for (int i = 0; i < 100; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<1>(tmem_base, kTmemCols);
    }
}

// What cutting the last wave along K costs this kernel, in its own K steps of 256 elements (measured:
// 112 tiles of 16 steps on 148 SMs take 15.0 us cut, 13 steps per worker, against 12.9 us whole, at
// 0.43 us per step): the clearing launch, a second epilogue per worker and the bulk reductions.
constexpr double kCutOverheadSteps = 7.0;

template <int XH>
int launch_impl(DeviceCtx* ctx, const Problem& p, cudaStream_t stream)
{
    const int x_pad = (p.m + 15) & ~15;
    const int tiles = (p.n + kRowsW - 1) / kRowsW;
    const uint64_t pitch = static_cast<uint64_t>(p.k) / 2;
    CUtensorMap tm_w, tm_x, tm_y;
    const bool tma_store = p.n % 4 == 0 && (reinterpret_cast<uintptr_t>(p.y) & 15u) == 0 && !getenv_flag_direct_store();
    int rc = make_tensor_map_2d(ctx, &tm_w, p.w, 1, pitch, p.n, pitch, kBKBytes, kRowsW, true);
    if (rc != INT4L_OK) return rc;
    rc = make_tensor_map_2d(ctx, &tm_x, p.x, 1, pitch, p.m, pitch, kBKBytes, x_pad, false);
    if (rc != INT4L_OK) return rc;
    if (tma_store) {
        rc = make_tensor_map_2d(ctx, &tm_y, p.y, 4, p.n, p.m, static_cast<uint64_t>(p.n) * 4, 32, 32, true);
        if (rc != INT4L_OK) return rc;
    } else {
        tm_y = tm_x;  // unused by the kernel
    }
    const int tail = tail_mode();
    const bool can_add = tail < 0 || tail == 2;
    const Schedule sched = plan_schedule(tiles, 1, (p.k + 255) / 256, ctx->sm_count, can_add, false, nullptr, tail == 2, 1.0, kCutOverheadSteps);
    if (sched.sk_tiles > 0) {
        rc = launch_clear_cut_tiles(static_cast<int*>(p.y), p.m, p.n, sched, kRowsW, x_pad, true, stream);
        if (rc != INT4L_OK) return rc;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sched.workers, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = Geo<XH>::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    // Behind a clearing kernel: start while it runs (the epilogue waits for it, see the kernel).
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = sched.sk_tiles > 0 ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_s4_fewrows_kernel<XH>, tm_w, tm_x, tm_y, tma_store ? 1 : 0, static_cast<int*>(p.y), p.n, p.m, x_pad,
                                             sched, ctx->status_dev, p.bias);
    count_launch();
    if (e != cudaSuccess) { cudaGetLastError(); return INT4L_ERR_CUDA; }
    return INT4L_OK;
}

}  // namespace

bool fewrows_supports(const Problem& p)
{
    return p.m <= 2 * kHalfRowsX && p.scaled.y16 == nullptr && !p.w_expanded;
}

int setup_fewrows(DeviceCtx*)
{
    cudaError_t e = cudaFuncSetAttribute(gemm_s4_fewrows_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<1>::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_s4_fewrows_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<2>::kSmemBytes);
    return e == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

int launch_fewrows(DeviceCtx* ctx, const Problem& p, cudaStream_t stream)
{
    if (!fewrows_supports(p)) return INT4L_ERR_UNSUPPORTED;
    return p.m <= kHalfRowsX ? launch_impl<1>(ctx, p, stream) : launch_impl<2>(ctx, p, stream);
}

}  // namespace i4l
