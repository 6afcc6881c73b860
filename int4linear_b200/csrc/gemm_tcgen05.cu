// Main GEMM kernel: packed s4 operands -> TMA -> shared-memory ring ->
// in-smem s4->s8 unpack -> tcgen05.mma kind::i8 (int32 accumulators in tensor
// memory) -> TMEM->register->(smem->TMA store | direct store) epilogue.
//
// Replaces the device side of the reference's kernels/linear_v21.h:471-753
// (cp.async ring, XOR swizzle, ldmatrix, mma.sync m16n8k64, int2 stores).
//
// Work decomposition
//   Persistent CTAs (one per SM) walk output tiles.  With CTAS == 1 a CTA owns a
//   128 x BN tile.  With CTAS == 2 a cluster of two CTAs owns a 256 x BN tile and
//   runs it as one cta_group::2 UMMA: each CTA loads and unpacks its own 128 rows
//   of X and its own BN/2 rows of W (no multicast: every byte is fetched by the
//   CTA that unpacks it), CTA 0 issues the instruction for the pair, and each
//   CTA's tensor memory receives the accumulators of its own 128 rows.  Halving
//   the W work per CTA matters because shared-memory bandwidth, not the tensor
//   pipe, is what limits this kernel.  K advances in blocks of 128 elements
//   (64 packed bytes per row).
//   Warp roles (448 threads):
//     warp 0      TMA producer: packed X tile (128 x 64 B) and W tile (BN x 64 B)
//                 per K block into the "packed" ring; OOB rows/bytes read as 0,
//                 which implements every M, N and K tail.
//     warps 6-13  unpack, as two groups of four warps that take alternate K
//                 blocks: read the packed ring, expand nibbles to bytes, write the
//                 "unpacked" ring in the UMMA K-major 128-byte-swizzled layout,
//                 release the packed slot.
//     warp 1      UMMA issuer: four 128 x BN x 32 tcgen05.mma per K block into one
//                 of two TMEM accumulator buffers; tcgen05.commit releases the
//                 unpacked slot / publishes the finished accumulator.
//     warps 2-5   epilogue: tcgen05.ld the accumulator (one TMEM sub-partition of
//                 32 lanes each), undo the scaling, write Y (int32 through staged TMA
//                 stores -- to one matrix, or to every rank's copy when the result is
//                 gathered -- or dequantised bf16).  Overlaps the next tile's main
//                 loop through the second accumulator buffer.
//
// The unpack
//   A packed 32-bit word x holds nibbles e0..e7.  (x << 4) & 0xF0F0F0F0 is four
//   bytes equal to 16*e0, 16*e2, 16*e4, 16*e6 as signed 8-bit values, and
//   x & 0xF0F0F0F0 is 16*e1, 16*e3, 16*e5, 16*e7: three ALU operations for
//   eight elements, sign handled for free (-8 -> -128).  Even and odd elements
//   end up de-interleaved, i.e. K is permuted inside each 32-element group;
//   X and W go through the same permutation, and a dot product does not care
//   in which order K is summed.  The accumulator is therefore exactly
//   256 * y, and the epilogue shifts it right by 8 (arithmetic, exact).
//   |256 * y| <= 256 * 64 * K < 2^31 needs K < 131072.
#include <cstdlib>

#include "common.h"
#include "ptx.cuh"
#include "epilogue.cuh"
#include "schedule.cuh"

namespace i4l {

namespace {

constexpr int kBM = 128;          // tile rows (UMMA M)
constexpr int kBKBytes = 64;      // packed bytes per row per K block (128 elements)
constexpr int kGroups = 2;         // unpack groups, each converting every kGroups-th K block
constexpr int kWarpsPerGroup = 4;   // measured: 8 unpack warps in all are enough, 16 only add contention
constexpr int kUnpackWarps = kGroups * kWarpsPerGroup;
constexpr int kThreads = 32 * (2 + 4 + kUnpackWarps);
constexpr int kStoreStageBytes = 4 * 2 * 4096;  // 4 epilogue warps x 2 buffers x (32 rows x 128 B)

// PREW: the W operand arrives already expanded to bytes (int4_linear_prepare_weights), so
// TMA drops its tile straight into the expanded ring and only X goes through the unpack.
template <int BN, int P, int U, int CTAS, bool PREW = false>
struct Cfg {
    static constexpr bool kPreW = PREW;
    static constexpr int kBN = BN;
    static constexpr int kP = P;
    static constexpr int kU = U;
    static constexpr int kCtas = CTAS;
    static constexpr int kTileM = kBM * CTAS;                    // rows of the (cluster) tile
    static constexpr int kRowsW = BN / CTAS;                     // W rows this CTA loads and unpacks
    static constexpr int kPkRows = kBM + (PREW ? 0 : kRowsW);      // rows that go through the unpack
    static constexpr int kPkStage = kPkRows * kBKBytes;            // packed X then (unless PREW) packed W
    static constexpr int kUpStage = (kBM + kRowsW) * 2 * kBKBytes; // s8 X (16 KB) then s8 W
    static constexpr int kTmemCols = 2 * BN;                     // two accumulator buffers
    static constexpr int kNumBarriers = 2 * P + 2 * U + 4 + U;     // the last U: "expanded W has landed" (PREW)
    static constexpr int kSmemBytes = 1024 /*alignment slack*/ + U * kUpStage + P * kPkStage +
                                      kStoreStageBytes + kNumBarriers * 8 + 16;
    static_assert(P >= kGroups && U >= kGroups, "every unpack group needs a slot of its own");
    // Every use of a packed slot must be consumed by the same unpack group.  A wait names a phase by
    // its parity only, and TMA loads do not land in the order they were issued: a group that runs
    // ahead could otherwise ask for a slot's next use while the use before it -- the other group's --
    // is still in flight, find the parity it wants (left by the use before that) and read a slot
    // that has not arrived.  The same holds for the slots TMA fills with expanded weights.  (Slots
    // released by tcgen05.commit complete in issue order; for those U >= kGroups is enough.)
    static_assert(P % kGroups == 0 && (!PREW || U % kGroups == 0), "a TMA-filled slot must stay with one unpack group");
    static_assert(kTmemCols == 128 || kTmemCols == 256 || kTmemCols == 512, "TMEM columns: power of two");
    static_assert(kSmemBytes <= 232448, "shared memory budget");
};

// Destination tensor maps of the gathering variant: the full Y of every rank of the node.
constexpr int kMaxPeers = 8;
struct PeerMaps {
    CUtensorMap map[kMaxPeers];
};

// Kernel body.  y_maps[0 .. n_y_maps) are the TMA-store destinations: the caller's Y normally;
// with peer gathering, every rank's full-width Y, this rank's block starting col_shift columns in.
template <class C, bool kTmaStore>
__device__ __forceinline__ void
gemm_s4_tcgen05_body(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const CUtensorMap& tm_wh,
                     const CUtensorMap* y_maps, int n_y_maps, int col_shift,
                     int* __restrict__ y, int m, int n, int k,
                     const Schedule& sched, int* status, const int* __restrict__ bias,
                     const ScaledOut& so)
{
    constexpr int BN = C::kBN, P = C::kP, U = C::kU, CTAS = C::kCtas;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - raw);

    const uint32_t up_base = base;
    const uint32_t pk_base = up_base + U * C::kUpStage;
    const uint32_t st_base = pk_base + P * C::kPkStage;
    const uint32_t bar_base = st_base + kStoreStageBytes;
    auto pk_full  = [&](int i) { return bar_base + 8u * i; };
    auto pk_empty = [&](int i) { return bar_base + 8u * (P + i); };
    auto up_full  = [&](int i) { return bar_base + 8u * (2 * P + i); };
    auto up_empty = [&](int i) { return bar_base + 8u * (2 * P + U + i); };
    auto tm_full  = [&](int i) { return bar_base + 8u * (2 * P + 2 * U + i); };
    auto tm_empty = [&](int i) { return bar_base + 8u * (2 * P + 2 * U + 2 + i); };
    auto w_full   = [&](int i) { return bar_base + 8u * (2 * P + 2 * U + 4 + i); };
    const uint32_t misc_off = (bar_base - base) + 8u * C::kNumBarriers;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + misc_off + 4);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    // Position in the pair (0 = the CTA that issues UMMA) and the id / count of work streams.
    const uint32_t cta_rank = CTAS == 2 ? cluster_cta_rank() : 0u;
    const int worker = CTAS == 2 ? static_cast<int>(cluster_id_x()) : static_cast<int>(blockIdx.x);
    const int workers = CTAS == 2 ? static_cast<int>(cluster_count_x()) : static_cast<int>(gridDim.x);

    // Barrier set-up by the lanes of warp 2 in parallel (one barrier each; a single thread takes
    // over a thousand cycles for the two dozen of them), tensor-map prefetch by thread 0.
    if (warp == 2) {
        static_assert(C::kNumBarriers <= 32, "one lane per barrier");
        if (lane < C::kNumBarriers) {
            // pk_full | pk_empty | up_full | up_empty | tm_full | tm_empty | w_full.  up_full and
            // tm_empty of CTA 0 collect the arrivals of both CTAs of a pair.
            uint32_t count = 1;
            if (lane >= P && lane < 2 * P) count = kWarpsPerGroup;
            else if (lane >= 2 * P && lane < 2 * P + U) count = kWarpsPerGroup * CTAS;
            else if (lane >= 2 * P + 2 * U + 2 && lane < 2 * P + 2 * U + 4) count = 4 * CTAS;
            mbar_init(bar_base + 8u * lane, count);
        }
        if (lane == 0) *abort_flag = 0;
        mbar_init_fence();
    } else if (tid == 0) {
        tma_prefetch_desc(&tm_x);
        tma_prefetch_desc(&tm_w);
        if (kTmaStore) tma_prefetch_desc(y_maps);
    }
    // Start-up order.  The TMA producer and the unpack warps need only this CTA's barriers, so they
    // start right after the CTA-wide barrier; the tensor-memory allocation (warp 1) is awaited
    // only by the warps that use tensor memory (named barrier 1 over warps 1-5), and the pair's
    // cluster barrier -- "the other CTA's barriers exist" -- is split into an arrive here and a
    // wait in each role just before its first access to the peer.
    __syncthreads();
    if constexpr (CTAS == 2) {
        if (warp == 0) cluster_arrive_relaxed(); else cluster_arrive_release();
    }
    uint32_t tmem_base = 0;
    if (warp >= 1 && warp < 6) {
        if (warp == 1) {
            tmem_alloc<CTAS>(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
            tmem_relinquish<CTAS>();
            tc_fence_before_sync();
        }
        named_barrier_sync(1, 160);
        tc_fence_after_sync();
        tmem_base = *tmem_slot;
        if constexpr (CTAS == 2) cluster_wait();
    }

    // Every role walks the same list of segments (schedule.cuh): whole tiles, then half-width
    // items or the K ranges of the tiles that are cut along K.

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool alive = true;
            Segment sg;
            for (int si = 0; alive && segment_of(sched, worker, BN, si, &sg); ++si) {
                int tm, tn;
                tile_coord(sched, sg.tile, &tm, &tn);
                const int rows_w = sg.width / CTAS;
                for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                    const uint32_t s = it % P, r = it / P;
                    if (!mbar_wait(pk_empty(s), (r & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                    mbar_expect_tx(pk_full(s), C::kPreW ? C::kPkStage : (kBM + rows_w) * kBKBytes);
                    const uint32_t dst = pk_base + s * C::kPkStage;
                    tma_load_2d(dst, &tm_x, pk_full(s), kb * kBKBytes, (tm * CTAS + cta_rank) * kBM);
                    if constexpr (!C::kPreW) {
                        tma_load_2d(dst + kBM * kBKBytes, sg.width == BN ? &tm_w : &tm_wh, pk_full(s), kb * kBKBytes,
                                    tn * BN + sg.col_off + cta_rank * rows_w);
                    } else {
                        // Expanded W goes directly into the slot the UMMA reads; that slot is free
                        // once the UMMAs of its previous use have been committed.
                        const uint32_t us = it % U, ur = it / U;
                        if (!mbar_wait(up_empty(us), (ur & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                        mbar_expect_tx(w_full(us), C::kRowsW * 128);
                        tma_load_2d(up_base + us * C::kUpStage + kBM * 128, &tm_w, w_full(us), kb * 128,
                                    tn * BN + cta_rank * C::kRowsW);
                    }
                }
            }
        }
        if constexpr (CTAS == 2) cluster_wait_divergent();  // the producer never touches the peer
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------- UMMA issuer
        if (lane == 0 && cta_rank == 0) {
            uint32_t it = 0, local_tile = 0;
            bool alive = true;
            Segment sg;
            for (int si = 0; alive && segment_of(sched, worker, BN, si, &sg); ++si, ++local_tile) {
                const uint32_t idesc = sg.width == BN ? umma_idesc_s8(C::kTileM, BN) : umma_idesc_s8(C::kTileM, BN / 2);
                const uint32_t buf = local_tile & 1u, br = local_tile >> 1;
                if (!mbar_wait(tm_empty(buf), (br & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                    const uint32_t s = it % U, r = it / U;
                    if (!mbar_wait(up_full(s), r & 1u, abort_flag)) { alive = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a_addr = up_base + s * C::kUpStage;
                    const uint64_t a_desc = umma_desc_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_sw128(a_addr + kBM * 128);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // 32 bytes of K per instruction: advance the start address field by 32 >> 4.
                        umma_i8<CTAS>(d_tmem, a_desc + 2u * j, b_desc + 2u * j, idesc, (kb != sg.kb0 || j != 0) ? 1u : 0u);
                    }
                    if constexpr (CTAS == 2) umma_commit_2cta(up_empty(s), 3); else umma_commit(up_empty(s));
                }
                if (alive) {
                    if constexpr (CTAS == 2) umma_commit_2cta(tm_full(buf), 3); else umma_commit(tm_full(buf));
                }
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // ---------------------------------------------------------- epilogue
        const int sp = warp & 3;  // TMEM sub-partition this warp may read
        const uint32_t stage0 = st_base + (warp - 2) * 8192;
        uint32_t local_tile = 0;
        uint32_t chunk_no = 0;
        bool alive = true;
        Segment sg;
        // With tiles cut along K this grid was allowed to start before the clearing kernel in front of
        // it had finished; nothing is added into Y until that kernel has completed.
        if (sched.sk_tiles > 0) asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int si = 0; alive && segment_of(sched, worker, BN, si, &sg); ++si, ++local_tile) {
            int tm, tn;
            tile_coord(sched, sg.tile, &tm, &tn);
            const int col_off = sg.col_off, width = sg.width;
            const uint32_t buf = local_tile & 1u, br = local_tile >> 1;
            if (!mbar_wait_warp(tm_full(buf), br & 1u, abort_flag)) { alive = false; break; }
            tc_fence_after_sync();
            const int row0 = (tm * CTAS + static_cast<int>(cta_rank)) * kBM + sp * 32;
            const int col0 = tn * BN + col_off;
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(sp * 32) << 16) + buf * BN;
            if (so.y16 != nullptr) {
                // Dequantised bf16 output; y_maps[0] then describes the bf16 matrix.
                if constexpr (kTmaStore) {
                    if (so.fp16) drain_accumulator_scaled_tma<true>(t_addr, width, row0, col0, m, n, so, y_maps, stage0, chunk_no, lane);
                    else drain_accumulator_scaled_tma<false>(t_addr, width, row0, col0, m, n, so, y_maps, stage0, chunk_no, lane);
                }
                else drain_accumulator_scaled(t_addr, width, row0, col0, m, n, so, lane);
            } else if (sg.mode != kSegStore) {
                // A share of a tile that is cut along K: added into Y, which the clearing kernel in
                // front of this launch has zeroed; the share that holds K block 0 brings the bias.
                drain_accumulator<kTmaStore, true>(t_addr, width, row0, col0, m, n, y, sg.mode == kSegAddFirst ? bias : nullptr,
                                                   y_maps, n_y_maps, col_shift, stage0, chunk_no, lane);
            } else {
                drain_accumulator<kTmaStore, false>(t_addr, width, row0, col0, m, n, y, bias, y_maps, n_y_maps, col_shift, stage0, chunk_no, lane);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if constexpr (CTAS == 2) mbar_arrive_cluster(tm_empty(buf), 0); else mbar_arrive(tm_empty(buf));
            }
        }
        if (kTmaStore && lane == 0) tma_store_wait_all<0>();
        __syncwarp();
    } else {
        // ------------------------------------------------------------ unpack
        // The unpack warps form kGroups independent groups; group g converts K blocks
        // g, g + kGroups, ...  A block's conversion is a chain of latencies (wait, shared
        // loads, shared stores, proxy fence, arrive), so several blocks must be in flight
        // at once to keep the tensor pipe fed.
        const int uw = warp - 6;
        const int group = uw / kWarpsPerGroup;
        const int gtid = (uw % kWarpsPerGroup) * 32 + lane;
        constexpr int kGroupThreads = kWarpsPerGroup * 32;
        constexpr int kChunks = C::kPkRows * 4;  // 16-byte packed chunks per stage
        constexpr int kPerThread = kChunks / kGroupThreads;
        static_assert(kChunks % kGroupThreads == 0, "unpack loop must divide evenly");
        uint32_t it = 0;
        bool alive = true;
        // The pair's barrier completes long before the first TMA data arrives, so waiting for it
        // here (warp still convergent) costs nothing.
        if constexpr (CTAS == 2) cluster_wait();
        Segment sg;
        for (int si = 0; alive && segment_of(sched, worker, BN, si, &sg); ++si) {
            // 16-byte chunks to convert in this item's stages (a half-width item has fewer W rows)
            const int chunks = C::kPreW ? kChunks : (sg.width == BN ? kChunks : (kBM + C::kRowsW / 2) * 4);
            for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                if (static_cast<int>(it % kGroups) != group) continue;
                const uint32_t ps = it % P, pr = it / P;
                const uint32_t us = it % U, ur = it / U;
                if (!mbar_wait(pk_full(ps), pr & 1u, abort_flag)) { alive = false; break; }
                const uint32_t src = pk_base + ps * C::kPkStage;
                const uint32_t dst = up_base + us * C::kUpStage;
                // All loads first, so their latencies overlap.
                uint4 x[kPerThread];
#pragma unroll
                for (int i = 0; i < kPerThread; ++i)
                    if (i * kGroupThreads + gtid < chunks) x[i] = lds128(src + (i * kGroupThreads + gtid) * 16);
                if (!mbar_wait(up_empty(us), (ur & 1u) ^ 1u, abort_flag)) { alive = false; break; }
#pragma unroll
                for (int i = 0; i < kPerThread; ++i) {
                    const int q = i * kGroupThreads + gtid;
                    if (q >= chunks) break;
                    const int r = q >> 2, c = q & 3;
                    uint4 lo, hi;
                    lo.x = (x[i].x << 4) & 0xF0F0F0F0u; hi.x = x[i].x & 0xF0F0F0F0u;
                    lo.y = (x[i].y << 4) & 0xF0F0F0F0u; hi.y = x[i].y & 0xF0F0F0F0u;
                    lo.z = (x[i].z << 4) & 0xF0F0F0F0u; hi.z = x[i].z & 0xF0F0F0F0u;
                    lo.w = (x[i].w << 4) & 0xF0F0F0F0u; hi.w = x[i].w & 0xF0F0F0F0u;
                    const uint32_t rowaddr = dst + r * 128;
                    const uint32_t sw = r & 7;
                    sts128(rowaddr + (((2 * c) ^ sw) << 4), lo);
                    sts128(rowaddr + (((2 * c + 1) ^ sw) << 4), hi);
                }
                fence_proxy_async_smem();
                if constexpr (C::kPreW) {
                    // The slot is complete only when TMA has also delivered its expanded W rows.
                    if (!mbar_wait(w_full(us), ur & 1u, abort_flag)) { alive = false; break; }
                }
                __syncwarp();
                if (lane == 0) {
                    if constexpr (CTAS == 2) mbar_arrive_cluster(up_full(us), 0); else mbar_arrive(up_full(us));
                    mbar_arrive(pk_empty(ps));
                }
            }
        }
    }

    // ------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // Something never arrived.  Report, give copies in flight time to land,
        // then release tensor memory so the SM stays usable.
        if (tid == 0) atomicExch(status, INT4L_ERR_DEVICE_TIMEOUT);
        for (int i = 0; i < 100; ++i) __nanosleep(1000);
        __syncthreads();
    }
    // A pair frees its tensor memory together, and neither CTA may leave while the
    // other can still signal its barriers.
    if constexpr (CTAS == 2) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<CTAS>(tmem_base, C::kTmemCols);
    }
}

template <class C, bool kTmaStore>
__global__ void __launch_bounds__(kThreads, 1)
gemm_s4_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_x,
                       const __grid_constant__ CUtensorMap tm_w,
                       const __grid_constant__ CUtensorMap tm_wh,
                       const __grid_constant__ CUtensorMap tm_y,
                       int* __restrict__ y, int m, int n, int k,
                       const Schedule sched, int* status, const int* __restrict__ bias,
                       const ScaledOut so)
{
    gemm_s4_tcgen05_body<C, kTmaStore>(tm_x, tm_w, tm_wh, &tm_y, 1, 0, y, m, n, k, sched, status, bias, so);
}

// GEMM fused with the all-gather of its result: the epilogue stores this rank's column block of Y
// into the full-width Y of every rank of the node -- ordinary TMA stores whose destination
// happens to be peer memory mapped over NVLink (no multicast, no loads from peers) -- so the
// exchange overlaps the tiles still being computed instead of following the GEMM as a collective.
template <class C>
__global__ void __launch_bounds__(kThreads, 1)
gemm_s4_tcgen05_gather_kernel(const __grid_constant__ CUtensorMap tm_x,
                              const __grid_constant__ CUtensorMap tm_w,
                              const __grid_constant__ CUtensorMap tm_wh,
                              const __grid_constant__ PeerMaps peers, int n_peers, int col_shift,
                              int m, int n, int k, const Schedule sched, int* status,
                              const int* __restrict__ bias)
{
    gemm_s4_tcgen05_body<C, true>(tm_x, tm_w, tm_wh, peers.map, n_peers, col_shift, nullptr, m, n, k, sched,
                                  status, bias, ScaledOut{});
}

// Clears the tiles the next GEMM launch cuts along K (its shares only add into them).  One block per
// tile, whole 16-byte stores where the row pitch allows; rows and columns beyond Y are skipped.
// transposed: the tiles are tiles of Y transposed (gemm_fewrows.cu); m and n stay Y's own rows and columns.
__global__ void __launch_bounds__(256)
clear_cut_tiles_kernel(int* __restrict__ y, int m, int n, const Schedule sched, int tile_m, int bn, bool transposed)
{
    // The GEMM behind this kernel is launched with programmatic stream serialisation: it may start
    // right away and run its main loops while the tiles are being cleared; its epilogue warps wait
    // for this grid to have completed before their first addition.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    int tm, tn;
    tile_coord(sched, sched.whole + static_cast<int>(blockIdx.x), &tm, &tn);
    const int row0 = transposed ? tn * bn : tm * tile_m, col0 = transposed ? tm * tile_m : tn * bn;
    const int rows = min(transposed ? bn : tile_m, m - row0), cols = min(transposed ? tile_m : bn, n - col0);
    if (rows <= 0 || cols <= 0) return;
    const bool vec_ok = (n & 3) == 0 && (reinterpret_cast<uintptr_t>(y) & 15u) == 0 && (cols & 3) == 0;
    if (vec_ok) {
        const int per_row = cols >> 2;
        for (int i = threadIdx.x; i < rows * per_row; i += blockDim.x) {
            const int r = i / per_row, c = (i - r * per_row) << 2;
            *reinterpret_cast<int4*>(y + static_cast<size_t>(row0 + r) * n + col0 + c) = make_int4(0, 0, 0, 0);
        }
    } else {
        for (int i = threadIdx.x; i < rows * cols; i += blockDim.x) {
            const int r = i / cols, c = i - r * cols;
            y[static_cast<size_t>(row0 + r) * n + col0 + c] = 0;
        }
    }
}

}  // namespace

int launch_clear_cut_tiles(int* y, int m, int n, const Schedule& sched, int tile_m, int bn, bool transposed, cudaStream_t stream)
{
    clear_cut_tiles_kernel<<<sched.sk_tiles, 256, 0, stream>>>(y, m, n, sched, tile_m, bn, transposed);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

namespace {

using Cfg256 = Cfg<256, 4, 2, 1>;
using Cfg128 = Cfg<128, 4, 3, 1>;
using Cfg64 = Cfg<64, 4, 4, 1>;
using Cfg256x2 = Cfg<256, 4, 4, 2>;  // 256 x 256 tile on a CTA pair (a fourth expanded slot is worth 4 %)
using Cfg256x2W = Cfg<256, 4, 4, 2, true>;  // the same with pre-expanded weights
using Cfg128W = Cfg<128, 4, 4, 1, true>;

// Time of one K block (and so of one tile) of a tile shape relative to the 256 x 256 pair tile, from
// CUDA-graph replays (no launch overhead in the figures) at K = 1024 and 4096.
constexpr double block_time_of(int bn, int ctas)
{
    return ctas == 2 ? 1.0 : (bn == 256 ? 1.7 : (bn == 128 ? 1.1 : 0.9));
}

template <class C, bool kTmaStore>
int launch_cfg(DeviceCtx* ctx, const Problem& p, cudaStream_t stream, const GatherDst* gather = nullptr)
{
    const int tiles_m = (p.m + C::kTileM - 1) / C::kTileM;
    const int tiles_n = (p.n + C::kBN - 1) / C::kBN;
    const uint64_t pitch = static_cast<uint64_t>(p.k) / 2;
    CUtensorMap tm_x, tm_w, tm_wh, tm_y;
    int rc = make_tensor_map_2d(ctx, &tm_x, p.x, 1, pitch, p.m, pitch, kBKBytes, kBM, false);
    if (rc != INT4L_OK) return rc;
    if (C::kPreW)  // expanded weights: K bytes per row, 128-byte swizzled boxes
        rc = make_tensor_map_2d(ctx, &tm_w, p.w, 1, static_cast<uint64_t>(p.k), p.n, static_cast<uint64_t>(p.k), 128, C::kRowsW, true);
    else
        rc = make_tensor_map_2d(ctx, &tm_w, p.w, 1, pitch, p.n, pitch, kBKBytes, C::kRowsW, false);
    if (rc != INT4L_OK) return rc;
    if (kTmaStore && p.scaled.y16 != nullptr) {
        rc = make_tensor_map_2d(ctx, &tm_y, p.scaled.y16, 2, p.n, p.m, static_cast<uint64_t>(p.n) * 2, 64, 32, true);
        if (rc != INT4L_OK) return rc;
    } else if (kTmaStore && gather == nullptr) {
        rc = make_tensor_map_2d(ctx, &tm_y, p.y, 4, p.n, p.m, static_cast<uint64_t>(p.n) * 4, 32, 32, true);
        if (rc != INT4L_OK) return rc;
    } else {
        tm_y = tm_x;  // unused by the kernel
    }
    // The last, partial wave of tiles: cut along K where partial sums can be added into Y (int32
    // output on this GPU) and that is cheaper, else as half-width items, else whole (schedule.cuh).
    const int max_workers = C::kCtas == 2 ? ctx->max_pairs : ctx->sm_count;
    const int tail = tail_mode();
    const bool can_add = (tail < 0 || tail == 2) && p.scaled.y16 == nullptr && gather == nullptr;
    const bool can_halve = (tail < 0 || tail == 1) && !C::kPreW && C::kCtas == 2;
    const Schedule sched = plan_schedule(tiles_m, tiles_n, (p.k + 127) / 128, max_workers, can_add, can_halve, nullptr, tail == 2,
                                         block_time_of(C::kBN, C::kCtas));
    tm_wh = tm_x;  // unused unless tiles are halved
    if (sched.half_tiles > 0) {
        rc = make_tensor_map_2d(ctx, &tm_wh, p.w, 1, pitch, p.n, pitch, kBKBytes, C::kRowsW / 2, false);
        if (rc != INT4L_OK) return rc;
    }
    if (sched.sk_tiles > 0) {
        // The cut tiles only receive additions: clear them first, on the same stream.
        rc = launch_clear_cut_tiles(static_cast<int*>(p.y), p.m, p.n, sched, C::kTileM, C::kBN, false, stream);
        if (rc != INT4L_OK) return rc;
    }
    const int workers = sched.workers;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(workers * C::kCtas, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = C::kCtas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // Behind a clearing kernel: start while it runs (the epilogue waits for it, see the kernel).
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = sched.sk_tiles > 0 ? 2 : 1;
    cudaError_t e;
    if constexpr (kTmaStore && !C::kPreW) {
        if (gather != nullptr) {
            PeerMaps peers;
            for (int d = 0; d < gather->world; ++d) {
                rc = make_tensor_map_2d(ctx, &peers.map[d], gather->y_full[d], 4, gather->n_total, p.m,
                                        static_cast<uint64_t>(gather->n_total) * 4, 32, 32, true);
                if (rc != INT4L_OK) return rc;
            }
            for (int d = gather->world; d < kMaxPeers; ++d) peers.map[d] = peers.map[0];
            e = cudaLaunchKernelEx(&cfg, gemm_s4_tcgen05_gather_kernel<C>, tm_x, tm_w, tm_wh, peers, gather->world,
                                   gather->col_offset, p.m, p.n, p.k, sched, ctx->status_dev, p.bias);
            count_launch();
            if (e != cudaSuccess) { cudaGetLastError(); return INT4L_ERR_CUDA; }
            return INT4L_OK;
        }
    }
    e = cudaLaunchKernelEx(&cfg, gemm_s4_tcgen05_kernel<C, kTmaStore>, tm_x, tm_w, tm_wh, tm_y,
                           static_cast<int*>(p.y), p.m, p.n, p.k, sched, ctx->status_dev, p.bias, p.scaled);
    count_launch();
    if (e != cudaSuccess) { cudaGetLastError(); return INT4L_ERR_CUDA; }
    return INT4L_OK;
}

template <class C>
int set_attr()
{
    cudaError_t e = cudaFuncSetAttribute(gemm_s4_tcgen05_kernel<C, true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return INT4L_ERR_CUDA;
    e = cudaFuncSetAttribute(gemm_s4_tcgen05_kernel<C, false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    return e == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

}  // namespace

int setup_tcgen05(DeviceCtx* ctx)
{
    int rc = set_attr<Cfg256>();
    if (rc == INT4L_OK) rc = set_attr<Cfg128>();
    if (rc == INT4L_OK) rc = set_attr<Cfg64>();
    if (rc == INT4L_OK) rc = set_attr<Cfg256x2>();
    if (rc == INT4L_OK) rc = set_attr<Cfg256x2W>();
    if (rc == INT4L_OK) rc = set_attr<Cfg128W>();
    if (rc == INT4L_OK && cudaFuncSetAttribute(gemm_s4_tcgen05_gather_kernel<Cfg256x2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               Cfg256x2::kSmemBytes) != cudaSuccess) rc = INT4L_ERR_CUDA;
    if (rc == INT4L_OK && cudaFuncSetAttribute(gemm_s4_tcgen05_gather_kernel<Cfg128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               Cfg128::kSmemBytes) != cudaSuccess) rc = INT4L_ERR_CUDA;
    if (rc != INT4L_OK) return rc;
    // How many CTA pairs the device can hold at once (pairs must sit in one GPC-level
    // neighbourhood, so this can be below sm_count / 2).
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * ctx->sm_count, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg256x2::kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int pairs = 0;
    if (cudaOccupancyMaxActiveClusters(&pairs, gemm_s4_tcgen05_kernel<Cfg256x2, true>, &cfg) != cudaSuccess || pairs <= 0) {
        cudaGetLastError();
        pairs = ctx->sm_count / 2;
    }
    ctx->max_pairs = pairs < ctx->sm_count / 2 ? pairs : ctx->sm_count / 2;
    return INT4L_OK;
}

// Tile-width choice: the widest N tile that still yields at least one tile per
// SM, because a wide tile re-reads X less often but a grid smaller than the
// machine leaves SMs idle.
int launch_tcgen05(DeviceCtx* ctx, const Problem& p, cudaStream_t stream)
{
    auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    const bool tma_store = !getenv_flag_direct_store() &&
                           (p.scaled.y16 == nullptr
                                ? p.n % 4 == 0
                                : (p.n % 8 == 0 && aligned16(p.scaled.y16)));
    if (p.w_expanded) {
        // Pre-expanded weights: CTA pairs whenever there is more than one row block, else one CTA.
        if (p.m > 128)
            return tma_store ? launch_cfg<Cfg256x2W, true>(ctx, p, stream) : launch_cfg<Cfg256x2W, false>(ctx, p, stream);
        return tma_store ? launch_cfg<Cfg128W, true>(ctx, p, stream) : launch_cfg<Cfg128W, false>(ctx, p, stream);
    }
    // A few rows of X: operands swapped and W through tensor memory (gemm_fewrows.cu).  From 65 rows on
    // only with at least 32 tiles of W rows: below that the 128 x 64 / 128 x 128 tiles of this kernel
    // put more CTAs to work (128 x 1024 x 1024: 7.5 us here, 8.1 there; 128 x 6144 x 4096: 15.5 / 13.9);
    // and from 113 rows on only with K >= 4096 (128 x 8192 x 1024: 8.5 us here, 9.1 there).
    if (fewrows_supports(p) && (fewrows_mode() == 1 || (fewrows_mode() < 0 && forced_tile_n() == 0 && forced_pairs() < 0 &&
                                                          (p.m <= 64 || (p.n >= 4096 && (p.m <= 112 || p.k >= 4096))))))
        return launch_fewrows(ctx, p, stream);
    // Tile choice by a small cost model fitted to measurements on B200: cost = (tile times the
    // busiest worker runs) x (time of one tile relative to a 256 x 256 pair tile).  A wider tile
    // re-expands X less often per output, a narrower one fills more SMs when the problem is small.
    // The schedule's own estimate of the busiest worker's time (whole waves plus the K-cut or
    // half-width tail) stands in for the wave count.
    const int kb_count = (p.k + 127) / 128;
    const int tail = tail_mode();
    const bool can_add = (tail < 0 || tail == 2) && p.scaled.y16 == nullptr;
    auto waves = [&](int tile_m, int bn, int workers, bool can_halve) {
        double c = 0.0;
        plan_schedule((p.m + tile_m - 1) / tile_m, (p.n + bn - 1) / bn, kb_count, workers, can_add, can_halve, &c, tail == 2,
                      block_time_of(bn, tile_m == 256 ? 2 : 1));
        return c;
    };
    const double cost_pairs = p.m > 128 ? waves(256, 256, ctx->max_pairs, tail < 0 || tail == 1)
                                        : 1e30;  // a lone row block would leave CTA 1 idle
    // Tile times relative to the pair tile, from CUDA-graph replays (no launch overhead in the
    // figures) at K = 1024 and 4096: 128 x 256 on one CTA 1.7, 128 x 128 1.1, 128 x 64 0.9.
    const double cost256 = waves(kBM, 256, ctx->sm_count, false) * block_time_of(256, 1);
    const double cost128 = waves(kBM, 128, ctx->sm_count, false) * block_time_of(128, 1);
    const double cost64 = waves(kBM, 64, ctx->sm_count, false) * block_time_of(64, 1);
    int bn = 256;
    double best = cost256;
    if (cost128 < best) { best = cost128; bn = 128; }
    if (cost64 < best) { best = cost64; bn = 64; }
    bool pairs = cost_pairs <= best;
    const int forced = forced_tile_n();
    if (forced == 64 || forced == 128 || forced == 256) { bn = forced; pairs = false; }
    if (forced_pairs() >= 0) pairs = forced_pairs() != 0;
    if (pairs) return tma_store ? launch_cfg<Cfg256x2, true>(ctx, p, stream) : launch_cfg<Cfg256x2, false>(ctx, p, stream);
    if (bn == 256) return tma_store ? launch_cfg<Cfg256, true>(ctx, p, stream) : launch_cfg<Cfg256, false>(ctx, p, stream);
    if (bn == 128) return tma_store ? launch_cfg<Cfg128, true>(ctx, p, stream) : launch_cfg<Cfg128, false>(ctx, p, stream);
    return tma_store ? launch_cfg<Cfg64, true>(ctx, p, stream) : launch_cfg<Cfg64, false>(ctx, p, stream);
}

// GEMM + all-gather through peer stores (see gemm_s4_tcgen05_gather_kernel).  p.n is this rank's
// column count; p.y is not used.
int launch_tcgen05_gather(DeviceCtx* ctx, const Problem& p, const GatherDst& g, cudaStream_t stream)
{
    if (g.world < 1 || g.world > kMaxPeers) return INT4L_ERR_INVALID_ARG;
    // Store chunks are 32 columns wide: a block that ends inside a chunk would spill into the
    // neighbouring rank's columns; TMA stores want a 16-byte row pitch.
    if (p.n % 32 != 0 || g.col_offset % 32 != 0 || g.n_total % 4 != 0 || g.col_offset + p.n > g.n_total)
        return INT4L_ERR_UNSUPPORTED;
    if (p.m > 128) return launch_cfg<Cfg256x2, true>(ctx, p, stream, &g);
    return launch_cfg<Cfg128, true>(ctx, p, stream, &g);
}

}  // namespace i4l
