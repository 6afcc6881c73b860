// GEMM kernel with the X operand in tensor memory ("TS" form of tcgen05.mma).
//
// Same operator, ring structure and unpack arithmetic as gemm_tcgen05.cu, for CTA pairs only,
// with one change aimed at what limits that kernel -- the shared-memory data path.  There the
// expanded X tile is written to shared memory by the unpack warps and read back by the tensor
// core: 16 KB + 16 KB per K block and CTA.  Here the warps that expand X write it straight from
// registers into tensor memory (tcgen05.st) and the UMMA takes its A operand from there, so X
// costs shared memory only its packed 8 KB (TMA write + one read).  Per K block and CTA:
//     packed ring   (128 + 96) x 64 B   written by TMA, read once by the unpack warps
//     W, expanded   96 x 128 B          written by the unpack warps, read by the tensor core
// against 4 UMMAs of 256 x 192 x 32.
//
// Tensor memory (512 columns): two 192-column accumulator buffers + four 32-column X stages,
// which is why the tile is 256 x 192 and not 256 x 256.
//
// X layout in tensor memory: lane = tile row, 32-bit column c of a K block holds K bytes
// 4c..4c+3 of the expanded row; UMMA j of a K block reads columns 8j..8j+7.  The expanded row is
// [even elements of packed chunk j | odd elements of packed chunk j] for j = 0..3 -- the same order
// the W rows have in shared memory, so both operands carry the same K permutation.
//
// A thread that writes tensor memory must sit in the warp whose (index % 4) matches the lane
// quarter it writes, and needs its whole packed row (4 x 16 B at a 64-byte row pitch); the packed
// X tile is therefore loaded with the 64-byte TMA swizzle, which makes those row-strided 16-byte
// reads conflict-free.
#include "common.h"
#include "ptx.cuh"
#include "epilogue.cuh"

#define I4L_TRACE_EXPORT int4_linear_debug_trace_ts
#include "trace.cuh"

namespace i4l {

namespace {

constexpr int kBM = 128;                 // rows per CTA
constexpr int kBN = 192;                 // columns per pair tile
constexpr int kRowsW = kBN / 2;          // W rows each CTA loads and expands
constexpr int kBKBytes = 64;
constexpr int kGroups = 2;               // unpack groups taking alternate K blocks
constexpr int kWarpsX = 4, kWarpsW = 4;  // per group
constexpr int kWarpsPerGroup = kWarpsX + kWarpsW;
constexpr int kThreads = 32 * (6 + kGroups * kWarpsPerGroup);
constexpr int kP = 6;                    // packed stages
constexpr int kU = 4;                    // expanded stages (W in smem, X in TMEM)
constexpr int kPkStage = (kBM + kRowsW) * kBKBytes;
constexpr int kUpStage = kRowsW * 2 * kBKBytes;
constexpr int kStoreStageBytes = 4 * 2 * 4096;
constexpr int kNumBarriers = 2 * kP + 2 * kU + 4;
constexpr int kSmemBytes = 1024 + kU * kUpStage + kP * kPkStage + kStoreStageBytes + kNumBarriers * 8 + 16;
constexpr int kTmemCols = 512;
constexpr int kTmemXCol = 2 * kBN;       // first column of the X stages
static_assert(kTmemXCol + 32 * kU <= kTmemCols, "tensor memory budget");
static_assert(kUpStage % 1024 == 0 && kPkStage % 1024 == 0, "stage bases must keep the swizzle alignment");
static_assert((kRowsW * 4) % (kWarpsW * 32) == 0, "W unpack loop must divide evenly");
static_assert(kSmemBytes <= 232448, "shared memory budget");

template <bool kTmaStore>
__global__ void __launch_bounds__(kThreads, 1)
gemm_s4_tcgen05_ts_kernel(const __grid_constant__ CUtensorMap tm_x,
                          const __grid_constant__ CUtensorMap tm_w,
                          const __grid_constant__ CUtensorMap tm_y,
                          int* __restrict__ y, int m, int n, int k,
                          int tiles_m, int tiles_n, int* status, const int* __restrict__ bias)
{
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
    const uint32_t cta_rank = cluster_cta_rank();
    const int worker = static_cast<int>(cluster_id_x());
    const int workers = static_cast<int>(cluster_count_x());

    if (tid == 0) {
        for (int i = 0; i < kP; ++i) { mbar_init(pk_full(i), 1); mbar_init(pk_empty(i), kWarpsPerGroup); }
        for (int i = 0; i < kU; ++i) { mbar_init(up_full(i), kWarpsPerGroup * 2); mbar_init(up_empty(i), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(tm_full(i), 1); mbar_init(tm_empty(i), 8); }
        *abort_flag = 0;
        mbar_init_fence();
        tma_prefetch_desc(&tm_x);
        tma_prefetch_desc(&tm_w);
        if (kTmaStore) tma_prefetch_desc(&tm_y);
    }
    if (warp == 1) {
        tmem_alloc<2>(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        tmem_relinquish<2>();
    }
    tc_fence_before_sync();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int num_tiles = tiles_m * tiles_n;
    const int kb_count = (k + 127) / 128;
    constexpr int kGroupM = 16;
    auto tile_coord = [&](int tile, int& tm, int& tn) {
        const int group_size = kGroupM * tiles_n;
        const int group = tile / group_size;
        const int first_m = group * kGroupM;
        const int gm = min(tiles_m - first_m, kGroupM);
        const int in_group = tile - group * group_size;
        tm = first_m + in_group % gm;
        tn = in_group / gm;
    };

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool alive = true;
            for (int tile = worker; alive && tile < num_tiles; tile += workers) {
                int tm, tn;
                tile_coord(tile, tm, tn);
                for (int kb = 0; kb < kb_count; ++kb, ++it) {
                    const uint32_t s = it % kP, r = it / kP;
                    if (!mbar_wait(pk_empty(s), (r & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                    mbar_expect_tx(pk_full(s), kPkStage);
                    const uint32_t dst = pk_base + s * kPkStage;
                    tma_load_2d(dst, &tm_x, pk_full(s), kb * kBKBytes, (tm * 2 + cta_rank) * kBM);
                    tma_load_2d(dst + kBM * kBKBytes, &tm_w, pk_full(s), kb * kBKBytes, tn * kBN + cta_rank * kRowsW);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------- UMMA issuer
        if (lane == 0 && cta_rank == 0) {
            constexpr uint32_t idesc = umma_idesc_s8(2 * kBM, kBN);
            uint32_t it = 0, local_tile = 0;
            bool alive = true;
            for (int tile = worker; alive && tile < num_tiles; tile += workers, ++local_tile) {
                const uint32_t buf = local_tile & 1u, br = local_tile >> 1;
                if (!mbar_wait(tm_empty(buf), (br & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * kBN;
                for (int kb = 0; kb < kb_count; ++kb, ++it) {
                    const uint32_t s = it % kU, r = it / kU;
                    I4L_TRACE_PUT(1, it, 0);
                    if (!mbar_wait(up_full(s), r & 1u, abort_flag)) { alive = false; break; }
                    I4L_TRACE_PUT(1, it, 1);
                    tc_fence_after_sync();
                    const uint64_t b_desc = umma_desc_sw128(up_base + s * kUpStage);
                    const uint32_t a_tmem = tmem_base + kTmemXCol + 32u * s;
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        umma_i8_ts<2>(d_tmem, a_tmem + 8u * j, b_desc + 2u * j, idesc, (kb | j) != 0 ? 1u : 0u);
                    umma_commit_2cta(up_empty(s), 3);
                    I4L_TRACE_PUT(1, it, 2);
                }
                if (alive) umma_commit_2cta(tm_full(buf), 3);
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // ---------------------------------------------------------- epilogue
        const int sp = warp & 3;
        const uint32_t stage0 = st_base + (warp - 2) * 8192;
        uint32_t local_tile = 0, chunk_no = 0;
        bool alive = true;
        for (int tile = worker; alive && tile < num_tiles; tile += workers, ++local_tile) {
            int tm, tn;
            tile_coord(tile, tm, tn);
            const uint32_t buf = local_tile & 1u, br = local_tile >> 1;
            if (!mbar_wait(tm_full(buf), br & 1u, abort_flag)) { alive = false; break; }
            tc_fence_after_sync();
            const int row0 = (tm * 2 + static_cast<int>(cta_rank)) * kBM + sp * 32;
            const int col0 = tn * kBN;
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(sp * 32) << 16) + buf * kBN;
            drain_accumulator<kTmaStore>(t_addr, kBN, row0, col0, m, n, y, bias, &tm_y, 1, 0, stage0, chunk_no, lane);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tm_empty(buf), 0);
        }
        if (kTmaStore && lane == 0) tma_store_wait_all<0>();
        __syncwarp();
    } else {
        // ------------------------------------------------------------ unpack
        const int uw = warp - 6;
        const int group = uw / kWarpsPerGroup;
        const int wg = uw % kWarpsPerGroup;
        const bool x_warp = wg < kWarpsX;
        // X warps: one thread per tile row; the lane quarter is fixed by the warp index.
        const int xrow = (warp & 3) * 32 + lane;
        const uint32_t xsw = (xrow >> 1) & 3;
        // W warps: 16-byte chunks of the packed W tile, strided over the group's W threads.
        const int wtid = (wg - kWarpsX) * 32 + lane;
        constexpr int kWThreads = kWarpsW * 32;
        constexpr int kWPerThread = kRowsW * 4 / kWThreads;
        uint32_t it = 0;
        bool alive = true;
        for (int tile = worker; alive && tile < num_tiles; tile += workers) {
            for (int kb = 0; kb < kb_count; ++kb, ++it) {
                if (static_cast<int>(it % kGroups) != group) continue;
                const uint32_t ps = it % kP, pr = it / kP;
                const uint32_t us = it % kU, ur = it / kU;
                [[maybe_unused]] const bool tr = lane == 0 && (wg == 0 || wg == kWarpsX);
                [[maybe_unused]] const int trole = x_warp ? 2 : 4;
                if (tr) I4L_TRACE_PUT(trole, it, 0);
                if (!mbar_wait(pk_full(ps), pr & 1u, abort_flag)) { alive = false; break; }
                if (tr) I4L_TRACE_PUT(trole, it, 1);
                const uint32_t src = pk_base + ps * kPkStage;
                if (x_warp) {
                    uint4 x[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) x[c] = lds128(src + xrow * 64 + ((c ^ xsw) << 4));
                    if (!mbar_wait(up_empty(us), (ur & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                    tc_fence_after_sync();
                    if (tr) I4L_TRACE_PUT(trole, it, 2);
                    uint32_t v[32];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint32_t w4[4] = {x[c].x, x[c].y, x[c].z, x[c].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            v[8 * c + e] = (w4[e] << 4) & 0xF0F0F0F0u;
                            v[8 * c + 4 + e] = w4[e] & 0xF0F0F0F0u;
                        }
                    }
                    tmem_st_32x32(tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + kTmemXCol + 32u * us, v);
                    tmem_st_wait();
                    tc_fence_before_sync();
                } else {
                    uint4 x[kWPerThread];
#pragma unroll
                    for (int i = 0; i < kWPerThread; ++i)
                        x[i] = lds128(src + kBM * kBKBytes + (i * kWThreads + wtid) * 16);
                    if (!mbar_wait(up_empty(us), (ur & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                    if (tr) I4L_TRACE_PUT(trole, it, 2);
                    const uint32_t dst = up_base + us * kUpStage;
#pragma unroll
                    for (int i = 0; i < kWPerThread; ++i) {
                        const int q = i * kWThreads + wtid;
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
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_cluster(up_full(us), 0);
                    mbar_arrive(pk_empty(ps));
                }
                if (tr) I4L_TRACE_PUT(trole, it, 3);
            }
        }
    }

    // ------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0) atomicExch(status, INT4L_ERR_DEVICE_TIMEOUT);
        for (int i = 0; i < 100; ++i) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<2>(tmem_base, kTmemCols);
    }
}

template <bool kTmaStore>
int launch_ts_impl(DeviceCtx* ctx, const Problem& p, cudaStream_t stream)
{
    const int tiles_m = (p.m + 2 * kBM - 1) / (2 * kBM);
    const int tiles_n = (p.n + kBN - 1) / kBN;
    const uint64_t pitch = static_cast<uint64_t>(p.k) / 2;
    CUtensorMap tm_x, tm_w, tm_y;
    int rc = make_tensor_map_2d(ctx, &tm_x, p.x, 1, pitch, p.m, pitch, kBKBytes, kBM, false, true);
    if (rc != INT4L_OK) return rc;
    rc = make_tensor_map_2d(ctx, &tm_w, p.w, 1, pitch, p.n, pitch, kBKBytes, kRowsW, false);
    if (rc != INT4L_OK) return rc;
    if (kTmaStore) {
        rc = make_tensor_map_2d(ctx, &tm_y, p.y, 4, p.n, p.m, static_cast<uint64_t>(p.n) * 4, 32, 32, true);
        if (rc != INT4L_OK) return rc;
    } else {
        tm_y = tm_x;
    }
    const int workers = min(tiles_m * tiles_n, ctx->max_pairs);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(workers * 2, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_s4_tcgen05_ts_kernel<kTmaStore>, tm_x, tm_w, tm_y,
                                       static_cast<int*>(p.y), p.m, p.n, p.k, tiles_m, tiles_n, ctx->status_dev, p.bias);
    count_launch();
    if (e != cudaSuccess) { cudaGetLastError(); return INT4L_ERR_CUDA; }
    return INT4L_OK;
}

}  // namespace

int setup_tcgen05_ts(DeviceCtx*)
{
    cudaError_t e = cudaFuncSetAttribute(gemm_s4_tcgen05_ts_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_s4_tcgen05_ts_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    return e == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

int launch_tcgen05_ts(DeviceCtx* ctx, const Problem& p, cudaStream_t stream)
{
    const bool tma_store = (p.n % 4 == 0) && !getenv_flag_direct_store();
    return tma_store ? launch_ts_impl<true>(ctx, p, stream) : launch_ts_impl<false>(ctx, p, stream);
}

}  // namespace i4l
