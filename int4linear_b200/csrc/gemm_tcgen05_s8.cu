// Two-pass path, second pass: GEMM on operands that were already expanded to bytes.
//
// The fused kernel (gemm_tcgen05.cu) is limited by the shared-memory data path: every K block
// it writes the expanded operands to shared memory with ordinary stores while the tensor core
// reads the previous ones from the same banks.  For large compute-bound shapes it is cheaper to
// expand both operands ONCE in a streaming pre-pass (packer.cu: expand kernel, HBM-bound, the
// operands are a small part of the traffic of such shapes) and then run this kernel, in which
// nothing but TMA writes and tensor-core reads touches shared memory:
//     warp 0      TMA: X' tile (128 x 128 B) and W' tile (rows x 128 B) per K block of 128
//                 elements straight into the 128-byte-swizzled ring the UMMA reads
//     warp 1      tcgen05.mma kind::i8 issue (CTA 0 of a pair issues for both); in the other
//                 CTA of a pair this warp forwards "my tile has landed" to CTA 0
//     warps 2-5   epilogue (epilogue.cuh), overlapped through two TMEM accumulator buffers
// X' / W' are M x K and N x K bytes: per 32 elements the 16 even ones then the 16 odd ones, each
// byte 16 x value -- the same byte order the fused kernel's unpack produces, so the arithmetic
// (and the result, bit for bit) is the same: accumulator = 256 * y, shifted back in the epilogue.
#include "common.h"
#include "ptx.cuh"
#include "epilogue.cuh"

namespace i4l {

namespace {

constexpr int kBM = 128;
constexpr int kThreads = 32 * 6;
constexpr int kStoreStageBytes = 4 * 2 * 4096;

template <int BN, int S, int CTAS>
struct CfgS8 {
    static constexpr int kBN = BN, kS = S, kCtas = CTAS;
    static constexpr int kTileM = kBM * CTAS;
    static constexpr int kRowsW = BN / CTAS;
    static constexpr int kStage = (kBM + kRowsW) * 128;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kNumBarriers = 3 * S + 4;  // full, empty, peer_full, tm_full[2], tm_empty[2]
    static constexpr int kSmemBytes = 1024 + S * kStage + kStoreStageBytes + kNumBarriers * 8 + 16;
    static_assert(kTmemCols == 128 || kTmemCols == 256 || kTmemCols == 512, "TMEM columns: power of two");
    static_assert(kSmemBytes <= 232448, "shared memory budget");
};

template <class C, bool kTmaStore>
__global__ void __launch_bounds__(kThreads, 1)
gemm_s8_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_x,
                       const __grid_constant__ CUtensorMap tm_w,
                       const __grid_constant__ CUtensorMap tm_y,
                       int* __restrict__ y, int m, int n, int k,
                       int tiles_m, int tiles_n, int* status, const int* __restrict__ bias)
{
    constexpr int BN = C::kBN, S = C::kS, CTAS = C::kCtas;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - raw);

    const uint32_t ring = base;
    const uint32_t st_base = ring + S * C::kStage;
    const uint32_t bar_base = st_base + kStoreStageBytes;
    auto full      = [&](int i) { return bar_base + 8u * i; };
    auto empty     = [&](int i) { return bar_base + 8u * (S + i); };
    auto peer_full = [&](int i) { return bar_base + 8u * (2 * S + i); };
    auto tm_full   = [&](int i) { return bar_base + 8u * (3 * S + i); };
    auto tm_empty  = [&](int i) { return bar_base + 8u * (3 * S + 2 + i); };
    const uint32_t misc_off = (bar_base - base) + 8u * C::kNumBarriers;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + misc_off + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t cta_rank = CTAS == 2 ? cluster_cta_rank() : 0u;
    const int worker = CTAS == 2 ? static_cast<int>(cluster_id_x()) : static_cast<int>(blockIdx.x);
    const int workers = CTAS == 2 ? static_cast<int>(cluster_count_x()) : static_cast<int>(gridDim.x);

    if (tid == 0) {
        for (int i = 0; i < S; ++i) { mbar_init(full(i), 1); mbar_init(empty(i), 1); mbar_init(peer_full(i), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(tm_full(i), 1); mbar_init(tm_empty(i), 4 * CTAS); }
        *abort_flag = 0;
        mbar_init_fence();
        tma_prefetch_desc(&tm_x);
        tma_prefetch_desc(&tm_w);
        if (kTmaStore) tma_prefetch_desc(&tm_y);
    }
    if (warp == 1) {
        tmem_alloc<CTAS>(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
        tmem_relinquish<CTAS>();
    }
    tc_fence_before_sync();
    if constexpr (CTAS == 2) cluster_sync_all(); else __syncthreads();
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
                    const uint32_t s = it % S, r = it / S;
                    if (!mbar_wait(empty(s), (r & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                    mbar_expect_tx(full(s), C::kStage);
                    const uint32_t dst = ring + s * C::kStage;
                    tma_load_2d(dst, &tm_x, full(s), kb * 128, (tm * CTAS + cta_rank) * kBM);
                    tma_load_2d(dst + kBM * 128, &tm_w, full(s), kb * 128, tn * BN + cta_rank * C::kRowsW);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && cta_rank == 0) {
            // ----------------------------------------------------- UMMA issuer
            constexpr uint32_t idesc = umma_idesc_s8(C::kTileM, BN);
            uint32_t it = 0, local_tile = 0;
            bool alive = true;
            for (int tile = worker; alive && tile < num_tiles; tile += workers, ++local_tile) {
                const uint32_t buf = local_tile & 1u, br = local_tile >> 1;
                if (!mbar_wait(tm_empty(buf), (br & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < kb_count; ++kb, ++it) {
                    const uint32_t s = it % S, r = it / S;
                    if (!mbar_wait(full(s), r & 1u, abort_flag)) { alive = false; break; }
                    if constexpr (CTAS == 2) {
                        if (!mbar_wait(peer_full(s), r & 1u, abort_flag)) { alive = false; break; }
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = ring + s * C::kStage;
                    const uint64_t a_desc = umma_desc_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_sw128(a_addr + kBM * 128);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        umma_i8<CTAS>(d_tmem, a_desc + 2u * j, b_desc + 2u * j, idesc, (kb | j) != 0 ? 1u : 0u);
                    if constexpr (CTAS == 2) umma_commit_2cta(empty(s), 3); else umma_commit(empty(s));
                }
                if (alive) {
                    if constexpr (CTAS == 2) umma_commit_2cta(tm_full(buf), 3); else umma_commit(tm_full(buf));
                }
            }
        } else if (lane == 0 && CTAS == 2) {
            // ------------- second CTA of a pair: tell CTA 0 when this CTA's tiles have landed
            uint32_t it = 0;
            bool alive = true;
            for (int tile = worker; alive && tile < num_tiles; tile += workers) {
                for (int kb = 0; kb < kb_count; ++kb, ++it) {
                    const uint32_t s = it % S, r = it / S;
                    if (!mbar_wait(full(s), r & 1u, abort_flag)) { alive = false; break; }
                    mbar_arrive_cluster(peer_full(s), 0);
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------- epilogue
        const int sp = warp & 3;
        const uint32_t stage0 = st_base + (warp - 2) * 8192;
        uint32_t local_tile = 0, chunk_no = 0;
        bool alive = true;
        for (int tile = worker; alive && tile < num_tiles; tile += workers, ++local_tile) {
            int tm, tn;
            tile_coord(tile, tm, tn);
            const uint32_t buf = local_tile & 1u, br = local_tile >> 1;
            if (!mbar_wait_warp(tm_full(buf), br & 1u, abort_flag)) { alive = false; break; }
            tc_fence_after_sync();
            const int row0 = (tm * CTAS + static_cast<int>(cta_rank)) * kBM + sp * 32;
            const int col0 = tn * BN;
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(sp * 32) << 16) + buf * BN;
            drain_accumulator<kTmaStore>(t_addr, BN, row0, col0, m, n, y, bias, &tm_y, 1, 0, stage0, chunk_no, lane);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if constexpr (CTAS == 2) mbar_arrive_cluster(tm_empty(buf), 0); else mbar_arrive(tm_empty(buf));
            }
        }
        if (kTmaStore && lane == 0) tma_store_wait_all<0>();
        __syncwarp();
    }

    // ------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0) atomicExch(status, INT4L_ERR_DEVICE_TIMEOUT);
        for (int i = 0; i < 100; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if constexpr (CTAS == 2) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<CTAS>(tmem_base, C::kTmemCols);
    }
}

using CfgS8Pair = CfgS8<256, 6, 2>;
using CfgS8One = CfgS8<128, 6, 1>;

template <class C, bool kTmaStore>
int launch_s8_cfg(DeviceCtx* ctx, const Problem& p, const void* x_bytes, const void* w_bytes, cudaStream_t stream)
{
    const int tiles_m = (p.m + C::kTileM - 1) / C::kTileM;
    const int tiles_n = (p.n + C::kBN - 1) / C::kBN;
    const uint64_t pitch = static_cast<uint64_t>(p.k);
    CUtensorMap tm_x, tm_w, tm_y;
    int rc = make_tensor_map_2d(ctx, &tm_x, x_bytes, 1, pitch, p.m, pitch, 128, kBM, true);
    if (rc != INT4L_OK) return rc;
    rc = make_tensor_map_2d(ctx, &tm_w, w_bytes, 1, pitch, p.n, pitch, 128, C::kRowsW, true);
    if (rc != INT4L_OK) return rc;
    if (kTmaStore) {
        rc = make_tensor_map_2d(ctx, &tm_y, p.y, 4, p.n, p.m, static_cast<uint64_t>(p.n) * 4, 32, 32, true);
        if (rc != INT4L_OK) return rc;
    } else {
        tm_y = tm_x;
    }
    const int max_workers = C::kCtas == 2 ? ctx->max_pairs : ctx->sm_count;
    const int workers = min(tiles_m * tiles_n, max_workers);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(workers * C::kCtas, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = C::kCtas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_s8_tcgen05_kernel<C, kTmaStore>, tm_x, tm_w, tm_y,
                                       static_cast<int*>(p.y), p.m, p.n, p.k, tiles_m, tiles_n, ctx->status_dev, p.bias);
    count_launch();
    if (e != cudaSuccess) { cudaGetLastError(); return INT4L_ERR_CUDA; }
    return INT4L_OK;
}

template <class C>
int set_attr_s8()
{
    cudaError_t e = cudaFuncSetAttribute(gemm_s8_tcgen05_kernel<C, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_s8_tcgen05_kernel<C, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    return e == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

}  // namespace

int setup_tcgen05_s8(DeviceCtx* ctx)
{
    int rc = set_attr_s8<CfgS8Pair>();
    if (rc == INT4L_OK) rc = set_attr_s8<CfgS8One>();
    if (rc != INT4L_OK || ctx->max_pairs > 0) return rc;
    // A context that has not learnt yet how many CTA pairs the device holds at once (the
    // static-scratch entry point builds its own) asks for this kernel's figure.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * ctx->sm_count, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = CfgS8Pair::kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int pairs = 0;
    if (cudaOccupancyMaxActiveClusters(&pairs, gemm_s8_tcgen05_kernel<CfgS8Pair, true>, &cfg) != cudaSuccess || pairs <= 0) {
        cudaGetLastError();
        pairs = ctx->sm_count / 2;
    }
    ctx->max_pairs = pairs < ctx->sm_count / 2 ? pairs : ctx->sm_count / 2;
    return rc;
}

// x_bytes: M x K bytes, w_bytes: N x K bytes (both made by the expand kernel); p.x / p.w are ignored.
int launch_tcgen05_s8(DeviceCtx* ctx, const Problem& p, const void* x_bytes, const void* w_bytes, cudaStream_t stream)
{
    const bool tma_store = (p.n % 4 == 0) && !getenv_flag_direct_store();
    if (p.m > 128)
        return tma_store ? launch_s8_cfg<CfgS8Pair, true>(ctx, p, x_bytes, w_bytes, stream)
                         : launch_s8_cfg<CfgS8Pair, false>(ctx, p, x_bytes, w_bytes, stream);
    return tma_store ? launch_s8_cfg<CfgS8One, true>(ctx, p, x_bytes, w_bytes, stream)
                     : launch_s8_cfg<CfgS8One, false>(ctx, p, x_bytes, w_bytes, stream);
}

}  // namespace i4l
