/*
 * Drop-in replacement for the reference's kernels/linear_v21.h.
 *
 * Put this directory in front of the reference tree on the include path
 * (-I<this repo>/int4linear_b200/compat -I<reference>) and the reference's
 * harnesses build unchanged:
 *
 *   test/test_correctness.cu   calls  linear_v21_launch(x_d, w_d, y_d, m, n, k)
 *                              (declared at kernels/linear_v21.h:760 of the
 *                              reference).  Here it resolves to the symbol of the same
 *                              name exported by libint4linear_b200.so, i.e. to the
 *                              sm_100a kernels.
 *   test/benchmark.cu          instantiates the kernel template itself
 *                              (test/benchmark.cu:46-72): it needs LOG2_WARP_SIZE,
 *                              LinearConfig<8,7,7,6,6,4> with its tile constants and
 *                              kSmemSize, the aggregate LinearArgs, and a __global__
 *                              template linear_v21_kernel<Config>(LinearArgs) that it
 *                              launches with a grid and block derived from those
 *                              constants and 96 KiB of dynamic shared memory.
 *
 * The template kernel below honours exactly that launch geometry (one CTA per
 * kThreadblockShapeM x kThreadblockShapeN tile, kWarpsPerThreadblockM x
 * kWarpsPerThreadblockN warps, kSmemSize bytes of dynamic shared memory) and the operand
 * format, is bit-exact, and needs nothing but the LinearArgs block: for the
 * configuration the reference uses, LinearConfig<8,7,7,6,6,4>, it is a self-contained
 * Blackwell kernel -- packed operands from global memory into registers, the same s4->s8
 * expansion as the library's kernels into 128-byte-swizzled shared memory, tcgen05.mma
 * kind::i8 into two 128 x 128 int32 accumulators in tensor memory, a shared-memory staged
 * epilogue with 128-byte coalesced stores -- with no tensor-map descriptor, no cluster and no
 * host-side set-up beyond the launch itself.  Other configurations run a plain warp-level
 * mma.sync kernel.  The library's persistent TMA kernels behind linear_v21_launch are
 * faster still (they keep four stages in flight and pair CTAs); this template is for call
 * sites that launch the kernel themselves.
 */
#ifndef INT4LINEAR_B200_COMPAT_LINEAR_V21_H_
#define INT4LINEAR_B200_COMPAT_LINEAR_V21_H_

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LOG2_WARP_SIZE 5

/* Same template parameters and member names as the reference's configuration type
 * (kernels/linear_v21.h:28-56): log2 of the CTA tile in M, N, K, log2 of the warp tile
 * in M, N, and a stage count (kept for source compatibility; this kernel stages
 * nothing). */
template <int L2TM, int L2TN, int L2TK, int L2WM, int L2WN, int STAGES = 3>
struct LinearConfig {
    static constexpr int kThreadblockShapeM = 1 << L2TM;
    static constexpr int kThreadblockShapeN = 1 << L2TN;
    static constexpr int kThreadblockShapeK = 1 << L2TK;
    static constexpr int kWarpShapeM = 1 << L2WM;
    static constexpr int kWarpShapeN = 1 << L2WN;
    static constexpr int kWarpsPerThreadblockM = kThreadblockShapeM / kWarpShapeM;
    static constexpr int kWarpsPerThreadblockN = kThreadblockShapeN / kWarpShapeN;
    static constexpr int kStages = STAGES;
    /* Bytes the caller passes as dynamic shared memory; the value the reference's
     * formula gives for the same parameters, so hard-coded opt-in limits still fit. */
    static constexpr int kSmemSize =
        STAGES * (kThreadblockShapeK / 8) * (kThreadblockShapeM + kThreadblockShapeN) * 4;
};

/* Field names and order of the reference's argument block (kernels/linear_v21.h:62-69). */
struct LinearArgs {
    void* X_ptr; /* M x K packed s4, row pitch K/2 bytes */
    void* W_ptr; /* N x K packed s4, row pitch K/2 bytes */
    void* Y_ptr; /* M x N int32 */
    int m;
    int n;
    int k;
};

namespace int4linear_b200_compat {

__device__ __forceinline__ void mma_m16n8k64_s4(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k64.row.col.s32.s4.s4.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

/* Word the tensor-memory kernel raises (to 5, the library's INT4L_ERR_DEVICE_TIMEOUT) when one of
 * its bounded waits expires or its shared memory is not laid out as it needs; every translation
 * unit that includes this header has its own copy.  linear_v21_kernel_status() reads and clears it. */
static __device__ int g_kernel_status;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ bool bar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

/* Bounded wait (one second of wall clock): false, with *abort_flag raised, when it runs out. */
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag)
{
    uint64_t t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
        if (bar_try(bar, parity)) return true;
        if ((spin & 63u) == 63u) {
            if (*abort_flag) return false;
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0 || now < t0) t0 = now;  /* restart the budget if the timer steps back */
            else if (now - t0 > 1000000000ull) { *abort_flag = 1; return false; }
        }
    }
}

/* Shared-memory descriptor of a K-major operand tile: rows of 128 bytes, 128-byte swizzle, 8-row
 * atoms of 1024 bytes one after the other (start address >> 4; stride between atoms 1024 >> 4 in
 * bits 32-45; descriptor version 1 in bits 46-47; layout 2 = SWIZZLE_128B in bits 61-63). */
__device__ __forceinline__ uint64_t operand_desc(uint32_t addr)
{
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

/* kind::i8 instruction descriptor: s32 accumulator, signed 8-bit A and B, both K-major, M x N. */
__device__ __forceinline__ constexpr uint32_t instr_desc(int m, int n)
{
    return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ uint4 load_packed(const uint8_t* base, int row, int rows, size_t pitch, int byte, int row_bytes)
{
    uint4 v = make_uint4(0u, 0u, 0u, 0u);  /* rows and bytes outside the matrix read as zero: every M, N and K tail */
    if (row < rows && byte < row_bytes)
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(base + static_cast<size_t>(row) * pitch + byte));
    return v;
}

/* 16 packed bytes (32 elements) -> 16 bytes of the even and 16 bytes of the odd elements, each byte
 * 16 x the element, written as chunks 2c and 2c + 1 of row r of a swizzled 128-byte-row tile. */
__device__ __forceinline__ void expand_store(uint32_t tile, int r, int c, uint4 p)
{
    const uint32_t row = tile + static_cast<uint32_t>(r) * 128u, sw = static_cast<uint32_t>(r) & 7u;
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(row + (((2u * c) ^ sw) << 4)),
                 "r"((p.x << 4) & 0xF0F0F0F0u), "r"((p.y << 4) & 0xF0F0F0F0u), "r"((p.z << 4) & 0xF0F0F0F0u), "r"((p.w << 4) & 0xF0F0F0F0u) : "memory");
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(row + (((2u * c + 1u) ^ sw) << 4)),
                 "r"(p.x & 0xF0F0F0F0u), "r"(p.y & 0xF0F0F0F0u), "r"(p.z & 0xF0F0F0F0u), "r"(p.w & 0xF0F0F0F0u) : "memory");
}

/* The tensor-memory kernel body for a 256 x TN tile (TN = 64, 128 or 256), 256 threads, K blocks of
 * 128 elements, two shared-memory stages of (256 + TN) x 128 bytes.
 *   every thread   loads its share of the packed X and W tile of K block kb + 2 into registers
 *                  (16-byte streaming loads), waits until the MMAs that read stage kb & 1 two blocks
 *                  ago have finished, expands K block kb from registers into that stage;
 *   warp 0, lane 0 once all eight warps have written the stage, issues two groups of four
 *                  128 x TN x 32 tcgen05.mma (rows 0-127 and 128-255 of the tile share the W operand)
 *                  and commits them to the stage's barrier;
 *   epilogue       warp w drains TMEM lanes 32 (w % 4) .. of accumulator w / 4, shifts the sums back
 *                  by 8 bits (both operands were multiplied by 16), transposes 32 x 32 blocks through
 *                  shared memory and stores whole 128-byte lines. */
template <int TN>
__device__ __forceinline__ void tensor_memory_tile(const LinearArgs& args, uint8_t* smem)
{
    constexpr int kStage = (256 + TN) * 128;
    constexpr int kChunksX = 256 * 4 / 256, kChunksW = TN * 4 / 256;  /* 16-byte packed chunks per thread and K block */
    constexpr int kLoads = kChunksX + kChunksW;
    constexpr uint32_t kCols = 2 * TN < 32 ? 32 : 2 * TN;              /* tensor-memory columns: two accumulators */
    __shared__ __align__(8) unsigned long long bars[4];                 /* written[2], consumed[2] */
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint8_t* __restrict__ x = static_cast<const uint8_t*>(args.X_ptr);
    const uint8_t* __restrict__ w = static_cast<const uint8_t*>(args.W_ptr);
    int* __restrict__ y = static_cast<int*>(args.Y_ptr);
    const int m = args.m, n = args.n, row_bytes = args.k >> 1;
    const size_t pitch = static_cast<size_t>(row_bytes);
    const int kb_count = (args.k + 127) >> 7;
    const int row0 = blockIdx.y * 256, col0 = blockIdx.x * TN;
    const uint32_t base = smem_addr(smem);
    const uint32_t written0 = smem_addr(&bars[0]), consumed0 = smem_addr(&bars[2]);

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(written0 + 8u * i), "r"(8u) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(consumed0 + 8u * i), "r"(1u) : "memory");
        }
        abort_word = (base & 1023u) ? 1 : 0;  /* the operand tiles must start on 1024-byte boundaries */
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_slot)), "r"(kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;

    /* chunk i of this thread: rows (i * 64 + tid / 4) of X for i < kChunksX, then of W; 16-byte column tid % 4 */
    const int sub_row = tid >> 2, c = tid & 3;
    auto load_block = [&](int kb, uint4 (&r)[kLoads]) {
        const int byte = kb * 64 + c * 16;
#pragma unroll
        for (int i = 0; i < kChunksX; ++i) r[i] = load_packed(x, row0 + i * 64 + sub_row, m, pitch, byte, kb < kb_count ? row_bytes : 0);
#pragma unroll
        for (int i = 0; i < kChunksW; ++i) r[kChunksX + i] = load_packed(w, col0 + i * 64 + sub_row, n, pitch, byte, kb < kb_count ? row_bytes : 0);
    };

    uint4 regs[3][kLoads];
    load_block(0, regs[0]);
    load_block(1, regs[1]);
    bool alive = !*abort_flag;
    constexpr uint32_t idesc = instr_desc(128, TN);
    for (int kb0 = 0; alive && kb0 < kb_count; kb0 += 3) {
#pragma unroll
        for (int u = 0; u < 3; ++u) {
            const int kb = kb0 + u;
            if (kb >= kb_count) break;
            const uint32_t s = static_cast<uint32_t>(kb) & 1u, use = static_cast<uint32_t>(kb) >> 1;
            load_block(kb + 2, regs[(u + 2) % 3]);
            /* stage s is free once the MMAs of its previous use have been committed */
            if (use > 0 && !bar_wait(consumed0 + 8u * s, (use - 1u) & 1u, abort_flag)) { alive = false; break; }
            const uint32_t stage = base + s * kStage;
#pragma unroll
            for (int i = 0; i < kChunksX; ++i) {
                const int r = i * 64 + sub_row;  /* rows 0-127: first operand tile, 128-255: second */
                expand_store(stage + (r >> 7) * 16384u, r & 127, c, regs[u][i]);
            }
#pragma unroll
            for (int i = 0; i < kChunksW; ++i) expand_store(stage + 32768u, i * 64 + sub_row, c, regs[u][kChunksX + i]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(written0 + 8u * s) : "memory");
            if (warp == 0) {
                if (lane == 0) {
                    if (bar_wait(written0 + 8u * s, use & 1u, abort_flag)) {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint64_t b_desc = operand_desc(stage + 32768u);
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            const uint64_t a_desc = operand_desc(stage + half * 16384u);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint32_t accumulate = (kb | j) != 0 ? 1u : 0u;
                                asm volatile(
                                    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n"
                                    ::"r"(tmem + half * TN), "l"(a_desc + 2u * j), "l"(b_desc + 2u * j), "r"(idesc), "r"(accumulate) : "memory");
                            }
                        }
                        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(consumed0 + 8u * s) : "memory");
                    }
                }
                __syncwarp();
            }
        }
    }
    /* the commit of the last K block covers every MMA before it */
    if (alive) {
        const uint32_t last = static_cast<uint32_t>(kb_count - 1);
        alive = bar_wait(consumed0 + 8u * (last & 1u), (last >> 1) & 1u, abort_flag);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();  /* nobody reads the operand stages any more: they become the epilogue's staging space */

    if (!*abort_flag) {
        const int half = warp >> 2, quarter = warp & 3;
        const int out_row0 = row0 + half * 128 + quarter * 32;
        const uint32_t stg = base + static_cast<uint32_t>(warp) * 4096u;  /* 32 rows x 128 bytes per warp */
        const bool vec_ok = (n & 3) == 0 && (reinterpret_cast<uintptr_t>(y) & 15u) == 0;
#pragma unroll 1
        for (int cc = 0; cc < TN; cc += 32) {
            if (out_row0 >= m || col0 + cc >= n) break;
            uint32_t v[32];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                  "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                  "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                  "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                : "r"(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + half * TN + cc)
                : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            /* lane = output row: write it as eight 16-byte chunks, chunk index XOR row % 8 */
#pragma unroll
            for (int q = 0; q < 8; ++q)
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(stg + lane * 128u + ((static_cast<uint32_t>(q) ^ (lane & 7u)) << 4)),
                             "r"(static_cast<uint32_t>(static_cast<int>(v[4 * q]) >> 8)), "r"(static_cast<uint32_t>(static_cast<int>(v[4 * q + 1]) >> 8)),
                             "r"(static_cast<uint32_t>(static_cast<int>(v[4 * q + 2]) >> 8)), "r"(static_cast<uint32_t>(static_cast<int>(v[4 * q + 3]) >> 8)) : "memory");
            __syncwarp();
            /* eight lanes per row: every store instruction of the warp writes four whole 128-byte lines */
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = i * 4 + (lane >> 3), q = lane & 7;
                uint4 o;
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(o.x), "=r"(o.y), "=r"(o.z), "=r"(o.w)
                             : "r"(stg + r * 128u + ((static_cast<uint32_t>(q) ^ (static_cast<uint32_t>(r) & 7u)) << 4)));
                const int row = out_row0 + r, col = col0 + cc + 4 * q;
                if (row < m) {
                    int* dst = y + static_cast<size_t>(row) * n + col;
                    if (vec_ok && col + 3 < n) {
                        *reinterpret_cast<uint4*>(dst) = o;
                    } else {
                        if (col < n) dst[0] = static_cast<int>(o.x);
                        if (col + 1 < n) dst[1] = static_cast<int>(o.y);
                        if (col + 2 < n) dst[2] = static_cast<int>(o.z);
                        if (col + 3 < n) dst[3] = static_cast<int>(o.w);
                    }
                }
            }
            __syncwarp();
        }
    } else if (tid == 0) {
        atomicExch(&g_kernel_status, 5);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kCols) : "memory");
    }
}

/* Any other configuration: fragments straight from global memory through the read-only cache into
 * warp-level mma.sync m16n8k64 s4, 16 columns of accumulators at a time. */
template <typename Config>
__device__ __forceinline__ void warp_mma_tile(const LinearArgs& args)
{
    const uint32_t* __restrict__ x = static_cast<const uint32_t*>(args.X_ptr);
    const uint32_t* __restrict__ w = static_cast<const uint32_t*>(args.W_ptr);
    int* __restrict__ y = static_cast<int*>(args.Y_ptr);
    const int m = args.m, n = args.n, words = args.k >> 3;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int grp = lane >> 2, quad = lane & 3;
    const int warp_m = warp / Config::kWarpsPerThreadblockN;
    const int warp_n = warp % Config::kWarpsPerThreadblockN;
    const int row_base = blockIdx.y * Config::kThreadblockShapeM + warp_m * Config::kWarpShapeM;
    const int col_base = blockIdx.x * Config::kThreadblockShapeN + warp_n * Config::kWarpShapeN;
    constexpr int kMI = Config::kWarpShapeM / 16;  /* 16-row pieces per warp tile */
    constexpr int kNJ = 2;                         /* 8-column pieces per pass */

    for (int col_pass = 0; col_pass < Config::kWarpShapeN; col_pass += 8 * kNJ) {
        int acc[kMI][kNJ][4];
#pragma unroll
        for (int i = 0; i < kMI; ++i)
#pragma unroll
            for (int j = 0; j < kNJ; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[i][j][e] = 0;

        for (int kw = 0; kw < words; kw += 8) {
            const bool upper = kw + 4 < words;
            uint32_t b[kNJ][2];
#pragma unroll
            for (int j = 0; j < kNJ; ++j) {
                const int c = col_base + col_pass + 8 * j + grp;
                const uint32_t* p = w + static_cast<size_t>(c) * words + kw + quad;
                b[j][0] = c < n ? __ldg(p) : 0u;
                b[j][1] = (c < n && upper) ? __ldg(p + 4) : 0u;
            }
#pragma unroll
            for (int i = 0; i < kMI; ++i) {
                const int r0 = row_base + 16 * i + grp, r1 = r0 + 8;
                const uint32_t* p0 = x + static_cast<size_t>(r0) * words + kw + quad;
                const uint32_t* p1 = x + static_cast<size_t>(r1) * words + kw + quad;
                const uint32_t a0 = r0 < m ? __ldg(p0) : 0u;
                const uint32_t a1 = r1 < m ? __ldg(p1) : 0u;
                const uint32_t a2 = (r0 < m && upper) ? __ldg(p0 + 4) : 0u;
                const uint32_t a3 = (r1 < m && upper) ? __ldg(p1 + 4) : 0u;
#pragma unroll
                for (int j = 0; j < kNJ; ++j) mma_m16n8k64_s4(acc[i][j], a0, a1, a2, a3, b[j][0], b[j][1]);
            }
        }

#pragma unroll
        for (int i = 0; i < kMI; ++i)
#pragma unroll
            for (int j = 0; j < kNJ; ++j) {
                const int c = col_base + col_pass + 8 * j + 2 * quad;
                const int r0 = row_base + 16 * i + grp, r1 = r0 + 8;
                if (r0 < m && c < n) y[static_cast<size_t>(r0) * n + c] = acc[i][j][0];
                if (r0 < m && c + 1 < n) y[static_cast<size_t>(r0) * n + c + 1] = acc[i][j][1];
                if (r1 < m && c < n) y[static_cast<size_t>(r1) * n + c] = acc[i][j][2];
                if (r1 < m && c + 1 < n) y[static_cast<size_t>(r1) * n + c + 1] = acc[i][j][3];
            }
    }
}

/* Whether the tensor-memory body fits a configuration: 256-row tiles, 64 / 128 / 256 columns, 256
 * threads, and at least two stages' worth of the dynamic shared memory the harness will pass. */
template <typename Config>
struct UsesTensorMemory {
    static constexpr int kThreads = Config::kWarpsPerThreadblockM * Config::kWarpsPerThreadblockN * 32;
    static constexpr bool value =
        Config::kThreadblockShapeM == 256 && kThreads == 256 &&
        (Config::kThreadblockShapeN == 64 || Config::kThreadblockShapeN == 128 || Config::kThreadblockShapeN == 256) &&
        Config::kSmemSize >= 2 * (256 + Config::kThreadblockShapeN) * 128;
};

}  // namespace int4linear_b200_compat

/* One CTA per output tile, blockIdx.x along N and blockIdx.y along M as the reference's harness
 * launches it (test/benchmark.cu:55-61), Config::kSmemSize bytes of dynamic shared memory.
 * Requires k % 32 == 0 like the reference kernel (16-byte row pitch) and k < 131072; any m, n. */
template <typename Config>
__global__ void __launch_bounds__(Config::kWarpsPerThreadblockM * Config::kWarpsPerThreadblockN * 32)
linear_v21_kernel(LinearArgs args)
{
    if constexpr (int4linear_b200_compat::UsesTensorMemory<Config>::value) {
        extern __shared__ __align__(1024) uint8_t linear_v21_dynamic_smem[];
        int4linear_b200_compat::tensor_memory_tile<Config::kThreadblockShapeN>(args, linear_v21_dynamic_smem);
    } else {
        int4linear_b200_compat::warp_mma_tile<Config>(args);
    }
}

/* Status of the template kernel's launches from this translation unit since the last call: 0, or 5
 * when a kernel gave up on a wait (the device stays usable).  Synchronises the device. */
static inline int linear_v21_kernel_status()
{
    int word = 0;
    if (cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpyFromSymbol(&word, int4linear_b200_compat::g_kernel_status, sizeof(int)) != cudaSuccess)
        return 4;
    if (word != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(int4linear_b200_compat::g_kernel_status, &zero, sizeof(int));
    }
    return word;
}

/* Exported by libint4linear_b200.so (C++ linkage, as in the reference). */
void linear_v21_launch(void* x_packed_d, void* w_packed_d, void* y_d, int m, int n, int k);

#endif /* INT4LINEAR_B200_COMPAT_LINEAR_V21_H_ */
