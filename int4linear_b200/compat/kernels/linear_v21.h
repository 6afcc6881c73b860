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
 * kWarpsPerThreadblockN warps) and the operand format, and is bit-exact, but it is
 * a plain warp-level mma.sync kernel: a kernel that only receives LinearArgs
 * cannot be handed TMA descriptors, so the tensor-memory path lives behind
 * linear_v21_launch.  Use the launcher (or the C ABI in include/int4linear_b200.h)
 * for performance; use this template to keep old call sites compiling.
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

}  // namespace int4linear_b200_compat

/* One CTA per output tile, blockIdx.x along N and blockIdx.y along M as the
 * reference's harness launches it (test/benchmark.cu:55-61).  Fragments come straight
 * from global memory through the read-only cache; the warp tile is walked in 16 x 8
 * pieces, 16 columns of accumulators at a time to bound register use.  Requires
 * k % 32 == 0 like the reference kernel; any m, n. */
template <typename Config>
__global__ void linear_v21_kernel(LinearArgs args)
{
    using namespace int4linear_b200_compat;
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

/* Exported by libint4linear_b200.so (C++ linkage, as in the reference). */
void linear_v21_launch(void* x_packed_d, void* w_packed_d, void* y_d, int m, int n, int k);

#endif /* INT4LINEAR_B200_COMPAT_LINEAR_V21_H_ */
