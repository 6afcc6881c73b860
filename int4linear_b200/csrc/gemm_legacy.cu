// Legacy-instruction path: the same operator on the warp-level
// mma.sync.m16n8k64 s4 instruction the reference is built around
// (kernels/linear_v21.h:95-106), kept as the comparison point for the tcgen05
// path and as an independently derived second implementation to cross-check it.
// It is deliberately simple -- fragments are fetched straight from global memory
// through the read-only cache, one 64 x 64 tile per CTA -- and is not meant to be
// fast.
#include "common.h"

namespace i4l {

namespace {

__device__ __forceinline__ void mma_s4(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k64.row.col.s32.s4.s4.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 4 warps as 2 x 2; each warp computes 32 x 32 outputs = 2 x 4 MMA tiles.
__global__ void __launch_bounds__(128)
gemm_s4_legacy_kernel(const uint32_t* __restrict__ x, const uint32_t* __restrict__ w, int* __restrict__ y,
                      int m, int n, int k, const int* __restrict__ bias)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int row0 = blockIdx.y * 64 + (warp >> 1) * 32;
    const int col0 = blockIdx.x * 64 + (warp & 1) * 32;
    const int words = k >> 3;  // 32-bit words per row

    int acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0;

    // One instruction covers 64 K elements = 8 words; lane q holds word q
    // (elements 8q..8q+7) and word 4+q (elements 32+8q..).
    for (int kw = 0; kw < words; kw += 8) {
        const bool hi_ok = kw + 4 < words;  // k % 64 == 32 leaves the upper half empty
        uint32_t a[2][4], b[4][2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r_lo = row0 + i * 16 + g, r_hi = r_lo + 8;
            const uint32_t* p_lo = x + static_cast<size_t>(r_lo) * words + kw + q;
            const uint32_t* p_hi = x + static_cast<size_t>(r_hi) * words + kw + q;
            a[i][0] = r_lo < m ? __ldg(p_lo) : 0u;
            a[i][1] = r_hi < m ? __ldg(p_hi) : 0u;
            a[i][2] = (r_lo < m && hi_ok) ? __ldg(p_lo + 4) : 0u;
            a[i][3] = (r_hi < m && hi_ok) ? __ldg(p_hi + 4) : 0u;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = col0 + j * 8 + g;
            const uint32_t* p = w + static_cast<size_t>(c) * words + kw + q;
            b[j][0] = c < n ? __ldg(p) : 0u;
            b[j][1] = (c < n && hi_ok) ? __ldg(p + 4) : 0u;
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                mma_s4(acc[i][j], a[i][0], a[i][1], a[i][2], a[i][3], b[j][0], b[j][1]);
    }

#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = col0 + j * 8 + 2 * q;
            const int r_lo = row0 + i * 16 + g, r_hi = r_lo + 8;
            if (bias != nullptr) {
                const int b0 = c < n ? __ldg(bias + c) : 0, b1 = c + 1 < n ? __ldg(bias + c + 1) : 0;
                acc[i][j][0] += b0; acc[i][j][1] += b1; acc[i][j][2] += b0; acc[i][j][3] += b1;
            }
            if (r_lo < m) {
                if (c < n) y[static_cast<size_t>(r_lo) * n + c] = acc[i][j][0];
                if (c + 1 < n) y[static_cast<size_t>(r_lo) * n + c + 1] = acc[i][j][1];
            }
            if (r_hi < m) {
                if (c < n) y[static_cast<size_t>(r_hi) * n + c] = acc[i][j][2];
                if (c + 1 < n) y[static_cast<size_t>(r_hi) * n + c + 1] = acc[i][j][3];
            }
        }
}

}  // namespace

int launch_legacy(DeviceCtx*, const Problem& p, cudaStream_t stream)
{
    dim3 grid((p.n + 63) / 64, (p.m + 63) / 64);
    gemm_s4_legacy_kernel<<<grid, 128, 0, stream>>>(static_cast<const uint32_t*>(p.x),
                                                     static_cast<const uint32_t*>(p.w),
                                                     static_cast<int*>(p.y), p.m, p.n, p.k, p.bias);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

}  // namespace i4l
