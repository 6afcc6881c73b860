// Decode-shape kernel (m <= 64): HBM-bound streaming of the packed weights.
//
// For a handful of activation rows the operator is one pass over W (N x K/2
// bytes) with almost no arithmetic per byte, so the design goal is to keep
// every SM pulling from HBM and to touch each weight byte exactly once, with no
// shared-memory round trip for W at all:
//   * each CTA owns a contiguous run of 8-row groups of W (so that it streams one
//     contiguous span of memory) and keeps the whole packed X (<= 64 rows) in
//     shared memory;
//   * each warp takes (group, K-slice) units; a lane loads 16 contiguous bytes of a
//     W row straight into registers (8 rows x 64 B per warp instruction), expands
//     the nibbles in registers and feeds warp-level mma.sync m16n8k32 s8;
//   * K-slice partial sums meet in a small shared-memory accumulator
//     (red.shared.add), and the CTA writes its Y columns once, coalesced.
// There is no split-K through global memory, no atomics on Y and no scratch.
//
// Same x16 nibble expansion as the main kernel: a packed word x gives
// (x << 4) & 0xF0F0F0F0 (even elements) and x & 0xF0F0F0F0 (odd elements), each
// byte 16 times the element; these two registers are exactly the (k 0-15,
// k 16-31) halves of one m16n8k32 fragment.  X words go through the same
// expansion, so both operands see the same K permutation; the int32 sum is
// 256 * y and is shifted back by 8.
//
// Replaces, for these shapes, the reference's kernels/linear_v21.h:471-753
// (which runs them as 256 x 128 tiles that are almost entirely padding).
#include "common.h"
#include "ptx.cuh"

namespace i4l {

namespace {

constexpr int kWarps = 16;
constexpr int kSkinnyThreads = kWarps * 32;
constexpr int kSlices = 8;  // K slices a group's work is spread over

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MB = number of 16-row blocks of X (m <= 16 * MB).
template <int MB>
__global__ void __launch_bounds__(kSkinnyThreads, 1)
gemm_s4_skinny_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ w, int* __restrict__ y,
                      int m, int n, int k, int groups_total, int groups_per_cta_max, int x_pitch)
{
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* xs = smem;                                                  // [MB*16][x_pitch]
    int* acc = reinterpret_cast<int*>(smem + MB * 16 * x_pitch);        // [groups][MB*16][8]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, q = lane & 3;
    const int row_bytes = k >> 1;

    // This CTA's run of 8-row groups.
    const int g_begin = static_cast<int>(static_cast<long long>(blockIdx.x) * groups_total / gridDim.x);
    const int g_end = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * groups_total / gridDim.x);
    const int n_groups = g_end - g_begin;

    // Stage packed X (rows >= m as zeros) and clear the accumulator.
    {
        const int chunks_per_row = row_bytes >> 4;
        const int total = MB * 16 * chunks_per_row;
        for (int i = tid; i < total; i += kSkinnyThreads) {
            const int r = i / chunks_per_row, c = i - r * chunks_per_row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < m) v = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * row_bytes + c * 16);
            *reinterpret_cast<uint4*>(xs + r * x_pitch + c * 16) = v;
        }
        for (int i = tid; i < n_groups * MB * 128; i += kSkinnyThreads) acc[i] = 0;
    }
    __syncthreads();

    // K in blocks of 128 elements (64 bytes per row); a lane owns bytes
    // [16q, 16q+16) of each block.  Slices are contiguous runs of blocks.
    const int kb_count = (k + 127) >> 7;
    const int slice = warp % kSlices;
    const int kb_begin = slice * kb_count / kSlices;
    const int kb_end = (slice + 1) * kb_count / kSlices;
    const int lane_off = q * 16;

    for (int gi = warp / kSlices; gi < n_groups; gi += kWarps / kSlices) {
        const int wrow = (g_begin + gi) * 8 + g;
        const bool row_ok = wrow < n;
        const uint8_t* wp = w + static_cast<size_t>(row_ok ? wrow : 0) * row_bytes + lane_off;
        int c[MB][4];
#pragma unroll
        for (int b = 0; b < MB; ++b) { c[b][0] = c[b][1] = c[b][2] = c[b][3] = 0; }

        for (int kb0 = kb_begin; kb0 < kb_end; kb0 += 4) {
            uint4 wv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int kb = kb0 + u;
                const bool ok = row_ok && kb < kb_end && (kb * 64 + lane_off) < row_bytes;
                wv[u] = ok ? ldg_stream(wp + kb * 64) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int kb = kb0 + u;
                if (kb >= kb_end) break;
                const uint32_t ww[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
                uint32_t b_lo[4], b_hi[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    b_lo[e] = (ww[e] << 4) & 0xF0F0F0F0u;
                    b_hi[e] = ww[e] & 0xF0F0F0F0u;
                }
#pragma unroll
                for (int b = 0; b < MB; ++b) {
                    const uint8_t* xa = xs + (b * 16 + g) * x_pitch + kb * 64 + lane_off;
                    const uint4 x0 = *reinterpret_cast<const uint4*>(xa);
                    const uint4 x1 = *reinterpret_cast<const uint4*>(xa + 8 * x_pitch);
                    const uint32_t xa0[4] = {x0.x, x0.y, x0.z, x0.w};
                    const uint32_t xa1[4] = {x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        mma_s8(c[b],
                               (xa0[e] << 4) & 0xF0F0F0F0u, (xa1[e] << 4) & 0xF0F0F0F0u,
                               xa0[e] & 0xF0F0F0F0u, xa1[e] & 0xF0F0F0F0u,
                               b_lo[e], b_hi[e]);
                    }
                }
            }
        }
        // Fragment -> accumulator: c0,c1 = (row g, cols 2q,2q+1); c2,c3 = row g+8.
        if (kb_begin < kb_end) {
#pragma unroll
            for (int b = 0; b < MB; ++b) {
                int* a = acc + (gi * MB * 16 + b * 16) * 8;
                atomicAdd(a + g * 8 + 2 * q, c[b][0] >> 8);
                atomicAdd(a + g * 8 + 2 * q + 1, c[b][1] >> 8);
                atomicAdd(a + (g + 8) * 8 + 2 * q, c[b][2] >> 8);
                atomicAdd(a + (g + 8) * 8 + 2 * q + 1, c[b][3] >> 8);
            }
        }
    }
    __syncthreads();

    // Y[r][g_begin*8 .. g_end*8): consecutive threads write consecutive columns.
    const int cols = n_groups * 8;
    const int col_base = g_begin * 8;
    for (int i = tid; i < m * cols; i += kSkinnyThreads) {
        const int r = i / cols, cc = i - r * cols;
        const int col = col_base + cc;
        if (col < n) y[static_cast<size_t>(r) * n + col] = acc[((cc >> 3) * MB * 16 + r) * 8 + (cc & 7)];
    }
}

struct SkinnyPlan {
    int mb, grid, groups_total, groups_per_cta_max, x_pitch;
    size_t smem;
};

bool plan_skinny(const DeviceCtx* ctx, const Problem& p, SkinnyPlan* out)
{
    if (p.m > 64) return false;
    SkinnyPlan s;
    s.mb = p.m <= 16 ? 1 : (p.m <= 32 ? 2 : 4);
    s.groups_total = (p.n + 7) / 8;
    s.grid = s.groups_total < ctx->sm_count ? s.groups_total : ctx->sm_count;
    s.groups_per_cta_max = (s.groups_total + s.grid - 1) / s.grid;
    // Row pitch of X in shared memory: == 64 (mod 128) so that the eight rows a
    // quarter-warp reads land in distinct 16-byte bank groups.
    const int row_bytes = p.k / 2;
    s.x_pitch = ((row_bytes + 127) / 128) * 128 + 64;
    s.smem = static_cast<size_t>(s.mb) * 16 * s.x_pitch +
             static_cast<size_t>(s.groups_per_cta_max) * s.mb * 128 * sizeof(int);
    if (s.smem > 200 * 1024) return false;
    *out = s;
    return true;
}

}  // namespace

bool skinny_supports(const DeviceCtx* ctx, const Problem& p)
{
    SkinnyPlan s;
    return plan_skinny(ctx, p, &s);
}

int setup_skinny(DeviceCtx*)
{
    cudaError_t e = cudaFuncSetAttribute(gemm_s4_skinny_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_s4_skinny_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_s4_skinny_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    return e == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

int launch_skinny(DeviceCtx* ctx, const Problem& p, cudaStream_t stream)
{
    SkinnyPlan s;
    if (!plan_skinny(ctx, p, &s)) return INT4L_ERR_UNSUPPORTED;
    const uint8_t* x = static_cast<const uint8_t*>(p.x);
    const uint8_t* w = static_cast<const uint8_t*>(p.w);
    int* y = static_cast<int*>(p.y);
    if (s.mb == 1)
        gemm_s4_skinny_kernel<1><<<s.grid, kSkinnyThreads, s.smem, stream>>>(x, w, y, p.m, p.n, p.k, s.groups_total, s.groups_per_cta_max, s.x_pitch);
    else if (s.mb == 2)
        gemm_s4_skinny_kernel<2><<<s.grid, kSkinnyThreads, s.smem, stream>>>(x, w, y, p.m, p.n, p.k, s.groups_total, s.groups_per_cta_max, s.x_pitch);
    else
        gemm_s4_skinny_kernel<4><<<s.grid, kSkinnyThreads, s.smem, stream>>>(x, w, y, p.m, p.n, p.k, s.groups_total, s.groups_per_cta_max, s.x_pitch);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

}  // namespace i4l
