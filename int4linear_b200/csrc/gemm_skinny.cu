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
#include <cstdlib>

#include <cuda_bf16.h>

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

// Final write of one output: the exact int32 (plus optional int32 bias), or the dequantised
// bfloat16 with the same arithmetic as the tensor-memory kernels' epilogue.
__device__ __forceinline__ void write_out(int* __restrict__ y, const int* __restrict__ bias, const ScaledOut& so,
                                          int r, int col, int n, int acc)
{
    if (so.y16 != nullptr) {
        const float rs = so.row_scale != nullptr ? __ldg(so.row_scale + r) : 1.0f;
        const float cs = so.col_scale != nullptr ? __ldg(so.col_scale + col) : 1.0f;
        const float b = so.bias != nullptr ? __ldg(so.bias + col) : 0.0f;
        static_cast<unsigned short*>(so.y16)[static_cast<size_t>(r) * n + col] =
            scaled_to_bits(fmaf(static_cast<float>(acc) * rs, cs, b), so.fp16);
    } else {
        y[static_cast<size_t>(r) * n + col] = acc + (bias ? __ldg(bias + col) : 0);
    }
}

// MB = number of 16-row blocks of X (m <= 16 * MB).
template <int MB>
__global__ void __launch_bounds__(kSkinnyThreads, 1)
gemm_s4_skinny_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ w, int* __restrict__ y,
                      int m, int n, int k, int groups_total, int groups_per_cta_max, int x_pitch, const int* __restrict__ bias,
                      const ScaledOut so)
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
        if (col < n) write_out(y, bias, so, r, col, n, acc[((cc >> 3) * MB * 16 + r) * 8 + (cc & 7)]);
    }
}


// Register-resident variant for m <= 16 and K <= 8192 (the decode shape proper).
// Each warp (16 or 32 per CTA) owns a fixed slice of K (KBW blocks of 128 elements) for every
// W group of the CTA, so its X fragments are loaded and expanded ONCE into registers and
// the inner loop is nothing but: one 16-byte streaming load per lane and K block, eight
// ALU operations to expand it, four MMAs.  Weight loads for several groups ahead are kept
// in flight, and the first of them are issued before anything else happens in the kernel,
// so HBM is busy from the first cycle; X never goes through shared memory.
template <int KBW, int D, int MINB, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, MINB)
gemm_s4_skinny_reg_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ w, int* __restrict__ y,
                          int m, int n, int k, int groups_total, int overlap, const int* __restrict__ bias,
                          const ScaledOut so)
{
    // D = groups of weight loads in flight per warp; WARPS * KBW K blocks are covered by one CTA.
    constexpr int kThreadsHere = WARPS * 32;
    // overlap: 0 = ordinary launch.  1, 2 = launched with programmatic stream serialisation:
    // this grid may start while the preceding work in the stream is still running, and lets its
    // own successor do the same.  Everything it reads before griddepcontrol.wait must therefore
    // not be written by that preceding work: the weights (1), or the weights and X (2).
    if (overlap) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(16) uint8_t smem[];
    int* acc = reinterpret_cast<int*>(smem);  // [groups][16][8]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, q = lane & 3;
    const int row_bytes = k >> 1;
    const int g_begin = static_cast<int>(static_cast<long long>(blockIdx.x) * groups_total / gridDim.x);
    const int g_end = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * groups_total / gridDim.x);
    const int n_groups = g_end - g_begin;

    // Byte offset of this lane's 16 bytes inside a row, per K block of the warp's slice.
    const int col0 = warp * KBW * 64 + q * 16;
    bool col_ok[KBW];
#pragma unroll
    for (int u = 0; u < KBW; ++u) col_ok[u] = col0 + u * 64 < row_bytes;

    auto load_group = [&](int gi, uint4 (&dst)[KBW]) {
        const int wrow = (g_begin + gi) * 8 + g;
        const bool ok = gi < n_groups && wrow < n;
        const uint8_t* p = w + static_cast<size_t>(ok ? wrow : 0) * row_bytes + col0;
#pragma unroll
        for (int u = 0; u < KBW; ++u)
            dst[u] = (ok && col_ok[u]) ? ldg_stream(p + u * 64) : make_uint4(0, 0, 0, 0);
    };

    uint4 wv[D][KBW];
#pragma unroll
    for (int d = 0; d < D; ++d) load_group(d, wv[d]);

    if (overlap == 1) asm volatile("griddepcontrol.wait;" ::: "memory");

    // X words of this warp's K slice, rows g and g + 8, kept PACKED (two registers per MMA): the
    // nibble expansion is redone for every group -- six ALU operations per MMA -- because the
    // registers this saves hold weight loads in flight, which is what the kernel's speed hangs on.
    uint32_t xa[KBW][4], xb[KBW][4];
#pragma unroll
    for (int u = 0; u < KBW; ++u) {
        uint4 x0 = make_uint4(0, 0, 0, 0), x1 = make_uint4(0, 0, 0, 0);
        if (col_ok[u]) {
            if (g < m) x0 = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(g) * row_bytes + col0 + u * 64);
            if (g + 8 < m) x1 = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(g + 8) * row_bytes + col0 + u * 64);
        }
        xa[u][0] = x0.x; xa[u][1] = x0.y; xa[u][2] = x0.z; xa[u][3] = x0.w;
        xb[u][0] = x1.x; xb[u][1] = x1.y; xb[u][2] = x1.z; xb[u][3] = x1.w;
    }

    for (int i = tid; i < n_groups * 128; i += kThreadsHere) acc[i] = 0;
    __syncthreads();

    for (int gi0 = 0; gi0 < n_groups; gi0 += D) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const int gi = gi0 + d;
            if (gi < n_groups) {
                int c[4] = {0, 0, 0, 0};
#pragma unroll
                for (int u = 0; u < KBW; ++u) {
                    const uint32_t ww[4] = {wv[d][u].x, wv[d][u].y, wv[d][u].z, wv[d][u].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        mma_s8(c, (xa[u][e] << 4) & 0xF0F0F0F0u, (xb[u][e] << 4) & 0xF0F0F0F0u,
                               xa[u][e] & 0xF0F0F0F0u, xb[u][e] & 0xF0F0F0F0u,
                               (ww[e] << 4) & 0xF0F0F0F0u, ww[e] & 0xF0F0F0F0u);
                }
                load_group(gi + D, wv[d]);
                int* o = acc + gi * 128;
                atomicAdd(o + g * 8 + 2 * q, c[0] >> 8);
                atomicAdd(o + g * 8 + 2 * q + 1, c[1] >> 8);
                atomicAdd(o + (g + 8) * 8 + 2 * q, c[2] >> 8);
                atomicAdd(o + (g + 8) * 8 + 2 * q + 1, c[3] >> 8);
            }
        }
    }
    __syncthreads();

    if (overlap == 2) asm volatile("griddepcontrol.wait;" ::: "memory");
    const int cols = n_groups * 8;
    const int col_base = g_begin * 8;
    for (int i = tid; i < m * cols; i += kThreadsHere) {
        const int r = i / cols, cc = i - r * cols;
        const int col = col_base + cc;
        if (col < n) write_out(y, bias, so, r, col, n, acc[((cc >> 3) * 16 + r) * 8 + (cc & 7)]);
    }
}


// Tensor-map variant for m <= 16 and K outside the range of the register variant.
// Every warp owns K slices of 128 packed bytes (256 elements).  For a slice it asks TMA
// for a box of [R rows x 128 B] of W -- all rows of the CTA's run at once when they fit,
// so that the whole weight slab of the CTA is requested in the first microsecond of the
// kernel and HBM can stream without waiting for anybody's registers -- into a private,
// 128-byte-swizzled buffer, and then walks the rows eight at a time with ldmatrix, which
// hands lane (g, q) four bytes of row g for each of four 16-byte chunks: exactly one
// m16n8k32 B fragment per register after the nibble expansion.  X fragments (the same
// bytes of rows g and g + 8 of X) stay in registers for the slice.
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__global__ void __launch_bounds__(kSkinnyThreads, 1)
gemm_s4_skinny_tma_kernel(const __grid_constant__ CUtensorMap tm_w, const uint8_t* __restrict__ x,
                          int* __restrict__ y, int m, int n, int k, int groups_total,
                          int stage_rows, int n_buffers, int* status, const int* __restrict__ bias)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - raw);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, q = lane & 3;
    const int row_bytes = k >> 1;
    const int n_slices = (row_bytes + 127) >> 7;
    const int g_begin = static_cast<int>(static_cast<long long>(blockIdx.x) * groups_total / gridDim.x);
    const int g_end = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * groups_total / gridDim.x);
    const int n_groups = g_end - g_begin;
    const int stage_groups = stage_rows >> 3;
    const int passes = (n_groups + stage_groups - 1) / stage_groups;

    // Layout: [16 warps][n_buffers][stage_rows x 128 B] | barriers [16][4] | abort | acc
    const uint32_t stage_bytes = static_cast<uint32_t>(stage_rows) * 128u;
    const uint32_t buf0 = base + (warp * n_buffers) * stage_bytes;
    const uint32_t bar_off = 16u * n_buffers * stage_bytes;
    const uint32_t bar0 = base + bar_off + warp * 32u;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + bar_off + 16 * 32);
    int* acc = reinterpret_cast<int*>(gbase + bar_off + 16 * 32 + 16);  // [groups][16][8]

    // Items of this warp in consumption order: slice-major over its slices, row passes inside.
    const int my_slices = warp < n_slices ? (n_slices - warp + 15) / 16 : 0;
    const int n_items = my_slices * passes;
    auto issue = [&](int item) {
        const int s = warp + 16 * (item / passes), p = item % passes;
        const int b = item % n_buffers;
        mbar_expect_tx(bar0 + 8u * b, stage_bytes);
        tma_load_2d(buf0 + b * stage_bytes, &tm_w, bar0 + 8u * b, s * 128, (g_begin + p * stage_groups) * 8);
    };

    if (tid == 0) *abort_flag = 0;
    if (lane == 0) {
        for (int b = 0; b < n_buffers; ++b) mbar_init(bar0 + 8u * b, 1);
        mbar_init_fence();
        for (int it = 0; it < n_items && it < n_buffers; ++it) issue(it);
    }
    for (int i = tid; i < n_groups * 128; i += kSkinnyThreads) acc[i] = 0;
    __syncthreads();

    uint32_t a[2][4][4];  // [half of the slice][16-byte chunk][a0..a3]
    int cur_slice = -1;
    bool alive = true;
    for (int item = 0; alive && item < n_items; ++item) {
        const int s = warp + 16 * (item / passes), p = item % passes;
        const int b = item % n_buffers;
        if (s != cur_slice) {
            cur_slice = s;
            // X words for this slice: byte offset of chunk j in half h is s*128 + h*64 + 16j + 4q.
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int off = s * 128 + h * 64 + j * 16 + q * 4;
                    uint32_t r0 = 0, r1 = 0;
                    if (off < row_bytes) {
                        if (g < m) r0 = __ldg(reinterpret_cast<const uint32_t*>(x + static_cast<size_t>(g) * row_bytes + off));
                        if (g + 8 < m) r1 = __ldg(reinterpret_cast<const uint32_t*>(x + static_cast<size_t>(g + 8) * row_bytes + off));
                    }
                    a[h][j][0] = (r0 << 4) & 0xF0F0F0F0u;
                    a[h][j][1] = (r1 << 4) & 0xF0F0F0F0u;
                    a[h][j][2] = r0 & 0xF0F0F0F0u;
                    a[h][j][3] = r1 & 0xF0F0F0F0u;
                }
        }
        if (!mbar_wait(bar0 + 8u * b, (item / n_buffers) & 1u, abort_flag)) { alive = false; break; }
        const uint32_t buf = buf0 + b * stage_bytes;
        const int groups_here = min(stage_groups, n_groups - p * stage_groups);
        // ldmatrix row address of this lane: row (lane & 7) of the group, chunk (lane >> 3).
        const uint32_t lrow = lane & 7, lchunk = lane >> 3;
        for (int gi = 0; gi < groups_here; ++gi) {
            const uint32_t rowaddr = buf + (gi * 8 + lrow) * 128u;
            uint32_t w0[4], w1[4];
            ldmatrix_x4(rowaddr + ((lchunk ^ lrow) << 4), w0);
            ldmatrix_x4(rowaddr + (((4 + lchunk) ^ lrow) << 4), w1);
            int c[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 4; ++j)
                mma_s8(c, a[0][j][0], a[0][j][1], a[0][j][2], a[0][j][3], (w0[j] << 4) & 0xF0F0F0F0u, w0[j] & 0xF0F0F0F0u);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                mma_s8(c, a[1][j][0], a[1][j][1], a[1][j][2], a[1][j][3], (w1[j] << 4) & 0xF0F0F0F0u, w1[j] & 0xF0F0F0F0u);
            int* o = acc + (p * stage_groups + gi) * 128;
            atomicAdd(o + g * 8 + 2 * q, c[0] >> 8);
            atomicAdd(o + g * 8 + 2 * q + 1, c[1] >> 8);
            atomicAdd(o + (g + 8) * 8 + 2 * q, c[2] >> 8);
            atomicAdd(o + (g + 8) * 8 + 2 * q + 1, c[3] >> 8);
        }
        // Refill this buffer with the item that will use it next.
        if (item + n_buffers < n_items) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) issue(item + n_buffers);
        }
    }
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0) atomicExch(status, INT4L_ERR_DEVICE_TIMEOUT);
        for (int i = 0; i < 100; ++i) __nanosleep(1000);
        return;
    }

    const int cols = n_groups * 8;
    const int col_base = g_begin * 8;
    for (int i = tid; i < m * cols; i += kSkinnyThreads) {
        const int r = i / cols, cc = i - r * cols;
        const int col = col_base + cc;
        if (col < n) y[static_cast<size_t>(r) * n + col] = acc[((cc >> 3) * 16 + r) * 8 + (cc & 7)] + (bias ? __ldg(bias + col) : 0);
    }
}

// Experiment knobs of the decode kernels, read from the environment once per process (a decode
// launch lasts microseconds; a getenv per launch would show):
//   INT4L_SKINNY_CTAS_PER_SM = 1 | 2   CTAs per SM of the register variant
//   INT4L_SKINNY_ROWS / INT4L_SKINNY_BUFS   stage geometry of the TMA variant
//   INT4L_SKINNY_DEPTH = 8   eight instead of four groups of weight loads in flight per warp (K <= 2048)
//   INT4L_SKINNY_EVEN_GRID = 1   equal shares of 8-row groups per CTA instead of a CTA in every slot
struct SkinnyEnv {
    int ctas_per_sm = 0, stage_rows = 0, n_buffers = 2, depth = 0, even_grid = 0;
};
const SkinnyEnv& skinny_env()
{
    static const SkinnyEnv env = [] {
        SkinnyEnv v;
        if (const char* e = getenv("INT4L_SKINNY_CTAS_PER_SM")) v.ctas_per_sm = atoi(e) == 1 ? 1 : 2;
        if (const char* e = getenv("INT4L_SKINNY_DEPTH")) v.depth = atoi(e);
        if (const char* e = getenv("INT4L_SKINNY_EVEN_GRID")) v.even_grid = atoi(e);
        if (const char* e = getenv("INT4L_SKINNY_ROWS")) {
            v.stage_rows = atoi(e);
            if (const char* b = getenv("INT4L_SKINNY_BUFS")) v.n_buffers = atoi(b);
        }
        return v;
    }();
    return env;
}

struct SkinnyPlan {
    int mb, grid, groups_total, groups_per_cta_max, x_pitch;
    size_t smem;
};

// Experiment knob INT4L_SKINNY: 0 automatic (register variant, else TMA variant, else the
// shared-memory variant), 1 never the TMA variant, 2 shared-memory variant only, 3 never the
// register variant.
int skinny_variant()
{
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("INT4L_SKINNY");
        v = e ? atoi(e) : 0;
    }
    return v;
}

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

template <int KBW, int D, int MINB, int WARPS>
cudaError_t reg_attr()
{
    return cudaFuncSetAttribute(gemm_s4_skinny_reg_kernel<KBW, D, MINB, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
}

template <int KBW, int D, int MINB, int WARPS>
cudaError_t reg_launch(cudaLaunchConfig_t cfg, int slots_per_sm_cap, const DeviceCtx* ctx, const Problem& p, int groups_total, int overlap,
                       bool even_grid)
{
    // Every CTA gets the same number of 8-row groups (the last one possibly fewer): the launch
    // lasts as long as its busiest CTA, and one group more or less is a sixth of the work.
    const int slots = (MINB < slots_per_sm_cap ? MINB : slots_per_sm_cap) * ctx->sm_count;
    const int per_cta = (groups_total + slots - 1) / slots;
    int grid = (groups_total + per_cta - 1) / per_cta;
    if (!even_grid) grid = groups_total < slots ? groups_total : slots;
    const int per_cta_max = (groups_total + grid - 1) / grid;
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(per_cta_max) * 128 * sizeof(int);
    return cudaLaunchKernelEx(&cfg, gemm_s4_skinny_reg_kernel<KBW, D, MINB, WARPS>, static_cast<const uint8_t*>(p.x),
                              static_cast<const uint8_t*>(p.w), static_cast<int*>(p.y), p.m, p.n, p.k, groups_total, overlap,
                              p.bias, p.scaled);
}

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
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_s4_skinny_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess) e = reg_attr<1, 4, 2, 16>();
    if (e == cudaSuccess) e = reg_attr<1, 8, 2, 16>();
    if (e == cudaSuccess) e = reg_attr<2, 2, 2, 16>();
    if (e == cudaSuccess) e = reg_attr<4, 2, 1, 16>();
    return e == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

int launch_skinny(DeviceCtx* ctx, const Problem& p, cudaStream_t stream)
{
    SkinnyPlan s;
    if (!plan_skinny(ctx, p, &s)) return INT4L_ERR_UNSUPPORTED;
    const uint8_t* x = static_cast<const uint8_t*>(p.x);
    const uint8_t* w = static_cast<const uint8_t*>(p.w);
    int* y = static_cast<int*>(p.y);
    const int kb_count = (p.k + 127) / 128;
    if (p.m <= 16 && kb_count >= 16 && kb_count <= 64 && skinny_variant() != 2 && skinny_variant() != 3) {
        // Two CTAs per SM: consecutive launches (overlap modes) can then be resident together,
        // so one launch streams weights while the previous one merges and writes its result.
        const int overlap = p.overlap >= 0 ? p.overlap : stream_overlap_mode();
        // One CTA per SM when launches may fully overlap (two launches then share each SM);
        // otherwise two, which hides more latency inside a single launch.
        int ctas_per_sm = overlap == 2 ? 1 : 2;
        if (skinny_env().ctas_per_sm) ctas_per_sm = skinny_env().ctas_per_sm;
        cudaLaunchConfig_t cfg = {};
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = overlap ? 1 : 0;
        const bool even = skinny_env().even_grid != 0;
        const int variant = skinny_env().depth;  // experiment: 8 = eight instead of four groups in flight (K <= 2048)
        cudaError_t e;
        if (kb_count <= 16) {
            e = variant == 8 ? reg_launch<1, 8, 2, 16>(cfg, ctas_per_sm, ctx, p, s.groups_total, overlap, even)
                             : reg_launch<1, 4, 2, 16>(cfg, ctas_per_sm, ctx, p, s.groups_total, overlap, even);
        } else if (kb_count <= 32) {
            e = reg_launch<2, 2, 2, 16>(cfg, ctas_per_sm, ctx, p, s.groups_total, overlap, even);
        } else {
            e = reg_launch<4, 2, 1, 16>(cfg, ctas_per_sm, ctx, p, s.groups_total, overlap, even);
        }
        count_launch();
        if (e != cudaSuccess) { cudaGetLastError(); return INT4L_ERR_CUDA; }
        return INT4L_OK;
    }
    if (p.m <= 16 && p.k >= 256 && skinny_variant() != 2 && p.scaled.y16 == nullptr) {
        // Whole slab resident when it fits (one buffer per warp holding every row of the CTA's
        // run for the warp's slice), otherwise two 48-row buffers per warp.
        const int rows_max = s.groups_per_cta_max * 8;
        const int n_slices = (p.k / 2 + 127) / 128;
        const size_t fixed = 1024 + 16 * 32 + 16 + static_cast<size_t>(s.groups_per_cta_max) * 128 * sizeof(int);
        int stage_rows = rows_max, n_buffers = 1;
        if (rows_max > 256 || n_slices > 16 || fixed + 16ull * rows_max * 128 > 227 * 1024) {
            stage_rows = 48;
            n_buffers = 2;
        }
        if (skinny_env().stage_rows) {  // experiment: explicit stage geometry
            stage_rows = skinny_env().stage_rows;
            n_buffers = skinny_env().n_buffers;
        }
        const size_t smem = fixed + 16ull * n_buffers * stage_rows * 128;
        if (smem <= 227 * 1024 && skinny_variant() != 1) {
            CUtensorMap tm_w;
            const uint64_t pitch = static_cast<uint64_t>(p.k) / 2;
            int rc = make_tensor_map_2d(ctx, &tm_w, p.w, 1, pitch, p.n, pitch, 128, stage_rows, true);
            if (rc != INT4L_OK) return rc;
            gemm_s4_skinny_tma_kernel<<<s.grid, kSkinnyThreads, smem, stream>>>(
                tm_w, x, y, p.m, p.n, p.k, s.groups_total, stage_rows, n_buffers, ctx->status_dev, p.bias);
            count_launch();
            return cudaGetLastError() == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
        }
    }
    if (s.mb == 1)
        gemm_s4_skinny_kernel<1><<<s.grid, kSkinnyThreads, s.smem, stream>>>(x, w, y, p.m, p.n, p.k, s.groups_total, s.groups_per_cta_max, s.x_pitch, p.bias, p.scaled);
    else if (s.mb == 2)
        gemm_s4_skinny_kernel<2><<<s.grid, kSkinnyThreads, s.smem, stream>>>(x, w, y, p.m, p.n, p.k, s.groups_total, s.groups_per_cta_max, s.x_pitch, p.bias, p.scaled);
    else
        gemm_s4_skinny_kernel<4><<<s.grid, kSkinnyThreads, s.smem, stream>>>(x, w, y, p.m, p.n, p.k, s.groups_total, s.groups_per_cta_max, s.x_pitch, p.bias, p.scaled);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

}  // namespace i4l
