// Shared epilogue of the tensor-memory GEMM kernels: one warp drains its 32 TMEM lanes
// (32 output rows) x `width` accumulator columns (a multiple of 32) into Y.
//
// The accumulator holds 256 * y (both operands were expanded to 16 x value), so each value is
// shifted right by 8 (arithmetic, exact), the optional int32 bias of its column is added, and
// the 32 x 32 chunk goes out either
//   * through a 128-byte-swizzled shared-memory staging buffer and one TMA store (which clips
//     the M and N tails by itself; `n_maps` destinations, each shifted right by `col_shift`
//     columns); two staging buffers per warp alternate, and a buffer is
//     reused only after the store group that read it has finished reading; or
//   * with per-thread stores (any n, needed when the row pitch of Y is not a multiple of 16 B).
// Replaces the reference's per-thread int2 stores, kernels/linear_v21.h:661-710.
#pragma once

#include <cuda_bf16.h>

#include "common.h"
#include "ptx.cuh"

namespace i4l {

// kAdd: the values are partial sums of a tile that is cut along K and are ADDED into Y (a bulk
// reduction per staged block, or atomic adds on the per-thread path) instead of stored.
template <bool kTmaStore, bool kAdd = false>
__device__ __forceinline__ void drain_accumulator(uint32_t t_addr, int width, int row0, int col0, int m, int n,
                                                  int* __restrict__ y, const int* __restrict__ bias,
                                                  const CUtensorMap* tm_y, int n_maps, int col_shift,
                                                  uint32_t stage0, uint32_t& chunk_no,
                                                  int lane)
{
    const int row = row0 + lane;
    const bool vec_ok = (n & 3) == 0;
#pragma unroll 1
    for (int c = 0; c < width; c += 32) {
        // A chunk entirely outside Y is skipped as a whole, so that the staging buffers
        // alternate exactly with the store groups that were committed.
        if (kTmaStore && !(row0 < m && col0 + c < n)) continue;
        uint32_t v[32];
        tmem_ld_32x32(t_addr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = static_cast<uint32_t>(static_cast<int>(v[i]) >> 8);
        if (bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (col0 + c + i < n) v[i] += static_cast<uint32_t>(__ldg(bias + col0 + c + i));
        }
        if constexpr (kTmaStore) {
            const uint32_t stg = stage0 + (chunk_no & 1u) * 4096;
            // The store issued two chunks ago read this buffer; make sure it is done.
            if (lane == 0) tma_store_wait_read<1>();
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 8; ++q)
                sts128(stg + lane * 128 + ((q ^ (lane & 7)) << 4),
                       make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                // One store per destination matrix (one normally; every rank's copy of the full Y
                // when the result is gathered through peer memory), all from the same staging tile.
                if constexpr (kAdd) tma_reduce_add_2d(tm_y, stg, col_shift + col0 + c, row0);
                else
                    for (int d = 0; d < n_maps; ++d) tma_store_2d(tm_y + d, stg, col_shift + col0 + c, row0);
                tma_store_commit();
            }
            ++chunk_no;
        } else {
            if (row < m) {
                int* dst = y + static_cast<size_t>(row) * n + col0 + c;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int col = col0 + c + 4 * q;
                    if constexpr (kAdd) {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (col + e < n) atomicAdd(dst + 4 * q + e, static_cast<int>(v[4 * q + e]));
                    } else if (vec_ok && col + 3 < n) {
                        *reinterpret_cast<int4*>(dst + 4 * q) =
                            make_int4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (col + e < n) dst[4 * q + e] = static_cast<int>(v[4 * q + e]);
                    }
                }
            }
        }
    }
}

// The few-rows kernel spreads its UMMAs over two issuing threads with an accumulator each (second_acc:
// the other accumulator's distance in columns, or -1 when only one of them holds anything).
__device__ __forceinline__ void add_second_accumulator(uint32_t t_addr, uint32_t (&v)[32])
{
    uint32_t u[32];
    tmem_ld_32x32(t_addr, u);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] += u[i];
}

// Swapped operands (gemm_fewrows.cu): the accumulator is a tile of Y transposed -- lane = row of W =
// column of Y, accumulator column = row of X = row of Y.  w_rows and x_rows are Y's column and row
// counts.  The warp writes its 32 x 32 block transposed into a 128-byte-swizzled staging tile (for each
// accumulator column the 32 lanes fill one 128-byte row: no bank conflicts) and one bulk store -- or
// bulk reduction, for a share of a tile that is cut along K -- moves it into Y, clipping the tails.
// Needs a 16-byte row pitch of Y (columns % 4 == 0).
template <bool kAdd>
__device__ __forceinline__ void drain_accumulator_transposed_tma(uint32_t t_addr, int width, int row0, int col0, int w_rows, int x_rows,
                                                                 const int* __restrict__ bias, const CUtensorMap* tm_y,
                                                                 uint32_t stg, int lane, int second_acc = -1)
{
    const int ycol = row0 + lane;
    const int b = (bias != nullptr && ycol < w_rows) ? __ldg(bias + ycol) : 0;
    if (row0 >= w_rows) return;
#pragma unroll 1
    for (int c = 0; c < width; c += 32) {
        if (col0 + c >= x_rows) break;
        uint32_t v[32];
        tmem_ld_32x32(t_addr + c, v);
        tmem_ld_wait();
        if (second_acc >= 0) add_second_accumulator(t_addr + second_acc + c, v);
        // The store issued for the previous block read this tile; make sure it is done.
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 32; ++i)
            sts32(stg + i * 128 + ((((lane >> 2) ^ (i & 7))) << 4) + (lane & 3) * 4,
                  static_cast<uint32_t>((static_cast<int>(v[i]) >> 8) + b));
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            if constexpr (kAdd) tma_reduce_add_2d(tm_y, stg, row0, col0 + c);
            else tma_store_2d(tm_y, stg, row0, col0 + c);
            tma_store_commit();
        }
    }
}

// The same with per-thread stores, for any row pitch of Y: for each accumulator column the warp
// writes 32 neighbouring int32 of one row of Y (one 128-byte request), or adds them atomically.
template <bool kAdd>
__device__ __forceinline__ void drain_accumulator_transposed(uint32_t t_addr, int width, int row0, int col0, int w_rows, int x_rows,
                                                             int* __restrict__ y, const int* __restrict__ bias, int lane,
                                                             int second_acc = -1)
{
    const int ycol = row0 + lane;
    const bool col_ok = ycol < w_rows;
    const int b = (bias != nullptr && col_ok) ? __ldg(bias + ycol) : 0;
#pragma unroll 1
    for (int c = 0; c < width; c += 32) {
        if (col0 + c >= x_rows) break;
        uint32_t v[32];
        tmem_ld_32x32(t_addr + c, v);
        tmem_ld_wait();
        if (second_acc >= 0) add_second_accumulator(t_addr + second_acc + c, v);
        if (!col_ok) continue;
        int* dst = y + static_cast<size_t>(col0 + c) * w_rows + ycol;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (col0 + c + i < x_rows) {
                const int val = (static_cast<int>(v[i]) >> 8) + b;
                if constexpr (kAdd) atomicAdd(dst + static_cast<size_t>(i) * w_rows, val);
                else dst[static_cast<size_t>(i) * w_rows] = val;
            }
        }
    }
}

// Dequantising variant: float(acc) * row_scale[row] * col_scale[col] + bias[col], rounded to
// bfloat16 or half (round to nearest even), written with per-thread 16-byte stores (8 values) where the
// row pitch allows.  The int32 -> float conversion is exact (|acc| <= 64 K < 2^24).
__device__ __forceinline__ void drain_accumulator_scaled(uint32_t t_addr, int width, int row0, int col0, int m, int n,
                                                         const ScaledOut& so, int lane)
{
    const int row = row0 + lane;
    const bool vec_ok = (n & 7) == 0;
    const float rs = (so.row_scale != nullptr && row < m) ? __ldg(so.row_scale + row) : 1.0f;
    unsigned short* out = static_cast<unsigned short*>(so.y16);  // bfloat16 or half bit patterns
#pragma unroll 1
    for (int c = 0; c < width; c += 32) {
        if (col0 + c >= n) break;
        uint32_t v[32];
        tmem_ld_32x32(t_addr + c, v);
        tmem_ld_wait();
        if (row >= m) continue;
        __align__(16) unsigned short h[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int col = col0 + c + i;
            const float cs = (so.col_scale != nullptr && col < n) ? __ldg(so.col_scale + col) : 1.0f;
            const float b = (so.bias != nullptr && col < n) ? __ldg(so.bias + col) : 0.0f;
            const float f = static_cast<float>(static_cast<int>(v[i]) >> 8);
            h[i] = scaled_to_bits(fmaf(f * rs, cs, b), so.fp16);
        }
        unsigned short* dst = out + static_cast<size_t>(row) * n + col0 + c;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int col = col0 + c + 8 * q;
            if (vec_ok && col + 7 < n) {
                *reinterpret_cast<uint4*>(dst + 8 * q) = *reinterpret_cast<const uint4*>(h + 8 * q);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (col + e < n) dst[8 * q + e] = h[8 * q + e];
            }
        }
    }
}

// The same dequantising epilogue through shared-memory staging and TMA stores: 64 accumulator
// columns (two tensor-memory loads) become one 32 x 128-byte bf16 tile, written in the 128B-swizzled
// layout and stored with one bulk copy that clips the M and N tails.  Needs n % 8 == 0 (16-byte
// row pitch of Y).  Column scales and biases: lane l fetches those of columns l and l + 32 of the
// NEXT chunk while the current one is converted (two coalesced loads per vector instead of a
// dependent chain of per-column loads), and the values reach the other lanes by shuffle.
template <bool kHalf>
__device__ __forceinline__ void drain_accumulator_scaled_tma(uint32_t t_addr, int width, int row0, int col0, int m, int n,
                                                             const ScaledOut& so, const CUtensorMap* tm_y16,
                                                             uint32_t stage0, uint32_t& chunk_no, int lane)
{
    const int row = row0 + lane;
    const float rs = (so.row_scale != nullptr && row < m) ? __ldg(so.row_scale + row) : 1.0f;
    const int n_live = (row0 < m && col0 < n) ? (min(width, n - col0) + 63) / 64 : 0;
    float cs_next[2] = {1.0f, 1.0f}, b_next[2] = {0.0f, 0.0f};
    auto fetch = [&](int c) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int col = min(col0 + c + 32 * hf + lane, n - 1);  // clamped: columns beyond n are clipped by the store
            cs_next[hf] = so.col_scale != nullptr ? __ldg(so.col_scale + col) : 1.0f;
            b_next[hf] = so.bias != nullptr ? __ldg(so.bias + col) : 0.0f;
        }
    };
    if (n_live > 0) fetch(0);
#pragma unroll 1
    for (int i = 0; i < n_live; ++i) {
        const int c = i * 64;
        const float cs_cur[2] = {cs_next[0], cs_next[1]}, b_cur[2] = {b_next[0], b_next[1]};
        if (i + 1 < n_live) fetch(c + 64);
        uint32_t v[2][32];
        tmem_ld_32x32(t_addr + c, v[0]);
        tmem_ld_32x32(t_addr + c + 32, v[1]);
        tmem_ld_wait();
        uint32_t h[32];  // 64 16-bit values, two per register
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int hf = j >> 4, l0 = (2 * j) & 31;
            const float s0 = __shfl_sync(0xffffffffu, cs_cur[hf], l0), s1 = __shfl_sync(0xffffffffu, cs_cur[hf], l0 + 1);
            const float o0 = __shfl_sync(0xffffffffu, b_cur[hf], l0), o1 = __shfl_sync(0xffffffffu, b_cur[hf], l0 + 1);
            const float f0 = fmaf(static_cast<float>(static_cast<int>(v[hf][l0]) >> 8) * rs, s0, o0);
            const float f1 = fmaf(static_cast<float>(static_cast<int>(v[hf][l0 + 1]) >> 8) * rs, s1, o1);
            if constexpr (kHalf) {  // the format is a compile-time choice here: this loop is the hot one
                const __half2 pr = __floats2half2_rn(f0, f1);
                h[j] = *reinterpret_cast<const uint32_t*>(&pr);
            } else {
                const __nv_bfloat162 pr = __floats2bfloat162_rn(f0, f1);
                h[j] = *reinterpret_cast<const uint32_t*>(&pr);
            }
        }
        const uint32_t stg = stage0 + (chunk_no & 1u) * 4096;
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
#pragma unroll
        for (int q = 0; q < 8; ++q)
            sts128(stg + lane * 128 + ((q ^ (lane & 7)) << 4), make_uint4(h[4 * q], h[4 * q + 1], h[4 * q + 2], h[4 * q + 3]));
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(tm_y16, stg, col0 + c, row0);
            tma_store_commit();
        }
        ++chunk_no;
    }
}

}  // namespace i4l
