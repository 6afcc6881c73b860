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

template <bool kTmaStore>
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
                    if (vec_ok && col + 3 < n) {
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

// Dequantising variant: float(acc) * row_scale[row] * col_scale[col] + bias[col], rounded to
// bfloat16 (round to nearest even), written with per-thread 16-byte stores (8 values) where the
// row pitch allows.  The int32 -> float conversion is exact (|acc| <= 64 K < 2^24).
__device__ __forceinline__ void drain_accumulator_scaled(uint32_t t_addr, int width, int row0, int col0, int m, int n,
                                                         const ScaledOut& so, int lane)
{
    const int row = row0 + lane;
    const bool vec_ok = (n & 7) == 0;
    const float rs = (so.row_scale != nullptr && row < m) ? __ldg(so.row_scale + row) : 1.0f;
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(so.y16);
#pragma unroll 1
    for (int c = 0; c < width; c += 32) {
        if (col0 + c >= n) break;
        uint32_t v[32];
        tmem_ld_32x32(t_addr + c, v);
        tmem_ld_wait();
        if (row >= m) continue;
        __align__(16) __nv_bfloat16 h[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int col = col0 + c + i;
            const float cs = (so.col_scale != nullptr && col < n) ? __ldg(so.col_scale + col) : 1.0f;
            const float b = (so.bias != nullptr && col < n) ? __ldg(so.bias + col) : 0.0f;
            const float f = static_cast<float>(static_cast<int>(v[i]) >> 8);
            h[i] = __float2bfloat16_rn(fmaf(f * rs, cs, b));
        }
        __nv_bfloat16* dst = out + static_cast<size_t>(row) * n + col0 + c;
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

}  // namespace i4l
