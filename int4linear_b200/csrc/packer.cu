// Device-side nibble packer: the reference's host functions
//     void pack  (const int* src, int* dst, int m, int n)   utils/packer.cpp:3-18
//     void unpack(const int* src, int* dst, int m, int n)   utils/packer.cpp:20-31
// as HBM-bound kernels, so that operands produced on the GPU never have to visit the host
// to be packed.  Bit layout identical: element 8j+t of a row in bits [4t, 4t+4) of word j,
// rows padded with zero nibbles to a multiple of eight elements, unpack sign-extends.
// A second packer takes int8 sources (the natural output type of a quantiser).
//
// One thread produces one 32-bit packed word (pack) or consumes one (unpack); consecutive
// threads touch consecutive words, so every access is coalesced; 16-byte vector loads/stores
// are used whenever the row length keeps rows 16-byte aligned.
#include "common.h"

namespace i4l {

namespace {

constexpr int kPackThreads = 256;

template <typename SrcT>
__global__ void __launch_bounds__(kPackThreads)
pack_s4_kernel(const SrcT* __restrict__ src, uint32_t* __restrict__ dst, int rows, int cols, int words_per_row)
{
    const long long total = static_cast<long long>(rows) * words_per_row;
    const bool vec = (cols % 8) == 0 && (reinterpret_cast<uintptr_t>(src) % 16) == 0;
    for (long long w = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; w < total;
         w += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(w / words_per_row), j = static_cast<int>(w - static_cast<long long>(r) * words_per_row);
        const SrcT* p = src + static_cast<size_t>(r) * cols + j * 8;
        int e[8];
        if (vec) {
            if constexpr (sizeof(SrcT) == 4) {
                const int4 a = __ldg(reinterpret_cast<const int4*>(p));
                const int4 b = __ldg(reinterpret_cast<const int4*>(p) + 1);
                e[0] = a.x; e[1] = a.y; e[2] = a.z; e[3] = a.w; e[4] = b.x; e[5] = b.y; e[6] = b.z; e[7] = b.w;
            } else {
                const int2 a = __ldg(reinterpret_cast<const int2*>(p));
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    e[t] = (a.x >> (8 * t)) & 0xFF;
                    e[4 + t] = (a.y >> (8 * t)) & 0xFF;
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < 8; ++t) e[t] = (j * 8 + t < cols) ? static_cast<int>(p[t]) : 0;
        }
        uint32_t word = 0;
#pragma unroll
        for (int t = 0; t < 8; ++t) word |= (static_cast<uint32_t>(e[t]) & 0xFu) << (4 * t);
        dst[w] = word;
    }
}

__global__ void __launch_bounds__(kPackThreads)
unpack_s4_kernel(const uint32_t* __restrict__ src, int* __restrict__ dst, int rows, int cols, int words_per_row)
{
    const long long total = static_cast<long long>(rows) * words_per_row;
    const bool vec = (cols % 8) == 0 && (reinterpret_cast<uintptr_t>(dst) % 16) == 0;
    for (long long w = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; w < total;
         w += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(w / words_per_row), j = static_cast<int>(w - static_cast<long long>(r) * words_per_row);
        const uint32_t word = __ldg(src + w);
        int e[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) e[t] = static_cast<int>(word << (28 - 4 * t)) >> 28;  // sign-extending nibble extract
        int* p = dst + static_cast<size_t>(r) * cols + j * 8;
        if (vec) {
            reinterpret_cast<int4*>(p)[0] = make_int4(e[0], e[1], e[2], e[3]);
            reinterpret_cast<int4*>(p)[1] = make_int4(e[4], e[5], e[6], e[7]);
        } else {
#pragma unroll
            for (int t = 0; t < 8; ++t)
                if (j * 8 + t < cols) p[t] = e[t];
        }
    }
}

// Operand expansion (first pass of the two-pass path, and int4_linear_prepare_weights): each
// 16-byte packed chunk (32 elements) becomes 32 bytes -- the 16 even elements, then the 16 odd
// ones, every byte equal to 16 x element -- which is byte for byte what the fused GEMM's unpack
// warps write for that chunk.  HBM-bound: reads rows*K/2 bytes, writes rows*K.  One launch can
// expand two matrices (X and W); chunks [0, chunks_a) belong to the first.
__device__ __forceinline__ void expand_chunk(const uint4 x, uint4& lo, uint4& hi)
{
    lo.x = (x.x << 4) & 0xF0F0F0F0u; hi.x = x.x & 0xF0F0F0F0u;
    lo.y = (x.y << 4) & 0xF0F0F0F0u; hi.y = x.y & 0xF0F0F0F0u;
    lo.z = (x.z << 4) & 0xF0F0F0F0u; hi.z = x.z & 0xF0F0F0F0u;
    lo.w = (x.w << 4) & 0xF0F0F0F0u; hi.w = x.w & 0xF0F0F0F0u;
}

__global__ void __launch_bounds__(kPackThreads)
expand_kernel(const uint4* __restrict__ src_a, uint4* __restrict__ dst_a, long long chunks_a,
              const uint4* __restrict__ src_b, uint4* __restrict__ dst_b, long long chunks_b)
{
    constexpr int kUnroll = 4;  // independent 16-byte loads in flight per thread
    const long long total = chunks_a + chunks_b;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < total; i0 += stride * kUnroll) {
        uint4 x[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const long long i = i0 + u * stride;
            if (i < total) x[u] = i < chunks_a ? __ldg(src_a + i) : __ldg(src_b + (i - chunks_a));
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const long long i = i0 + u * stride;
            if (i < total) {
                uint4 lo, hi;
                expand_chunk(x[u], lo, hi);
                uint4* d = i < chunks_a ? dst_a + 2 * i : dst_b + 2 * (i - chunks_a);
                d[0] = lo;
                d[1] = hi;
            }
        }
    }
}

int grid_for(const DeviceCtx* ctx, long long words)
{
    long long blocks = (words + kPackThreads - 1) / kPackThreads;
    const long long cap = static_cast<long long>(ctx->sm_count) * 16;
    return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace

int launch_pack(DeviceCtx* ctx, const void* src, int src_elem_bytes, void* dst, int rows, int cols, cudaStream_t stream)
{
    const int wpr = (cols + 7) / 8;
    const long long words = static_cast<long long>(rows) * wpr;
    if (src_elem_bytes == 4)
        pack_s4_kernel<int><<<grid_for(ctx, words), kPackThreads, 0, stream>>>(static_cast<const int*>(src), static_cast<uint32_t*>(dst), rows, cols, wpr);
    else
        pack_s4_kernel<signed char><<<grid_for(ctx, words), kPackThreads, 0, stream>>>(static_cast<const signed char*>(src), static_cast<uint32_t*>(dst), rows, cols, wpr);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

int launch_expand(DeviceCtx* ctx, const void* a_packed, void* a_bytes, int rows_a,
                  const void* b_packed, void* b_bytes, int rows_b, int k, cudaStream_t stream)
{
    const long long chunks_a = static_cast<long long>(rows_a) * (k / 32);  // k % 32 == 0
    const long long chunks_b = static_cast<long long>(rows_b) * (k / 32);
    const long long per_block = static_cast<long long>(kPackThreads) * 4;
    long long blocks = (chunks_a + chunks_b + per_block - 1) / per_block;
    const long long cap = static_cast<long long>(ctx->sm_count) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    expand_kernel<<<static_cast<int>(blocks), kPackThreads, 0, stream>>>(
        static_cast<const uint4*>(a_packed), static_cast<uint4*>(a_bytes), chunks_a,
        static_cast<const uint4*>(b_packed), static_cast<uint4*>(b_bytes), chunks_b);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

int launch_expand_weights(DeviceCtx* ctx, const void* w_packed, void* w_expanded, int n, int k, cudaStream_t stream)
{
    return launch_expand(ctx, w_packed, w_expanded, n, nullptr, nullptr, 0, k, stream);
}

int launch_unpack(DeviceCtx* ctx, const void* src, void* dst, int rows, int cols, cudaStream_t stream)
{
    const int wpr = (cols + 7) / 8;
    const long long words = static_cast<long long>(rows) * wpr;
    unpack_s4_kernel<<<grid_for(ctx, words), kPackThreads, 0, stream>>>(static_cast<const uint32_t*>(src), static_cast<int*>(dst), rows, cols, wpr);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

}  // namespace i4l

// ------------------------------------------------------------------ host side
// Host packer with the reference's interface (utils/packer.h:5-6, utils/packer.cpp:3-31), so that a
// program written against the reference links against this library alone: src holds one element
// per int, a packed word holds eight nibbles, element 8w + j of a row in bits 4j .. 4j+3 of word w
// (low nibble = even index); a row is padded with zero nibbles to a whole word.  unpack
// sign-extends.  Plain loops over rows: these run outside any timed region, like the reference's.
void pack(const int* src, int* dst, const int m, const int n)
{
    const int wpr = (n + 7) / 8;
    for (int r = 0; r < m; ++r) {
        const int* s = src + static_cast<size_t>(r) * n;
        int* d = dst + static_cast<size_t>(r) * wpr;
        for (int w = 0; w < wpr; ++w) {
            uint32_t word = 0;
            const int left = n - 8 * w < 8 ? n - 8 * w : 8;
            for (int j = 0; j < left; ++j) word |= (static_cast<uint32_t>(s[8 * w + j]) & 0xFu) << (4 * j);
            d[w] = static_cast<int>(word);
        }
    }
}

void unpack(const int* src, int* dst, const int m, const int n)
{
    const int wpr = (n + 7) / 8;
    for (int r = 0; r < m; ++r) {
        const int* s = src + static_cast<size_t>(r) * wpr;
        int* d = dst + static_cast<size_t>(r) * n;
        for (int c = 0; c < n; ++c) {
            const uint32_t nib = (static_cast<uint32_t>(s[c >> 3]) >> (4 * (c & 7))) & 0xFu;
            d[c] = static_cast<int>(nib ^ 8u) - 8;  // sign extension of a 4-bit two's-complement value
        }
    }
}

extern "C" void int4_linear_pack_host(const int* src, int* dst, int m, int n) { pack(src, dst, m, n); }
extern "C" void int4_linear_unpack_host(const int* src, int* dst, int m, int n) { unpack(src, dst, m, n); }
