// Yardstick kernel for the decode shapes: a read-only pass over a buffer, written the way the
// decode kernels read their weights (one 16-byte streaming load per lane and step, several in
// flight, every SM busy), with an XOR of everything read as its only output.  What this takes for
// the bytes of a weight matrix is the floor for ONE launch of any kernel that has to read those
// bytes once from HBM: launch, ramp-up and drain included, no arithmetic, no result to write.
// bench.py reports it beside the decode kernel's own time.  No reference counterpart.
#include "common.h"

namespace i4l {

namespace {

constexpr int kProbeThreads = 512;
constexpr int kProbeInFlight = 8;

__global__ void __launch_bounds__(kProbeThreads, 2)
stream_read_kernel(const uint4* __restrict__ src, size_t n16, unsigned* __restrict__ sink)
{
    const size_t stride = static_cast<size_t>(gridDim.x) * kProbeThreads;
    size_t i = static_cast<size_t>(blockIdx.x) * kProbeThreads + threadIdx.x;
    uint4 acc = make_uint4(0, 0, 0, 0);
    while (i < n16) {
        uint4 v[kProbeInFlight];
#pragma unroll
        for (int u = 0; u < kProbeInFlight; ++u) {
            const size_t j = i + u * stride;
            if (j < n16)
                asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "l"(src + j));
            else
                v[u] = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < kProbeInFlight; ++u) { acc.x ^= v[u].x; acc.y ^= v[u].y; acc.z ^= v[u].z; acc.w ^= v[u].w; }
        i += kProbeInFlight * stride;
    }
    unsigned r = acc.x ^ acc.y ^ acc.z ^ acc.w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r ^= __shfl_xor_sync(0xffffffffu, r, o);
    if ((threadIdx.x & 31) == 0 && r != 0) atomicXor(sink, r);
}

}  // namespace

int launch_stream_read(DeviceCtx* ctx, const void* src, size_t bytes, unsigned* sink, cudaStream_t stream)
{
    const size_t n16 = bytes / 16;
    if (n16 == 0) return INT4L_ERR_INVALID_ARG;
    size_t blocks = (n16 + kProbeThreads - 1) / kProbeThreads;
    const size_t cap = static_cast<size_t>(2) * ctx->sm_count;
    if (blocks > cap) blocks = cap;
    stream_read_kernel<<<static_cast<unsigned>(blocks), kProbeThreads, 0, stream>>>(static_cast<const uint4*>(src), n16, sink);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? INT4L_OK : INT4L_ERR_CUDA;
}

}  // namespace i4l
