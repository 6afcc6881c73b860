// Optional timeline capture (compile with -DI4L_TRACE): the first worker of a kernel records a
// clock value at the hand-over points of each role for its first kTraceIters K blocks into a
// per-translation-unit device buffer, which the named export copies to the host.  Off in normal
// builds; exists to find where a pipeline stalls.  Include after defining I4L_TRACE_EXPORT to the
// name of the export function of the including file.
#pragma once

#ifdef I4L_TRACE
#define I4L_TRACE_CAT2(a, b) a##b
#define I4L_TRACE_CAT(a, b) I4L_TRACE_CAT2(a, b)
constexpr int kTraceIters = 192;
static __device__ long long i4l_trace_buf[2][5][kTraceIters][4];
#define I4L_TRACE_PUT(role, it, slot)                                                         \
    do {                                                                                      \
        if (worker == 0 && (it) < kTraceIters) i4l_trace_buf[cta_rank][role][it][slot] = clock64(); \
    } while (0)
// SM clock during the kernel: (clock64, globaltimer ns) of the first worker at entry and exit.
static __device__ long long i4l_trace_clk[2][2];
#define I4L_TRACE_CLK(slot)                                                                   \
    do {                                                                                      \
        if (worker == 0 && cta_rank == 0 && threadIdx.x == 0) {                               \
            i4l_trace_clk[slot][0] = clock64();                                               \
            i4l_trace_clk[slot][1] = static_cast<long long>(global_timer_ns());               \
        }                                                                                     \
    } while (0)
extern "C" int I4L_TRACE_CAT(I4L_TRACE_EXPORT, _clk)(void* dst)
{
    return cudaMemcpyFromSymbol(dst, i4l_trace_clk, sizeof(i4l_trace_clk)) == cudaSuccess ? 0 : -1;
}
extern "C" int I4L_TRACE_EXPORT(void* dst, int bytes)
{
    if (bytes > static_cast<int>(sizeof(i4l_trace_buf))) bytes = sizeof(i4l_trace_buf);
    return cudaMemcpyFromSymbol(dst, i4l_trace_buf, bytes) == cudaSuccess ? bytes : -1;
}
#else
#define I4L_TRACE_PUT(role, it, slot) do { } while (0)
#define I4L_TRACE_CLK(slot) do { } while (0)
#endif
