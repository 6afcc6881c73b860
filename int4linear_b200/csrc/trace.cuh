// Optional timeline capture (compile with -DI4L_TRACE): the first worker of a kernel records a
// clock value at the hand-over points of each role for its first kTraceIters K blocks into a
// per-translation-unit device buffer, which the named export copies to the host.  Off in normal
// builds; exists to find where a pipeline stalls.  Include after defining I4L_TRACE_EXPORT to the
// name of the export function of the including file.
#pragma once

#ifdef I4L_TRACE
constexpr int kTraceIters = 192;
static __device__ long long i4l_trace_buf[2][5][kTraceIters][4];
#define I4L_TRACE_PUT(role, it, slot)                                                         \
    do {                                                                                      \
        if (worker == 0 && (it) < kTraceIters) i4l_trace_buf[cta_rank][role][it][slot] = clock64(); \
    } while (0)
extern "C" int I4L_TRACE_EXPORT(void* dst, int bytes)
{
    if (bytes > static_cast<int>(sizeof(i4l_trace_buf))) bytes = sizeof(i4l_trace_buf);
    return cudaMemcpyFromSymbol(dst, i4l_trace_buf, bytes) == cudaSuccess ? bytes : -1;
}
#else
#define I4L_TRACE_PUT(role, it, slot) do { } while (0)
#endif
