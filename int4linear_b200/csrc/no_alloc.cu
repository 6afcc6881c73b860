// int4_linear_launch_static_scratch_async: the two-pass operator for callers that must not
// allocate device memory.
//
// Who that is: a process whose GPU memory already belongs to somebody else -- an inference
// server or a framework allocator that reserved the whole device up front, so that a cudaMalloc
// issued from inside a library either fails or eats into a budget it was never given; a
// latency-critical loop that cannot afford the device-wide synchronisation cudaMalloc and
// cudaFree imply; code running under a "no allocation after start-up" rule.  The regular
// two-pass path (int4_linear_set_two_pass(1)) grows a cudaMalloc'ed scratch buffer on demand
// and is therefore off limits to them.
//
// Here the scratch for the expanded operands is a fixed array in the library's own device data
// segment.  It costs kStaticScratchBytes on every GPU that loads the library, for the life of
// the process, and bounds the shapes this entry point accepts: (m + n) * k bytes must fit.
//
// The array's name is only a host-side handle in host code, not an address the GPU understands,
// so the first call on each device (with that device current) asks the runtime for the real
// device address with cudaGetSymbolAddress and keeps it.  That first call also opts the GEMM
// kernel into its shared-memory size and looks up the tensor-map encoder; make it before any
// stream capture starts on that device.  No call here, first or later, uses cudaMalloc,
// cudaFree, cudaHostAlloc or any other allocating routine.
//
// A bounded wait that expires inside these kernels raises a status word that also lives in the
// library's device image; int4_linear_last_status() fetches and clears it with a symbol copy (no
// allocation either), so a device-side timeout here is reported like one of the regular path.
//
// All calls on a device share the one array, and it still holds whatever the previous call
// left there.  Nothing in it needs to start at zero: the pre-pass overwrites every byte the GEMM
// then reads.  Two calls whose kernels can run at the same time on one device (different
// streams, or the same stream with launch overlap) would expand into the same bytes and race;
// keep calls of this entry point ordered on one stream per device.
#include <mutex>

#include "common.h"

namespace {

constexpr size_t kStaticScratchBytes = 64ull << 20;  // 64 MiB: (m + n) * k <= 67 108 864

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
// Word the kernels raise when one of their bounded waits expires (they need a valid address).
static __device__ int g_static_status;

constexpr int kMaxDevices = 64;
struct StaticCtx {
    bool ready = false;
    unsigned char* scratch = nullptr;  // device address of g_static_scratch on this device
    i4l::DeviceCtx ctx;                // the fields the launchers read; nothing here is allocated
};
StaticCtx g_static[kMaxDevices];
std::mutex g_static_mutex;

// Per-device set-up.  Returns nullptr and a status on failure.
StaticCtx* static_ctx(int* status)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        *status = INT4L_ERR_NO_DEVICE;
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticCtx* s = &g_static[dev];
    if (s->ready) { *status = INT4L_OK; return s; }

    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess || prop.major != 10) {
        cudaGetLastError();
        *status = INT4L_ERR_NO_DEVICE;
        return nullptr;
    }
    void* scratch = nullptr;
    void* status_word = nullptr;
    if (cudaGetSymbolAddress(&scratch, g_static_scratch) != cudaSuccess ||
        cudaGetSymbolAddress(&status_word, g_static_status) != cudaSuccess || scratch == nullptr) {
        cudaGetLastError();
        *status = INT4L_ERR_CUDA;
        return nullptr;
    }
    cudaDriverEntryPointQueryResult qres;
    void* encode = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &encode, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || encode == nullptr) {
        cudaGetLastError();
        *status = INT4L_ERR_CUDA;
        return nullptr;
    }
    s->ctx.device = dev;
    s->ctx.sm_count = prop.multiProcessorCount;
    s->ctx.max_pairs = 0;  // setup_tcgen05_s8 fills it in from an occupancy query
    s->ctx.cc_major = prop.major;
    s->ctx.cc_minor = prop.minor;
    s->ctx.status_dev = static_cast<int*>(status_word);
    s->ctx.encode_tiled = encode;
    const int rc = i4l::setup_tcgen05_s8(&s->ctx);  // cudaFuncSetAttribute only
    if (rc != INT4L_OK) { *status = rc; return nullptr; }
    s->scratch = static_cast<unsigned char*>(scratch);
    s->ready = true;
    *status = INT4L_OK;
    return s;
}

}  // namespace

namespace i4l {

// Status word of the static-scratch kernels on the current device: fetched from the device image
// and cleared when set.  INT4L_OK when this entry point has never run on the device.
int poll_static_scratch_status()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return INT4L_OK; }
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!g_static[dev].ready) return INT4L_OK;
    }
    int word = INT4L_OK;
    if (cudaMemcpyFromSymbol(&word, g_static_status, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return INT4L_ERR_CUDA; }
    if (word != INT4L_OK) {
        const int zero = INT4L_OK;
        if (cudaMemcpyToSymbol(g_static_status, &zero, sizeof(int)) != cudaSuccess) cudaGetLastError();
    }
    return word;
}

}  // namespace i4l

extern "C" int int4_linear_launch_static_scratch_async(const void* x_packed_d, const void* w_packed_d,
                                                       const int* bias_d, void* y_d, int m, int n, int k,
                                                       void* stream)
{
    if (!x_packed_d || !w_packed_d || !y_d || m <= 0 || n <= 0 || k <= 0) return INT4L_ERR_INVALID_ARG;
    if (k % 32 != 0 || k >= 131072) return INT4L_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x_packed_d) | reinterpret_cast<uintptr_t>(w_packed_d) |
         reinterpret_cast<uintptr_t>(y_d)) & 15u)
        return INT4L_ERR_MISALIGNED;
    if (bias_d != nullptr && (reinterpret_cast<uintptr_t>(bias_d) & 3u)) return INT4L_ERR_MISALIGNED;
    const unsigned long long need = (static_cast<unsigned long long>(m) + static_cast<unsigned long long>(n)) *
                                    static_cast<unsigned long long>(k);
    if (need > kStaticScratchBytes) return INT4L_ERR_TOO_LARGE;

    int rc = INT4L_OK;
    StaticCtx* s = static_ctx(&rc);
    if (s == nullptr) return rc;

    // X' (m * k bytes) then W' (n * k bytes); m * k is a multiple of 32, so W' stays 16-byte aligned.
    unsigned char* xb = s->scratch;
    unsigned char* wb = xb + static_cast<size_t>(m) * k;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    rc = i4l::launch_expand(&s->ctx, x_packed_d, xb, m, w_packed_d, wb, n, k, st);
    if (rc != INT4L_OK) return rc;
    i4l::Problem p{x_packed_d, w_packed_d, y_d, m, n, k, bias_d, false};
    return i4l::launch_tcgen05_s8(&s->ctx, p, xb, wb, st);
}
