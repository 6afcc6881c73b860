// C-ABI layer: argument checking, per-device set-up, shape dispatch, the
// blocking / asynchronous / host-buffer entry points, and status reporting.
// Mirrors the host launcher of the reference, kernels/linear_v21.cu:9-49.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.h"
#include "ptx.cuh"

namespace i4l {

namespace {

constexpr int kMaxDevices = 64;
DeviceCtx g_ctx[kMaxDevices];
bool g_ctx_ready[kMaxDevices];
std::mutex g_mutex;          // creation of the per-device contexts
std::mutex g_tm_mutex;       // tensor-map cache
std::mutex g_scratch_mutex;  // two-pass scratch (taken inside dispatch, which may run under g_mutex)
std::atomic<long long> g_launches{0};
std::atomic<int> g_path{-1};       // -1 = not yet read from the environment
std::atomic<int> g_tile_n{0};      // 0 = automatic
std::atomic<int> g_direct_store{-1};
std::atomic<int> g_overlap{-1};    // -1 = not yet read from the environment
std::atomic<int> g_two_pass{-2};   // -2 = not yet read from the environment
std::atomic<int> g_pairs{-2};      // -2 = not yet read from the environment
std::atomic<int> g_tail{-2};       // -2 = not yet read from the environment
std::atomic<int> g_fewrows{-2};    // few-rows kernel (M <= 64): -1 by shape, 0 never, 1 whenever it can run
thread_local int t_last_status = INT4L_OK;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int path_from_env()
{
    const char* e = std::getenv("INT4L_PATH");
    if (!e) return INT4L_PATH_AUTO;
    if (!std::strcmp(e, "tcgen05")) return INT4L_PATH_TCGEN05;
    if (!std::strcmp(e, "legacy")) return INT4L_PATH_LEGACY;
    if (!std::strcmp(e, "skinny")) return INT4L_PATH_SKINNY;
    return INT4L_PATH_AUTO;
}

int current_path()
{
    int p = g_path.load();
    if (p < 0) { p = path_from_env(); g_path.store(p); }
    return p;
}

int check_args(const void* x, const void* w, const void* y, int m, int n, int k)
{
    if (!x || !w || !y || m <= 0 || n <= 0 || k <= 0) return INT4L_ERR_INVALID_ARG;
    if (k % 32 != 0 || k >= 131072) return INT4L_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) & 15u)
        return INT4L_ERR_MISALIGNED;
    return INT4L_OK;
}

void report(int status, const char* what)
{
    t_last_status = status;
    if (status != INT4L_OK)
        std::fprintf(stderr, "CUDA FAILED: %s (%s)\n", int4_linear_status_string(status), what);
}

}  // namespace

void count_launch(int n) { g_launches.fetch_add(n); }

bool getenv_flag_direct_store()
{
    int v = g_direct_store.load();
    if (v < 0) {
        const char* e = std::getenv("INT4L_EPILOGUE");
        v = (e && !std::strcmp(e, "direct")) ? 1 : 0;
        g_direct_store.store(v);
    }
    return v != 0;
}

int forced_tile_n()
{
    int v = g_tile_n.load();
    if (v == 0) {
        static const int from_env = [] { const char* e = std::getenv("INT4L_TILE_N"); return e ? std::atoi(e) : 0; }();
        v = from_env;
    }
    return v;
}

int stream_overlap_mode()
{
    int v = g_overlap.load();
    if (v < 0) {
        const char* e = std::getenv("INT4L_OVERLAP");
        v = e ? std::atoi(e) : 0;
        if (v < 0 || v > 2) v = 0;
        g_overlap.store(v);
    }
    return v;
}

int two_pass_mode()
{
    int v = g_two_pass.load();
    if (v == -2) {
        const char* e = std::getenv("INT4L_TWO_PASS");
        v = e ? std::atoi(e) : -1;
        if (v < -1 || v > 1) v = -1;
        g_two_pass.store(v);
    }
    return v;
}

int forced_pairs()
{
    int v = g_pairs.load();
    if (v == -2) {
        const char* e = std::getenv("INT4L_PAIRS");
        v = e ? std::atoi(e) : -1;
        if (v < -1 || v > 1) v = -1;
        g_pairs.store(v);
    }
    return v;
}

int tail_mode()
{
    int v = g_tail.load();
    if (v == -2) {
        const char* e = std::getenv("INT4L_TAIL");
        v = -1;
        if (e && !std::strcmp(e, "none")) v = 0;
        else if (e && !std::strcmp(e, "half")) v = 1;
        else if (e && !std::strcmp(e, "kcut")) v = 2;
        g_tail.store(v);
    }
    return v;
}

int fewrows_mode()
{
    int v = g_fewrows.load();
    if (v == -2) {
        const char* e = std::getenv("INT4L_FEWROWS");
        v = e ? std::atoi(e) : -1;
        if (v < -1 || v > 1) v = -1;
        g_fewrows.store(v);
    }
    return v;
}

DeviceCtx* current_ctx(int* status)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        *status = INT4L_ERR_NO_DEVICE;
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceCtx* c = &g_ctx[dev];
    if (g_ctx_ready[dev]) { *status = INT4L_OK; return c; }

    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) { cudaGetLastError(); *status = INT4L_ERR_NO_DEVICE; return nullptr; }
    if (prop.major != 10) { *status = INT4L_ERR_NO_DEVICE; return nullptr; }
    c->device = dev;
    c->sm_count = prop.multiProcessorCount;
    c->cc_major = prop.major;
    c->cc_minor = prop.minor;

    void* host = nullptr;
    if (cudaHostAlloc(&host, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) { *status = INT4L_ERR_CUDA; return nullptr; }
    std::memset(host, 0, 64);
    void* devp = nullptr;
    if (cudaHostGetDevicePointer(&devp, host, 0) != cudaSuccess) { *status = INT4L_ERR_CUDA; return nullptr; }
    c->status_host = static_cast<volatile int*>(host);
    c->status_dev = static_cast<int*>(devp);

    cudaDriverEntryPointQueryResult qres;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !fn) {
        *status = INT4L_ERR_CUDA;
        return nullptr;
    }
    c->encode_tiled = fn;

    int rc = setup_tcgen05(c);
    if (rc == INT4L_OK) rc = setup_tcgen05_s8(c);
    if (rc == INT4L_OK) rc = setup_skinny(c);
    if (rc == INT4L_OK) rc = setup_fewrows(c);
    if (rc != INT4L_OK) { *status = rc; return nullptr; }
    c->attrs_set = true;
    g_ctx_ready[dev] = true;
    *status = INT4L_OK;
    return c;
}

int make_tensor_map_2d(DeviceCtx* ctx, CUtensorMap* out, const void* base, int elem_bytes,
                       uint64_t inner_elems, uint64_t rows, uint64_t row_pitch_bytes,
                       uint32_t box_inner, uint32_t box_rows, bool swizzle128, bool swizzle64)
{
    const int swizzle = swizzle128 ? 2 : (swizzle64 ? 1 : 0);
    {
        std::lock_guard<std::mutex> lock(g_tm_mutex);
        for (const TensorMapEntry& e : ctx->tm_cache) {
            if (e.base == base && e.inner == inner_elems && e.rows == rows && e.pitch == row_pitch_bytes &&
                e.box_inner == box_inner && e.box_rows == box_rows && e.elem_bytes == elem_bytes && e.swizzle == swizzle) {
                *out = e.map;
                return INT4L_OK;
            }
        }
    }
    const cuuint64_t dims[2] = {inner_elems, rows};
    const cuuint64_t strides[1] = {row_pitch_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
        out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_INT32 : (elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8), 2,
        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : (swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return INT4L_ERR_CUDA;
    // A tensor map describes addresses and shapes only, never contents, so a remembered one stays
    // valid for as long as the same pointer denotes an allocation of at least that extent.
    std::lock_guard<std::mutex> lock(g_tm_mutex);
    TensorMapEntry& e = ctx->tm_cache[ctx->tm_next];
    ctx->tm_next = (ctx->tm_next + 1) % DeviceCtx::kTensorMapCache;
    e.base = base; e.inner = inner_elems; e.rows = rows; e.pitch = row_pitch_bytes;
    e.box_inner = box_inner; e.box_rows = box_rows; e.elem_bytes = elem_bytes; e.swizzle = swizzle;
    e.map = *out;
    return INT4L_OK;
}

bool skinny_supports(const DeviceCtx* ctx, const Problem& p);

namespace {

int choose_path(const DeviceCtx* ctx, const Problem& p)
{
    const int forced = current_path();
    if (forced == INT4L_PATH_SKINNY) return skinny_supports(ctx, p) ? INT4L_PATH_SKINNY : INT4L_PATH_TCGEN05;
    if (forced != INT4L_PATH_AUTO) return forced;
    // Measured (CUDA-graph replays, weights from HBM): up to 16 rows the register kernels win; from
    // 17 to 32 rows they still do while the weights are small (4096 x 4096: 8.3 us against 9.6), and
    // the few-rows tensor-memory kernel wins from 32 M weight elements on (14336 x 4096: 13.0 us
    // against 18.5); from 33 rows on the tensor-memory family always.
    const bool fewrows_ok = fewrows_mode() != 0 && fewrows_supports(p);
    if (fewrows_mode() == 1 && fewrows_ok) return INT4L_PATH_TCGEN05;
    // Beyond K = 8192 the register kernel for up to 16 rows does not apply, and its fallback loses to
    // the few-rows kernel on large weights (16 x 4096 x 14336: 16.9 us against 13.4).
    const bool large = static_cast<long long>(p.n) * p.k >= (1ll << 25);
    const int skinny_rows = (fewrows_ok && large) ? (p.k > 8192 ? 0 : 16) : 32;
    if (p.m <= skinny_rows && skinny_supports(ctx, p)) return INT4L_PATH_SKINNY;
    return INT4L_PATH_TCGEN05;
}

int ensure_stage(void** buf, size_t* have, size_t need)
{
    if (*have >= need) return INT4L_OK;
    if (*buf) cudaFree(*buf);
    *buf = nullptr;
    *have = 0;
    if (cudaMalloc(buf, need) != cudaSuccess) { cudaGetLastError(); return INT4L_ERR_CUDA; }
    *have = need;
    return INT4L_OK;
}

// Two-pass path: expand both operands into `scratch` ((m + n) * k bytes), then the byte GEMM.
int run_two_pass(DeviceCtx* ctx, const Problem& p, void* scratch, cudaStream_t stream)
{
    uint8_t* xb = static_cast<uint8_t*>(scratch);
    uint8_t* wb = xb + static_cast<size_t>(p.m) * p.k;
    int rc = launch_expand(ctx, p.x, xb, p.m, p.w, wb, p.n, p.k, stream);
    if (rc != INT4L_OK) return rc;
    return launch_tcgen05_s8(ctx, p, xb, wb, stream);
}

// The two-pass path is opt-in only: measured on B200 it equals the fused kernel from 8192 x 8192
// outputs upwards (K = 8192) and is slower below, for 2.5x the operand traffic and a scratch buffer.
bool two_pass_wanted() { return two_pass_mode() == 1; }

int dispatch(DeviceCtx* ctx, const Problem& p, cudaStream_t stream)
{
    switch (choose_path(ctx, p)) {
        case INT4L_PATH_SKINNY: return launch_skinny(ctx, p, stream);
        case INT4L_PATH_LEGACY: return launch_legacy(ctx, p, stream);
        default: break;
    }
    if (two_pass_wanted() && forced_pairs() < 0 && forced_tile_n() == 0) {
        const size_t need = (static_cast<size_t>(p.m) + p.n) * p.k;
        bool have;
        {
            std::lock_guard<std::mutex> lock(g_scratch_mutex);
            have = ensure_stage(&ctx->scratch, &ctx->scratch_bytes, need) == INT4L_OK;
        }
        if (have) return run_two_pass(ctx, p, ctx->scratch, stream);
    }
    return launch_tcgen05(ctx, p, stream);
}

int poll_device_status(DeviceCtx* ctx)
{
    if (!ctx || !ctx->status_host) return INT4L_OK;
    int s = *ctx->status_host;
    if (s != INT4L_OK) *ctx->status_host = INT4L_OK;
    return s;
}

// Large host-buffer problems are cut into up to eight row blocks of X / Y and run as a
// three-stream pipeline -- upload of block i+1, GEMM of block i and download of block i-1 overlap --
// because the download of Y (4 bytes per output) is by far the longest leg and PCIe is full duplex.
int host_pipelined(DeviceCtx* ctx, const void* x_h, const void* w_h, void* y_h, int m, int n, int k, bool reuse_w)
{
    if (ctx->host_up == nullptr) {
        bool ok = cudaStreamCreateWithFlags(&ctx->host_up, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaStreamCreateWithFlags(&ctx->host_run, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaStreamCreateWithFlags(&ctx->host_down, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaEventCreateWithFlags(&ctx->host_ev_w, cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; ok && i < 8; ++i)
            ok = cudaEventCreateWithFlags(&ctx->host_ev_x[i], cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&ctx->host_ev_y[i], cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; ok && i < 4; ++i)
            ok = cudaEventCreateWithFlags(&ctx->host_ev_wc[i], cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&ctx->host_ev_yc[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) { cudaGetLastError(); ctx->host_up = nullptr; return INT4L_ERR_CUDA; }
    }
    const size_t row_x = static_cast<size_t>(k) / 2, row_y = static_cast<size_t>(n) * 4;
    const int block = ((m + 7) / 8 + 255) / 256 * 256;  // rows per block, a multiple of the tile height
    const uint8_t* xh = static_cast<const uint8_t*>(x_h);
    uint8_t* yh = static_cast<uint8_t*>(y_h);
    uint8_t* xd = static_cast<uint8_t*>(ctx->stage_x);
    uint8_t* yd = static_cast<uint8_t*>(ctx->stage_y);
    bool ok = true;
    int rc = INT4L_OK;
    // The download of Y is the longest leg (4 bytes per output against half a byte per operand
    // element), so it should start as early as possible.  When W has to be uploaded too, it goes up
    // in four column chunks behind the first row block of X, and that row block is computed chunk
    // by chunk as they land: the first download starts after 1/8 of X and 1/4 of W instead of after
    // all of W.  The chunk results are compact slabs in the staging area of that row block and go
    // to their place in y_h with a strided copy.
    int first = 0;  // row blocks already done by the chunked start
    const int chunk_n = ((n + 3) / 4 + 255) / 256 * 256;
    if (!reuse_w && n >= 4 * 256) {
        const uint8_t* wh = static_cast<const uint8_t*>(w_h);
        uint8_t* wd = static_cast<uint8_t*>(ctx->stage_w);
        const int rows = m < block ? m : block;
        ok = cudaMemcpyAsync(xd, xh, rows * row_x, cudaMemcpyHostToDevice, ctx->host_up) == cudaSuccess;
        size_t slab = 0;
        for (int j = 0, c0 = 0; ok && c0 < n; ++j, c0 += chunk_n) {
            const int cw = n - c0 < chunk_n ? n - c0 : chunk_n;
            ok = cudaMemcpyAsync(wd + c0 * row_x, wh + c0 * row_x, cw * row_x, cudaMemcpyHostToDevice, ctx->host_up) == cudaSuccess &&
                 cudaEventRecord(ctx->host_ev_wc[j], ctx->host_up) == cudaSuccess &&
                 cudaStreamWaitEvent(ctx->host_run, ctx->host_ev_wc[j], 0) == cudaSuccess;
            if (!ok) break;
            Problem p{xd, wd + c0 * row_x, yd + slab, rows, cw, k};
            rc = dispatch(ctx, p, ctx->host_run);
            if (rc != INT4L_OK) break;
            ok = cudaEventRecord(ctx->host_ev_yc[j], ctx->host_run) == cudaSuccess &&
                 cudaStreamWaitEvent(ctx->host_down, ctx->host_ev_yc[j], 0) == cudaSuccess &&
                 cudaMemcpy2DAsync(yh + static_cast<size_t>(c0) * 4, row_y, yd + slab, static_cast<size_t>(cw) * 4,
                                   static_cast<size_t>(cw) * 4, rows, cudaMemcpyDeviceToHost, ctx->host_down) == cudaSuccess;
            slab += static_cast<size_t>(rows) * cw * 4;
        }
        first = 1;
    } else if (!reuse_w) {
        ok = cudaMemcpyAsync(ctx->stage_w, w_h, static_cast<size_t>(n) * row_x, cudaMemcpyHostToDevice, ctx->host_up) == cudaSuccess &&
             cudaEventRecord(ctx->host_ev_w, ctx->host_up) == cudaSuccess &&
             cudaStreamWaitEvent(ctx->host_run, ctx->host_ev_w, 0) == cudaSuccess;
    }
    for (int i = first, r0 = first * block; ok && rc == INT4L_OK && r0 < m; ++i, r0 += block) {
        const int rows = m - r0 < block ? m - r0 : block;
        ok = cudaMemcpyAsync(xd + r0 * row_x, xh + r0 * row_x, rows * row_x, cudaMemcpyHostToDevice, ctx->host_up) == cudaSuccess &&
             cudaEventRecord(ctx->host_ev_x[i], ctx->host_up) == cudaSuccess &&
             cudaStreamWaitEvent(ctx->host_run, ctx->host_ev_x[i], 0) == cudaSuccess;
        if (!ok) break;
        Problem p{xd + r0 * row_x, ctx->stage_w, yd + r0 * row_y, rows, n, k};
        rc = dispatch(ctx, p, ctx->host_run);
        if (rc != INT4L_OK) break;
        ok = cudaEventRecord(ctx->host_ev_y[i], ctx->host_run) == cudaSuccess &&
             cudaStreamWaitEvent(ctx->host_down, ctx->host_ev_y[i], 0) == cudaSuccess &&
             cudaMemcpyAsync(yh + r0 * row_y, yd + r0 * row_y, rows * row_y, cudaMemcpyDeviceToHost, ctx->host_down) == cudaSuccess;
    }
    // Drain all three streams whatever happened, so that no copy is left in flight on return.
    const bool drained = cudaStreamSynchronize(ctx->host_up) == cudaSuccess &&
                         cudaStreamSynchronize(ctx->host_run) == cudaSuccess &&
                         cudaStreamSynchronize(ctx->host_down) == cudaSuccess;
    if (rc != INT4L_OK) return rc;
    if (!ok || !drained) { cudaGetLastError(); return INT4L_ERR_CUDA; }
    return INT4L_OK;
}

}  // namespace

// Self-test of the failure path: one warp waits, with the given budget, on an mbarrier that
// nothing ever arrives at -- the situation a wrong descriptor or a lost arrival would create in a
// GEMM kernel -- and must come back by itself and raise the status word like the real kernels do.
__global__ void selftest_timeout_kernel(int* status, unsigned long long budget_ns)
{
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        mbar_init_fence();
    }
    __syncthreads();
    const bool arrived = mbar_wait(smem_u32(&bar), 0, &abort_flag, budget_ns);
    __syncthreads();
    if (threadIdx.x == 0 && !arrived && abort_flag) atomicExch(status, INT4L_ERR_DEVICE_TIMEOUT);
}

}  // namespace i4l

using namespace i4l;

extern "C" {

int int4_linear_launch_async(const void* x, const void* w, void* y, int m, int n, int k, void* stream)
{
    int rc = check_args(x, w, y, m, n, k);
    if (rc != INT4L_OK) { t_last_status = rc; return rc; }
    DeviceCtx* ctx = current_ctx(&rc);
    if (!ctx) { t_last_status = rc; return rc; }
    Problem p{x, w, y, m, n, k};
    rc = dispatch(ctx, p, static_cast<cudaStream_t>(stream));
    t_last_status = rc;
    return rc;
}

int int4_linear_bias_launch_async(const void* x, const void* w, const int* bias_d, void* y, int m, int n, int k, void* stream)
{
    int rc = check_args(x, w, y, m, n, k);
    if (rc == INT4L_OK && bias_d != nullptr && (reinterpret_cast<uintptr_t>(bias_d) & 3u)) rc = INT4L_ERR_MISALIGNED;
    if (rc != INT4L_OK) { t_last_status = rc; return rc; }
    DeviceCtx* ctx = current_ctx(&rc);
    if (!ctx) { t_last_status = rc; return rc; }
    Problem p{x, w, y, m, n, k, bias_d};
    rc = dispatch(ctx, p, static_cast<cudaStream_t>(stream));
    t_last_status = rc;
    return rc;
}

int int4_linear_decode_launch_async(const void* x, const void* w, const int* bias_d, void* y, int m, int n, int k,
                                    int promises, void* stream)
{
    int rc = check_args(x, w, y, m, n, k);
    if (rc == INT4L_OK && bias_d != nullptr && (reinterpret_cast<uintptr_t>(bias_d) & 3u)) rc = INT4L_ERR_MISALIGNED;
    if (rc == INT4L_OK && (promises < 0 || promises > 3 || promises == INT4L_PROMISE_X_NOT_PENDING)) rc = INT4L_ERR_INVALID_ARG;
    if (rc != INT4L_OK) { t_last_status = rc; return rc; }
    DeviceCtx* ctx = current_ctx(&rc);
    if (!ctx) { t_last_status = rc; return rc; }
    Problem p{x, w, y, m, n, k, bias_d};
    p.overlap = promises == 0 ? 0 : (promises == INT4L_PROMISE_WEIGHTS_STATIONARY ? 1 : 2);
    rc = dispatch(ctx, p, static_cast<cudaStream_t>(stream));
    t_last_status = rc;
    return rc;
}

int int4_linear_prepare_weights(const void* w_packed_d, void* w_expanded_d, int n, int k, void* stream)
{
    int rc = check_args(w_packed_d, w_packed_d, w_expanded_d, 1, n, k);
    if (rc != INT4L_OK) { t_last_status = rc; return rc; }
    DeviceCtx* ctx = current_ctx(&rc);
    if (ctx) rc = launch_expand_weights(ctx, w_packed_d, w_expanded_d, n, k, static_cast<cudaStream_t>(stream));
    t_last_status = rc;
    return rc;
}

int int4_linear_launch_prepared_async(const void* x, const void* w_expanded_d, const int* bias_d, void* y,
                                      int m, int n, int k, void* stream)
{
    int rc = check_args(x, w_expanded_d, y, m, n, k);
    if (rc == INT4L_OK && bias_d != nullptr && (reinterpret_cast<uintptr_t>(bias_d) & 3u)) rc = INT4L_ERR_MISALIGNED;
    if (rc != INT4L_OK) { t_last_status = rc; return rc; }
    DeviceCtx* ctx = current_ctx(&rc);
    if (!ctx) { t_last_status = rc; return rc; }
    Problem p{x, w_expanded_d, y, m, n, k, bias_d, true};
    rc = launch_tcgen05(ctx, p, static_cast<cudaStream_t>(stream));
    t_last_status = rc;
    return rc;
}

int int4_linear_launch_expanded_async(const void* x_expanded_d, const void* w_expanded_d, const int* bias_d, void* y,
                                      int m, int n, int k, void* stream)
{
    int rc = check_args(x_expanded_d, w_expanded_d, y, m, n, k);
    if (rc == INT4L_OK && bias_d != nullptr && (reinterpret_cast<uintptr_t>(bias_d) & 3u)) rc = INT4L_ERR_MISALIGNED;
    if (rc != INT4L_OK) { t_last_status = rc; return rc; }
    DeviceCtx* ctx = current_ctx(&rc);
    if (!ctx) { t_last_status = rc; return rc; }
    Problem p{nullptr, nullptr, y, m, n, k, bias_d};
    rc = launch_tcgen05_s8(ctx, p, x_expanded_d, w_expanded_d, static_cast<cudaStream_t>(stream));
    t_last_status = rc;
    return rc;
}

static int scaled_launch(const void* x, const void* w, const float* row_scale_d, const float* col_scale_d,
                         const float* bias_d, void* y16_d, int fp16, int m, int n, int k, void* stream)
{
    int rc = check_args(x, w, y16_d, m, n, k);
    if (rc != INT4L_OK) { t_last_status = rc; return rc; }
    DeviceCtx* ctx = current_ctx(&rc);
    if (!ctx) { t_last_status = rc; return rc; }
    Problem p{x, w, y16_d, m, n, k};
    p.scaled.row_scale = row_scale_d;
    p.scaled.col_scale = col_scale_d;
    p.scaled.bias = bias_d;
    p.scaled.y16 = y16_d;
    p.scaled.fp16 = fp16;
    // Decode shapes keep their streaming kernels; the legacy path has no scaled epilogue.
    rc = choose_path(ctx, p) == INT4L_PATH_SKINNY ? launch_skinny(ctx, p, static_cast<cudaStream_t>(stream))
                                                  : launch_tcgen05(ctx, p, static_cast<cudaStream_t>(stream));
    t_last_status = rc;
    return rc;
}

int int4_linear_scaled_launch_async(const void* x, const void* w, const float* row_scale_d, const float* col_scale_d,
                                    const float* bias_d, void* y_bf16_d, int m, int n, int k, void* stream)
{
    return scaled_launch(x, w, row_scale_d, col_scale_d, bias_d, y_bf16_d, 0, m, n, k, stream);
}

int int4_linear_scaled_f16_launch_async(const void* x, const void* w, const float* row_scale_d, const float* col_scale_d,
                                        const float* bias_d, void* y_f16_d, int m, int n, int k, void* stream)
{
    return scaled_launch(x, w, row_scale_d, col_scale_d, bias_d, y_f16_d, 1, m, n, k, stream);
}

int int4_linear_launch_gather_async(const void* x, const void* w_shard, const int* bias_d, void* const* y_full_ptrs,
                                    int world, int col_offset, int m, int n_local, int n_total, int k, void* stream)
{
    if (!y_full_ptrs || world < 1 || world > 8 || n_total <= 0 || col_offset < 0) { t_last_status = INT4L_ERR_INVALID_ARG; return INT4L_ERR_INVALID_ARG; }
    for (int d = 0; d < world; ++d)
        if (!y_full_ptrs[d] || (reinterpret_cast<uintptr_t>(y_full_ptrs[d]) & 15u)) { t_last_status = INT4L_ERR_INVALID_ARG; return INT4L_ERR_INVALID_ARG; }
    int rc = check_args(x, w_shard, y_full_ptrs[0], m, n_local, k);
    if (rc != INT4L_OK) { t_last_status = rc; return rc; }
    DeviceCtx* ctx = current_ctx(&rc);
    if (!ctx) { t_last_status = rc; return rc; }
    Problem p{x, w_shard, nullptr, m, n_local, k, bias_d};
    GatherDst g{y_full_ptrs, world, col_offset, n_total};
    rc = launch_tcgen05_gather(ctx, p, g, static_cast<cudaStream_t>(stream));
    t_last_status = rc;
    return rc;
}

void int4_linear_launch(void* x, void* w, void* y, int m, int n, int k)
{
    int rc = int4_linear_launch_async(x, w, y, m, n, k, nullptr);
    if (rc != INT4L_OK) { report(rc, "launch"); return; }
    if (cudaDeviceSynchronize() != cudaSuccess) { cudaGetLastError(); report(INT4L_ERR_CUDA, "synchronize"); return; }
    int st = INT4L_OK;
    DeviceCtx* ctx = current_ctx(&st);
    st = poll_device_status(ctx);
    report(st, "kernel");
}

int int4_linear_host(const void* x_h, const void* w_h, void* y_h, int m, int n, int k, int w_resident)
{
    int rc = check_args(x_h, w_h, y_h, m, n, k);
    if (rc == INT4L_ERR_MISALIGNED) rc = INT4L_OK;  // host buffers need no alignment
    if (rc != INT4L_OK) { t_last_status = rc; return rc; }
    DeviceCtx* ctx = current_ctx(&rc);
    if (!ctx) { t_last_status = rc; return rc; }
    const size_t xb = static_cast<size_t>(m) * k / 2, wb = static_cast<size_t>(n) * k / 2;
    const size_t yb = static_cast<size_t>(m) * n * 4;
    {
        // One host-buffer call at a time per DEVICE (the staging buffers and the three pipeline
        // streams belong to the device's context); calls on different devices run concurrently.
        std::lock_guard<std::mutex> lock(ctx->host_mutex);
        const bool w_buf_grew = ctx->stage_w_bytes < wb;
        rc = ensure_stage(&ctx->stage_x, &ctx->stage_x_bytes, xb);
        if (rc == INT4L_OK) rc = ensure_stage(&ctx->stage_w, &ctx->stage_w_bytes, wb);
        if (rc == INT4L_OK) rc = ensure_stage(&ctx->stage_y, &ctx->stage_y_bytes, yb);
        if (rc != INT4L_OK) { t_last_status = rc; return rc; }
        const bool reuse = w_resident && !w_buf_grew && ctx->stage_w_src == w_h && ctx->stage_w_src_bytes == wb;
        if (m >= 1024 && yb >= (16u << 20)) {
            rc = host_pipelined(ctx, x_h, w_h, y_h, m, n, k, reuse);
            // The weights count as resident only when their upload went through.
            if (rc != INT4L_OK) { ctx->stage_w_src = nullptr; ctx->stage_w_src_bytes = 0; t_last_status = rc; return rc; }
            if (!reuse) { ctx->stage_w_src = w_h; ctx->stage_w_src_bytes = wb; }
        } else {
            cudaError_t e = cudaMemcpyAsync(ctx->stage_x, x_h, xb, cudaMemcpyHostToDevice, nullptr);
            if (e == cudaSuccess && !reuse) {
                e = cudaMemcpyAsync(ctx->stage_w, w_h, wb, cudaMemcpyHostToDevice, nullptr);
                ctx->stage_w_src = e == cudaSuccess ? w_h : nullptr;
                ctx->stage_w_src_bytes = e == cudaSuccess ? wb : 0;
            }
            if (e != cudaSuccess) { cudaGetLastError(); t_last_status = INT4L_ERR_CUDA; return INT4L_ERR_CUDA; }
            Problem p{ctx->stage_x, ctx->stage_w, ctx->stage_y, m, n, k};
            rc = dispatch(ctx, p, nullptr);
            if (rc != INT4L_OK) { t_last_status = rc; return rc; }
            e = cudaMemcpyAsync(y_h, ctx->stage_y, yb, cudaMemcpyDeviceToHost, nullptr);
            if (e == cudaSuccess) e = cudaStreamSynchronize(nullptr);
            if (e != cudaSuccess) { cudaGetLastError(); t_last_status = INT4L_ERR_CUDA; return INT4L_ERR_CUDA; }
        }
    }
    rc = poll_device_status(ctx);
    t_last_status = rc;
    return rc;
}

int int4_linear_pack_i32(const int* src_d, void* dst_d, int rows, int cols, void* stream)
{
    if (!src_d || !dst_d || rows <= 0 || cols <= 0) { t_last_status = INT4L_ERR_INVALID_ARG; return INT4L_ERR_INVALID_ARG; }
    int rc = INT4L_OK;
    DeviceCtx* ctx = current_ctx(&rc);
    if (ctx) rc = launch_pack(ctx, src_d, 4, dst_d, rows, cols, static_cast<cudaStream_t>(stream));
    t_last_status = rc;
    return rc;
}

int int4_linear_pack_i8(const signed char* src_d, void* dst_d, int rows, int cols, void* stream)
{
    if (!src_d || !dst_d || rows <= 0 || cols <= 0) { t_last_status = INT4L_ERR_INVALID_ARG; return INT4L_ERR_INVALID_ARG; }
    int rc = INT4L_OK;
    DeviceCtx* ctx = current_ctx(&rc);
    if (ctx) rc = launch_pack(ctx, src_d, 1, dst_d, rows, cols, static_cast<cudaStream_t>(stream));
    t_last_status = rc;
    return rc;
}

int int4_linear_unpack_i32(const void* src_d, int* dst_d, int rows, int cols, void* stream)
{
    if (!src_d || !dst_d || rows <= 0 || cols <= 0) { t_last_status = INT4L_ERR_INVALID_ARG; return INT4L_ERR_INVALID_ARG; }
    int rc = INT4L_OK;
    DeviceCtx* ctx = current_ctx(&rc);
    if (ctx) rc = launch_unpack(ctx, src_d, dst_d, rows, cols, static_cast<cudaStream_t>(stream));
    t_last_status = rc;
    return rc;
}

int int4_linear_probe_stream_read(const void* src_d, unsigned long long bytes, unsigned* sink_d, void* stream)
{
    if (!src_d || !sink_d || bytes < 16 || (reinterpret_cast<uintptr_t>(src_d) & 15u)) return INT4L_ERR_INVALID_ARG;
    int rc = INT4L_OK;
    DeviceCtx* ctx = current_ctx(&rc);
    if (!ctx) return rc;
    return launch_stream_read(ctx, src_d, static_cast<size_t>(bytes), sink_d, static_cast<cudaStream_t>(stream));
}

int int4_linear_selftest_timeout(int budget_ms)
{
    if (budget_ms < 1 || budget_ms > 100) return INT4L_ERR_INVALID_ARG;
    int rc = INT4L_OK;
    DeviceCtx* ctx = current_ctx(&rc);
    if (!ctx) return rc;
    selftest_timeout_kernel<<<1, 32>>>(ctx->status_dev, static_cast<unsigned long long>(budget_ms) * 1000000ull);
    count_launch();
    if (cudaGetLastError() != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) { cudaGetLastError(); return INT4L_ERR_CUDA; }
    return INT4L_OK;
}

int int4_linear_last_status(void)
{
    int st = INT4L_OK;
    int dev = -1;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices && g_ctx_ready[dev])
        st = poll_device_status(&g_ctx[dev]);
    else
        cudaGetLastError();
    if (st == INT4L_OK) st = poll_static_scratch_status();
    if (st != INT4L_OK) t_last_status = st;
    return t_last_status;
}

const char* int4_linear_status_string(int status)
{
    switch (status) {
        case INT4L_OK: return "ok";
        case INT4L_ERR_INVALID_ARG: return "invalid argument";
        case INT4L_ERR_UNSUPPORTED: return "unsupported shape (need k % 32 == 0 and k < 131072)";
        case INT4L_ERR_MISALIGNED: return "pointer not 16-byte aligned";
        case INT4L_ERR_CUDA: return "CUDA call failed";
        case INT4L_ERR_DEVICE_TIMEOUT: return "in-kernel wait timed out";
        case INT4L_ERR_NO_DEVICE: return "no sm_100 device";
        case INT4L_ERR_TOO_LARGE: return "size beyond the fixed capacity of this entry point";
        default: return "unknown status";
    }
}

int int4_linear_set_path(int path)
{
    int prev = current_path();
    if (path >= INT4L_PATH_AUTO && path <= INT4L_PATH_SKINNY) g_path.store(path);
    return prev;
}

int int4_linear_set_two_pass(int mode)
{
    if (mode < -1 || mode > 1) return INT4L_ERR_INVALID_ARG;
    g_two_pass.store(mode);
    return INT4L_OK;
}

int int4_linear_set_tuning(int tile_n, int direct_store, int cta_pairs)
{
    if (tile_n != 0 && tile_n != 64 && tile_n != 128 && tile_n != 256) return INT4L_ERR_INVALID_ARG;
    if (cta_pairs < -1 || cta_pairs > 1) return INT4L_ERR_INVALID_ARG;
    g_tile_n.store(tile_n);
    g_direct_store.store(direct_store ? 1 : 0);
    g_pairs.store(cta_pairs);
    return INT4L_OK;
}

int int4_linear_set_fewrows(int mode)
{
    if (mode < -1 || mode > 1) return INT4L_ERR_INVALID_ARG;
    g_fewrows.store(mode);
    return INT4L_OK;
}

int int4_linear_set_tail(int mode)
{
    if (mode < -1 || mode > 2) return INT4L_ERR_INVALID_ARG;
    g_tail.store(mode);
    return INT4L_OK;
}

int int4_linear_set_overlap(int mode)
{
    if (mode < 0 || mode > 2) return -INT4L_ERR_INVALID_ARG;
    const int prev = stream_overlap_mode();
    g_overlap.store(mode);
    return prev;
}

int int4_linear_path_for(int m, int n, int k)
{
    int rc = INT4L_OK;
    DeviceCtx* ctx = current_ctx(&rc);
    if (!ctx) return -rc;
    Problem p{nullptr, nullptr, nullptr, m, n, k};
    return choose_path(ctx, p);
}

int int4_linear_device_info(int what)
{
    int rc = INT4L_OK;
    DeviceCtx* ctx = current_ctx(&rc);
    if (!ctx) return -rc;
    if (what == 0) return ctx->sm_count;
    if (what == 1) return ctx->max_pairs;
    return -INT4L_ERR_INVALID_ARG;
}

long long int4_linear_launch_count(void) { return g_launches.load(); }

int int4_linear_version(void) { return 100; }

}  // extern "C"

// The reference declares its launcher with C++ linkage (kernels/linear_v21.h:760);
// exporting the same symbol lets test/test_correctness.cu link against this
// library unchanged.
void linear_v21_launch(void* x_packed_d, void* w_packed_d, void* y_d, int m, int n, int k)
{
    int4_linear_launch(x_packed_d, w_packed_d, y_d, m, n, k);
}
