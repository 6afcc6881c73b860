// Internal declarations shared by the kernels and the C-ABI layer.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/int4linear_b200.h"

namespace i4l {

// Problem description handed to every kernel launcher.  Operand format is the
// reference's (kernels/linear_v21.h:62-69): X is M x K and W is N x K, both
// packed two signed nibbles per byte (low nibble = even index) with a row
// pitch of K/2 bytes; Y is M x N int32, row-major.
// Optional scaled 16-bit float output: Y16[i][j] = f16(float(acc[i][j]) * row_scale[i] * col_scale[j] + bias[j]),
// any of the three vectors may be null (factor 1 / addend 0).  Active when y16 is set; the int32 Y is
// then not written.
struct ScaledOut {
    const float* row_scale = nullptr;  // m per-row (per-token) factors
    const float* col_scale = nullptr;  // n per-column (per-channel) factors
    const float* bias = nullptr;       // n addends
    void* y16 = nullptr;               // m x n 16-bit floats, row-major
    int fp16 = 0;                      // 0: bfloat16, 1: IEEE half
};

#ifdef __CUDACC__
// The 16-bit pattern of a scaled output value in the chosen format (round to nearest even).
__device__ __forceinline__ unsigned short scaled_to_bits(float v, int fp16)
{
    return fp16 ? __half_as_ushort(__float2half_rn(v)) : __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
#endif

struct Problem {
    const void* x;
    const void* w;
    void* y;
    int m, n, k;
    // Optional int32 bias of length N added to every row of Y (nullptr = none).  Not part of the
    // reference operator (its README lists bias as future work); exact integer arithmetic.
    const int* bias = nullptr;
    // True when `w` is not the packed matrix but its byte expansion made by
    // int4_linear_prepare_weights (N x K bytes).
    bool w_expanded = false;
    ScaledOut scaled;
    // Launch-overlap promise of this call (int4_linear_decode_launch_async): -1 = the process-wide
    // setting of int4_linear_set_overlap, else 0, 1 or 2 with the same meaning.
    int overlap = -1;
};

// One remembered tensor map: encoding costs a driver call of a microsecond or two, and a
// serving loop presents the same few (pointer, shape, box) combinations over and over.
struct TensorMapEntry {
    const void* base = nullptr;
    uint64_t inner = 0, rows = 0, pitch = 0;
    uint32_t box_inner = 0, box_rows = 0;
    int elem_bytes = 0, swizzle = 0;
    CUtensorMap map;
};

// Per-device state created on the first call on that device.
struct DeviceCtx {
    static constexpr int kTensorMapCache = 32;
    TensorMapEntry tm_cache[kTensorMapCache];
    int tm_next = 0;  // round-robin replacement
    int device = -1;
    int sm_count = 0;
    int max_pairs = 0;  // co-resident 2-CTA clusters of the GEMM kernel
    int cc_major = 0, cc_minor = 0;
    // Host-mapped word the kernels raise when a bounded wait expires.
    volatile int* status_host = nullptr;
    int* status_dev = nullptr;
    // cuTensorMapEncodeTiled, resolved through the runtime (no libcuda link).
    void* encode_tiled = nullptr;
    // Device scratch owned by the host-buffer entry point; host_mutex serialises its users on
    // this device only.
    std::mutex host_mutex;
    void* stage_x = nullptr; size_t stage_x_bytes = 0;
    void* stage_w = nullptr; size_t stage_w_bytes = 0;
    void* stage_y = nullptr; size_t stage_y_bytes = 0;
    // Streams and events of the pipelined host-buffer path (created on first use).
    cudaStream_t host_up = nullptr, host_run = nullptr, host_down = nullptr;
    cudaEvent_t host_ev_w = nullptr, host_ev_x[8] = {}, host_ev_y[8] = {};
    cudaEvent_t host_ev_wc[4] = {}, host_ev_yc[4] = {};  // W column chunks of the first row block
    const void* stage_w_src = nullptr;  // host weights currently resident in stage_w
    size_t stage_w_src_bytes = 0;
    // Scratch of the two-pass path (expanded operands), grown on demand.
    void* scratch = nullptr; size_t scratch_bytes = 0;
    bool attrs_set = false;
};

// Returns the context of the current device (nullptr + status on failure).
DeviceCtx* current_ctx(int* status);

// Builds a 2-D tiled tensor map over a row-major byte/word matrix.
//   elem_bytes 1 -> UINT8 elements, 4 -> INT32 elements.
//   swizzle128 selects CU_TENSOR_MAP_SWIZZLE_128B (inner box must be 128 B),
//   swizzle64 CU_TENSOR_MAP_SWIZZLE_64B (inner box 64 B).
int make_tensor_map_2d(DeviceCtx* ctx, CUtensorMap* out, const void* base, int elem_bytes,
                       uint64_t inner_elems, uint64_t rows, uint64_t row_pitch_bytes,
                       uint32_t box_inner, uint32_t box_rows, bool swizzle128, bool swizzle64 = false);

// Destinations of the gathering GEMM: the full-width Y (m x n_total int32) of every rank.
struct GatherDst {
    void* const* y_full;  // `world` device pointers (this rank's own buffer and mapped peer buffers)
    int world;
    int col_offset;       // first column of this rank's block
    int n_total;
};

// Kernel launchers.  Each returns an INT4L_* status; none of them synchronises.
int launch_tcgen05(DeviceCtx* ctx, const Problem& p, cudaStream_t stream);
// GEMM on operands already expanded to bytes (second pass of the two-pass path).
int launch_tcgen05_s8(DeviceCtx* ctx, const Problem& p, const void* x_bytes, const void* w_bytes, cudaStream_t stream);
int launch_tcgen05_gather(DeviceCtx* ctx, const Problem& p, const GatherDst& g, cudaStream_t stream);
int launch_skinny(DeviceCtx* ctx, const Problem& p, cudaStream_t stream);
int launch_legacy(DeviceCtx* ctx, const Problem& p, cudaStream_t stream);

// Device-side packer (packer.cu).  src_elem_bytes: 4 = int32 per element, 1 = int8.
int launch_pack(DeviceCtx* ctx, const void* src, int src_elem_bytes, void* dst, int rows, int cols, cudaStream_t stream);
// Expands one or two packed matrices (rows x k/2 bytes) to rows x k bytes in one launch.
int launch_expand(DeviceCtx* ctx, const void* a_packed, void* a_bytes, int rows_a,
                  const void* b_packed, void* b_bytes, int rows_b, int k, cudaStream_t stream);
int launch_expand_weights(DeviceCtx* ctx, const void* w_packed, void* w_expanded, int n, int k, cudaStream_t stream);
int launch_unpack(DeviceCtx* ctx, const void* src, void* dst, int rows, int cols, cudaStream_t stream);

// Read-only streaming pass over `bytes` bytes (probe.cu): the one-launch floor of the decode shapes.
int launch_stream_read(DeviceCtx* ctx, const void* src, size_t bytes, unsigned* sink, cudaStream_t stream);

// Few rows of X (M <= 64): operands swapped, W through tensor memory (gemm_fewrows.cu).
bool fewrows_supports(const Problem& p);
int launch_fewrows(DeviceCtx* ctx, const Problem& p, cudaStream_t stream);
int setup_fewrows(DeviceCtx* ctx);
// Clears the tiles a following GEMM launch cuts along K (gemm_tcgen05.cu); transposed: tiles of Y transposed.
struct Schedule;
int launch_clear_cut_tiles(int* y, int m, int n, const Schedule& sched, int tile_m, int bn, bool transposed, cudaStream_t stream);

// One-off function attribute set-up (dynamic shared memory opt-in).
int setup_tcgen05(DeviceCtx* ctx);
int setup_tcgen05_s8(DeviceCtx* ctx);
int setup_skinny(DeviceCtx* ctx);

// Device-side status of the static-scratch entry point on the current device (no_alloc.cu).
int poll_static_scratch_status();

// Launch counter (kernels of this library launched by this process).
void count_launch(int n = 1);

// True when the decode-shape kernel can run this problem (m <= 64 and X fits
// in shared memory).
bool skinny_supports(const DeviceCtx* ctx, const Problem& p);

// Experiment knobs (int4_linear_set_tuning / INT4L_EPILOGUE, INT4L_TILE_N).
bool getenv_flag_direct_store();
int forced_tile_n();
int stream_overlap_mode();  // int4_linear_set_overlap: 0 off, 1 weights stationary, 2 weights and X
int two_pass_mode();  // -1 automatic, 0 never, 1 whenever the tensor-memory family is used
int fewrows_mode();  // int4_linear_set_fewrows: -1 by shape, 0 never, 1 whenever the kernel can run
int tail_mode();  // int4_linear_set_tail: -1 automatic, 0 whole tiles only, 1 half-width items, 2 cut along K
int forced_pairs();  // -1 automatic, 0 never use CTA pairs, 1 always (m > 128)

}  // namespace i4l
