/*
 * int4linear_b200 -- C ABI of the Blackwell (sm_100a) INT4 linear layer
 *
 *     Y[M x N] (int32) = X[M x K] (s4) * W[N x K]^T (s4)
 *
 * Operand format (identical to myeongs-song/Int4Linear):
 *   X  M rows of K signed 4-bit values, two per byte, low nibble = even index,
 *      i.e. eight per little-endian 32-bit word exactly as utils/packer.cpp:3-18
 *      writes them; row pitch K/2 bytes.
 *   W  N rows of K values in the same packing ("column-major K x N").
 *   Y  M x N int32, row-major, fully overwritten.
 *
 * Shape contract: m, n, k > 0; k % 32 == 0 (16-byte row pitch); k < 131072
 * (the kernels multiply 16*x by 16*w in int32 and shift the sum back).
 * X, W and Y must be 16-byte aligned.  Any m and n are accepted.
 *
 * The first call on a device sets that device up (a host-mapped status word, kernel
 * attributes, one driver entry point); issue it before any CUDA-graph capture.
 * All functions are thread-safe per device.  Nothing here falls back to a
 * CPU implementation: without an sm_100 GPU every compute entry point fails
 * with INT4L_ERR_NO_DEVICE.
 */
#ifndef INT4LINEAR_B200_H_
#define INT4LINEAR_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes returned by the int-returning entry points and by
 * int4_linear_last_status(). */
#define INT4L_OK                  0
#define INT4L_ERR_INVALID_ARG     1  /* null pointer or non-positive dimension   */
#define INT4L_ERR_UNSUPPORTED     2  /* k % 32 != 0 or k >= 131072               */
#define INT4L_ERR_MISALIGNED      3  /* a pointer is not 16-byte aligned         */
#define INT4L_ERR_CUDA            4  /* a CUDA runtime/driver call failed        */
#define INT4L_ERR_DEVICE_TIMEOUT  5  /* a bounded in-kernel wait expired         */
#define INT4L_ERR_NO_DEVICE       6  /* current device is not sm_100             */
#define INT4L_ERR_TOO_LARGE       7  /* size beyond a fixed-capacity entry point */

/* Kernel families selectable with int4_linear_set_path(). */
#define INT4L_PATH_AUTO     0  /* shape dispatch (default)                                   */
#define INT4L_PATH_TCGEN05  1  /* TMA -> s4->s8 unpack -> tcgen05.mma kind::i8 -> TMEM        */
#define INT4L_PATH_LEGACY   2  /* warp-level mma.sync m16n8k64 s4 (pre-Blackwell instruction) */
#define INT4L_PATH_SKINNY   3  /* register-streaming kernels, m <= 64 (chosen for m <= 32)    */

/*
 * Drop-in for `void linear_v21_launch(void*, void*, void*, int, int, int)`
 * (kernels/linear_v21.h:760, body kernels/linear_v21.cu:9-49): device
 * pointers, current device, default stream, returns after the result is
 * complete (the reference ends with cudaDeviceSynchronize, linear_v21.cu:39).
 * Like the reference it returns nothing; on failure it prints one
 * "CUDA FAILED: ..." line to stderr (the reference's wording,
 * kernels/linear_v10.cu:33-38) and records the code for
 * int4_linear_last_status().  The library also exports the C++ symbol
 * linear_v21_launch with the same behaviour so the reference's
 * test/test_correctness.cu links unchanged.
 */
void int4_linear_launch(void* x_packed_d, void* w_packed_d, void* y_d, int m, int n, int k);

/*
 * Same operator, asynchronous on `stream` (a cudaStream_t; NULL = default
 * stream) and returning a status code.  No reference counterpart: the
 * reference launcher is blocking; this is what a multi-GPU driver or a graph
 * capture needs.  A device-side timeout is only visible later through
 * int4_linear_last_status().
 */
int int4_linear_launch_async(const void* x_packed_d, const void* w_packed_d, void* y_d,
                             int m, int n, int k, void* stream);

/*
 * The operator with a fused bias: Y[i][j] = sum_l X[i][l] * W[j][l] + bias[j], all int32 and
 * exact.  bias_d is a device pointer to n ints (NULL = no bias, identical to
 * int4_linear_launch_async).  No reference counterpart: the reference lists bias addition as
 * future work (README.md:72); the add happens in the kernels' epilogue, so Y is still written
 * exactly once.
 */
int int4_linear_bias_launch_async(const void* x_packed_d, const void* w_packed_d, const int* bias_d,
                                  void* y_d, int m, int n, int k, void* stream);

/*
 * The operator for a stream of small-batch (decode) launches, with per-call promises instead of
 * the process-wide switch of int4_linear_set_overlap.  `promises` is a bit set:
 *   INT4L_PROMISE_WEIGHTS_STATIONARY  w_packed_d is not written by anything queued before this
 *                                     launch in `stream` (a linear layer's weights never are);
 *   INT4L_PROMISE_X_NOT_PENDING       the same for x_packed_d (valid only together with the first).
 * With a promise the launch may begin while its predecessor in the stream is still running
 * (programmatic dependent launch) and stream the promised operands early; everything it was not
 * promised is read, and Y is written, only after the predecessor has completed.  For shapes that
 * the decode kernels do not serve (m > 32) the promises are ignored.  0 = an ordinary launch.
 * bias_d as in int4_linear_bias_launch_async.  No reference counterpart: the reference launcher
 * synchronises the device after every call (kernels/linear_v21.cu:39).
 */
#define INT4L_PROMISE_WEIGHTS_STATIONARY 1
#define INT4L_PROMISE_X_NOT_PENDING      2
int int4_linear_decode_launch_async(const void* x_packed_d, const void* w_packed_d, const int* bias_d, void* y_d,
                                    int m, int n, int k, int promises, void* stream);

/*
 * The operator with a dequantising epilogue and bfloat16 output:
 *     Y16[i][j] = bf16( float(sum_l X[i][l] * W[j][l]) * row_scale[i] * col_scale[j] + bias[j] )
 * row_scale_d (m floats, per-token), col_scale_d (n floats, per-channel) and bias_d (n floats)
 * are device pointers, each may be NULL (factor 1 / addend 0); y_bf16_d is m x n bfloat16,
 * row-major, 16-byte aligned.  The integer sum is exact, its conversion to float is exact, the
 * scaling is one float multiply and one fused multiply-add, the result is rounded to nearest
 * even.  Halves the bytes of Y, the dominant stream of large shapes.  Runs on the tensor-memory
 * kernels and, for decode shapes, on the streaming kernels (same bits from both); the legacy path
 * has no such epilogue.  No reference counterpart (its output is int32 only).
 */
int int4_linear_scaled_launch_async(const void* x_packed_d, const void* w_packed_d, const float* row_scale_d,
                                    const float* col_scale_d, const float* bias_d, void* y_bf16_d,
                                    int m, int n, int k, void* stream);

/*
 * The same with IEEE half-precision output (y_f16_d: m x n halves).  The scaled value must fit the
 * half range (|v| < 65504), else it rounds to infinity as the conversion instruction does.
 */
int int4_linear_scaled_f16_launch_async(const void* x_packed_d, const void* w_packed_d, const float* row_scale_d,
                                    const float* col_scale_d, const float* bias_d, void* y_f16_d,
                                    int m, int n, int k, void* stream);

/*
 * N-sharded GEMM fused with the all-gather of its result.  This rank holds n_local rows of W
 * (columns [col_offset, col_offset + n_local) of the full Y) and the full X; y_full_ptrs is a HOST
 * array of `world` (<= 8) device pointers to the m x n_total int32 result buffer of every rank
 * of the node -- the rank's own buffer and its peers' buffers mapped into this process (CUDA
 * IPC / symmetric memory).  The kernel's epilogue stores the rank's column block into all of them
 * with TMA stores over NVLink while later tiles are still being computed; no multicast and no
 * loads from peer memory are involved.  Every rank calls this with its own shard; the full Y is
 * complete on a rank once ALL ranks' kernels have finished (synchronise the ranks afterwards,
 * e.g. with a barrier).  Needs n_local % 32 == 0, col_offset % 32 == 0, n_total % 4 == 0.
 * No reference counterpart (the reference is single-GPU).
 */
int int4_linear_launch_gather_async(const void* x_packed_d, const void* w_shard_packed_d, const int* bias_d,
                                    void* const* y_full_ptrs, int world, int col_offset,
                                    int m, int n_local, int n_total, int k, void* stream);

/*
 * Weight-stationary pre-layout.  int4_linear_prepare_weights expands a packed W (n rows of k/2
 * bytes) once into n rows of k bytes in the byte order the GEMM's tensor-core stage consumes
 * (w_expanded_d: n * k bytes, 16-byte aligned); int4_linear_launch_prepared_async then runs the
 * operator with that buffer in place of the packed weights, so that only the activations go
 * through the in-kernel unpack.  Same results bit for bit; costs twice the weight memory and is
 * meant for compute-bound shapes (decode shapes should keep the packed form: they are bound by
 * weight bytes).  bias_d as in int4_linear_bias_launch_async (NULL = none).  No reference
 * counterpart: the reference has one weight format.
 */
int int4_linear_prepare_weights(const void* w_packed_d, void* w_expanded_d, int n, int k, void* stream);
int int4_linear_launch_prepared_async(const void* x_packed_d, const void* w_expanded_d, const int* bias_d,
                                      void* y_d, int m, int n, int k, void* stream);

/*
 * The operator on operands that were BOTH expanded beforehand with int4_linear_prepare_weights
 * (which expands any packed matrix: pass X and its row count as well): x_expanded_d is m x k
 * bytes, w_expanded_d n x k bytes.  A pure 8-bit GEMM -- TMA straight into the ring the tensor
 * core reads, no unpack stage -- with the same results bit for bit.  It is the second pass of the
 * two-pass path made callable by itself, for callers that keep activations expanded across
 * several layers, and it is what bench.py times to measure the 8-bit tensor rate this library's
 * own pipeline reaches on the device.  No reference counterpart.
 */
int int4_linear_launch_expanded_async(const void* x_expanded_d, const void* w_expanded_d, const int* bias_d,
                                      void* y_d, int m, int n, int k, void* stream);

/*
 * The two-pass operator (expand pre-pass + byte GEMM, see int4_linear_set_two_pass) for callers
 * that are not allowed to allocate device memory: servers or frameworks that have handed the
 * whole GPU to their own allocator, loops that cannot take the device-wide synchronisation of
 * cudaMalloc/cudaFree, code under a no-allocation-after-start-up rule.  It has no counterpart
 * in the reference.  Its scratch is a fixed 64 MiB array inside the library's device image --
 * present on every GPU that loads the library, until the process exits -- so it accepts only
 * (m + n) * k <= 67 108 864 and returns INT4L_ERR_TOO_LARGE beyond that.  It never calls
 * cudaMalloc, cudaFree or any other allocating routine.  The first call on a device resolves the
 * array's device address and sets kernel attributes; issue it before any stream capture on that
 * device.  The array is shared by all calls and keeps the previous call's bytes (each call
 * overwrites what it reads, nothing has to be cleared); calls that could overlap on one GPU race
 * on it, so keep them ordered on one stream per device.  Same arguments and results as
 * int4_linear_bias_launch_async; a device-side timeout is reported by int4_linear_last_status
 * (which reads this entry point's status word back with a symbol copy, again without allocating).
 */
int int4_linear_launch_static_scratch_async(const void* x_packed_d, const void* w_packed_d, const int* bias_d,
                                            void* y_d, int m, int n, int k, void* stream);

/*
 * Host-buffer form of the call sequence in test/test_correctness.cu:53-63
 * (cudaMalloc x3, cudaMemcpy H2D x2, launch, cudaMemcpy D2H): operands and
 * result live in host memory; the library stages them through device buffers
 * it keeps between calls.  `w_resident` != 0 says the weights behind
 * `w_packed_h` are unchanged since the previous call with the same pointer
 * and size, so their upload is skipped (a linear layer's weights are
 * stationary; activations and the result always move).
 */
int int4_linear_host(const void* x_packed_h, const void* w_packed_h, void* y_h,
                     int m, int n, int k, int w_resident);

/*
 * Host packer with the reference's semantics (`pack` / `unpack`, utils/packer.h:5-6,
 * utils/packer.cpp:3-31): src / dst are HOST arrays, m x n ints with one signed 4-bit value each
 * on the unpacked side and m x ceil(n / 8) ints on the packed side (low nibble = even index, rows
 * padded with zero nibbles).  The library also exports the C++ symbols `pack` and `unpack`
 * themselves (declared in compat/utils/packer.h).
 */
void int4_linear_pack_host(const int* src_h, int* dst_h, int m, int n);
void int4_linear_unpack_host(const int* src_h, int* dst_h, int m, int n);

/*
 * Device-side forms of `void pack(const int* src, int* dst, int m, int n)` and
 * `void unpack(...)` (utils/packer.h:5-6, utils/packer.cpp:3-31): same bit layout, same
 * row padding to a multiple of eight elements, but source and destination are DEVICE
 * pointers and the work is a kernel on `stream`.  rows/cols take the place of the
 * reference's m/n.  dst of pack (src of unpack) holds rows * ceil(cols/8) 32-bit words.
 * int4_linear_pack_i8 takes one signed byte per element instead of one int.
 */
int int4_linear_pack_i32(const int* src_d, void* dst_d, int rows, int cols, void* stream);
int int4_linear_pack_i8(const signed char* src_d, void* dst_d, int rows, int cols, void* stream);
int int4_linear_unpack_i32(const void* src_d, int* dst_d, int rows, int cols, void* stream);

/* Status of the most recent call on the current device; also polls the word
 * the kernels raise when a bounded wait expires (and clears it). */
int int4_linear_last_status(void);

/* Measurement aid for the HBM-bound decode shapes: one read-only streaming pass over `bytes`
 * bytes at src_d (16-byte aligned), issued like the decode kernels' weight loads, XOR of the data
 * into *sink_d.  Its time for the bytes of a weight matrix is the floor for one launch of a kernel
 * that must read them once; bench.py reports it beside the decode kernel.  No reference
 * counterpart. */
int int4_linear_probe_stream_read(const void* src_d, unsigned long long bytes, unsigned* sink_d, void* stream);

/* Self-test of the in-kernel failure handling, safe to run on a shared GPU: launches one warp
 * that waits for at most budget_ms (1..100) on a barrier nothing will ever signal, exactly as a
 * GEMM kernel would after a lost arrival.  The kernel must return by itself; afterwards
 * int4_linear_last_status() reports INT4L_ERR_DEVICE_TIMEOUT once and the device stays usable.
 * Returns INT4L_OK when the kernel was run and came back. */
int int4_linear_selftest_timeout(int budget_ms);

/* Static string for a status code. */
const char* int4_linear_status_string(int status);

/* Forces one kernel family (INT4L_PATH_*) for subsequent calls of this
 * process; returns the previous setting.  The environment variable
 * INT4L_PATH=auto|tcgen05|legacy|skinny sets the initial value. */
int int4_linear_set_path(int path);

/* Tuning overrides for the tcgen05 family, for experiments and tests:
 * tile_n in {0 = automatic, 64, 128, 256} fixes the N extent of the
 * single-CTA output tile; direct_store != 0 makes the epilogue write Y with
 * per-thread vector stores instead of shared-memory staging + TMA stores
 * (always used when n % 4 != 0); cta_pairs = 1 forces the 256 x 256 tile on a
 * two-CTA cluster (cta_group::2), 0 forbids pairs, -1 leaves the choice to the
 * dispatcher.
 * Environment: INT4L_TILE_N, INT4L_EPILOGUE=direct, INT4L_PAIRS. */
int int4_linear_set_tuning(int tile_n, int direct_store, int cta_pairs);

/* How the tensor-memory kernels run a last wave of output tiles that does not fill the GPU:
 * 0 as whole tiles; 1 as half-width items when at most half of the CTA pairs would be busy (about
 * three quarters of a tile time instead of a whole one); 2 cut along K into equal shares for all
 * workers, every share ADDING its partial sums into Y (bulk reductions; integer addition, so the
 * result is bit-identical whatever the order) after a small kernel, launched in front of the GEMM
 * on the same stream, has cleared those tiles; -1 (default) whichever of the three the schedule's
 * cost estimate prefers.  Mode 2 applies to int32 output on one GPU.  The results are identical in
 * all modes.  Replaces the fixed one-CTA-per-tile grid of kernels/linear_v21.cu:20-37.
 * Returns INT4L_OK or INT4L_ERR_INVALID_ARG.  Environment: INT4L_TAIL=none|half|kcut. */
int int4_linear_set_tail(int mode);

/* Few rows of X (M <= 128, int32 output): a kernel of its own (csrc/gemm_fewrows.cu) runs the
 * tensor-memory GEMM with its operands swapped -- the 128-row side of each tile holds rows of W,
 * the narrow side (16 .. 64, once or twice) the rows of X, the accumulator is a tile of Y transposed
 * and the epilogue writes it back transposed -- and passes W through tensor memory instead of shared
 * memory, so that neither the tensor pipe nor the nibble expansion is spent on a 128-row X tile
 * that is mostly padding.  -1 (default): by shape -- 17 <= M <= 64 (from 17 to 32 only on large
 * weights), 65 <= M <= 128 when N >= 4096 (from 113 rows on: and K >= 4096), and M <= 16 where the decode kernels cannot run or K >
 * 8192; 0: never; 1: whenever M <= 128.  Results are identical either way.  The reference runs
 * every M on its one 256 x 128 tile (kernels/linear_v21.cu:12).
 * Returns INT4L_OK or INT4L_ERR_INVALID_ARG.  Environment: INT4L_FEWROWS=0|1. */
int int4_linear_set_fewrows(int mode);

/* Overlap of back-to-back decode-shape launches in one stream (programmatic dependent
 * launch).  0 (default): every launch waits for the preceding work in its stream, as any
 * kernel does.  1: the caller promises that the WEIGHTS passed to a launch are not written by
 * the work queued before it in the stream (stationary weights): the launch may start early
 * and prefetch weights while its predecessor finishes; X is read and Y written only after
 * the predecessor has completed.  2: the same promise for the weights AND X.
 * Returns the previous mode, or -INT4L_ERR_INVALID_ARG.  Environment: INT4L_OVERLAP.
 * No reference counterpart (the reference launcher synchronises the device after every call). */
int int4_linear_set_overlap(int mode);

/* Two-pass execution (opt-in): a streaming pre-pass expands both packed operands to bytes in a
 * scratch buffer the library keeps per device ((m + n) * k bytes, allocated with cudaMalloc on
 * first need and grown when a larger shape arrives), then a GEMM kernel reads them with nothing
 * but TMA and the tensor core on the shared-memory path.  Results are identical.  Measured on
 * B200 it is within +-5 % of the fused kernel for the largest shapes and slower for smaller
 * ones, so the dispatcher never picks it by itself.  mode: 1 = use it whenever the
 * tensor-memory family runs; 0 or -1 = fused single-kernel path only (default; no scratch).
 * Returns INT4L_OK, or INT4L_ERR_INVALID_ARG for any other mode (setting unchanged).
 * Environment: INT4L_TWO_PASS.  Because the first use of a larger shape allocates, make that
 * call before capturing a CUDA graph.  The scratch is one buffer per device: two-pass launches
 * that could run concurrently on one device (different streams) must not be issued. */
int int4_linear_set_two_pass(int mode);

/* Which family the dispatcher would use for a shape (INT4L_PATH_*). */
int int4_linear_path_for(int m, int n, int k);

/* Facts about the current device as this library sees them:
 * what = 0 number of SMs, 1 number of two-CTA clusters of the GEMM kernel that
 * can be resident at once.  Negative return = -status. */
int int4_linear_device_info(int what);

/* Number of kernels this library has launched in this process. */
long long int4_linear_launch_count(void);

/* Library version as major*10000 + minor*100 + patch. */
int int4_linear_version(void);

#ifdef __cplusplus
}
#endif

#endif /* INT4LINEAR_B200_H_ */
