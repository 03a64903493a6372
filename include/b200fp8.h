/*
 * b200fp8 — C ABI of the B200 (sm_100a) FP8 rowwise-scaled GEMM library.
 *
 *   Y[M,N] = bf16( (X_e4m3[M,K] · W_e4m3[N,K]^T) ⊙ x_scale[M] ⊗ w_scale[N]  (+ bias[N]) )     fp32 accumulation
 *
 * This is the boundary a TritonBench `fp8_gemm_rowwise` backend binds.  In the reference the
 * same boundary is the call from a backend closure into FBGEMM:
 *   tritonbench/operators/fp8_gemm_rowwise/operator.py:187-199  (`_triton`  -> matmul_fp8_row)
 *   tritonbench/operators/fp8_gemm_rowwise/operator.py:201-217  (`_cutlass_or_ck` -> torch.ops.fbgemm.f8f8bf16_rowwise)
 *   tritonbench/operators/fp8_gemm_rowwise/operator.py:219-235  (`_cublas` -> f8f8bf16_cublas + scale_fp8_row)
 *
 * Rules of the ABI
 *   - plain pointers and sizes only; no C++ or torch types cross it;
 *   - every function returns a b200fp8_status (0 = OK) and never exits or throws;
 *   - the device-pointer entry points allocate nothing, never synchronise and enqueue all work
 *     on the stream they are given, so a call can be captured in a CUDA graph (the reference
 *     times this operator by graph replay: operator.py:156, components/do_bench/run.py:190-199);
 *   - the caller owns every buffer, including the workspace.
 */
#ifndef B200FP8_H_
#define B200FP8_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200FP8_ABI_VERSION 1

typedef enum b200fp8_status {
  B200FP8_OK = 0,
  B200FP8_BAD_ARG = 1,               /* null pointer, non-positive size, leading dimension < row length */
  B200FP8_UNSUPPORTED_ARCH = 2,      /* device is not compute capability 10.x */
  B200FP8_UNSUPPORTED_ALIGNMENT = 3, /* the forced variant needs 16-byte aligned rows / pointers */
  B200FP8_WORKSPACE_TOO_SMALL = 4,
  B200FP8_LAUNCH_FAILED = 5,         /* a CUDA runtime / driver call failed; see b200fp8_last_cuda_error */
  B200FP8_DEVICE_TIMEOUT = 6,        /* a bounded wait inside a kernel ran out (read by b200fp8_query_status) */
  B200FP8_TOO_LARGE = 7              /* size beyond a stated maximum of the entry point */
} b200fp8_status;

/* `flags` bits 0-3: kernel variant.  0 lets the library choose from (M, N, K). */
#define B200FP8_VARIANT_AUTO 0u
#define B200FP8_VARIANT_TC_1CTA 1u   /* tcgen05 128x256x128 tiles, one CTA per tile                       */
#define B200FP8_VARIANT_TC_2CTA 2u   /* tcgen05 256x256x128 tiles, cta_group::2 CTA pair per tile         */
#define B200FP8_VARIANT_SKINNY 3u    /* M <= 128: swap-AB tcgen05 stream-K, persistent; for outputs too wide for TC_SPLITK */
#define B200FP8_VARIANT_SIMT 4u      /* CUDA-core kernel, any alignment; slow, used as an on-GPU cross-check */
#define B200FP8_VARIANT_TC_SPLITK 5u /* few tiles (decode, small M x N): one 128 x BN tile (BN <= 256) per cluster of
                                        1/2/4/8 CTAs that split K and reduce over distributed shared memory, or one
                                        128 x BN tile (BN <= 512) per CTA when that covers the output in one wave */
#define B200FP8_VARIANT_GEMV 6u      /* M <= 4: CUDA-core GEMV, every warp streams whole rows of W with 128-bit loads and
                                        finishes them with a warp-shuffle reduction; K a multiple of 16.  Never chosen by
                                        AUTO: measured slower than TC_SPLITK (the e4m3 conversions and fp32 multiply-adds
                                        need more issue slots than the memory gives time for)                            */
#define B200FP8_VARIANT_MASK 0xFu
#define B200FP8_FLAG_NO_TMA_STORE 0x10u /* tcgen05 variants: write Y with plain stores instead of TMA        */
/* TC_SPLITK, SKINNY and GEMV kernels only (TC_SPLITK and SKINNY are what `auto` picks for M <= 128): launch with programmatic stream
 * serialization, so the kernel may start while the kernel before it in the stream still runs.  It reads W
 * (only W) before that kernel has completed, everything else after.  The caller promises that no work still
 * in flight writes W.  The producer + quantiser kernels (b200fp8_fused_row_quantize: activations only) let such a
 * dependent start as soon as they are running (griddepcontrol.launch_dependents), so a decode GEMM behind them
 * overlaps the quantiser; the plain row and block quantisers, which also serve weights, do not. */
#define B200FP8_FLAG_PDL 0x20u
/* Y holds IEEE fp16 instead of bf16 (the output type of TritonBench's `fp8_gemm` operator with per-tensor
 * scales, tritonbench/operators/fp8_gemm/fp8_gemm.py:88-101); same 16-bit storage, same leading dimension. */
#define B200FP8_FLAG_OUT_FP16 0x40u

/* TC_SPLITK only, bits 8-16: force the tile width (a multiple of 16 x split, at most 256; with split 1 also a
 * multiple of 64 from 320 to 448, a wide tile multiplied as two column halves) and the cluster size (1, 2, 4 or
 * 8) instead of the library's cost model; 0 in a field lets the library choose it.
 * Any combination is correct; the knob exists for tuning and for tests. */
#define B200FP8_FLAG_SPLITK_CONFIG(block_n, split) ((((uint32_t)(block_n) / 16u) << 8) | ((uint32_t)(split) << 13))

/* Size of the bytes at the start of every workspace that hold the device status word. */
#define B200FP8_WORKSPACE_HEADER_BYTES 256u

int b200fp8_abi_version(void);

const char* b200fp8_status_string(int status);

/* Last CUDA error code (cudaError_t / CUresult value) seen by this thread inside the library. */
int b200fp8_last_cuda_error(void);

/*
 * Workspace a call with these sizes and flags needs, in bytes (always >= the header).
 * The workspace must be zero when first used (b200fp8_workspace_init); the library leaves
 * it zero after every call that completes, so one initialisation serves any number of calls.
 * Replaces: the output/temporary allocation FBGEMM's wrappers do per call (operator.py:187-235).
 */
size_t b200fp8_workspace_bytes(int64_t M, int64_t N, int64_t K, uint32_t flags);

/* Zero a workspace on `cuda_stream` (cudaMemsetAsync; capturable). */
int b200fp8_workspace_init(void* workspace, size_t workspace_bytes, void* cuda_stream);

/*
 * The GEMM.  All pointers are device pointers on the current device.
 *   xq [M,K] e4m3, row pitch ldx bytes;  wq [N,K] e4m3, row pitch ldw bytes (both K contiguous)
 *   x_scale [M], w_scale [N] fp32;  bias_bf16 [N] or NULL;  y_bf16 [M,N] bf16, row pitch ldy elements.
 * Replaces: the three backend calls cited at the top of this file.
 */
int b200fp8_gemm_rowwise(const void* xq, const void* wq, const float* x_scale, const float* w_scale,
                         const void* bias_bf16, void* y_bf16, int64_t M, int64_t N, int64_t K, int64_t ldx,
                         int64_t ldw, int64_t ldy, void* workspace, size_t workspace_bytes, uint32_t flags,
                         void* cuda_stream);

/*
 * The GEMM with its result written to several buffers at once: the fused form of "GEMM, then all-gather of Y" of
 * a run that shards X by rows over the GPUs of one node.  y_copies[0..num_copies) are device pointers, valid in
 * this process, to where THIS call's M rows of Y belong inside each copy of the gathered matrix: y_copies[0] in
 * the caller's own buffer, the others inside the other GPUs' buffers mapped into this process (CUDA IPC, see
 * b200fp8_shared_buffer_*).  All copies share the row pitch ldy (elements, a multiple of 8) and must be 16-byte
 * aligned.  The epilogue TMA-stores every 32 x 64 box of a tile to all copies (peer copies travel over NVLink as
 * plain stores; no kernel reads another GPU's memory), tile by tile while the next tile is multiplied, so the
 * exchange overlaps the arithmetic.  At most 8 copies.  Large-M kernels only (flags: AUTO, TC_1CTA, TC_2CTA,
 * OUT_FP16).  The call returns when the kernel is enqueued; rows written into another GPU's buffer may be read
 * there only after that GPU's process has synchronised with this stream (a barrier between the ranks).
 * Replaces: nothing in the reference (it has no multi-GPU code); the unfused form is b200fp8_gemm_rowwise
 * followed by an NCCL all-gather.
 */
int b200fp8_gemm_rowwise_gather(const void* xq, const void* wq, const float* x_scale, const float* w_scale,
                                const void* bias_bf16, void* const* y_copies, int num_copies, int64_t M, int64_t N,
                                int64_t K, int64_t ldx, int64_t ldw, int64_t ldy, void* workspace,
                                size_t workspace_bytes, uint32_t flags, void* cuda_stream);
/*
 * Device buffers another process of the same node can map, for the gathered Y above.  create: cudaMalloc on the
 * current device plus its CUDA IPC handle (B200FP8_IPC_HANDLE_BYTES bytes, to be sent to the other processes by
 * whatever channel the caller has); open: map a buffer created by another process, on another GPU, into this one
 * (peer access is enabled on first use); close undoes open, destroy undoes create.  Replaces: nothing in the
 * reference.
 */
#define B200FP8_IPC_HANDLE_BYTES 64u
int b200fp8_shared_buffer_create(size_t bytes, void** device_ptr, void* handle_out, size_t handle_bytes);
int b200fp8_shared_buffer_open(const void* handle_in, size_t handle_bytes, void** device_ptr);
int b200fp8_shared_buffer_close(void* device_ptr);
int b200fp8_shared_buffer_destroy(void* device_ptr);

/*
 * The same GEMM for M <= 128 WITHOUT any caller-provided workspace and without a single allocation.
 * (No counterpart in the reference: FBGEMM's wrappers allocate their output and temporaries per call.)
 *
 * For whom: a host that has handed all device memory to its own arena and lets no library call
 * cudaMalloc (an inference server that sizes its KV cache to the last free byte, a runtime that
 * forbids allocation once serving has started), and therefore cannot size and pass a workspace
 * either.  The kernel is the stream-K decode kernel; its scratch (status word, arrival counters,
 * fp32 partial sums) lives in a fixed 8 MiB array in device global memory that belongs to the
 * loaded library: every GPU that loads the library holds those 8 MiB until the process exits.
 *
 *   - M > 128, or a shape whose partial sums need more than the 8 MiB, returns B200FP8_TOO_LARGE
 *     (the scratch a decode problem needs grows with M only: every problem with M <= 48 fits);
 *   - calls no cudaMalloc / cudaFree and no allocating library routine; it enqueues one small
 *     cudaMemsetAsync (status word + the counters this call uses) and the kernel on `cuda_stream`;
 *   - the FIRST call on each device looks up the array's device address (cudaGetSymbolAddress) and
 *     raises the kernel's shared-memory limit: make that first call before any stream capture;
 *   - all calls share the one array: two calls that overlap on the GPU (different streams, or
 *     concurrent graphs) race on it.  Order them on one stream or with events.
 * b200fp8_noalloc_status reads the status word of the array after the caller synchronised.
 */
int b200fp8_gemm_rowwise_noalloc(const void* xq, const void* wq, const float* x_scale, const float* w_scale,
                                 const void* bias_bf16, void* y_bf16, int64_t M, int64_t N, int64_t K, int64_t ldx,
                                 int64_t ldw, int64_t ldy, void* cuda_stream);
int b200fp8_noalloc_status(uint32_t* device_status);

/*
 * Grouped form (mixture-of-experts): the rows of xq [M_total, K] are partitioned, in order, into num_groups
 * groups of group_rows[g] rows (an int32 array in DEVICE memory, read by the kernel: no host round trip when
 * the sizes come from a router kernel); group g is multiplied with rows [g*N, (g+1)*N) of the stacked
 * wq [num_groups*N, K]; x_scale [M_total], w_scale [num_groups*N]; y [M_total, N].  Rows beyond the sum of the
 * group sizes are left untouched.  Needs only the workspace header (256 bytes).  `flags`: variant AUTO, TC_1CTA
 * (128-row tiles per group) or TC_2CTA (a CTA pair per 256-row tile of a group; AUTO picks it when M_total x N has
 * enough such tiles for the pairs the device runs at once), NO_TMA_STORE, OUT_FP16.
 * Replaces: `grouped_gemm_fp8_rowwise(group_A, group_B, m_sizes, a_scale, b_scale)` and
 * `torch.ops.fbgemm.f8f8bf16_rowwise_grouped_stacked` in
 * tritonbench/operators/fp8_gemm_rowwise_grouped/operator.py:412-470.
 */
int b200fp8_gemm_rowwise_grouped(const void* xq, const void* wq, const float* x_scale, const float* w_scale,
                                 const int32_t* group_rows, int64_t num_groups, void* y_bf16, int64_t M_total,
                                 int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldy, void* workspace,
                                 size_t workspace_bytes, uint32_t flags, void* cuda_stream);

/*
 * Block-scaled form: one fp32 scale per 128x128 block of X and of W,
 *   Y[m,n] = bf16( sum_kb (sum_{k in block kb} X[m,k] W[n,k]) * x_scale[m/128][kb] * w_scale[n/128][kb] ),
 * x_scale [ceil(M/128)][ld_xs], w_scale [ceil(N/128)][ld_ws] fp32 (row pitches in elements, >= ceil(K/128)).
 * Every k-block's product is accumulated in tensor memory on its own and promoted into fp32 registers with
 * that block's scale.  Needs only the workspace header.
 * Replaces: `matmul_fp8_block(xq, wq, x_scale, w_scale)` and `torch.ops.fbgemm.f8f8bf16_blockwise` in
 * tritonbench/operators/fp8_gemm_blockwise/operator.py:139-149.
 */
int b200fp8_gemm_blockwise(const void* xq, const void* wq, const float* x_scale, const float* w_scale, void* y_bf16,
                           int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldy, int64_t ld_xs,
                           int64_t ld_ws, void* workspace, size_t workspace_bytes, uint32_t flags, void* cuda_stream);

/*
 * Rowwise e4m3 quantiser: x [rows, cols] (row pitch ldx ELEMENTS) -> q [rows, cols] e4m3 bytes (row pitch ldq
 * bytes) and scale [rows] fp32 such that x ~ float(q) * scale.  One pass over HBM, asynchronous on the stream.
 *   x_dtype  B200FP8_DTYPE_BF16 / _FP16 / _FP32
 *   recipe   B200FP8_QUANT_OPERATOR: bit-exact with the operator's `fp8_row_quantize`
 *            (tritonbench/operators/fp8_gemm_rowwise/operator.py:136-145: arithmetic in x's dtype,
 *            multiplier 448 / clamp(rowmax, 1e-12), fp16 multiplier clamped to 65504, returns 1 / multiplier);
 *            B200FP8_QUANT_FP32 (fp32 x only): scale = max(rowabsmax, 1e-12) / 448, q = e4m3(clamp(x / scale)).
 * Replaces: the five eager torch kernels per operand of operator.py:136-145 called from operator.py:280-297.
 */
#define B200FP8_DTYPE_BF16 0
#define B200FP8_DTYPE_FP16 1
#define B200FP8_DTYPE_FP32 2
#define B200FP8_QUANT_OPERATOR 0
#define B200FP8_QUANT_FP32 1
int b200fp8_row_quantize(const void* x, int x_dtype, int recipe, int64_t rows, int64_t cols, int64_t ldx, void* q,
                         int64_t ldq, float* scale, void* cuda_stream);

/*
 * 128x128 block quantiser, the operand format of b200fp8_gemm_blockwise: per block the multiplier 448 / blockmax
 * (blockmax clamped below at 1e-12 in x's dtype, the division in fp32, 1 where it is infinite), q = e4m3(x * mult)
 * without a clamp, scale[block row][block column] = 1 / mult.  Rows and columns beyond the matrix count as zeros.
 * scale is [ceil(rows/128)][ld_scale] fp32 with ld_scale >= ceil(cols/128).  Bit-exact with the reference's
 * `fp8_block_quantize` (tritonbench/operators/fp8_gemm_blockwise/operator.py:87-120), which it replaces: eight eager torch
 * kernels and a padded copy of x.
 */
int b200fp8_block_quantize(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ldx, void* q, int64_t ldq,
                           float* scale, int64_t ld_scale, void* cuda_stream);

/*
 * Producer + rowwise quantiser in one pass: the activation that feeds the GEMM is computed from its bf16 inputs,
 * quantised (scale = max(rowabsmax(y), 1e-12) / 448, q = e4m3(clamp(y * (1 / scale)))) and written as e4m3 bytes plus
 * one fp32 scale per row, without the bf16 activation being stored.  fp32 arithmetic; the SiLU uses the hardware
 * exponential and reciprocal (about 2 ulp).
 *   B200FP8_PRODUCER_RMS_NORM  y[k] = x1[k] * rsqrt(mean_k(x1^2) + eps) * x2[k], x2 the weight vector [cols] (ld2 ignored)
 *   B200FP8_PRODUCER_SILU_MUL  y[k] = x1[k] / (1 + exp(-x1[k])) * x2[k],         x2 [rows, cols] with row pitch ld2
 *   round_bf16 != 0            y is rounded to bf16 before the quantisation (= producer kernel, then quantiser)
 * Replaces: `rms_norm_fp8_rowwise_quant(x1, wd)` / `silu_mul_fp8_rowwise_quant(x1, x2)` and, with round_bf16,
 * `rms_norm` / `silu_mul` followed by `quantize_fp8_row`
 * (tritonbench/operators/fp8_fused_quant_gemm_rowwise/operator.py:86-131; those kernels are Meta-internal and absent
 * from the reference tree, so eps and the fp32 arithmetic are this library's definition).
 */
#define B200FP8_PRODUCER_RMS_NORM 1
#define B200FP8_PRODUCER_SILU_MUL 2
int b200fp8_fused_row_quantize(int producer, const void* x1_bf16, const void* x2_bf16, int64_t rows, int64_t cols,
                               int64_t ld1, int64_t ld2, float eps, int round_bf16, void* q, int64_t ldq, float* scale,
                               void* cuda_stream);

/*
 * Read the device status word of a workspace.  Call after the stream has been synchronised.
 * Returns B200FP8_OK or B200FP8_DEVICE_TIMEOUT; *device_status receives the raw word
 * (code << 24 | site).  Replaces: the reference's exit-on-error helper macros
 * (tritonbench/operators/mixed_gemm/kernels/helper.h:40-64) with a status code.
 */
int b200fp8_query_status(const void* workspace, uint32_t* device_status);

/*
 * Self-test of the failure path: launches one CTA that waits on a barrier nothing will ever arrive on, with a
 * limit of `limit_us` microseconds (at most one second).  The wait runs out, the kernel ends normally, and after a
 * synchronise b200fp8_query_status(workspace) returns B200FP8_DEVICE_TIMEOUT.  Nothing faults, traps or hangs;
 * re-initialise the workspace afterwards.  Replaces: nothing in the reference (its native code exits the process
 * on error, tritonbench/operators/mixed_gemm/kernels/helper.h:40-64).
 */
int b200fp8_selftest_wait_timeout(void* workspace, uint32_t limit_us, void* cuda_stream);

/*
 * Human-readable plan for a problem size: variant, tile, grid, pipeline depth, workspace.
 * Writes a NUL-terminated string of at most n-1 characters.
 * Replaces: the backend knobs the reference passes to FBGEMM (operator.py:187-199).
 */
int b200fp8_describe_plan(int64_t M, int64_t N, int64_t K, uint32_t flags, char* buf, size_t n);

/*
 * Host-buffer form, the call a host program without its own device memory makes:
 * inputs and output live in host memory (pinned for full PCIe speed), device staging
 * buffers belong to the context.  One call = copy in, GEMM, copy out, synchronise; the context's device is
 * made current for the duration of the call.  Larger problems are cut into panels of 1024 rows of X and 2048
 * rows of W that go up alternately; after every upload the strip of Y that has just become computable is multiplied
 * by one GEMM and sent down by one copy (a pitched copy into the host array when the strip is narrower than Y), so
 * both PCIe directions and the GPU work at once.
 * Whatever the call returns, no copy is in flight on the caller's buffers when it returns.
 * Replaces: `input_cast(.to(device))` + backend call + result read in
 * tritonbench/utils/triton_op.py:846-850,1221-1232.
 */
typedef struct b200fp8_host_ctx b200fp8_host_ctx;
int b200fp8_host_ctx_create(int64_t M, int64_t N, int64_t K, uint32_t flags, b200fp8_host_ctx** out);
int b200fp8_host_ctx_destroy(b200fp8_host_ctx* ctx);
int b200fp8_gemm_rowwise_host(b200fp8_host_ctx* ctx, const void* xq, const void* wq, const float* x_scale,
                              const float* w_scale, const void* bias_bf16, void* y_bf16);
/*
 * Serving form.  The context keeps the W, w_scale and bias of the last upload on the device: an upload is this
 * call, or any b200fp8_gemm_rowwise_host call that passed wq.  A b200fp8_gemm_rowwise_host call with wq == NULL
 * reuses them (its w_scale and bias_bf16 arguments are ignored; BAD_ARG if nothing was uploaded yet): only X and
 * x_scale go up, and Y comes down in whole row panels.  set_weights(ctx, NULL, NULL, NULL) forgets the weights.
 * Synchronous.  Replaces: the reference keeps `wq` on the device across the timed calls of one input
 * (tritonbench/utils/triton_op.py:846-850 casts the inputs once, 1221-1232 times the call).
 */
int b200fp8_host_ctx_set_weights(b200fp8_host_ctx* ctx, const void* wq, const float* w_scale, const void* bias_bf16);
/*
 * Tuning knob: panel sizes of the pipeline above (rows of X per panel, rows of W = columns of Y per panel).
 * A panel smaller than its dimension must be a multiple of 128 rows / 256 columns; at most 64 panels per
 * dimension.  Any setting gives a Y within the kernels' tolerance of any other (strips of different shapes may
 * run different kernel plans).  Replaces: nothing in the reference.
 */
int b200fp8_host_ctx_set_panels(b200fp8_host_ctx* ctx, int64_t panel_rows, int64_t panel_cols);

#ifdef __cplusplus
}
#endif
#endif /* B200FP8_H_ */
