/*
 * mnq.h -- C ABI of libmnq.so: B200 (sm_100a) kernels for MetalNative's fused
 * INT4/INT8 dequantise + matmul operator.
 *
 * Every entry point takes plain device pointers and sizes, enqueues work on the
 * CUDA stream it is given and returns without synchronising.  The caller owns all
 * buffers (inputs, output and workspace); unless an entry point says otherwise
 * the library allocates nothing.  No C++ exception crosses this boundary: each
 * call returns an mnq_status and, on failure, mnq_last_error() gives the message
 * for the calling thread.  Validation runs on the host before any launch.
 *
 * Data layouts are the reference's (shaders/matmul_dequant_kernel.metal:55-72):
 *   activations    [M, K]        fp16 or bf16, row-major, leading dimension lda
 *   weights_packed [N, K/2]      uint8, two 4-bit values per byte, element k in
 *                                the low nibble for even k, high nibble for odd k
 *                  [N, K]        int8
 *   scales, zeros  [N, ceil(K/group_size)]   fp16 or bf16
 *   out            [M, N]        dtype of the activations, leading dimension ldc
 * with  w[n,k] = (q - 8) * s - z  (int4, q the unsigned nibble)
 *       w[n,k] =  q      * s - z  (int8, q signed)
 * and   out[m,n] = sum_k activations[m,k] * w[n,k], accumulated in fp32.
 */
#ifndef MNQ_H
#define MNQ_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define MNQ_API __attribute__((visibility("default")))
#else
#define MNQ_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes: the values of the reference's MetalNativeError enum
 * (include/metal_native/core/error.h:21-31). */
typedef enum mnq_status {
    MNQ_SUCCESS = 0,
    MNQ_DEVICE_NOT_FOUND = 1,
    MNQ_ALLOCATION_FAILED = 2,
    MNQ_KERNEL_COMPILATION_FAILED = 3,
    MNQ_INVALID_ARGUMENT = 4,
    MNQ_OUT_OF_MEMORY = 5,
    MNQ_TIMEOUT_ERROR = 6,
    MNQ_INTERNAL_ERROR = 7,
    MNQ_NOT_IMPLEMENTED = 8
} mnq_status;

/* Replaces enum class QuantType {INT4, INT8}
 * (include/metal_native/ops/matmul.h:59-63). */
typedef enum mnq_quant { MNQ_INT4 = 0, MNQ_INT8 = 1 } mnq_quant;

/* Element types that cross the boundary. */
typedef enum mnq_dtype { MNQ_FP16 = 0, MNQ_BF16 = 1, MNQ_FP32 = 2 } mnq_dtype;

/* Kernel families the dispatcher chooses from (mnq_dequant_matmul_ex). */
typedef enum mnq_path {
    MNQ_PATH_AUTO = 0,
    MNQ_PATH_GEMV = 1,    /* M <= 32: streams packed rows, unpacks in registers */
    MNQ_PATH_GEMM = 2,    /* tcgen05 / TMEM tensor-core tiles */
    MNQ_PATH_GENERIC = 3  /* any shape or alignment; guarded scalar loads */
} mnq_path;

/* What is applied to the fp32 result before the store: the values of the reference's
 * enum class MatmulEpilogue {None, Bias, BiasReLU, BiasSiLU, ResidualAdd}
 * (include/metal_native/ops/fused_matmul.h:18-24). */
typedef enum mnq_epilogue {
    MNQ_EPI_NONE = 0,
    MNQ_EPI_BIAS = 1,       /* out = x W^T + bias            bias [N], broadcast over rows */
    MNQ_EPI_BIAS_RELU = 2,  /* out = max(0, x W^T + bias) */
    MNQ_EPI_BIAS_SILU = 3,  /* out = silu(x W^T + bias), silu(v) = v / (1 + exp(-v)) */
    MNQ_EPI_RESIDUAL = 4    /* out = x W^T + residual        residual [M, N] */
} mnq_epilogue;

/* Process-wide options (mnq_set_option / mnq_get_option). */
typedef enum mnq_option {
    /* Non-zero: the caller promises that weights_packed, scales and zeros are never written by
     * work that is still in flight when an operator call starts (model state, loaded once).  The
     * decode kernels then request their first weight tiles before they wait for the previous
     * kernel in the stream to finish.  Default 0. */
    MNQ_OPT_WEIGHTS_IMMUTABLE = 0,
    /* Polls (of about 100 ns each) a sharded call waits for another rank before it gives up and
     * sets bit 2 of the device status word.  Default 1 << 22 (about 0.4 s). */
    MNQ_OPT_PEER_WAIT_POLLS = 1,
    /* Largest token count M that takes the decode (GEMV) kernels; above it the tensor-core
     * kernel runs.  0..32, initialised from the environment variable METAL_NATIVE_GEMV_MAX_M
     * when set.  Default 0: chosen per problem from B200 measurements (16 for int8 weights with
     * one scale per row and for layers of fewer than 8192 rows and less than 24 MB, 32 for every other
     * format; bf16 activations with group-wise scales stay on the decode kernels up to 64 tokens).  The
     * reference's counterpart is the fixed `use_vecmat = (M <= 8)` (src/ops/matmul.mm:946). */
    MNQ_OPT_GEMV_MAX_M = 2,
    /* Non-zero: bf16 activations with group-wise scales (or zeros) above the decode threshold use ONE
     * fp16 weight tile per k-block, as fp16 activations do, instead of two bf16 tiles (hi + lo): the
     * activations are converted once per call to fp16 times a per-token power of two, scales and zeros
     * are normalised per row.  About twice as fast up to 128 tokens (measured on the Llama-3-8B shapes:
     * 34 against 70 us at 64 tokens) and 1.1-1.3 times at 512; every weight is rounded to 11 significant
     * bits instead of 16, which adds noise of about 2.8e-4 of the output RMS (rel-L2 stays under 1e-3).
     * Needs room in the workspace (mnq_workspace_bytes accounts for it while the option is set).
     * Default 0. */
    MNQ_OPT_BF16_FP16_TILES = 3
} mnq_option;

/* Optional overrides for mnq_dequant_matmul_ex.  Zero in a field means "let the
 * library decide"; a zero-filled struct behaves like passing NULL. */
typedef struct mnq_tuning {
    int32_t path;                /* mnq_path */
    int32_t split_k;             /* GEMV: number of K chunks */
    int32_t warps_per_cta;       /* GEMV: 16 output rows per warp at a time */
    int32_t gemv_variant;        /* kernel variant, 0 auto.  GEMV path: 1 register-prefetch kernel, 2 shared-memory
                                    streaming kernel.  GEMM path: 1 single-CTA tiles, 2 CTA pairs (cta_group::2),
                                    3 never two CTAs per SM, 4 two CTAs per SM whenever a tile allows it, 5 no raw-integer
                                    tiles, 6 weight tiles always through shared memory (never tensor memory), 7 no cut of the last round's tiles along K, 8 bf16 activations with
                                    group-wise scales: two bf16 tiles per k-block even with MNQ_OPT_BF16_FP16_TILES set.  Streaming GEMV: 9 the batched-decode kernel even on small layers of few rows, 3 the general kernel even where the compact or the batched one would
                                    run, 4 no kernel that reads prepared activations (the compact kernel up to 8 tokens,
                                    the general one above) */
    int32_t piece_bytes;         /* streaming GEMV: packed bytes per row per stage (multiple of 64) */
    int32_t stages;              /* streaming GEMV: stages per warp (2..8) */
    int32_t ctas_per_sm;         /* streaming GEMV: resident CTAs per SM the plan assumes */
    int32_t row_blocks_per_warp; /* streaming GEMV: consecutive 16-row blocks per warp */
} mnq_tuning;

/* Name of a status code ("Success", "InvalidArgument", ...): the strings of the
 * reference's error_to_string (src/core/error.cpp:14-26). */
MNQ_API const char* mnq_status_name(int status);

/* Message of the last failed call made by this thread ("" if none).  The text
 * after the "<StatusName>: " prefix the reference puts in MNException::what()
 * (src/core/error.cpp:60-63). */
MNQ_API const char* mnq_last_error(void);

/* Workspace the fused operator may need for the given problem, in bytes (it
 * depends only on the arguments, never on device state).  The workspace holds
 * arrival counters (its first 64 KiB) followed by split-K partial sums.  It must be
 * zero-filled once before its first use; every call leaves the counters at zero
 * again, so one buffer can be reused by successive calls, of any shapes, on the
 * same stream.  Calls that may run
 * concurrently need separate workspaces. */
MNQ_API size_t mnq_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size, int32_t quant_type);

/* Fused dequantise + matmul.  Replaces
 *   MNTensor dequant_matmul(activations, weights_packed, scales, zeros, group_size, quant_type)
 * (include/metal_native/ops/matmul.h:77-82; host side src/ops/matmul.mm:903-1029).
 *
 * Differences from the reference's host function, all at the boundary:
 *   - the caller passes `out` (the reference allocates and returns it);
 *   - act_dtype may be MNQ_BF16 as well as MNQ_FP16 (out has the same dtype);
 *     scale_dtype is the dtype of scales and zeros and may differ from it;
 *   - group_size may be any positive multiple of 32, or any value >= K for one
 *     scale per output row ("per-channel"); the reference accepts 32, 64, 128;
 *   - zeros may be NULL, meaning all zero;
 *   - every row m < M is computed (the reference's M <= 8 kernels write row 0 only).
 * K must be even for int4.  lda >= K, ldc >= N, in elements.
 * `workspace` may be NULL when workspace_bytes is 0; if the workspace is smaller
 * than mnq_workspace_bytes() the call still succeeds with less K-parallelism. */
MNQ_API int mnq_dequant_matmul(const void* activations, const void* weights_packed, const void* scales,
                       const void* zeros, void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                       int64_t ldc, int32_t group_size, int32_t quant_type, int32_t act_dtype,
                       int32_t scale_dtype, void* workspace, size_t workspace_bytes, void* stream);

/* Same, with overrides (tests and tuning).  `tuning` may be NULL. */
MNQ_API int mnq_dequant_matmul_ex(const void* activations, const void* weights_packed, const void* scales,
                          const void* zeros, void* out, int64_t M, int64_t N, int64_t K,
                          int64_t lda, int64_t ldc, int32_t group_size, int32_t quant_type,
                          int32_t act_dtype, int32_t scale_dtype, void* workspace,
                          size_t workspace_bytes, void* stream, const mnq_tuning* tuning);

/* Which kernel family mnq_dequant_matmul would run for these arguments
 * (an mnq_path value other than AUTO), or a negative mnq_status on bad arguments.
 * Pure host logic: usable without a GPU.  The reference's counterpart is the
 * `use_vecmat = (M <= 8)` choice in src/ops/matmul.mm:946-956. */
MNQ_API int mnq_select_path(int64_t M, int64_t N, int64_t K, int64_t lda, int32_t group_size,
                    int32_t quant_type, int32_t act_dtype, const void* activations,
                    const void* weights_packed, const void* scales, const void* zeros);

/* Same question with the dtype of scales and zeros given (mnq_select_path assumes fp16): the
 * tensor-core kernel multiplies fp16 activations by fp16 scales only, so fp16 activations with
 * bf16 scales and M above the decode threshold run the any-shape kernel (MNQ_PATH_GENERIC),
 * which is correct but slow. */
MNQ_API int mnq_select_path_ex(int64_t M, int64_t N, int64_t K, int64_t lda, int32_t group_size,
                       int32_t quant_type, int32_t act_dtype, int32_t scale_dtype, const void* activations,
                       const void* weights_packed, const void* scales, const void* zeros);

/* Sets / reads a process-wide option (mnq_option).  mnq_set_option returns MNQ_INVALID_ARGUMENT
 * for an unknown option or a value outside its range; mnq_get_option returns -1 for an unknown
 * option.  Thread-safe; a call already enqueued keeps the value it was launched with. */
MNQ_API int mnq_set_option(int32_t option, int64_t value);
MNQ_API int64_t mnq_get_option(int32_t option);

/* Fused dequantise + matmul with an epilogue, and optionally an fp32 output.  Replaces
 *   MNTensor fused_matmul(a, b, epilogue, bias, residual, ...)
 * (include/metal_native/ops/fused_matmul.h:64-70) for the quantised operator: the reference
 * applies its epilogues to the unquantised matmul (shaders/matmul_fused_epilogue.metal:97-124);
 * here the same arithmetic follows the dequant-matmul's fp32 accumulation, before the only store:
 * fp32 add of bias[n] (or residual[m, n]), the activation in fp32, one rounding to the output type.
 *   epilogue  an mnq_epilogue value; bias is [N] and residual [M, ldr] (ldr >= N, in elements), both
 *             in the activation dtype; the one the epilogue does not use may be NULL.  As in the
 *             reference a missing required tensor is MNQ_INVALID_ARGUMENT.
 *   out_dtype the activation dtype (then out is what mnq_dequant_matmul returns, with the epilogue
 *             applied) or MNQ_FP32: out is float [M, ldc] holding the value before the final
 *             rounding -- the accumulators themselves, for checking a 16-bit kernel against an fp32
 *             expectation without the output rounding in the way.
 * Other arguments as for mnq_dequant_matmul. */
MNQ_API int mnq_dequant_matmul_fused(const void* activations, const void* weights_packed, const void* scales,
                             const void* zeros, void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                             int64_t ldc, int32_t group_size, int32_t quant_type, int32_t act_dtype,
                             int32_t scale_dtype, int32_t out_dtype, int32_t epilogue, const void* bias,
                             const void* residual, int64_t ldr, void* workspace, size_t workspace_bytes,
                             void* stream);

/* Dequantise a whole weight matrix with the fused operator's formula (scale and
 * zero, [N, ceil(K/g)] indexing): out[n,k] = (q-8)*s - z  or  q*s - z, evaluated
 * in fp32 as a product then a subtraction (the product is exact), then rounded to nearest even if out_dtype is
 * fp16 or bf16.  The fp32 output is bit-identical to the reference's CPU helpers
 * dequant_reference_int4 / dequant_reference_int8
 * (tests/cpp/test_dequant_matmul.mm:119-188).  out is [N, K] row-major. */
MNQ_API int mnq_dequantize(const void* weights_packed, const void* scales, const void* zeros, void* out,
                   int64_t N, int64_t K, int32_t group_size, int32_t quant_type,
                   int32_t scale_dtype, int32_t out_dtype, void* stream);

/* The reference's standalone dequantise kernels
 *   dequantize_int8_to_fp16[_vec]  (shaders/dequantize_kernel.metal:9-22, 58-96)
 *   dequantize_int4_to_fp16[_vec]  (shaders/dequantize_kernel.metal:26-54, 100-163)
 * as launched by QuantWeightCache::get_dequantized
 * (src/memory/quant_weight_cache.mm:65-153): scale only, no zero-point, flat
 * group index i / group_size, fp16 scales, fp16 output of num_elements values. */
MNQ_API int mnq_dequantize_flat(const void* input, const void* scales_fp16, void* out_fp16,
                        int64_t num_elements, int32_t group_size, int32_t quant_type, void* stream);

/* Reads (and, if `clear` is non-zero, resets) the device-side status word of the
 * current device; synchronises the device.  Bits 0 and 1: a decode / tensor-core kernel gave
 * up a bounded wait for an asynchronous copy; bit 2: a sharded call gave up waiting for
 * another rank (MNQ_OPT_PEER_WAIT_POLLS).  In each case the output of that call is incomplete
 * (reported by the shim as TimeoutError, the reference's MetalNativeError::TimeoutError,
 * include/metal_native/core/error.h:28); the arrival counters of the workspace are back at
 * zero, so the workspace can be used again.  No counterpart call in the reference. */
MNQ_API int mnq_device_status(uint32_t* status, int32_t clear);

/* Fused dequantise + matmul for callers that cannot allocate device memory.
 * No counterpart in the reference (its operator allocates its own output).
 *
 * Same arguments and results as mnq_dequant_matmul, minus the workspace: the split-K
 * scratch the decode kernels need lives in a fixed array inside the library,
 * MNQ_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the library, kept
 * until the process exits.  It is meant for code that is handed only its inputs and
 * outputs and must not call cudaMalloc or any allocator: plugins of a host runtime that
 * owns all device memory, callbacks running inside an allocator, serving loops with a
 * frozen memory budget.  The call itself allocates nothing (no cudaMalloc, cudaFree or
 * allocating library routine).
 *
 *  - Limit: a problem whose scratch demand, mnq_workspace_bytes(M, N, K, ...), exceeds
 *    MNQ_STATIC_SCRATCH_BYTES is refused with MNQ_INVALID_ARGUMENT; nothing is launched.
 *  - The first call on each device looks up the array's device address (a synchronous
 *    runtime query): make that first call before any stream capture begins.
 *  - All calls on a device share the one array.  Each call clears the arrival counters
 *    it needs on `stream` before launching, but two calls that overlap on the GPU
 *    (different streams, or different threads) race on it and give wrong results:
 *    serialise them, or use mnq_dequant_matmul with separate workspaces. */
#define MNQ_STATIC_SCRATCH_BYTES (4u << 20)
MNQ_API int mnq_dequant_matmul_static(const void* activations, const void* weights_packed, const void* scales,
                              const void* zeros, void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                              int64_t ldc, int32_t group_size, int32_t quant_type, int32_t act_dtype,
                              int32_t scale_dtype, void* stream);

/* Fused gate+up projection with the SwiGLU activation in the epilogue (decode sizes):
 *   out[m, j] = silu(g) * u,  g = x[m,:] . W[j,:],  u = x[m,:] . W[H + j,:],  silu(g) = g / (1 + exp(-g))
 * for the fused weight matrix W = [gate rows; up rows] of shape [2H, K] (scales and zeros [2H, G]).
 * The reference computes the two projections with dequant_matmul and applies fast::swiglu(gate, up)
 * as a separate kernel (include/metal_native/future/fast_ops.h:86-90, shaders/fused_swiglu.metal:48-84:
 * fp32 math, 16-bit store); here a 16-row MMA tile holds 8 gate rows and their 8 up rows, so both
 * sums of an output sit in one thread's accumulators and the [M, 2H] intermediate is never written.
 * out is [M, H] in the activation dtype.  Takes what the streaming decode kernel takes with K unsplit
 * (M <= 32 among others); otherwise MNQ_NOT_IMPLEMENTED. */
MNQ_API int mnq_dequant_matmul_swiglu(const void* activations, const void* weights_packed, const void* scales,
                                      const void* zeros, void* out, int64_t M, int64_t H, int64_t K, int64_t lda,
                                      int64_t ldc, int32_t group_size, int32_t quant_type, int32_t act_dtype,
                                      int32_t scale_dtype, void* stream);

/* Fused residual addition + RMSNorm, the operator that produces the activations of the MLP these
 * projections belong to: out = rms_norm(input + residual) * weight, row by row.  Replaces the
 * reference's fast::fused_residual_norm (include/metal_native/future/fast_ops.h:99-107) and keeps the
 * arithmetic of its kernels (shaders/fused_residual_norm.metal:43-76): the sum is rounded to the
 * 16-bit type and that rounded value is normalised, the mean of squares is taken over the unrounded
 * sums in fp32, rms_inv = rsqrt(mean + eps), one rounding at the store.  input, residual, out:
 * [rows, hidden] with row strides ld_* (elements); weight: [hidden]; all of `dtype` (MNQ_FP16 or
 * MNQ_BF16; the reference has fp16 and fp32).  sum_out, if not NULL, receives the rounded sums (the
 * block's new residual stream; the reference discards them).  out may alias input or residual. */
MNQ_API int mnq_residual_rmsnorm(const void* input, const void* residual, const void* weight, void* out,
                                 void* sum_out, int64_t rows, int64_t hidden, int64_t ld_in, int64_t ld_res,
                                 int64_t ld_out, int64_t ld_sum, float eps, int32_t dtype, void* stream);

/* The fused operator for activations and output in HOST memory (pinned for the copies to be
 * asynchronous), weights, scales and zeros resident on the device.  The reference's tensors live in
 * memory both the CPU and the GPU address (MTLStorageModeShared, src/core/tensor_helpers.mm:13-48), so
 * its callers hand `dequant_matmul` buffers they filled on the CPU and read the result on the CPU
 * after `synchronize()`; on a discrete GPU the same calling pattern needs the two copies, and this
 * entry point enqueues them with the kernel: host -> device of [M, K] activations (contiguous),
 * the operator, device -> host of the [M, N] output (contiguous), all on `stream`, returning
 * without synchronising.  `workspace` must hold mnq_host_workspace_bytes(...) bytes: the operator's
 * scratch (zero-filled once, as for mnq_dequant_matmul) followed by the device copies of the
 * activations and the output. */
MNQ_API size_t mnq_host_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size, int32_t quant_type);
MNQ_API int mnq_dequant_matmul_host(const void* activations_host, const void* weights_packed, const void* scales,
                                    const void* zeros, void* out_host, int64_t M, int64_t N, int64_t K,
                                    int32_t group_size, int32_t quant_type, int32_t act_dtype, int32_t scale_dtype,
                                    void* workspace, size_t workspace_bytes, void* stream);

/* Column-sharded fused operator with the all-gather folded into the kernel.  No counterpart in
 * the reference (it drives one device); this is the N-sharded form of mnq_dequant_matmul for
 * `world` GPUs of one node, one process per GPU, each holding rows [n_offset, n_offset + N_local)
 * of the weights, scales and zeros and the whole activation block.
 *
 * out_peers and flag_peers are HOST arrays of `world` device pointers, the same on every rank:
 * out_peers[g] is rank g's gathered output [M, ldc] (ldc >= the full N) and flag_peers[g] points to
 * MNQ_GATHER_FLAG_WORDS 32-bit words on rank g, zero before the first call and never touched by
 * the caller afterwards; all of them must be addressable from this GPU (peer-mapped, e.g. torch
 * symmetric memory or cudaIpc handles).  The kernel stores every output element of this rank's
 * slice into all `world` buffers (after each rank has announced, through the flag words, that it
 * has begun the same call and so no longer reads the previous result), and its last CTA
 * publishes the call's number in every rank's flag block and waits, with a bounded spin, until
 * every rank has done the same here: when the call's work completes on `stream`, the gathered
 * [M, N] output is complete in out_peers[rank].  A rank that never shows up makes the waits give
 * up (bit 2 of mnq_device_status); they never hang the GPU.
 *
 * Rules for the caller: every rank makes the same sequence of calls on a given set of buffers;
 * whatever reads the gathered output is enqueued on `stream` before this rank's next call on it.
 * The call numbers live in the flag blocks, so the calls may be captured in a CUDA graph and
 * replayed.  Only problems the streaming decode kernel takes (M <= 32 among others) are accepted;
 * others return MNQ_NOT_IMPLEMENTED and are gathered with a collective instead. */
#define MNQ_GATHER_FLAG_WORDS 32
MNQ_API int mnq_dequant_matmul_gather(const void* activations, const void* weights_packed, const void* scales,
                                      const void* zeros, void* const* out_peers, uint32_t* const* flag_peers,
                                      int32_t world, int32_t rank, int64_t n_offset, int64_t M,
                                      int64_t N_local, int64_t K, int64_t lda, int64_t ldc, int32_t group_size,
                                      int32_t quant_type, int32_t act_dtype, int32_t scale_dtype, void* workspace,
                                      size_t workspace_bytes, void* stream);

/* Library version, "major.minor.patch". */
MNQ_API const char* mnq_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MNQ_H */
