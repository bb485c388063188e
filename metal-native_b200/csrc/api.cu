// C ABI of libmnq.so (declared in include/mnq.h): argument validation, kernel
// selection and error reporting.  Mirrors the host side of the reference operator,
// src/ops/matmul.mm:903-1029: the same checks in the same order with the same
// messages, followed by the checks the reference leaves out (scales/zeros presence,
// leading dimensions, even K for int4), all before any launch.
#include <cuda.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "mnq_common.cuh"

namespace mnq {

int launch_dequantize_matrix(const void* wq, const void* scales, const void* zeros, void* out,
                             int64_t N, int64_t K, int32_t group_size, int32_t G, int32_t quant,
                             int32_t scale_dtype, int32_t out_dtype, int sm_count, cudaStream_t stream);
int launch_dequantize_flat(const void* in, const void* scales, void* out, int64_t num_elements,
                           int32_t group_size, int32_t quant, int sm_count, cudaStream_t stream);

namespace {
thread_local char g_error[512] = "";
}

int fail(int status, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return status;
}

// ---------------------------------------------------------------------------
// Process-wide options
// ---------------------------------------------------------------------------
namespace {
constexpr int kNumOptions = 4;
std::atomic<int64_t> g_options[kNumOptions] = {{0}, {int64_t(1) << 22}, {0}, {0}};
std::once_flag g_options_env;

bool option_in_range(int option, int64_t v)
{
    switch (option) {
        case MNQ_OPT_WEIGHTS_IMMUTABLE: return v == 0 || v == 1;
        case MNQ_OPT_BF16_FP16_TILES: return v == 0 || v == 1;
        case MNQ_OPT_PEER_WAIT_POLLS: return v >= 1 && v <= (int64_t(1) << 31) - 1;
        case MNQ_OPT_GEMV_MAX_M: return v >= 0 && v <= 32;   // 0: chosen per problem
        default: return false;
    }
}
// The decode / tensor-core threshold may come from the environment, read once; the reference
// advertises its per-phase strategies the same way, as strings (src/inference/phase_pipeline.mm:28-40).
void options_from_env()
{
    const char* e = getenv("METAL_NATIVE_GEMV_MAX_M");
    if (!e || !*e) return;
    char* end = nullptr;
    const long v = strtol(e, &end, 10);
    if (end && *end == 0 && option_in_range(MNQ_OPT_GEMV_MAX_M, v)) g_options[MNQ_OPT_GEMV_MAX_M].store(v);
}
}  // namespace

int64_t option_value(int option)
{
    std::call_once(g_options_env, options_from_env);
    if (option < 0 || option >= kNumOptions) return -1;
    return g_options[option].load(std::memory_order_relaxed);
}

// A kernel's shared-memory attribute has to be set once per device, not once per launch: one bit
// per device ordinal says whether it has been.  (Two threads racing through the first launch both
// set the attribute, which is harmless; the bit is set only after the attribute is.)
bool attribute_done_on_device(const std::atomic<uint64_t>& flags)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    return (flags.load(std::memory_order_acquire) >> dev) & 1u;
}
void mark_attribute_done_on_device(std::atomic<uint64_t>& flags)
{
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) flags.fetch_or(uint64_t(1) << dev, std::memory_order_acq_rel);
}

int check_cuda(cudaError_t e, const char* what)
{
    if (e == cudaSuccess) return MNQ_SUCCESS;
    const int status = (e == cudaErrorMemoryAllocation) ? MNQ_OUT_OF_MEMORY
                     : (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) ? MNQ_DEVICE_NOT_FOUND
                     : MNQ_INTERNAL_ERROR;
    return fail(status, "%s: %s", what, cudaGetErrorString(e));
}

int encode_tensor_map_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                         uint64_t dim0, uint64_t dim1, uint64_t pitch_bytes, uint32_t box0, uint32_t box1,
                         CUtensorMapSwizzle swizzle)
{
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;   // resolved once per process; the pointer never changes
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
            return fail(MNQ_INTERNAL_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    if (reinterpret_cast<uintptr_t>(base) % 16 || pitch_bytes % 16 || (static_cast<uint64_t>(box0) * elem_bytes) % 16)
        return fail(MNQ_INVALID_ARGUMENT, "tensor map: base, pitch and box width must be multiples of 16 bytes");
    // A descriptor is a pure function of these arguments, and a decode step asks for the same few over
    // and over: a small direct-mapped table saves the driver call (about a microsecond) on a hit.
    struct Entry {
        const void* base; uint64_t dim0, dim1, pitch; uint32_t box0, box1; int dtype, elem_bytes, swizzle; bool valid;
        CUtensorMap map;
    };
    static Entry table[64];
    static std::mutex table_lock;
    const uint64_t h = (reinterpret_cast<uintptr_t>(base) >> 8) * 0x9E3779B97F4A7C15ull + dim1 * 31 + box1 * 7 + box0 + swizzle;
    Entry& e = table[(h >> 32) & 63];
    {
        std::lock_guard<std::mutex> g(table_lock);
        if (e.valid && e.base == base && e.dim0 == dim0 && e.dim1 == dim1 && e.pitch == pitch_bytes && e.box0 == box0 &&
            e.box1 == box1 && e.dtype == static_cast<int>(dtype) && e.elem_bytes == elem_bytes && e.swizzle == static_cast<int>(swizzle)) {
            *out = e.map;
            return MNQ_SUCCESS;
        }
    }
    const cuuint64_t dims[2] = {dim0, dim1};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box0, box1};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(out, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MNQ_INTERNAL_ERROR, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    {
        std::lock_guard<std::mutex> g(table_lock);
        e.base = base; e.dim0 = dim0; e.dim1 = dim1; e.pitch = pitch_bytes; e.box0 = box0; e.box1 = box1;
        e.dtype = static_cast<int>(dtype); e.elem_bytes = elem_bytes; e.swizzle = static_cast<int>(swizzle);
        e.map = *out; e.valid = true;
    }
    return MNQ_SUCCESS;
}

namespace {

// SM count of the current device; one attribute query per device per process.
int current_sm_count(int* out)
{
    static int cached[64];
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc) return rc;
    if (dev >= 0 && dev < 64 && cached[dev] > 0) { *out = cached[dev]; return MNQ_SUCCESS; }
    int sms = 0;
    rc = check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev),
                    "cudaDeviceGetAttribute(MultiProcessorCount)");
    if (rc) return rc;
    if (dev >= 0 && dev < 64) cached[dev] = sms;
    *out = sms;
    return MNQ_SUCCESS;
}

// Host-only validation shared by mnq_dequant_matmul_ex and mnq_select_path.
int validate_matmul(const void* x, const void* wq, const void* scales, const void* out, bool need_out,
                    int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldc, int32_t group_size,
                    int32_t quant, int32_t act_dtype, int32_t scale_dtype)
{
    // src/ops/matmul.mm:913-915 (Float16 only there; bf16 is this library's extension)
    if (act_dtype != MNQ_FP16 && act_dtype != MNQ_BF16)
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: activations must be Float16 or BFloat16");
    // src/ops/matmul.mm:916-918 accepts 32, 64, 128; here any multiple of 32, or >= K for one
    // scale per output row
    if (group_size <= 0 || (group_size < K && group_size % 32 != 0))
        return fail(MNQ_INVALID_ARGUMENT,
                    "dequant_matmul: group_size must be a positive multiple of 32 (32, 64, 128, ...) or >= K");
    if (quant != MNQ_INT4 && quant != MNQ_INT8)
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: quant_type must be INT4 or INT8");
    if (scale_dtype != MNQ_FP16 && scale_dtype != MNQ_BF16)
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: scales must be Float16 or BFloat16");
    if (M < 0 || N < 0 || K < 0)
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: negative dimension");
    // src/ops/matmul.mm:926-934 checks weights_packed.shape[1] == K/2; an odd K would make the
    // kernels' (K+1)/2 row stride disagree with that, so it is rejected outright
    if (quant == MNQ_INT4 && (K & 1))
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: INT4 weights must be [N, K/2] (K must be even)");
    if (lda < K) return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: lda must be >= K");
    if (ldc < N) return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: ldc must be >= N");
    if (M > 0 && N > 0) {
        if (K > 0 && (!x || !wq || !scales))
            return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: null activations, weights_packed or scales");
        if (need_out && !out) return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: null output");
    }
    return MNQ_SUCCESS;
}

void fill_args(MatmulArgs& a, const void* x, const void* wq, const void* scales, const void* zeros,
               void* out, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldc, int32_t group_size,
               int32_t quant, int32_t act_dtype, int32_t scale_dtype, void* workspace,
               size_t workspace_bytes, void* stream)
{
    a.x = x; a.wq = wq; a.scales = scales; a.zeros = zeros; a.out = out;
    a.M = M; a.N = N; a.K = K; a.lda = lda; a.ldc = ldc;
    a.group_size = group_size;
    a.G = (K <= 0) ? 0 : static_cast<int32_t>((K + group_size - 1) / group_size);
    a.quant = quant; a.act_dtype = act_dtype; a.scale_dtype = scale_dtype;
    a.workspace = workspace; a.workspace_bytes = workspace ? workspace_bytes : 0;
    a.stream = static_cast<cudaStream_t>(stream);
    a.sm_count = 148;
    a.gather = GatherArgs{};
    a.swiglu_h = 0;
    a.epi = Epilogue{};
}

// Largest token count the decode kernels take.  MNQ_OPT_GEMV_MAX_M when set (1..32); otherwise by
// what was measured on B200.  The decode kernels feed warp MMAs, whose rate (one m16n8k16 per 8
// cycles and SM sub-partition) bounds them from about 16 tokens on; the tensor-core kernel's cost is
// flat up to 128 tokens but it has to expand every weight to 16 bits in shared memory.  int8 weights
// with one scale per row run raw-integer tiles there, which overtake the decode kernels once those need
// three token tiles (17 tokens); for every other format the decode kernels stay ahead up to their limit of 32.
int64_t gemv_max_m_for(int64_t K, int32_t group_size, int32_t quant, int32_t act_dtype)
{
    (void)act_dtype;
    const int64_t set = option_value(MNQ_OPT_GEMV_MAX_M);
    if (set > 0) return set;
    if (quant == MNQ_INT8 && group_size >= K) return 16;
    return 32;
}

// Decode kernels up to the threshold, the tensor-core kernel above it, the any-shape kernel for
// whatever neither takes.
int choose_path(const MatmulArgs& a)
{
    int64_t gemv_max_m = gemv_max_m_for(a.K, a.group_size, a.quant, a.act_dtype);
    // small layers of few rows: the tensor-core kernel from 17 tokens (not where it needs two bf16 tiles per k-block)
    if (option_value(MNQ_OPT_GEMV_MAX_M) == 0 && gemv_max_m > 16 && few_rows_small_layer(a) &&
        !(a.act_dtype == MNQ_BF16 && (a.group_size < a.K || a.zeros != nullptr)))
        gemv_max_m = 16;
    if (a.M <= gemv_max_m && gemv_supported(a)) return MNQ_PATH_GEMV;
    // 33 to 64 tokens of bf16 activations where the tensor-core kernel would need two bf16 tiles per
    // k-block (group-wise scales, the caller has not opted for fp16 tiles): the batched-decode
    // kernel with six or eight token tiles is faster (measured: 31-50 against 70 us on the Llama-3-8B
    // shapes).  Only while the threshold is left to the library.
    if (a.M > 32 && a.M <= 64 && a.act_dtype == MNQ_BF16 && option_value(MNQ_OPT_GEMV_MAX_M) == 0 &&
        option_value(MNQ_OPT_BF16_FP16_TILES) == 0 && a.group_size < a.K && gemv_supported(a))
        return MNQ_PATH_GEMV;
    if (a.M > gemv_max_m && gemm_supported(a)) return MNQ_PATH_GEMM;
    if (a.M <= 32 && gemv_supported(a)) return MNQ_PATH_GEMV;   // e.g. K not a multiple of 64
    return MNQ_PATH_GENERIC;
}

template <typename T>
__global__ void zero_rows_kernel(void* out, int64_t M, int64_t N, int64_t ldc, const Epilogue epi)
{
    const int64_t total = M * N;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x)
        store_result<T>(epi, out, ldc, static_cast<int>(i / N), static_cast<int>(i % N), 0.f);
}

}  // namespace
}  // namespace mnq

using namespace mnq;

extern "C" {

const char* mnq_status_name(int status)
{
    switch (status) {
        case MNQ_SUCCESS: return "Success";
        case MNQ_DEVICE_NOT_FOUND: return "DeviceNotFound";
        case MNQ_ALLOCATION_FAILED: return "AllocationFailed";
        case MNQ_KERNEL_COMPILATION_FAILED: return "KernelCompilationFailed";
        case MNQ_INVALID_ARGUMENT: return "InvalidArgument";
        case MNQ_OUT_OF_MEMORY: return "OutOfMemory";
        case MNQ_TIMEOUT_ERROR: return "TimeoutError";
        case MNQ_INTERNAL_ERROR: return "InternalError";
        case MNQ_NOT_IMPLEMENTED: return "NotImplemented";
        default: return "Unknown";
    }
}

const char* mnq_last_error(void) { return g_error; }

const char* mnq_version(void) { return "0.1.0"; }

int mnq_device_status(uint32_t* status, int32_t clear)
{
    if (!status) return fail(MNQ_INVALID_ARGUMENT, "device_status: null status pointer");
    unsigned int v = 0;
    const int rc = read_device_status(&v, clear != 0);
    if (rc) return rc;
    *status = v;
    return MNQ_SUCCESS;
}

size_t mnq_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size, int32_t quant_type)
{
    if (M > 32) {   // (33 to 64 tokens of bf16 activations may take the batched-decode kernel: enough for both)
        const size_t g = gemm_workspace_bytes(M, N, K, group_size, quant_type);
        const size_t d = M <= 64 ? gemv_workspace_bytes(M, N, K, group_size, quant_type) : 0;
        return g > d ? g : d;
    }
    // 9..32 tokens take either family, depending on MNQ_OPT_GEMV_MAX_M and the dtypes: enough for both
    const size_t a = gemv_workspace_bytes(M, N, K, group_size, quant_type);
    const size_t b = M > 8 ? gemm_workspace_bytes(M, N, K, group_size, quant_type) : 0;
    return a > b ? a : b;
}

int mnq_set_option(int32_t option, int64_t value)
{
    option_value(option);   // the environment is read before the first explicit setting
    if (option < 0 || option >= kNumOptions) return fail(MNQ_INVALID_ARGUMENT, "set_option: unknown option %d", option);
    if (!option_in_range(option, value))
        return fail(MNQ_INVALID_ARGUMENT, "set_option: value %lld is out of range for option %d", (long long)value, option);
    g_options[option].store(value);
    return MNQ_SUCCESS;
}

int64_t mnq_get_option(int32_t option) { return option_value(option); }

int mnq_select_path_ex(int64_t M, int64_t N, int64_t K, int64_t lda, int32_t group_size, int32_t quant_type,
                       int32_t act_dtype, int32_t scale_dtype, const void* activations, const void* weights_packed,
                       const void* scales, const void* zeros)
{
    const int rc = validate_matmul(activations, weights_packed, scales, nullptr, false, M, N, K, lda, N,
                                   group_size, quant_type, act_dtype, scale_dtype);
    if (rc) return -rc;
    MatmulArgs a;
    fill_args(a, activations, weights_packed, scales, zeros, nullptr, M, N, K, lda, N, group_size,
              quant_type, act_dtype, scale_dtype, nullptr, 0, nullptr);
    // the answer must not depend on how much workspace a later call brings
    a.workspace = reinterpret_cast<void*>(uintptr_t(256));
    a.workspace_bytes = mnq_workspace_bytes(M, N, K, group_size, quant_type);
    return choose_path(a);
}

int mnq_select_path(int64_t M, int64_t N, int64_t K, int64_t lda, int32_t group_size, int32_t quant_type,
                    int32_t act_dtype, const void* activations, const void* weights_packed,
                    const void* scales, const void* zeros)
{
    return mnq_select_path_ex(M, N, K, lda, group_size, quant_type, act_dtype, MNQ_FP16, activations, weights_packed,
                              scales, zeros);
}

static int run_matmul(const void* activations, const void* weights_packed, const void* scales,
                      const void* zeros, void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                      int64_t ldc, int32_t group_size, int32_t quant_type, int32_t act_dtype,
                      int32_t scale_dtype, void* workspace, size_t workspace_bytes, void* stream,
                      const mnq_tuning* tuning, const Epilogue& epi)
{
    int rc = validate_matmul(activations, weights_packed, scales, out, true, M, N, K, lda, ldc, group_size,
                             quant_type, act_dtype, scale_dtype);
    if (rc) return rc;
    if (M == 0 || N == 0) return MNQ_SUCCESS;  // empty output: nothing to launch

    MatmulArgs a;
    fill_args(a, activations, weights_packed, scales, zeros, out, M, N, K, lda, ldc, group_size, quant_type,
              act_dtype, scale_dtype, workspace, workspace_bytes, stream);
    a.epi = epi;
    rc = current_sm_count(&a.sm_count);
    if (rc) return rc;

    if (K == 0) {  // empty reduction: the sum over no terms, then the epilogue
        const int64_t total = M * N;
        const int grid = static_cast<int>(total / 256 + 1 > 1024 ? 1024 : total / 256 + 1);
        if (act_dtype == MNQ_FP16)
            zero_rows_kernel<__half><<<grid, 256, 0, a.stream>>>(out, M, N, ldc, epi);
        else
            zero_rows_kernel<__nv_bfloat16><<<grid, 256, 0, a.stream>>>(out, M, N, ldc, epi);
        return check_cuda(cudaGetLastError(), "zero-fill launch");
    }

    int path = (tuning && tuning->path != MNQ_PATH_AUTO) ? tuning->path : choose_path(a);
    switch (path) {
        case MNQ_PATH_GEMV: return launch_gemv(a, tuning);
        case MNQ_PATH_GEMM: return launch_gemm(a, tuning);
        case MNQ_PATH_GENERIC: return launch_generic(a);
        default: return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: unknown path %d", path);
    }
}

int mnq_dequant_matmul_ex(const void* activations, const void* weights_packed, const void* scales,
                          const void* zeros, void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                          int64_t ldc, int32_t group_size, int32_t quant_type, int32_t act_dtype,
                          int32_t scale_dtype, void* workspace, size_t workspace_bytes, void* stream,
                          const mnq_tuning* tuning)
{
    return run_matmul(activations, weights_packed, scales, zeros, out, M, N, K, lda, ldc, group_size, quant_type,
                      act_dtype, scale_dtype, workspace, workspace_bytes, stream, tuning, Epilogue{});
}

int mnq_dequant_matmul_fused(const void* activations, const void* weights_packed, const void* scales,
                             const void* zeros, void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                             int64_t ldc, int32_t group_size, int32_t quant_type, int32_t act_dtype,
                             int32_t scale_dtype, int32_t out_dtype, int32_t epilogue, const void* bias,
                             const void* residual, int64_t ldr, void* workspace, size_t workspace_bytes,
                             void* stream)
{
    // include/metal_native/ops/fused_matmul.h:51-52: a required epilogue tensor that is missing is InvalidArgument
    if (epilogue < MNQ_EPI_NONE || epilogue > MNQ_EPI_RESIDUAL)
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_fused: unknown epilogue %d", epilogue);
    const bool needs_bias = epilogue == MNQ_EPI_BIAS || epilogue == MNQ_EPI_BIAS_RELU || epilogue == MNQ_EPI_BIAS_SILU;
    if (needs_bias && !bias && N > 0)
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_fused: this epilogue requires a bias tensor [N]");
    if (epilogue == MNQ_EPI_RESIDUAL) {
        if (!residual && M > 0 && N > 0)
            return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_fused: ResidualAdd requires a residual tensor [M, N]");
        if (ldr < N) return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_fused: ldr must be >= N");
    }
    if (out_dtype != act_dtype && out_dtype != MNQ_FP32)
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_fused: out_dtype must be the activation dtype or Float32");
    Epilogue epi{};
    epi.kind = epilogue;
    epi.out_f32 = out_dtype == MNQ_FP32 ? 1 : 0;
    epi.bias = needs_bias ? bias : nullptr;
    epi.residual = epilogue == MNQ_EPI_RESIDUAL ? residual : nullptr;
    epi.ldr = ldr;
    return run_matmul(activations, weights_packed, scales, zeros, out, M, N, K, lda, ldc, group_size, quant_type,
                      act_dtype, scale_dtype, workspace, workspace_bytes, stream, nullptr, epi);
}

int mnq_dequant_matmul_gather(const void* activations, const void* weights_packed, const void* scales,
                              const void* zeros, void* const* out_peers, uint32_t* const* flag_peers,
                              int32_t world, int32_t rank, int64_t n_offset, int64_t M,
                              int64_t N_local, int64_t K, int64_t lda, int64_t ldc, int32_t group_size,
                              int32_t quant_type, int32_t act_dtype, int32_t scale_dtype, void* workspace,
                              size_t workspace_bytes, void* stream)
{
    if (world < 1 || world > kMaxGatherRanks || rank < 0 || rank >= world)
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_gather: world must be 1..%d and 0 <= rank < world", kMaxGatherRanks);
    if (!out_peers || !flag_peers) return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_gather: null pointer table");
    for (int g = 0; g < world; ++g)
        if (!out_peers[g] || !flag_peers[g])
            return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_gather: null buffer for rank %d", g);
    if (n_offset < 0 || n_offset + N_local > ldc)
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_gather: columns [n_offset, n_offset + N_local) must lie inside ldc");
    int rc = validate_matmul(activations, weights_packed, scales, out_peers[rank], true, M, N_local, K, lda, N_local,
                             group_size, quant_type, act_dtype, scale_dtype);
    if (rc) return rc;
    if (M == 0 || N_local == 0 || K == 0)
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_gather: empty problems are not gathered (every rank must launch)");

    MatmulArgs a;
    fill_args(a, activations, weights_packed, scales, zeros, out_peers[rank], M, N_local, K, lda, ldc, group_size,
              quant_type, act_dtype, scale_dtype, workspace, workspace_bytes, stream);
    rc = current_sm_count(&a.sm_count);
    if (rc) return rc;
    a.gather.world = world;
    a.gather.rank = rank;
    a.gather.n_offset = n_offset;
    for (int g = 0; g < world; ++g) {
        a.gather.out_peer[g] = out_peers[g];
        a.gather.flag_peer[g] = flag_peers[g];
    }
    // the peer stores live in the streaming decode kernel's epilogue
    if (M > 32 || !gemv_stream_supported(a, nullptr))
        return fail(MNQ_NOT_IMPLEMENTED,
                    "dequant_matmul_gather: only problems the streaming decode kernel takes (M <= 32, rows a multiple "
                    "of 16 bytes, group_size a multiple of the k step); gather other shapes with a collective");
    return launch_gemv_stream(a, nullptr);
}

int mnq_dequant_matmul_swiglu(const void* activations, const void* weights_packed, const void* scales,
                              const void* zeros, void* out, int64_t M, int64_t H, int64_t K, int64_t lda,
                              int64_t ldc, int32_t group_size, int32_t quant_type, int32_t act_dtype,
                              int32_t scale_dtype, void* stream)
{
    if (H < 0) return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_swiglu: negative dimension");
    // the weights are the fused [2H, K] matrix; validate it as such, with an output of H columns
    int rc = validate_matmul(activations, weights_packed, scales, out, true, M, 2 * H, K, lda, 2 * H, group_size,
                             quant_type, act_dtype, scale_dtype);
    if (rc) return rc;
    if (ldc < H) return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_swiglu: ldc must be >= H");
    if (M == 0 || H == 0) return MNQ_SUCCESS;
    if (K == 0) return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_swiglu: K must be positive");
    MatmulArgs a;
    fill_args(a, activations, weights_packed, scales, zeros, out, M, 2 * H, K, lda, ldc, group_size, quant_type,
              act_dtype, scale_dtype, nullptr, 0, stream);
    rc = current_sm_count(&a.sm_count);
    if (rc) return rc;
    a.swiglu_h = H;
    if (M > 32 || !gemv_stream_supported(a, nullptr))
        return fail(MNQ_NOT_IMPLEMENTED,
                    "dequant_matmul_swiglu: only problems the streaming decode kernel takes without splitting K "
                    "(M <= 32, rows a multiple of 16 bytes, the activation block fits shared memory); "
                    "use dequant_matmul and apply the activation separately");
    return launch_gemv_stream(a, nullptr);
}

static size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

// Device address of a host buffer if it is pinned and mapped into this device's address space
// (cudaHostAlloc / cudaHostRegister memory, torch's pinned tensors), else null.  The answer for a pointer
// is remembered per thread: the query costs about a microsecond.
static void* device_pointer_of_pinned(const void* host)
{
    struct Seen { const void* host; void* dev; int device; };
    static thread_local Seen seen[8];
    static thread_local int next = 0;
    int device = 0;
    if (!host || cudaGetDevice(&device) != cudaSuccess) return nullptr;
    for (const Seen& s : seen)
        if (s.host == host && s.device == device) return s.dev;
    cudaPointerAttributes attr{};
    void* dev = nullptr;
    if (cudaPointerGetAttributes(&attr, host) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer)
        dev = attr.devicePointer;
    else
        cudaGetLastError();   // an unregistered pointer is not an error here
    seen[next] = Seen{host, dev, device};
    next = (next + 1) & 7;
    return dev;
}

// Copies a small activation block out of pinned, device-mapped host memory.  A kernel instead of a
// copy operation: the operator's kernel, launched programmatically dependent behind it, starts its
// set-up (and, with immutable weights, its weight stream) while this one is still fetching over the bus.
__global__ void __launch_bounds__(256) stage_activations_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n16)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = src[i];
}

// Operator scratch at the front of a host-call workspace.  Never shorter than the counter region:
// a workspace is shared by successive calls of any kind, and the device copies of activations and
// output that follow the scratch must not land where a later split-K call expects zeroed counters.
static size_t host_scratch_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size, int32_t quant_type)
{
    const size_t need = align256(mnq_workspace_bytes(M, N, K, group_size, quant_type));
    return need > mnq::kCounterBytes ? need : mnq::kCounterBytes;
}

size_t mnq_host_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size, int32_t quant_type)
{
    if (M <= 0 || N <= 0 || K < 0) return 0;
    return host_scratch_bytes(M, N, K, group_size, quant_type) + align256(static_cast<size_t>(M) * K * 2) +
           align256(static_cast<size_t>(M) * N * 2);
}

int mnq_dequant_matmul_host(const void* activations_host, const void* weights_packed, const void* scales,
                            const void* zeros, void* out_host, int64_t M, int64_t N, int64_t K,
                            int32_t group_size, int32_t quant_type, int32_t act_dtype, int32_t scale_dtype,
                            void* workspace, size_t workspace_bytes, void* stream)
{
    int rc = validate_matmul(activations_host, weights_packed, scales, out_host, true, M, N, K, K, N, group_size,
                             quant_type, act_dtype, scale_dtype);
    if (rc) return rc;
    if (M == 0 || N == 0) return MNQ_SUCCESS;
    const size_t need = mnq_host_workspace_bytes(M, N, K, group_size, quant_type);
    if (!workspace || workspace_bytes < need)
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_host: workspace of %zu bytes needed (mnq_host_workspace_bytes), got %zu",
                    need, workspace ? workspace_bytes : static_cast<size_t>(0));
    // workspace: [operator scratch][activations][output]
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    const size_t scratch = host_scratch_bytes(M, N, K, group_size, quant_type);
    const size_t op_scratch = mnq_workspace_bytes(M, N, K, group_size, quant_type);
    unsigned char* x_dev = ws + scratch;
    unsigned char* out_dev = x_dev + align256(static_cast<size_t>(M) * K * 2);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // (The activations are staged in device memory even when they sit in pinned, device-mapped memory:
    // every CTA reads its K range of them, and three hundred reads over the bus cost far more than one.)
    if (K > 0) {
        const size_t x_bytes = static_cast<size_t>(M) * K * 2;
        const void* x_mapped = (M <= 32 && x_bytes % 16 == 0) ? device_pointer_of_pinned(activations_host) : nullptr;
        if (x_mapped && reinterpret_cast<uintptr_t>(x_mapped) % 16 == 0) {
            const size_t n16 = x_bytes / 16;
            const unsigned blocks = static_cast<unsigned>(n16 / 256 + 1 > 16 ? 16 : n16 / 256 + 1);
            stage_activations_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint4*>(x_mapped), reinterpret_cast<uint4*>(x_dev), n16);
            rc = check_cuda(cudaGetLastError(), "activation staging launch");
        } else {
            rc = check_cuda(cudaMemcpyAsync(x_dev, activations_host, x_bytes, cudaMemcpyHostToDevice, st),
                            "cudaMemcpyAsync(activations to device)");
        }
        if (rc) return rc;
    }
    // A decode-sized result goes straight from the kernel's epilogue into pinned, device-mapped host
    // memory (every output is written once, as posted writes): the copy back and its launch are saved.
    void* out_mapped = (M <= 32) ? device_pointer_of_pinned(out_host) : nullptr;
    rc = mnq_dequant_matmul(x_dev, weights_packed, scales, zeros, out_mapped ? out_mapped : out_dev, M, N, K, K, N, group_size,
                            quant_type, act_dtype, scale_dtype, op_scratch ? ws : nullptr, op_scratch ? scratch : 0, stream);
    if (rc || out_mapped) return rc;
    return check_cuda(cudaMemcpyAsync(out_host, out_dev, static_cast<size_t>(M) * N * 2, cudaMemcpyDeviceToHost, st),
                      "cudaMemcpyAsync(output to host)");
}

int mnq_dequant_matmul(const void* activations, const void* weights_packed, const void* scales,
                       const void* zeros, void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                       int64_t ldc, int32_t group_size, int32_t quant_type, int32_t act_dtype,
                       int32_t scale_dtype, void* workspace, size_t workspace_bytes, void* stream)
{
    return mnq_dequant_matmul_ex(activations, weights_packed, scales, zeros, out, M, N, K, lda, ldc,
                                 group_size, quant_type, act_dtype, scale_dtype, workspace,
                                 workspace_bytes, stream, nullptr);
}

int mnq_dequantize(const void* weights_packed, const void* scales, const void* zeros, void* out, int64_t N,
                   int64_t K, int32_t group_size, int32_t quant_type, int32_t scale_dtype,
                   int32_t out_dtype, void* stream)
{
    if (quant_type != MNQ_INT4 && quant_type != MNQ_INT8)
        return fail(MNQ_INVALID_ARGUMENT, "dequantize: quant_type must be INT4 or INT8");
    if (scale_dtype != MNQ_FP16 && scale_dtype != MNQ_BF16)
        return fail(MNQ_INVALID_ARGUMENT, "dequantize: scales must be Float16 or BFloat16");
    if (out_dtype != MNQ_FP16 && out_dtype != MNQ_BF16 && out_dtype != MNQ_FP32)
        return fail(MNQ_INVALID_ARGUMENT, "dequantize: output must be Float32, Float16 or BFloat16");
    if (N < 0 || K < 0 || group_size <= 0)
        return fail(MNQ_INVALID_ARGUMENT, "dequantize: bad dimensions or group_size");
    if (N == 0 || K == 0) return MNQ_SUCCESS;
    if (!weights_packed || !scales || !out)
        return fail(MNQ_INVALID_ARGUMENT, "dequantize: null weights_packed, scales or output");
    int sms = 148;
    const int rc = current_sm_count(&sms);
    if (rc) return rc;
    const int32_t G = static_cast<int32_t>((K + group_size - 1) / group_size);
    return launch_dequantize_matrix(weights_packed, scales, zeros, out, N, K, group_size, G, quant_type,
                                    scale_dtype, out_dtype, sms, static_cast<cudaStream_t>(stream));
}

int mnq_dequantize_flat(const void* input, const void* scales_fp16, void* out_fp16, int64_t num_elements,
                        int32_t group_size, int32_t quant_type, void* stream)
{
    if (quant_type != MNQ_INT4 && quant_type != MNQ_INT8)
        return fail(MNQ_INVALID_ARGUMENT, "dequantize_flat: quant_type must be INT4 or INT8");
    if (num_elements < 0 || group_size <= 0)
        return fail(MNQ_INVALID_ARGUMENT, "dequantize_flat: bad num_elements or group_size");
    if (num_elements == 0) return MNQ_SUCCESS;
    if (!input || !scales_fp16 || !out_fp16)
        return fail(MNQ_INVALID_ARGUMENT, "dequantize_flat: null input, scales or output");
    int sms = 148;
    const int rc = current_sm_count(&sms);
    if (rc) return rc;
    return launch_dequantize_flat(input, scales_fp16, out_fp16, num_elements, group_size, quant_type, sms,
                                  static_cast<cudaStream_t>(stream));
}

}  // extern "C"
