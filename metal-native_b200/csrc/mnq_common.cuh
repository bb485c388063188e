// Shared device helpers: dtype traits, cache-hinted loads, exact integer -> fp16/bf16
// unpacking of packed INT4 / INT8 weights, warp-level mma wrappers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/mnq.h"

namespace mnq {

// ---------------------------------------------------------------------------
// Host-side error plumbing (defined in api.cu)
// ---------------------------------------------------------------------------
int fail(int status, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);
bool attribute_done_on_device(const std::atomic<uint64_t>& flags);
void mark_attribute_done_on_device(std::atomic<uint64_t>& flags);

// ---------------------------------------------------------------------------
// 16-bit float traits
// ---------------------------------------------------------------------------
template <typename T> struct F16Traits;

template <> struct F16Traits<__half> {
    using T2 = __half2;
    static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
};
template <> struct F16Traits<__nv_bfloat16> {
    using T2 = __nv_bfloat162;
    static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};

// scales / zeros arrive as fp16 or bf16 bits; widening to fp32 is exact.
__device__ __forceinline__ float widen16(const void* base, size_t idx, int dtype)
{
    const uint16_t bits = __ldg(reinterpret_cast<const uint16_t*>(base) + idx);
    if (dtype == MNQ_BF16) return __uint_as_float(static_cast<uint32_t>(bits) << 16);
    return __half2float(__ushort_as_half(bits));
}

// ---------------------------------------------------------------------------
// Loads
// ---------------------------------------------------------------------------
// Weights are read exactly once: keep them out of L1 so the activations and scales
// staged through L1/shared memory are not evicted.
__device__ __forceinline__ uint4 ldg_stream_16(const void* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream_8(const void* p)
{
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream_4(const void* p)
{
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// ---------------------------------------------------------------------------
// Bit tricks
// ---------------------------------------------------------------------------
template <int LUT>
__device__ __forceinline__ uint32_t lop3(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(r) : "r"(a), "r"(b), "r"(c), "n"(LUT));
    return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
__device__ __forceinline__ uint32_t b2_as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __nv_bfloat162 u32_as_b2(uint32_t v) { return *reinterpret_cast<__nv_bfloat162*>(&v); }

// ---------------------------------------------------------------------------
// INT4: one 32-bit word = 8 nibbles n0..n7 (element k in nibble k).
// Produces (q - 8) as exact 16-bit floats, paired (n0,n4) (n1,n5) (n2,n6) (n3,n7):
// the pairing that costs no shifts for the even nibbles.  The activations are
// staged in the same order, so the pairing never has to be undone.
// ---------------------------------------------------------------------------
template <typename T> struct UnpackInt4;

template <> struct UnpackInt4<__half> {
    // 0x6400 = 1024.0h: OR-ing a nibble into the low mantissa bits gives 1024 + n
    // exactly; OR-ing it 4 bits higher gives 1024 + 16 n.
    static __device__ __forceinline__ void run(uint32_t w, uint32_t (&out)[4])
    {
        constexpr uint32_t LO = 0x000F000Fu, HI = 0x00F000F0u, MAGIC = 0x64006400u;
        const uint32_t w8 = w >> 8;
        const __half2 lo0 = u32_as_h2(lop3<0xEA>(w, LO, MAGIC));
        const __half2 hi0 = u32_as_h2(lop3<0xEA>(w, HI, MAGIC));
        const __half2 lo1 = u32_as_h2(lop3<0xEA>(w8, LO, MAGIC));
        const __half2 hi1 = u32_as_h2(lop3<0xEA>(w8, HI, MAGIC));
        const __half2 c1032 = __half2half2(__ushort_as_half(0x6408));  // 1032
        const __half2 sixteenth = __half2half2(__ushort_as_half(0x2C00));  // 1/16
        const __half2 m72 = __half2half2(__ushort_as_half(0xD480));  // -72
        out[0] = h2_as_u32(__hsub2(lo0, c1032));           // (n0-8, n4-8)
        out[1] = h2_as_u32(__hfma2(hi0, sixteenth, m72));  // (n1-8, n5-8): 64 + n - 72
        out[2] = h2_as_u32(__hsub2(lo1, c1032));           // (n2-8, n6-8)
        out[3] = h2_as_u32(__hfma2(hi1, sixteenth, m72));  // (n3-8, n7-8)
    }
};

template <> struct UnpackInt4<__nv_bfloat16> {
    // 0x4300 = 128.0bf16 (7 mantissa bits): 128 + n is exact for n < 128.
    static __device__ __forceinline__ void run(uint32_t w, uint32_t (&out)[4])
    {
        constexpr uint32_t LO = 0x000F000Fu, MAGIC = 0x43004300u;
        const __nv_bfloat162 c136 = __bfloat162bfloat162(__ushort_as_bfloat16(0x4308));  // 136
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 v = u32_as_b2(lop3<0xEA>(w >> (4 * i), LO, MAGIC));
            out[i] = b2_as_u32(__hsub2(v, c136));
        }
    }
};

// ---------------------------------------------------------------------------
// INT8: one 32-bit word = 4 signed bytes b0..b3.  Produces q as exact 16-bit
// floats, paired (b0,b1) (b2,b3).
// ---------------------------------------------------------------------------
template <typename T> struct UnpackInt8;

template <> struct UnpackInt8<__half> {
    static __device__ __forceinline__ void run(uint32_t w, uint32_t (&out)[2])
    {
        const uint32_t u = w ^ 0x80808080u;  // b + 128 in 0..255
        const __half2 c1152 = __half2half2(__ushort_as_half(0x6480));  // 1024 + 128
        out[0] = h2_as_u32(__hsub2(u32_as_h2(prmt(u, 0x64646464u, 0x4140u)), c1152));
        out[1] = h2_as_u32(__hsub2(u32_as_h2(prmt(u, 0x64646464u, 0x4342u)), c1152));
    }
};

template <> struct UnpackInt8<__nv_bfloat16> {
    // bf16 has 8 significant bits: 128 + (0..127) is exact, 128 + (128..255) is not.  So a byte b
    // becomes v = 0x4300 | (b & 0x7F) = 128 + (b mod 128) and c = 0x4300 | (b & 0x80), which is
    // 128.0 for b >= 0 and 256.0 (0x4380) for b < 0; v - c = b exactly in both cases.
    static __device__ __forceinline__ void run(uint32_t w, uint32_t (&out)[2])
    {
        const uint32_t lo7 = w & 0x7F7F7F7Fu, sgn = w & 0x80808080u;
        const uint32_t v01 = prmt(lo7, 0x43434343u, 0x5140u), v23 = prmt(lo7, 0x43434343u, 0x7362u);
        const uint32_t c01 = prmt(sgn, 0x43434343u, 0x5140u), c23 = prmt(sgn, 0x43434343u, 0x7362u);
        out[0] = b2_as_u32(__hsub2(u32_as_b2(v01), u32_as_b2(c01)));
        out[1] = b2_as_u32(__hsub2(u32_as_b2(v23), u32_as_b2(c23)));
    }
};

// ---------------------------------------------------------------------------
// Warp-level tensor-core step used by the decode path: D[16x8] += A[16x16] B[16x8],
// fp32 accumulate.  A = 16 weight rows, B = up to 8 activation rows (tokens).
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void mma_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1);

template <>
__device__ __forceinline__ void mma_16x8x16<__half>(float (&d)[4], uint32_t a0, uint32_t a1,
                                                    uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16x8x16<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1,
                                                           uint32_t a2, uint32_t a3, uint32_t b0,
                                                           uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------------------
// What happens to an fp32 result between the accumulator and memory: the reference's
// MatmulEpilogue (include/metal_native/ops/fused_matmul.h:18-24) as applied by its
// apply_epilogue (shaders/matmul_fused_epilogue.metal:97-124: fp32 arithmetic on the accumulated
// value, bias [N] broadcast over rows, residual [M, N], one rounding at the store), plus an fp32
// output mode that stores the value unrounded.
// ---------------------------------------------------------------------------
struct Epilogue {
    int32_t kind;          // mnq_epilogue
    int32_t out_f32;       // 1: out is float [M, ldc]
    const void* bias;      // [N] in the activation dtype (kinds BIAS, BIAS_RELU, BIAS_SILU)
    const void* residual;  // [M, ldr] in the activation dtype (kind RESIDUAL)
    long long ldr;
};

template <typename T>
__device__ __forceinline__ float epilogue_value(const Epilogue& e, float v, int m, int n)
{
    if (e.kind == MNQ_EPI_NONE) return v;
    if (e.kind == MNQ_EPI_RESIDUAL)
        return v + F16Traits<T>::to_float(static_cast<const T*>(e.residual)[(size_t)m * e.ldr + n]);
    v += F16Traits<T>::to_float(static_cast<const T*>(e.bias)[n]);
    if (e.kind == MNQ_EPI_BIAS_RELU) return fmaxf(0.f, v);
    if (e.kind == MNQ_EPI_BIAS_SILU) return v / (1.f + expf(-v));
    return v;
}

// out[m, n] = epilogue(v), rounded to T unless the fp32 output mode is on
template <typename T>
__device__ __forceinline__ void store_result(const Epilogue& e, void* out, long long ldc, int m, int n, float v)
{
    v = epilogue_value<T>(e, v, m, n);
    if (e.out_f32) static_cast<float*>(out)[(size_t)m * ldc + n] = v;
    else static_cast<T*>(out)[(size_t)m * ldc + n] = F16Traits<T>::from_float(v);
}

// ---------------------------------------------------------------------------
// Launch-argument bundles
// ---------------------------------------------------------------------------
// Column-sharded call: this rank's [M, N] result is stored into the gathered [M, ldc] buffer of
// every rank at column n_offset, through peer-mapped pointers, and the kernel returns only when
// every rank's slice has arrived in this rank's buffer.  Each rank owns a block of
// kGatherFlagWords 32-bit words, zero before the first call, written by its peers:
//   [0, 8)   arrival: word s = number of the last call whose slice from rank s is complete here
//   [8]      CTA counter of the running call (local use)      [9] number of completed calls (local)
//   [16, 24) ready: word s = number of the call rank s has begun, i.e. rank s no longer reads
//            the previous call's gathered output and its buffer may be overwritten
constexpr int kMaxGatherRanks = 8;
constexpr int kGatherFlagWords = 32;
constexpr int kGatherCounterWord = 8;
constexpr int kGatherEpochWord = 9;
constexpr int kGatherReadyBase = 16;
struct GatherArgs {
    int32_t world;                         // 0: plain call
    int32_t rank;
    int64_t n_offset;
    void* out_peer[kMaxGatherRanks];       // gathered output buffer of each rank
    uint32_t* flag_peer[kMaxGatherRanks];  // kGatherFlagWords words on each rank
};

struct MatmulArgs {
    const void* x;        // [M, K] act dtype
    const void* wq;       // packed weights
    const void* scales;   // [N, G]
    const void* zeros;    // [N, G] or null
    void* out;            // [M, N] act dtype
    int64_t M, N, K, lda, ldc;
    int32_t group_size;   // clamped to >= 1; >= K means one group per row
    int32_t G;            // groups per row = ceil(K / group_size)
    int32_t quant;        // mnq_quant
    int32_t act_dtype;    // mnq_dtype
    int32_t scale_dtype;  // mnq_dtype
    void* workspace;
    size_t workspace_bytes;
    cudaStream_t stream;
    int32_t sm_count;
    GatherArgs gather;    // world == 0 unless called through mnq_dequant_matmul_gather
    int64_t swiglu_h;     // > 0: weights are [2H, K] (gate rows, then up rows) and out is [M, H] = silu(gate) * up
    Epilogue epi;         // kind NONE and out_f32 0 unless called through mnq_dequant_matmul_fused
};

// Few rows and little data.  The batched-decode path costs two launches more than the other decode kernels
// (activation image, K-cut reduction), about 4 us, which layers like a 4096 x 4096 projection do not earn
// back: measured on B200, the compact and general streaming kernels are ahead there up to 16 tokens
// (8.6-10.2 against 12.9-16.6 us for 8 MB of int4) and the tensor-core kernel above (13.8 against 16.6-23 us).
inline int64_t packed_weight_bytes(const MatmulArgs& a) { return a.N * (a.quant == MNQ_INT4 ? a.K / 2 : a.K); }
inline bool few_rows_small_layer(const MatmulArgs& a) { return a.N < 8192 && packed_weight_bytes(a) < (int64_t(24) << 20); }

// Process-wide options (mnq_set_option); defined in api.cu.
int64_t option_value(int option);

// Split-K workspace layout, the same for every kernel and every problem shape: arrival
// counters (always left at zero by the kernel that used them) in the first kCounterBytes,
// fp32 partial sums (left dirty) after them.  Keeping the counter region fixed means a
// later call with another shape never finds stale partial sums where it expects zeroed
// counters.
constexpr size_t kCounterBytes = 64 * 1024;
constexpr int64_t kMaxCounters = kCounterBytes / 4;

// Launchers (each returns an mnq_status)
#ifdef CUDA_VERSION  // <cuda.h> included by the translation unit
// Encodes a 2-D tiled TMA descriptor through the driver entry point obtained at run time
// (no link-time dependency on libcuda).  dim0 is the contiguous dimension; sizes in
// elements, the row pitch in bytes (a multiple of 16), the base 16-byte aligned.
int encode_tensor_map_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                         uint64_t dim0, uint64_t dim1, uint64_t pitch_bytes, uint32_t box0, uint32_t box1,
                         CUtensorMapSwizzle swizzle);
#endif
// The streaming plan's figures the compact decode kernel (gemv_lean.cu) needs.
// Activations (tokens x chunk length) a CTA of 8 warps of that kernel stages: 8 blocks of 8 per thread.
constexpr int64_t kLeanMaxStaged = 8 * 256 * 8;
struct LeanShape {
    int warps, num_chunks, steps_per_chunk, total_steps, stages;
    int resident_ctas;   // CTAs the plan expects to be resident on the GPU at once
};
bool gemv_lean_supported(const MatmulArgs& a, const LeanShape& s);
#ifdef CUDA_VERSION
int launch_gemv_lean(const MatmulArgs& a, const LeanShape& s, const CUtensorMap& wmap);
#endif
int read_lean_status(unsigned int* out, bool clear);
// Batched decode, 9 to 32 tokens (gemv_mid.cu): activations prepared once per call in the workspace.
bool gemv_mid_supported(const MatmulArgs& a, const mnq_tuning* tuning);
size_t gemv_mid_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size, int32_t quant);
#ifdef CUDA_VERSION
int launch_gemv_mid(const MatmulArgs& a, const mnq_tuning* tuning, const CUtensorMap& wmap);
#endif
int launch_gemv_mid_wide(const MatmulArgs& a, const mnq_tuning* tuning);   // 33 to 64 tokens, bf16 activations
int read_mid_status(unsigned int* out, bool clear);
int launch_generic(const MatmulArgs& a);
bool gemv_supported(const MatmulArgs& a);
int launch_gemv(const MatmulArgs& a, const mnq_tuning* tuning);
bool gemv_stream_supported(const MatmulArgs& a, const mnq_tuning* tuning);
int launch_gemv_stream(const MatmulArgs& a, const mnq_tuning* tuning);
// out[m, n] = sum over splits of partial[split][m][n] (fp32 planes, index order), as fp16 / bf16
int launch_splitk_reduce(const float* partial, void* out, int M, int N, int64_t ldc, int splits, int32_t act_dtype,
                         const Epilogue& epi, cudaStream_t stream);
int read_device_status(unsigned int* out, bool clear);
size_t gemv_stream_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size, int32_t quant, bool* supported);
size_t gemv_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size, int32_t quant);
bool gemm_supported(const MatmulArgs& a);
size_t gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size, int32_t quant);
size_t gemm_split_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size);
int launch_gemm(const MatmulArgs& a, const mnq_tuning* tuning);

}  // namespace mnq
