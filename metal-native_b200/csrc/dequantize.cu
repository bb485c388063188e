// Standalone dequantisation kernels.
//
//  * dequantize_matrix_kernel: the fused operator's formula over a whole weight
//    matrix, w = (q-8)*s - z (int4) / q*s - z (int8) with [N, ceil(K/g)] scales and
//    zeros (reference: shaders/matmul_dequant_kernel.metal:29-49 and the CPU helpers
//    tests/cpp/test_dequant_matmul.mm:119-188).  fp32 output is the bit-exactness
//    witness; fp16 / bf16 output is that value rounded to nearest even.
//  * dequantize_flat_kernel: the reference's dequantize_int{4,8}_to_fp16 kernels
//    (shaders/dequantize_kernel.metal): scale only, flat group index.
//
// Both are pure streaming: 0.5-1 byte read and 2-4 bytes written per weight, so the
// bound is HBM write bandwidth.  Each thread converts 8 consecutive weights of one
// row (one 32-bit word of nibbles, or 8 bytes) and writes them with 16/32-byte stores.
#include "mnq_common.cuh"

namespace mnq {
namespace {

template <typename OutT> struct OutCvt;
template <> struct OutCvt<float> {
    static __device__ __forceinline__ float cvt(float v) { return v; }
};
template <> struct OutCvt<__half> {
    static __device__ __forceinline__ __half cvt(float v) { return __float2half_rn(v); }
};
template <> struct OutCvt<__nv_bfloat16> {
    static __device__ __forceinline__ __nv_bfloat16 cvt(float v) { return __float2bfloat16_rn(v); }
};

// Product then subtraction, each rounded once (no contraction): the instruction
// sequence of the reference's CPU helper.  (The product is exact anyway: at most
// 8 x 11 significant bits.)
__device__ __forceinline__ float dequant_value(int q_centred, float s, float z)
{
    return __fsub_rn(__fmul_rn(static_cast<float>(q_centred), s), z);
}

template <typename OutT, int N> struct alignas(sizeof(OutT) * N) Pack { OutT v[N]; };

// One thread = 8 consecutive k of one row.  Requires K % 8 == 0.
template <int QUANT, typename OutT>
__global__ void __launch_bounds__(256)
dequantize_matrix_vec8_kernel(const uint8_t* __restrict__ wq, const void* __restrict__ scales,
                              const void* __restrict__ zeros, OutT* __restrict__ out, int64_t N,
                              int64_t K, int32_t group_size, int32_t G, int32_t scale_dtype)
{
    const int64_t k8_per_row = K >> 3;
    const int64_t total = N * k8_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / k8_per_row;
        const int64_t k0 = (i - n * k8_per_row) << 3;
        int q[8];
        if (QUANT == MNQ_INT4) {
            const uint32_t w = ldg_stream_4(wq + n * (K >> 1) + (k0 >> 1));
#pragma unroll
            for (int e = 0; e < 8; ++e) q[e] = static_cast<int>((w >> (4 * e)) & 0xF) - 8;
        } else {
            const uint2 w = ldg_stream_8(wq + n * K + k0);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                q[e] = static_cast<int>(static_cast<int8_t>((w.x >> (8 * e)) & 0xFF));
                q[e + 4] = static_cast<int>(static_cast<int8_t>((w.y >> (8 * e)) & 0xFF));
            }
        }
        Pack<OutT, 8> o;
        int g_prev = -1;
        float s = 0.f, z = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int g = static_cast<int>((k0 + e) / group_size);
            if (g != g_prev) {
                s = widen16(scales, n * G + g, scale_dtype);
                z = zeros ? widen16(zeros, n * G + g, scale_dtype) : 0.f;
                g_prev = g;
            }
            o.v[e] = OutCvt<OutT>::cvt(dequant_value(q[e], s, z));
        }
        *reinterpret_cast<Pack<OutT, 8>*>(out + n * K + k0) = o;
    }
}

// Any K (int4: any even K or odd K with row stride (K+1)/2): one thread per element.
template <int QUANT, typename OutT>
__global__ void __launch_bounds__(256)
dequantize_matrix_scalar_kernel(const uint8_t* __restrict__ wq, const void* __restrict__ scales,
                                const void* __restrict__ zeros, OutT* __restrict__ out, int64_t N,
                                int64_t K, int32_t group_size, int32_t G, int32_t scale_dtype)
{
    const int64_t total = N * K;
    const int64_t row_bytes = (QUANT == MNQ_INT4) ? ((K + 1) >> 1) : K;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / K;
        const int64_t k = i - n * K;
        int q;
        if (QUANT == MNQ_INT4) {
            const uint8_t b = wq[n * row_bytes + (k >> 1)];
            q = static_cast<int>((k & 1) ? (b >> 4) : (b & 0xF)) - 8;
        } else {
            q = static_cast<int>(static_cast<int8_t>(wq[n * row_bytes + k]));
        }
        const int64_t g = k / group_size;
        const float s = widen16(scales, n * G + g, scale_dtype);
        const float z = zeros ? widen16(zeros, n * G + g, scale_dtype) : 0.f;
        out[i] = OutCvt<OutT>::cvt(dequant_value(q, s, z));
    }
}

// Reference semantics of shaders/dequantize_kernel.metal: out[i] = half(q) * s[i / g]
// in half arithmetic == RN_fp16 of the exact (fp32-representable) product.
template <int QUANT>
__global__ void __launch_bounds__(256)
dequantize_flat_kernel(const uint8_t* __restrict__ in, const __half* __restrict__ scales,
                       __half* __restrict__ out, int64_t num_elements, int32_t group_size, bool vec_ok)
{
    const int64_t n8 = (num_elements + 7) >> 3;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t e0 = i << 3;
        const bool full = vec_ok && (e0 + 8 <= num_elements);
        int q[8];
        if (full) {
            if (QUANT == MNQ_INT4) {
                const uint32_t w = ldg_stream_4(in + (e0 >> 1));
#pragma unroll
                for (int e = 0; e < 8; ++e) q[e] = static_cast<int>((w >> (4 * e)) & 0xF) - 8;
            } else {
                const uint2 w = ldg_stream_8(in + e0);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    q[e] = static_cast<int>(static_cast<int8_t>((w.x >> (8 * e)) & 0xFF));
                    q[e + 4] = static_cast<int>(static_cast<int8_t>((w.y >> (8 * e)) & 0xFF));
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int64_t idx = e0 + e;
                q[e] = 0;
                if (idx < num_elements) {
                    if (QUANT == MNQ_INT4) {
                        const uint8_t b = in[idx >> 1];
                        q[e] = static_cast<int>((idx & 1) ? (b >> 4) : (b & 0xF)) - 8;
                    } else {
                        q[e] = static_cast<int>(static_cast<int8_t>(in[idx]));
                    }
                }
            }
        }
        Pack<__half, 8> o;
        int64_t g_prev = -1;
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int64_t idx = e0 + e;
            if (idx < num_elements) {
                const int64_t g = idx / group_size;
                if (g != g_prev) { s = __half2float(__ldg(scales + g)); g_prev = g; }
                o.v[e] = __float2half_rn(__fmul_rn(static_cast<float>(q[e]), s));
            } else {
                o.v[e] = __ushort_as_half(0);
            }
        }
        if (full) {
            *reinterpret_cast<Pack<__half, 8>*>(out + e0) = o;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (e0 + e < num_elements) out[e0 + e] = o.v[e];
        }
    }
}

inline int grid_for(int64_t work_items, int sm_count)
{
    const int64_t blocks = (work_items + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count) * 16;  // grid-stride beyond this
    return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

template <int QUANT, typename OutT>
int launch_matrix(const void* wq, const void* scales, const void* zeros, void* out, int64_t N,
                  int64_t K, int32_t group_size, int32_t G, int32_t scale_dtype, int sm_count,
                  cudaStream_t stream)
{
    const bool aligned = (reinterpret_cast<uintptr_t>(wq) % 8 == 0) &&
                         (reinterpret_cast<uintptr_t>(out) % (8 * sizeof(OutT)) == 0);
    if (K % 8 == 0 && aligned) {
        dequantize_matrix_vec8_kernel<QUANT, OutT><<<grid_for(N * (K / 8), sm_count), 256, 0, stream>>>(
            static_cast<const uint8_t*>(wq), scales, zeros, static_cast<OutT*>(out), N, K, group_size,
            G, scale_dtype);
    } else {
        dequantize_matrix_scalar_kernel<QUANT, OutT><<<grid_for(N * K, sm_count), 256, 0, stream>>>(
            static_cast<const uint8_t*>(wq), scales, zeros, static_cast<OutT*>(out), N, K, group_size,
            G, scale_dtype);
    }
    return check_cuda(cudaGetLastError(), "dequantize launch");
}

}  // namespace

int launch_dequantize_matrix(const void* wq, const void* scales, const void* zeros, void* out,
                             int64_t N, int64_t K, int32_t group_size, int32_t G, int32_t quant,
                             int32_t scale_dtype, int32_t out_dtype, int sm_count, cudaStream_t stream)
{
#define MNQ_DQ(Q, T) \
    return launch_matrix<Q, T>(wq, scales, zeros, out, N, K, group_size, G, scale_dtype, sm_count, stream)
    if (quant == MNQ_INT4) {
        if (out_dtype == MNQ_FP32) MNQ_DQ(MNQ_INT4, float);
        if (out_dtype == MNQ_FP16) MNQ_DQ(MNQ_INT4, __half);
        MNQ_DQ(MNQ_INT4, __nv_bfloat16);
    }
    if (out_dtype == MNQ_FP32) MNQ_DQ(MNQ_INT8, float);
    if (out_dtype == MNQ_FP16) MNQ_DQ(MNQ_INT8, __half);
    MNQ_DQ(MNQ_INT8, __nv_bfloat16);
#undef MNQ_DQ
}

int launch_dequantize_flat(const void* in, const void* scales, void* out, int64_t num_elements,
                           int32_t group_size, int32_t quant, int sm_count, cudaStream_t stream)
{
    const bool vec_ok = (reinterpret_cast<uintptr_t>(in) % 8 == 0) &&
                        (reinterpret_cast<uintptr_t>(out) % 16 == 0);
    const int grid = grid_for((num_elements + 7) / 8, sm_count);
    if (quant == MNQ_INT4)
        dequantize_flat_kernel<MNQ_INT4><<<grid, 256, 0, stream>>>(
            static_cast<const uint8_t*>(in), static_cast<const __half*>(scales),
            static_cast<__half*>(out), num_elements, group_size, vec_ok);
    else
        dequantize_flat_kernel<MNQ_INT8><<<grid, 256, 0, stream>>>(
            static_cast<const uint8_t*>(in), static_cast<const __half*>(scales),
            static_cast<__half*>(out), num_elements, group_size, vec_ok);
    return check_cuda(cudaGetLastError(), "dequantize_flat launch");
}

}  // namespace mnq
