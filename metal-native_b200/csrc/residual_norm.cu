// Fused residual addition + RMSNorm, the operator that produces the MLP's activations in a Llama /
// Mistral block: out = rms_norm(input + residual) * weight.  Replaces the reference's
// fast::fused_residual_norm (include/metal_native/future/fast_ops.h:99-107) and its kernels
// fused_residual_rms_norm_fp16 / _large_fp16 / _regcache_fp16
// (shaders/fused_residual_norm.metal:43-76, 140-200, 269-330), whose arithmetic it keeps: the sum
// s = float(input) + float(residual) is rounded to the 16-bit type (that rounded value is what gets
// normalised), the mean of squares is taken over the UNROUNDED sums in fp32,
// rms_inv = rsqrt(mean + eps), out = round(float(round(s)) * rms_inv * float(weight)).
//
// HBM-bound: one CTA per row, the row held in registers between the two passes (16-byte loads, one
// read of input and residual, one write of the result), warp-shuffle + shared-memory reduction in a
// fixed order.  Rows longer than the register cache, or not 16-byte aligned, take a two-pass path
// that re-reads the rounded sums from the output, as the reference's plain kernel does.  The
// rounded sum, which is the block's new residual stream, can be stored too (sum_out).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "mnq_common.cuh"

namespace mnq {
namespace {

template <typename T> struct Pair16;
template <> struct Pair16<__half> {
    static __device__ __forceinline__ float2 unpack(uint32_t w) { return __half22float2(u32_as_h2(w)); }
    static __device__ __forceinline__ uint32_t pack(float a, float b) { return h2_as_u32(__floats2half2_rn(a, b)); }
};
template <> struct Pair16<__nv_bfloat16> {
    static __device__ __forceinline__ float2 unpack(uint32_t w)
    {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
    }
    static __device__ __forceinline__ uint32_t pack(float a, float b) { return b2_as_u32(__floats2bfloat162_rn(a, b)); }
};

constexpr int kNormThreads = 256;
constexpr int kNormChunks = 8;   // 16-byte chunks a thread keeps: rows up to 8 * 256 * 8 = 16384 elements

__device__ __forceinline__ float block_sum(float v, float* scratch)
{
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) total += scratch[w];   // the same order in every thread
    return total;
}

template <typename T>
__global__ void __launch_bounds__(kNormThreads)
residual_rmsnorm_kernel(const T* input, const T* residual, const T* __restrict__ weight, T* out, T* sum_out, long long hidden, long long ld_in, long long ld_res,
                        long long ld_out, long long ld_sum, float eps, int vec)
{
    __shared__ float scratch[kNormThreads / 32];
    const long long row = blockIdx.x;
    const T* in_row = input + row * ld_in;
    const T* res_row = residual + row * ld_res;
    T* out_row = out + row * ld_out;
    T* sum_row = sum_out ? sum_out + row * ld_sum : nullptr;
    // Launched programmatically dependent: nothing global is touched before the previous kernel is done.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (vec) {
        const int chunks = static_cast<int>(hidden / 8);
        uint4 h[kNormChunks];   // the rounded sums, 8 per chunk
        float sq = 0.f;
#pragma unroll
        for (int u = 0; u < kNormChunks; ++u) {
            const int c = threadIdx.x + u * kNormThreads;
            if (c < chunks) {
                // (plain loads: out or sum_out may be the same memory as input or residual)
                const uint4 a = reinterpret_cast<const uint4*>(in_row)[c];
                const uint4 b = reinterpret_cast<const uint4*>(res_row)[c];
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
                uint32_t hw[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 fa = Pair16<T>::unpack(aw[e]), fb = Pair16<T>::unpack(bw[e]);
                    const float s0 = fa.x + fb.x, s1 = fa.y + fb.y;
                    sq = fmaf(s0, s0, sq);
                    sq = fmaf(s1, s1, sq);
                    hw[e] = Pair16<T>::pack(s0, s1);
                }
                h[u] = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                if (sum_row) reinterpret_cast<uint4*>(sum_row)[c] = h[u];
            }
        }
        const float rms_inv = rsqrtf(block_sum(sq, scratch) / static_cast<float>(hidden) + eps);
#pragma unroll
        for (int u = 0; u < kNormChunks; ++u) {
            const int c = threadIdx.x + u * kNormThreads;
            if (c < chunks) {
                const uint4 w = __ldg(reinterpret_cast<const uint4*>(weight) + c);
                const uint32_t hw[4] = {h[u].x, h[u].y, h[u].z, h[u].w}, ww[4] = {w.x, w.y, w.z, w.w};
                uint32_t ow[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 fh = Pair16<T>::unpack(hw[e]), fw = Pair16<T>::unpack(ww[e]);
                    ow[e] = Pair16<T>::pack(fh.x * rms_inv * fw.x, fh.y * rms_inv * fw.y);
                }
                reinterpret_cast<uint4*>(out_row)[c] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
        }
        return;
    }
    // any length and alignment: the rounded sums go through the output row
    float sq = 0.f;
    for (long long i = threadIdx.x; i < hidden; i += kNormThreads) {
        const float s = F16Traits<T>::to_float(in_row[i]) + F16Traits<T>::to_float(res_row[i]);
        const T hr = F16Traits<T>::from_float(s);
        out_row[i] = hr;
        if (sum_row) sum_row[i] = hr;
        sq = fmaf(s, s, sq);
    }
    const float rms_inv = rsqrtf(block_sum(sq, scratch) / static_cast<float>(hidden) + eps);
    for (long long i = threadIdx.x; i < hidden; i += kNormThreads)   // (each thread re-reads what it wrote)
        out_row[i] = F16Traits<T>::from_float(F16Traits<T>::to_float(out_row[i]) * rms_inv * F16Traits<T>::to_float(weight[i]));
}

template <typename T>
int launch_norm(const void* input, const void* residual, const void* weight, void* out, void* sum_out, int64_t rows,
                int64_t hidden, int64_t ld_in, int64_t ld_res, int64_t ld_out, int64_t ld_sum, float eps, cudaStream_t stream)
{
    auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool vec = hidden % 8 == 0 && hidden <= static_cast<int64_t>(kNormChunks) * kNormThreads * 8 && aligned(input) &&
                     aligned(residual) && aligned(weight) && aligned(out) && (!sum_out || aligned(sum_out)) && ld_in % 8 == 0 &&
                     ld_res % 8 == 0 && ld_out % 8 == 0 && (!sum_out || ld_sum % 8 == 0);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(rows));
    cfg.blockDim = dim3(kNormThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, &residual_rmsnorm_kernel<T>, static_cast<const T*>(input),
                                         static_cast<const T*>(residual), static_cast<const T*>(weight), static_cast<T*>(out),
                                         static_cast<T*>(sum_out), (long long)hidden, (long long)ld_in, (long long)ld_res,
                                         (long long)ld_out, (long long)ld_sum, eps, vec ? 1 : 0),
                      "residual_rmsnorm launch");
}

}  // namespace
}  // namespace mnq

using namespace mnq;

extern "C" MNQ_API int mnq_residual_rmsnorm(const void* input, const void* residual, const void* weight, void* out,
                                            void* sum_out, int64_t rows, int64_t hidden, int64_t ld_in, int64_t ld_res,
                                            int64_t ld_out, int64_t ld_sum, float eps, int32_t dtype, void* stream)
{
    if (rows < 0 || hidden < 0) return fail(MNQ_INVALID_ARGUMENT, "fused_residual_norm: negative shape (%lld, %lld)", (long long)rows, (long long)hidden);
    if (dtype != MNQ_FP16 && dtype != MNQ_BF16) return fail(MNQ_INVALID_ARGUMENT, "fused_residual_norm: dtype must be fp16 or bf16");
    if (rows == 0 || hidden == 0) return MNQ_SUCCESS;
    if (!input || !residual || !weight || !out) return fail(MNQ_INVALID_ARGUMENT, "fused_residual_norm: null tensor");
    if (ld_in < hidden || ld_res < hidden || ld_out < hidden || (sum_out && ld_sum < hidden))
        return fail(MNQ_INVALID_ARGUMENT, "fused_residual_norm: a row stride is smaller than the row length %lld", (long long)hidden);
    if (rows > 2147483647LL) return fail(MNQ_INVALID_ARGUMENT, "fused_residual_norm: too many rows");
    if (!(eps >= 0.f)) return fail(MNQ_INVALID_ARGUMENT, "fused_residual_norm: eps must be non-negative");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == MNQ_FP16)
        return launch_norm<__half>(input, residual, weight, out, sum_out, rows, hidden, ld_in, ld_res, ld_out, ld_sum, eps, s);
    return launch_norm<__nv_bfloat16>(input, residual, weight, out, sum_out, rows, hidden, ld_in, ld_res, ld_out, ld_sum, eps, s);
}
