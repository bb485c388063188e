// Device helpers shared by the decode kernels (gemv_stream.cu, gemv_lean.cu): mbarrier and TMA
// wrappers, the warp MMA, the exact encodings of packed INT4 / INT8 weights that feed it, one
// 64-byte step of 16 rows, and the per-group scale / offset application.
#pragma once

#include <cuda.h>

#include "mnq_common.cuh"

namespace mnq {
namespace {

constexpr int kStepBytes = 64;  // packed bytes of one row consumed per step (4 lanes x 16)
constexpr unsigned kSpinLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)  // bounded; false = gave up
{
    for (unsigned i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// One TMA tile copy: box of the tensor map at element coordinates (x, y) -> shared memory.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// D = A * B + C with C passed by value, so that a chain can start from literal zeros.
template <typename T>
__device__ __forceinline__ void mma_c(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                      uint32_t b0, uint32_t b1, float c0, float c1, float c2, float c3);
template <>
__device__ __forceinline__ void mma_c<__half>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1, float c0, float c1,
                                              float c2, float c3)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}
template <>
__device__ __forceinline__ void mma_c<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                     uint32_t a3, uint32_t b0, uint32_t b1, float c0,
                                                     float c1, float c2, float c3)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}

// Encodings (see the header comment).  inv_alpha multiplies the scale; offset = beta + c.
// hi_x_scale: the high-nibble encoding of int4/fp16 is 16 times larger than the low-nibble
// one, so the activations those MMAs consume are staged pre-multiplied by 1/16 (exact in
// fp16 down to |x| = 2^-10; below that the lost bits are worth less than 2^-25 each) and
// both encodings accumulate into one fp32 chain.
template <int QUANT, typename T> struct Enc;
template <> struct Enc<MNQ_INT4, __half> {
    static constexpr float inv_alpha = 16777216.f, offset = 8.f;
    static constexpr bool hi_x_scale = true;
    // (n0,n4) (n1,n5) (n2,n6) (n3,n7) as L0 H0 L1 H1
    static __device__ __forceinline__ void run(uint32_t w, uint32_t& L0, uint32_t& H0, uint32_t& L1, uint32_t& H1)
    {
        const uint32_t w8 = w >> 8;
        L0 = w & 0x000F000Fu; H0 = w & 0x00F000F0u; L1 = w8 & 0x000F000Fu; H1 = w8 & 0x00F000F0u;
    }
};
template <> struct Enc<MNQ_INT4, __nv_bfloat16> {
    static constexpr float inv_alpha = 1.f, offset = 136.f;
    static constexpr bool hi_x_scale = false;
    static __device__ __forceinline__ void run(uint32_t w, uint32_t& L0, uint32_t& H0, uint32_t& L1, uint32_t& H1)
    {
        constexpr uint32_t M = 0x000F000Fu, MAGIC = 0x43004300u;
        L0 = lop3<0xEA>(w, M, MAGIC); H0 = lop3<0xEA>(w >> 4, M, MAGIC);
        L1 = lop3<0xEA>(w >> 8, M, MAGIC); H1 = lop3<0xEA>(w >> 12, M, MAGIC);
    }
};
template <> struct Enc<MNQ_INT8, __half> {
    static constexpr float inv_alpha = 16777216.f, offset = 128.f;
    static constexpr bool hi_x_scale = false;
    static __device__ __forceinline__ void run(uint32_t w, uint32_t& A0, uint32_t& A1)
    {
        const uint32_t u = w ^ 0x80808080u;
        A0 = prmt(u, 0u, 0x4140u); A1 = prmt(u, 0u, 0x4342u);
    }
};
template <> struct Enc<MNQ_INT8, __nv_bfloat16> {
    static constexpr float inv_alpha = 1.f, offset = 0.f;
    static constexpr bool hi_x_scale = false;
    static __device__ __forceinline__ void run(uint32_t w, uint32_t& A0, uint32_t& A1)
    {
        uint32_t o[2];
        UnpackInt8<__nv_bfloat16>::run(w, o);
        A0 = o[0]; A1 = o[1];
    }
};

// One step: 64 packed bytes of 16 rows against NT x 8 activation rows, accumulated into
// acc (one chain of 8 MMAs; with ZERO_START it starts from zero in this step).  xb[nt] points
// at this lane's 16 bytes of the step's first 8-block (int4) / 32 bytes (int8) in the staged
// activation row; all further offsets are compile-time constants.
template <int QUANT, typename T, int NT, bool ZERO_START>
__device__ __forceinline__ void step_mma(const uint4& wa, const uint4& wb, const unsigned char* const (&xb)[NT],
                                         float (&acc)[NT][4])
{
    const uint32_t aw[4] = {wa.x, wa.y, wa.z, wa.w};
    const uint32_t bw[4] = {wb.x, wb.y, wb.z, wb.w};
    if (QUANT == MNQ_INT4) {
#pragma unroll
        for (int jw = 0; jw < 4; ++jw) {
            uint32_t aL0, aH0, aL1, aH1, bL0, bH0, bL1, bH1;
            Enc<MNQ_INT4, T>::run(aw[jw], aL0, aH0, aL1, aH1);
            Enc<MNQ_INT4, T>::run(bw[jw], bL0, bH0, bL1, bH1);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint4 xv = *reinterpret_cast<const uint4*>(xb[nt] + jw * 64);
                if (ZERO_START && jw == 0)
                    mma_c<T>(acc[nt], aL0, bL0, aL1, bL1, xv.x, xv.y, 0.f, 0.f, 0.f, 0.f);
                else
                    mma_c<T>(acc[nt], aL0, bL0, aL1, bL1, xv.x, xv.y, acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
                mma_c<T>(acc[nt], aH0, bH0, aH1, bH1, xv.z, xv.w, acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
            }
        }
    } else {
#pragma unroll
        for (int jw = 0; jw < 4; jw += 2) {
            uint32_t a0, a1, b0, b1, c0, c1, d0, d1;
            Enc<MNQ_INT8, T>::run(aw[jw], a0, a1);
            Enc<MNQ_INT8, T>::run(bw[jw], b0, b1);
            Enc<MNQ_INT8, T>::run(aw[jw + 1], c0, c1);
            Enc<MNQ_INT8, T>::run(bw[jw + 1], d0, d1);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint4 xv = *reinterpret_cast<const uint4*>(xb[nt] + jw * 8);
                if (ZERO_START && jw == 0)
                    mma_c<T>(acc[nt], a0, b0, a1, b1, xv.x, xv.y, 0.f, 0.f, 0.f, 0.f);
                else
                    mma_c<T>(acc[nt], a0, b0, a1, b1, xv.x, xv.y, acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
                mma_c<T>(acc[nt], c0, d0, c1, d1, xv.z, xv.w, acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
            }
        }
    }
}

// tot += S * acc - Z * X for the lane's two rows (S0/Z0: row r, S1/Z1: row r+8).  xsum_lane
// points at this lane's pair of activation sums of the group (columns 2t, 2t+1 of tile 0).
template <int NT>
__device__ __forceinline__ void close_group(float (&tot)[NT][4], const float (&acc)[NT][4], float S0, float S1,
                                            float Z0, float Z1, const float* xsum_lane)
{
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const float2 X = *reinterpret_cast<const float2*>(xsum_lane + nt * 8);
        tot[nt][0] = fmaf(-Z0, X.x, fmaf(S0, acc[nt][0], tot[nt][0]));
        tot[nt][1] = fmaf(-Z0, X.y, fmaf(S0, acc[nt][1], tot[nt][1]));
        tot[nt][2] = fmaf(-Z1, X.x, fmaf(S1, acc[nt][2], tot[nt][2]));
        tot[nt][3] = fmaf(-Z1, X.y, fmaf(S1, acc[nt][3], tot[nt][3]));
    }
}

}  // namespace
}  // namespace mnq
