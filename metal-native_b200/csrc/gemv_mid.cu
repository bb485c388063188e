// Decode-shaped fused dequantise + matmul for 5 to 32 tokens, and up to 64 for bf16 activations (the
// batched-decode case; replaces,
// for those token counts, the reference's tiled kernels dequant_matmul_int{4,8}_fp16,
// shaders/matmul_dequant_kernel.metal:55-223, 351-479).  Same weight movement and arithmetic as
// the other decode kernels (gemv_stream.cu, gemv_lean.cu): one TMA tile copy per 16-row x 256-byte
// piece into a per-warp ring, packed integers fed to m16n8k16 warp MMAs through exact encodings,
// scale and offset applied per group in fp32.  What differs is where the activations come from.
//
// With this many tokens the activation block is as large as a CTA's shared memory, and staging it
// (convert, permute into MMA fragment order, group sums) in every CTA cost more than streaming
// the weights.  Here it is prepared ONCE per call by a small kernel, prepare_image_kernel, which
// writes the block to the workspace as the exact shared-memory image the MMAs read, cut along K
// into pieces of four steps: per piece the fp16 fragments of every token (rows padded so that
// the eight token rows of a fragment load fall on different banks), then the fp32 sum of every
// (step, token).  bf16 activations become fp16 times a per-token power of two.  The main kernel
// walks K piece by piece: image pieces come into a small ring with one bulk copy each, every warp
// multiplies the piece against the weight pieces of its row blocks and releases it, and the last
// warp to release a ring slot requests the piece that will reuse it, so a CTA holds a few pieces
// of activations, whatever K is, and the copies overlap the arithmetic.  (The copies hit L2, but
// they queue behind every SM's outstanding weight requests, so the ring is as deep as fits.)  A warp keeps the accumulators of its row block in registers
// over a sweep of K.  (The kernel can also carry two row blocks per warp, NB = 2, so that every
// activation fragment loaded from shared memory feeds both; that halves the warps a CTA can hold
// and measured slower on B200, where these token counts are bound by the warp-MMA rate, one
// m16n8k16 per 8 cycles and SM sub-partition, not by shared memory; it is not instantiated.)
//
// Row blocks are dealt out evenly over one CTA per SM and then over its warps; a layer with too
// few row blocks is also cut along K (grid.y), each cut writing an fp32 plane that a second
// small kernel adds in index order.  Every wait on an mbarrier is bounded: a wait that gives up
// sets bit 0 of the device status word and the CTA leaves.
#include <cuda.h>
#include <limits.h>

#include <algorithm>
#include <atomic>
#include <type_traits>

#include "gemv_mma_common.cuh"

namespace mnq {

__device__ unsigned int g_mid_status = 0;   // bit 0: a bounded wait for a weight tile or an activation piece gave up

namespace {

constexpr int kPieceBytes = 256;                        // packed bytes of one row per weight piece
constexpr int kPieceSteps = kPieceBytes / kStepBytes;   // 4
constexpr int kStageBytes = 16 * kPieceBytes;           // one weight-ring stage
constexpr int kMidMaxSmem = 226 * 1024;
// Fewer tokens than this run the compact kernel: preparing the activations costs a launch and a
// dependency (about 3.5 us), which five tokens' worth of per-CTA staging outweighs (measured).
constexpr int kMidMinTokens = 5;
// Above 32 tokens only bf16 activations come here (5 to 8 token tiles): with group-wise scales the
// tensor-core kernel needs two bf16 tiles per k-block for them, and eight token tiles on the warp MMA
// are still faster than that (measured on the Llama-3-8B shapes).
constexpr int kMidMaxTokens = 64;
constexpr int kPrepThreads = 1024;
constexpr int kPrepBatch = 4;                           // 8-blocks a thread holds: K <= 8 * 4 * 1024

// Geometry of one activation piece of the image, per weight format and token-tile count.
template <int QUANT, int NT> struct Image {
    static constexpr int STEP = (QUANT == MNQ_INT4) ? 128 : 64;     // k per step
    static constexpr int PIECE_K = STEP * kPieceSteps;              // k per piece: 512 / 256
    static constexpr int ROWS = 8 * NT;                             // token rows, zero-filled past M
    static constexpr int ROW_BYTES = PIECE_K * 2;
    static constexpr int PAD = (QUANT == MNQ_INT4) ? 64 : 16;       // staggers the 8 rows of a fragment load over the banks
    static constexpr int RS = ROW_BYTES + PAD;                      // row stride
    static constexpr int SUMS_OFF = ROWS * RS;                      // float [kPieceSteps][ROWS]
    static constexpr int BYTES = SUMS_OFF + kPieceSteps * ROWS * 4; // a multiple of 16
};
inline int image_piece_bytes(int quant, int nt)
{
    const int step = quant == MNQ_INT4 ? 128 : 64;
    const int rs = step * kPieceSteps * 2 + (quant == MNQ_INT4 ? 64 : 16);
    return 8 * nt * rs + kPieceSteps * 8 * nt * 4;
}

struct MidParams {
    const void* x;
    const unsigned short* scales;
    const unsigned short* zeros;   // may be null
    void* out;
    unsigned char* image;          // [pieces][Image::BYTES]
    float* tok_up;                 // [8 NT] power of two that undoes the token's bf16 -> fp16 rescale (1 for fp16)
    float* partial;                // [num_chunks][M][N] when K is cut
    long long lda, ldc;
    int M, N, K, G;
    int row_blocks;
    int pieces;                    // K pieces per row
    int pieces_per_chunk, num_chunks;
    int stages, xstages;
    int scale_bf16;
    int weights_immutable;
    Epilogue epi;
};

// ---------------------------------------------------------------------------------------------
// Activation image.  One CTA per token row (rows past M are written as zeros).
// ---------------------------------------------------------------------------------------------
template <int QUANT, typename T, int NT>
__global__ void __launch_bounds__(kPrepThreads)
prepare_image_kernel(const MidParams p)
{
    using Img = Image<QUANT, NT>;
    constexpr bool CONVERT_X = !std::is_same<T, __half>::value;
    constexpr int SEG = Img::STEP / 8;                     // 8-blocks per step
    constexpr int BPP = Img::PIECE_K / 8;                  // 8-blocks per piece
    __shared__ unsigned int x_max_bits;

    const int m = blockIdx.x;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int blocks = p.K / 8;                            // a multiple of BPP
    if (tid == 0) x_max_bits = 0u;
    // the next kernel in the stream may be scheduled at once: it waits for this grid to finish
    // before it reads the image
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (m >= p.M) {
        // token rows the MMA tiles have but the problem does not: zeros
        for (int i = tid; i < blocks; i += kPrepThreads) {
            const int pc = i / BPP, bl = i - pc * BPP;
            *reinterpret_cast<uint4*>(p.image + (size_t)pc * Img::BYTES + (size_t)m * Img::RS + bl * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        for (int i = tid; i < p.pieces * kPieceSteps; i += kPrepThreads)
            reinterpret_cast<float*>(p.image + (size_t)(i / kPieceSteps) * Img::BYTES + Img::SUMS_OFF)[(i % kPieceSteps) * Img::ROWS + m] = 0.f;
        if (tid == 0) p.tok_up[m] = 1.f;
        return;
    }

    const T* xg = static_cast<const T*>(p.x) + (size_t)m * p.lda;
    // the whole token row in registers: one round trip to memory
    uint4 xq[kPrepBatch];
#pragma unroll
    for (int u = 0; u < kPrepBatch; ++u) {
        const int i = u * kPrepThreads + tid;
        xq[u] = make_uint4(0u, 0u, 0u, 0u);
        if (i < blocks) xq[u] = __ldg(reinterpret_cast<const uint4*>(xg + (size_t)i * 8));
    }
    float x_down = 1.f;
    if (CONVERT_X) {
        // largest |x| of the token -> power-of-two scale that puts it just below 2^15
        __syncthreads();   // x_max_bits is zero
        unsigned int mx = 0;
#pragma unroll
        for (int u = 0; u < kPrepBatch; ++u) {
            const uint32_t w[4] = {xq[u].x, xq[u].y, xq[u].z, xq[u].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) mx = max(mx, max(w[e] & 0x7FFFu, (w[e] >> 16) & 0x7FFFu));
        }
        mx = __reduce_max_sync(0xffffffffu, mx);
        if (lane == 0 && mx) atomicMax(&x_max_bits, mx);
        __syncthreads();
        const int E = static_cast<int>(x_max_bits >> 7);   // biased bf16 exponent of the maximum
        int sh = (E == 0) ? 0 : (E - 127) - 14;
        sh = max(-100, min(100, sh));
        x_down = __int_as_float((127 - sh) << 23);
        if (tid == 0) p.tok_up[m] = __int_as_float((127 + sh) << 23);
    } else if (tid == 0) {
        p.tok_up[m] = 1.f;
    }

    // whole warps walk the blocks together (the step sums are shuffle reductions over aligned lane runs)
    {
#pragma unroll
        for (int u = 0; u < kPrepBatch; ++u) {
        const int i = u * kPrepThreads + tid;
        if (u * kPrepThreads + (tid & ~31) >= blocks) break;   // (warp-uniform)
        const bool valid = i < blocks;                      // blocks is a multiple of SEG: whole runs are valid or not
        uint32_t v[4] = {xq[u].x, xq[u].y, xq[u].z, xq[u].w};
        if (CONVERT_X) {   // bf16 -> fp16, times 2^-shift (exact unless the result is subnormal)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(v[e] << 16) * x_down;
                const float hi = __uint_as_float(v[e] & 0xFFFF0000u) * x_down;
                v[e] = h2_as_u32(__floats2half2_rn(lo, hi));
            }
        }
        float sum = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(u32_as_h2(v[e]));
            sum += f.x;
            sum += f.y;
        }
#pragma unroll
        for (int d = 1; d < SEG; d <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
        if (!valid) continue;
        const int pc = i / BPP, b = i - pc * BPP;          // piece, 8-block inside it
        unsigned char* piece = p.image + (size_t)pc * Img::BYTES;
        if ((lane & (SEG - 1)) == 0)
            reinterpret_cast<float*>(piece + Img::SUMS_OFF)[(b / SEG) * Img::ROWS + m] = sum;
        int pos;
        uint4 o;
        if (QUANT == MNQ_INT4) {
            // inside a 128-k step the 8-blocks are laid out [word j][lane t]; inside an 8-block the
            // order is k+0,k+4,k+2,k+6 | k+1,k+5,k+3,k+7 (low-nibble pairs, then high-nibble pairs, the
            // latter pre-multiplied by 1/16: see Enc<MNQ_INT4, __half>)
            const int step = b >> 4, bl = b & 15;
            pos = step * Img::STEP + ((bl & 3) * 4 + (bl >> 2)) * 8;
            const __half2 k16 = __half2half2(__ushort_as_half(0x2C00));   // 1/16
            o.x = prmt(v[0], v[2], 0x5410u);
            o.y = prmt(v[1], v[3], 0x5410u);
            o.z = h2_as_u32(__hmul2(u32_as_h2(prmt(v[0], v[2], 0x7632u)), k16));
            o.w = h2_as_u32(__hmul2(u32_as_h2(prmt(v[1], v[3], 0x7632u)), k16));
        } else {
            pos = b * 8;
            o = make_uint4(v[0], v[1], v[2], v[3]);
        }
        *reinterpret_cast<uint4*>(piece + (size_t)m * Img::RS + (size_t)pos * 2) = o;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// One step of NB row blocks: 64 packed bytes of each block's 16 rows against NT x 8 activation
// rows; every activation fragment is loaded once and used by all NB blocks.  Each block's chain
// of 8 MMAs starts from zero (GROUPED: the step is a group) or continues acc.
// ---------------------------------------------------------------------------------------------
template <int QUANT, typename MT, int NT, int NB, bool ZERO_START>
__device__ __forceinline__ void step_mma_nb(const uint4 (&wa)[NB], const uint4 (&wb)[NB],
                                            const unsigned char* const (&xb)[NT], float (&acc)[NB][NT][4])
{
    if (QUANT == MNQ_INT4) {
#pragma unroll
        for (int jw = 0; jw < 4; ++jw) {
            uint32_t aL0[NB], aH0[NB], aL1[NB], aH1[NB], bL0[NB], bH0[NB], bL1[NB], bH1[NB];
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                const uint32_t aw = jw == 0 ? wa[b].x : jw == 1 ? wa[b].y : jw == 2 ? wa[b].z : wa[b].w;
                const uint32_t bw = jw == 0 ? wb[b].x : jw == 1 ? wb[b].y : jw == 2 ? wb[b].z : wb[b].w;
                Enc<MNQ_INT4, MT>::run(aw, aL0[b], aH0[b], aL1[b], aH1[b]);
                Enc<MNQ_INT4, MT>::run(bw, bL0[b], bH0[b], bL1[b], bH1[b]);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint4 xv = *reinterpret_cast<const uint4*>(xb[nt] + jw * 64);
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    if (ZERO_START && jw == 0)
                        mma_c<MT>(acc[b][nt], aL0[b], bL0[b], aL1[b], bL1[b], xv.x, xv.y, 0.f, 0.f, 0.f, 0.f);
                    else
                        mma_c<MT>(acc[b][nt], aL0[b], bL0[b], aL1[b], bL1[b], xv.x, xv.y, acc[b][nt][0], acc[b][nt][1],
                                  acc[b][nt][2], acc[b][nt][3]);
                    mma_c<MT>(acc[b][nt], aH0[b], bH0[b], aH1[b], bH1[b], xv.z, xv.w, acc[b][nt][0], acc[b][nt][1],
                              acc[b][nt][2], acc[b][nt][3]);
                }
            }
        }
    } else {
#pragma unroll
        for (int jw = 0; jw < 4; jw += 2) {
            uint32_t a0[NB], a1[NB], b0[NB], b1[NB], c0[NB], c1[NB], d0[NB], d1[NB];
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                Enc<MNQ_INT8, MT>::run(jw == 0 ? wa[b].x : wa[b].z, a0[b], a1[b]);
                Enc<MNQ_INT8, MT>::run(jw == 0 ? wb[b].x : wb[b].z, b0[b], b1[b]);
                Enc<MNQ_INT8, MT>::run(jw == 0 ? wa[b].y : wa[b].w, c0[b], c1[b]);
                Enc<MNQ_INT8, MT>::run(jw == 0 ? wb[b].y : wb[b].w, d0[b], d1[b]);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint4 xv = *reinterpret_cast<const uint4*>(xb[nt] + jw * 8);
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    if (ZERO_START && jw == 0)
                        mma_c<MT>(acc[b][nt], a0[b], b0[b], a1[b], b1[b], xv.x, xv.y, 0.f, 0.f, 0.f, 0.f);
                    else
                        mma_c<MT>(acc[b][nt], a0[b], b0[b], a1[b], b1[b], xv.x, xv.y, acc[b][nt][0], acc[b][nt][1],
                                  acc[b][nt][2], acc[b][nt][3]);
                    mma_c<MT>(acc[b][nt], c0[b], d0[b], c1[b], d1[b], xv.z, xv.w, acc[b][nt][0], acc[b][nt][1],
                              acc[b][nt][2], acc[b][nt][3]);
                }
            }
        }
    }
}

__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// GROUPED: every step is one quantisation group; otherwise one group per row.
// NB: row blocks a warp carries through one sweep of K.
template <int QUANT, typename T, int NT, bool GROUPED, int NB>
__global__ void __launch_bounds__((NT >= 5 || (NT >= 4 && NB >= 2)) ? 256 : 512)
gemv_mid_kernel(const __grid_constant__ MidParams p, const __grid_constant__ CUtensorMap wmap)
{
    using MT = __half;
    using Img = Image<QUANT, NT>;
    constexpr int XSTAGE = (Img::BYTES + 127) & ~127;

    extern __shared__ __align__(128) unsigned char smem[];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int wc = blockDim.x >> 5;
    const int r = lane >> 2;
    const int t = lane & 3;

    // shared memory: activation ring, weight rings (one per warp), barriers, release counters
    unsigned char* xring = smem;
    unsigned char* wring0 = smem + p.xstages * XSTAGE;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(wring0 + wc * p.stages * kStageBytes);
    unsigned long long* xfull = bars;                                  // [xstages]
    unsigned long long* wbars = bars + p.xstages + warp * p.stages;    // [stages] of this warp
    unsigned int* xreleased = reinterpret_cast<unsigned int*>(bars + p.xstages + wc * p.stages);   // [xstages] warps done with the slot

    // this CTA's K pieces and row blocks; the row blocks are dealt evenly to CTAs, then to warps
    const int j0 = blockIdx.y * p.pieces_per_chunk;
    const int nj = min(p.pieces, j0 + p.pieces_per_chunk) - j0;
    const int cb0 = static_cast<int>((long long)blockIdx.x * p.row_blocks / gridDim.x);
    const int ncb = static_cast<int>(((long long)blockIdx.x + 1) * p.row_blocks / gridDim.x) - cb0;
    const int sweeps = ((ncb + wc - 1) / wc + NB - 1) / NB;   // the same for every warp of the CTA
    const int x_total = sweeps * nj;                          // activation pieces the CTA consumes

    if (tid == 0) {
        for (int s = 0; s < p.xstages; ++s) {
            mbar_init(smem_u32(&xfull[s]), 1);
            xreleased[s] = 0u;
        }
        for (int i = 0; i < wc * p.stages; ++i) mbar_init(smem_u32(&bars[p.xstages + i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // activation piece number `it` of this CTA (sweep-major, then K) into ring slot s
    auto request_x = [&](int it, int s) {
        const uint32_t bar = smem_u32(&xfull[s]);
        mbar_expect_tx(bar, static_cast<uint32_t>(Img::BYTES));
        bulk_copy_g2s(smem_u32(xring + s * XSTAGE), p.image + (size_t)(j0 + it % nj) * Img::BYTES,
                      static_cast<uint32_t>(Img::BYTES), bar);
    };

    const int wb0 = cb0 + static_cast<int>((long long)warp * ncb / wc);
    const int nrb = cb0 + static_cast<int>(((long long)warp + 1) * ncb / wc) - wb0;
    const int total_pieces = nrb * nj;
    unsigned char* ring = wring0 + warp * p.stages * kStageBytes;

    // weight pieces are requested in the order they are consumed: sweep, K piece, block of the sweep
    int iss_sweep = 0, iss_jj = 0, iss_b = 0, iss_stage = 0, iss_count = 0;
    auto blocks_in = [&](int sweep) { return max(0, min(NB, nrb - sweep * NB)); };
    auto issue_piece = [&]() {
        if (lane == 0) {
            const uint32_t bar = smem_u32(&wbars[iss_stage]);
            mbar_expect_tx(bar, static_cast<uint32_t>(kStageBytes));
            tma_load_2d(smem_u32(ring + iss_stage * kStageBytes), &wmap, ((j0 + iss_jj) * kPieceBytes) >> 2,
                        (wb0 + iss_sweep * NB + iss_b) * 16, bar);
        }
        ++iss_count;
        if (++iss_stage == p.stages) iss_stage = 0;
        if (++iss_b == blocks_in(iss_sweep)) {
            iss_b = 0;
            if (++iss_jj == nj) { iss_jj = 0; ++iss_sweep; }
        }
    };
    // (immutable weights: the whole ring before the dependency wait; holding part of it back until the
    // first activation pieces are requested, as the compact kernel does, measured slightly slower here)
    if (p.weights_immutable)
        for (int j = 0; j < p.stages && j < total_pieces; ++j) issue_piece();
    // Launched programmatically dependent: everything above touched only this CTA's shared memory
    // and, if the caller declared them immutable, the weights.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // (the image is written by the kernel before this one)
    if (tid == 0)
        for (int it = 0; it < p.xstages && it < x_total; ++it) request_x(it, it);
    if (!p.weights_immutable)
        for (int j = 0; j < p.stages && j < total_pieces; ++j) issue_piece();

    const bool scale_bf16 = p.scale_bf16 != 0;
    const bool has_zero = p.zeros != nullptr;
    auto widen2 = [&](uint32_t w, float& a, float& b) {
        if (scale_bf16) { a = __uint_as_float(w << 16); b = __uint_as_float(w & 0xFFFF0000u); }
        else { const float2 f = __half22float2(u32_as_h2(w)); a = f.x; b = f.y; }
    };
    struct ScaleRegs { uint2 s0, s1, z0, z1; };
    // pointers to the scales / zeros of this lane's two rows of block b of the sweep, at the next piece
    const unsigned short *sp0[NB], *sp1[NB], *zp0[NB], *zp1[NB];
    auto point_at = [&](int sweep) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            const int n0 = (wb0 + sweep * NB + b) * 16 + r, n1 = n0 + 8;   // (rows past N are clamped: never stored)
            const size_t g0 = GROUPED ? (size_t)j0 * kPieceSteps : 0;
            sp0[b] = p.scales + (size_t)min(n0, p.N - 1) * p.G + g0;
            sp1[b] = p.scales + (size_t)min(n1, p.N - 1) * p.G + g0;
            zp0[b] = zp1[b] = p.scales;
            if (has_zero) { zp0[b] = p.zeros + (size_t)min(n0, p.N - 1) * p.G + g0; zp1[b] = p.zeros + (size_t)min(n1, p.N - 1) * p.G + g0; }
        }
    };
    auto load_scales = [&](ScaleRegs (&q)[NB]) {   // the next four groups (GROUPED) of both rows of every block, then advance
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            q[b].z0 = q[b].z1 = make_uint2(0u, 0u);
            if (GROUPED) {
                q[b].s0 = __ldg(reinterpret_cast<const uint2*>(sp0[b])); q[b].s1 = __ldg(reinterpret_cast<const uint2*>(sp1[b]));
                sp0[b] += kPieceSteps; sp1[b] += kPieceSteps;
                if (has_zero) {
                    q[b].z0 = __ldg(reinterpret_cast<const uint2*>(zp0[b])); q[b].z1 = __ldg(reinterpret_cast<const uint2*>(zp1[b]));
                    zp0[b] += kPieceSteps; zp1[b] += kPieceSteps;
                }
            } else {
                q[b].s0 = make_uint2(__ldg(sp0[b]), 0u); q[b].s1 = make_uint2(__ldg(sp1[b]), 0u);
                if (has_zero) { q[b].z0.x = __ldg(zp0[b]); q[b].z1.x = __ldg(zp1[b]); }
            }
        }
    };

    const int x_lane_off = (QUANT == MNQ_INT4) ? t * 16 : t * 32;
    bool gave_up = false;
    int stage = 0;
    uint32_t parity = 0;
    int xs = 0;
    uint32_t xph = 0;
    for (int sweep = 0; sweep < sweeps && !gave_up; ++sweep) {
        const int nb = blocks_in(sweep);
        ScaleRegs sc_cur[NB], sc_nxt[NB];
        if (nb > 0) { point_at(sweep); load_scales(sc_cur); }
        float tot[NB][NT][4];      // GROUPED: the result; otherwise the raw sum over K
        float xacc[NT][2];         // !GROUPED: sum of the activations over this CTA's K range, tokens 2t, 2t+1 of every tile
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) tot[b][nt][i] = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) xacc[nt][0] = xacc[nt][1] = 0.f;

        for (int jj = 0; jj < nj; ++jj) {
            if (GROUPED && nb > 0 && jj + 1 < nj) load_scales(sc_nxt);
            if (!mbar_wait(smem_u32(&xfull[xs]), xph)) { gave_up = true; break; }
            const unsigned char* xpiece = xring + xs * XSTAGE;
            if (nb > 0) {
                // the weight pieces of this K piece: one per block of the sweep, in consecutive ring stages
                const unsigned char* wst[NB];
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    wst[b] = ring + stage * kStageBytes + r * kPieceBytes + t * 16;
                    if (b < nb) {
                        if (!mbar_wait(smem_u32(&wbars[stage]), parity)) { gave_up = true; break; }
                        if (++stage == p.stages) { stage = 0; parity ^= 1u; }
                    }
                }
                if (gave_up) break;
                const float* sums = reinterpret_cast<const float*>(xpiece + Img::SUMS_OFF) + 2 * t;
#pragma unroll
                for (int ps = 0; ps < kPieceSteps; ++ps) {
                    uint4 wa[NB], wb[NB];
#pragma unroll
                    for (int b = 0; b < NB; ++b) {
                        // a sweep's last, single block: the second operand repeats the first (its results are dropped)
                        wa[b] = *reinterpret_cast<const uint4*>(wst[b] + ps * kStepBytes);
                        wb[b] = *reinterpret_cast<const uint4*>(wst[b] + 8 * kPieceBytes + ps * kStepBytes);
                    }
                    const unsigned char* xb[NT];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) xb[nt] = xpiece + (nt * 8 + r) * Img::RS + x_lane_off + ps * Img::STEP * 2;
                    if (GROUPED) {
                        float a4[NB][NT][4];
                        step_mma_nb<QUANT, MT, NT, NB, true>(wa, wb, xb, a4);
#pragma unroll
                        for (int b = 0; b < NB; ++b) {
                            const uint32_t sw0 = (ps & 2) ? sc_cur[b].s0.y : sc_cur[b].s0.x, sw1 = (ps & 2) ? sc_cur[b].s1.y : sc_cur[b].s1.x;
                            const uint32_t zw0 = (ps & 2) ? sc_cur[b].z0.y : sc_cur[b].z0.x, zw1 = (ps & 2) ? sc_cur[b].z1.y : sc_cur[b].z1.x;
                            float s0a, s0b, s1a, s1b, z0a, z0b, z1a, z1b;
                            widen2(sw0, s0a, s0b); widen2(sw1, s1a, s1b); widen2(zw0, z0a, z0b); widen2(zw1, z1a, z1b);
                            const float s0 = (ps & 1) ? s0b : s0a, s1 = (ps & 1) ? s1b : s1a;
                            const float z0 = (ps & 1) ? z0b : z0a, z1 = (ps & 1) ? z1b : z1a;
                            // S = s / alpha, Z = (beta + c) s + z (see Enc)
                            close_group<NT>(tot[b], a4[b], s0 * Enc<QUANT, MT>::inv_alpha, s1 * Enc<QUANT, MT>::inv_alpha,
                                            fmaf(Enc<QUANT, MT>::offset, s0, z0), fmaf(Enc<QUANT, MT>::offset, s1, z1),
                                            sums + ps * Img::ROWS);
                        }
                    } else {
                        step_mma_nb<QUANT, MT, NT, NB, false>(wa, wb, xb, tot);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const float2 X = *reinterpret_cast<const float2*>(sums + ps * Img::ROWS + nt * 8);
                            xacc[nt][0] += X.x;
                            xacc[nt][1] += X.y;
                        }
                    }
                }
                if (GROUPED) {
#pragma unroll
                    for (int b = 0; b < NB; ++b) sc_cur[b] = sc_nxt[b];
                }
                __syncwarp();   // every lane is done reading these stages
                for (int b = 0; b < nb; ++b)
                    if (iss_count < total_pieces) issue_piece();
            }
            __syncwarp();       // ... and this activation piece
            if (lane == 0) {
                // the last warp to release the slot requests the piece that reuses it
                __threadfence_block();
                if (atomicAdd(&xreleased[xs], 1u) == static_cast<unsigned int>(wc - 1)) {
                    xreleased[xs] = 0u;
                    __threadfence_block();
                    const int nxt = sweep * nj + jj + p.xstages;
                    if (nxt < x_total) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        request_x(nxt, xs);
                    }
                }
            }
            if (++xs == p.xstages) { xs = 0; xph ^= 1u; }
        }
        if (gave_up) break;

        // ---- results of this sweep: accumulator i of tile nt is output (m = nt*8 + 2t + (i&1), n = n0 or n0 + 8)
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            if (b >= nb) break;
            const int n0 = (wb0 + sweep * NB + b) * 16 + r;
            float S0 = 1.f, S1 = 1.f, Z0 = 0.f, Z1 = 0.f;
            if (!GROUPED) {
                float s0, s1, z0 = 0.f, z1 = 0.f, unused;
                widen2(sc_cur[b].s0.x, s0, unused); widen2(sc_cur[b].s1.x, s1, unused);
                if (has_zero) { widen2(sc_cur[b].z0.x, z0, unused); widen2(sc_cur[b].z1.x, z1, unused); }
                S0 = s0 * Enc<QUANT, MT>::inv_alpha; S1 = s1 * Enc<QUANT, MT>::inv_alpha;
                Z0 = fmaf(Enc<QUANT, MT>::offset, s0, z0); Z1 = fmaf(Enc<QUANT, MT>::offset, s1, z1);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float2 up = *reinterpret_cast<const float2*>(p.tok_up + nt * 8 + 2 * t);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int m = nt * 8 + 2 * t + (i & 1);
                    const int n = (i & 2) ? n0 + 8 : n0;
                    float v = tot[b][nt][i];
                    if (!GROUPED) v = fmaf(-((i & 2) ? Z1 : Z0), xacc[nt][i & 1], ((i & 2) ? S1 : S0) * v);
                    v *= (i & 1) ? up.y : up.x;
                    if (m < p.M && n < p.N) {
                        if (p.num_chunks == 1) store_result<T>(p.epi, p.out, p.ldc, m, n, v);
                        else __stcg(&p.partial[((size_t)blockIdx.y * p.M + m) * p.N + n], v);
                    }
                }
            }
        }
    }
    if (gave_up && lane == 0) atomicOr(&g_mid_status, 1u);
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
struct MidPlan {
    int nt, nb, warps, stages, xstages, grid_x, num_chunks, pieces, pieces_per_chunk, piece_bytes;
    size_t smem, planes_bytes, image_off, image_bytes, need_ws;
};

bool plan_mid_with(const MatmulArgs& a, const mnq_tuning* tuning, size_t workspace_bytes, int want_warps, MidPlan* out)
{
    if (a.M < kMidMinTokens || a.M > kMidMaxTokens || a.swiglu_h > 0 || a.gather.world > 0) return false;
    if (a.M > 32 && a.act_dtype != MNQ_BF16) return false;
    const int step = a.quant == MNQ_INT4 ? 128 : 64;
    const int piece_k = step * kPieceSteps;
    if (a.K < piece_k || a.K % piece_k || a.N < 1 || a.N > (1 << 30) || a.K > 8 * kPrepBatch * kPrepThreads) return false;
    const bool grouped = a.group_size < a.K;
    if (grouped) {
        if (a.group_size != step || a.G % kPieceSteps) return false;   // a step is a group; 8-byte scale loads
        if (reinterpret_cast<uintptr_t>(a.scales) % 8 || (a.zeros && reinterpret_cast<uintptr_t>(a.zeros) % 8)) return false;
    }
    if (reinterpret_cast<uintptr_t>(a.x) % 16 || a.lda % 8 || reinterpret_cast<uintptr_t>(a.wq) % 16) return false;

    MidPlan pl{};
    pl.nt = static_cast<int>((a.M + 7) / 8);   // 1 to 8 token tiles (5 to 8: bf16 activations only)
    pl.nb = 1;
    const int max_warps = pl.nt >= 5 ? 8 : 16;   // (six and eight token tiles need about 200 registers per thread)
    pl.warps = std::min(want_warps, max_warps);
    if (tuning && tuning->warps_per_cta > 0) pl.warps = tuning->warps_per_cta;
    if (pl.warps > max_warps) pl.warps = max_warps;
    // two weight pieces in flight per row block a warp carries keep HBM busy; whatever shared memory
    // is left holds activation pieces
    pl.stages = 2 * pl.nb;
    if (tuning && tuning->stages > 0) pl.stages = tuning->stages;
    if (pl.stages < 2 * pl.nb) pl.stages = 2 * pl.nb;
    if (pl.stages > 8) pl.stages = 8;
    pl.pieces = static_cast<int>(a.K / piece_k);
    pl.piece_bytes = image_piece_bytes(a.quant, pl.nt);
    const int xstage = (pl.piece_bytes + 127) & ~127;
    for (;;) {
        const size_t fixed = static_cast<size_t>(pl.warps) * pl.stages * kStageBytes + 8 * (8 + pl.warps * pl.stages) + 64;
        pl.xstages = fixed < static_cast<size_t>(kMidMaxSmem) ? static_cast<int>((kMidMaxSmem - fixed) / xstage) : 0;
        if (pl.xstages > 8) pl.xstages = 8;
        if (pl.xstages > pl.pieces) pl.xstages = pl.pieces;
        pl.smem = static_cast<size_t>(pl.xstages) * xstage + fixed;
        if (pl.xstages >= 2 || (pl.xstages >= 1 && pl.pieces == 1)) break;
        if (pl.stages > 2 * pl.nb) { --pl.stages; continue; }
        if (pl.warps > 4) { --pl.warps; continue; }
        return false;
    }
    // One CTA per SM.  Few row blocks: K is cut so that every SM has work; the cost of a cut is the
    // plane traffic and the second kernel.  Time is counted in weight pieces per warp.
    const int64_t row_blocks = (a.N + 15) / 16;
    const int sms = a.sm_count;
    int best_c = 1;
    double best_cost = 1e30;
    const int cmax = (tuning && tuning->split_k > 0) ? tuning->split_k : 16;
    for (int c = (tuning && tuning->split_k > 0) ? tuning->split_k : 1; c <= cmax && c <= pl.pieces; ++c) {
        const int64_t gx = std::max<int64_t>(1, std::min<int64_t>(sms / c, row_blocks));
        const int64_t per_cta = (row_blocks + gx - 1) / gx;
        const int64_t per_warp = (per_cta + pl.warps - 1) / pl.warps;
        const int64_t sw = (per_warp + pl.nb - 1) / pl.nb;
        const int64_t ppc = (pl.pieces + c - 1) / c;
        const double cost = static_cast<double>(sw) * pl.nb * (ppc + 2) + (c > 1 ? 10.0 + 0.5 * c : 0.0);
        if (cost < best_cost - 1e-9) { best_cost = cost; best_c = c; }
    }
    for (int c = best_c;; --c) {
        pl.pieces_per_chunk = (pl.pieces + c - 1) / c;
        pl.num_chunks = (pl.pieces + pl.pieces_per_chunk - 1) / pl.pieces_per_chunk;
        pl.grid_x = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(sms / pl.num_chunks, row_blocks)));
        pl.planes_bytes = pl.num_chunks > 1 ? static_cast<size_t>(pl.num_chunks) * a.M * a.N * 4 : 0;
        pl.image_off = (kCounterBytes + pl.planes_bytes + 255) & ~size_t(255);
        pl.image_bytes = ((static_cast<size_t>(pl.pieces) * pl.piece_bytes + 255) & ~size_t(255)) + 256;   // + tok_up
        pl.need_ws = pl.image_off + pl.image_bytes;
        if (pl.need_ws <= workspace_bytes) break;
        if (c == 1) return false;
    }
    *out = pl;
    return true;
}

// 16 warps per CTA for big layers, 8 for small ones (under 48 MB of packed weights): a small layer
// is over in a few microseconds, and the extra warps mostly add weight requests in flight, behind
// which the activation pieces queue (measured on the Qwen2.5-7B, Llama-3-8B and Llama-3-70B shapes).
bool plan_mid(const MatmulArgs& a, const mnq_tuning* tuning, size_t workspace_bytes, MidPlan* out)
{
    const int64_t packed = a.N * (a.quant == MNQ_INT4 ? a.K / 2 : a.K);
    return plan_mid_with(a, tuning, workspace_bytes, packed >= (int64_t(48) << 20) ? 16 : 8, out);
}

template <int QUANT, typename T, int NT, bool GROUPED, int NB>
int launch_mid_one(const MidParams& p, const CUtensorMap& wmap, const MidPlan& pl, cudaStream_t stream)
{
    auto* prep = &prepare_image_kernel<QUANT, T, NT>;
    auto* kern = &gemv_mid_kernel<QUANT, T, NT, GROUPED, NB>;
    static std::atomic<uint64_t> attr_set{0};   // (one flag word per template instantiation)
    if (!attribute_done_on_device(attr_set)) {
        const int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMidMaxSmem),
                                  "cudaFuncSetAttribute(gemv_mid)");
        if (rc) return rc;
        mark_attribute_done_on_device(attr_set);
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(8 * NT);
    cfg.blockDim = dim3(kPrepThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int rc = check_cuda(cudaLaunchKernelEx(&cfg, prep, p), "prepare_image launch");
    if (rc) return rc;
    cfg.gridDim = dim3(static_cast<unsigned>(pl.grid_x), static_cast<unsigned>(pl.num_chunks), 1);
    cfg.blockDim = dim3(pl.warps * 32);
    cfg.dynamicSmemBytes = pl.smem;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, p, wmap), "gemv_mid launch");
}

}  // namespace

bool gemv_mid_supported(const MatmulArgs& a, const mnq_tuning* tuning)
{
    MidPlan pl;
    return plan_mid(a, tuning, a.workspace ? a.workspace_bytes : 0, &pl);
}

size_t gemv_mid_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size, int32_t quant)
{
    MatmulArgs a{};
    a.x = a.wq = a.scales = a.zeros = reinterpret_cast<const void*>(uintptr_t(4096));
    a.M = M; a.N = N; a.K = K; a.lda = K; a.ldc = N;
    a.group_size = group_size;
    a.G = K > 0 ? static_cast<int32_t>((K + group_size - 1) / group_size) : 0;
    a.quant = quant; a.act_dtype = M > 32 ? MNQ_BF16 : MNQ_FP16; a.scale_dtype = MNQ_FP16;
    a.sm_count = 148;
    MidPlan pl;
    if (!plan_mid(a, nullptr, ~size_t(0), &pl)) return 0;
    return pl.need_ws;
}

int launch_gemv_mid(const MatmulArgs& a, const mnq_tuning* tuning, const CUtensorMap& wmap)
{
    MidPlan pl;
    if (!plan_mid(a, tuning, a.workspace ? a.workspace_bytes : 0, &pl))
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: no batched-decode plan for this problem");
    MidParams p{};
    p.x = a.x;
    p.scales = static_cast<const unsigned short*>(a.scales);
    p.zeros = static_cast<const unsigned short*>(a.zeros);
    p.out = a.out;
    unsigned char* ws = static_cast<unsigned char*>(a.workspace);
    p.image = ws + pl.image_off;
    p.tok_up = reinterpret_cast<float*>(ws + pl.image_off + pl.image_bytes - 256);
    p.partial = reinterpret_cast<float*>(ws + kCounterBytes);
    p.lda = a.lda; p.ldc = a.ldc;
    p.M = static_cast<int>(a.M); p.N = static_cast<int>(a.N); p.K = static_cast<int>(a.K); p.G = a.G;
    p.row_blocks = static_cast<int>((a.N + 15) / 16);
    p.pieces = pl.pieces; p.pieces_per_chunk = pl.pieces_per_chunk; p.num_chunks = pl.num_chunks;
    p.stages = pl.stages; p.xstages = pl.xstages;
    p.scale_bf16 = a.scale_dtype == MNQ_BF16 ? 1 : 0;
    p.weights_immutable = option_value(MNQ_OPT_WEIGHTS_IMMUTABLE) != 0 ? 1 : 0;
    p.epi = a.epi;
    const bool grouped = a.group_size < a.K;
    int rc;
#define MNQ_MID_WIDE(Q)                                                                                      \
    rc = pl.nt == 5 ? (grouped ? launch_mid_one<Q, __nv_bfloat16, 5, true, 1>(p, wmap, pl, a.stream)         \
                               : launch_mid_one<Q, __nv_bfloat16, 5, false, 1>(p, wmap, pl, a.stream))       \
       : pl.nt == 6 ? (grouped ? launch_mid_one<Q, __nv_bfloat16, 6, true, 1>(p, wmap, pl, a.stream)         \
                               : launch_mid_one<Q, __nv_bfloat16, 6, false, 1>(p, wmap, pl, a.stream))       \
       : pl.nt == 7 ? (grouped ? launch_mid_one<Q, __nv_bfloat16, 7, true, 1>(p, wmap, pl, a.stream)         \
                               : launch_mid_one<Q, __nv_bfloat16, 7, false, 1>(p, wmap, pl, a.stream))       \
                    : (grouped ? launch_mid_one<Q, __nv_bfloat16, 8, true, 1>(p, wmap, pl, a.stream)         \
                               : launch_mid_one<Q, __nv_bfloat16, 8, false, 1>(p, wmap, pl, a.stream))
#define MNQ_MID(Q, T)                                                                                        \
    rc = pl.nt == 1 ? (grouped ? launch_mid_one<Q, T, 1, true, 1>(p, wmap, pl, a.stream)                     \
                               : launch_mid_one<Q, T, 1, false, 1>(p, wmap, pl, a.stream))                   \
       : pl.nt == 4 ? (grouped ? launch_mid_one<Q, T, 4, true, 1>(p, wmap, pl, a.stream)                     \
                               : launch_mid_one<Q, T, 4, false, 1>(p, wmap, pl, a.stream))                   \
       : pl.nt == 3 ? (grouped ? launch_mid_one<Q, T, 3, true, 1>(p, wmap, pl, a.stream)                     \
                               : launch_mid_one<Q, T, 3, false, 1>(p, wmap, pl, a.stream))                   \
                    : (grouped ? launch_mid_one<Q, T, 2, true, 1>(p, wmap, pl, a.stream)                     \
                               : launch_mid_one<Q, T, 2, false, 1>(p, wmap, pl, a.stream))
    if (pl.nt > 4) {   // bf16 only (plan_mid)
        if (a.quant == MNQ_INT4) MNQ_MID_WIDE(MNQ_INT4);
        else MNQ_MID_WIDE(MNQ_INT8);
    } else if (a.quant == MNQ_INT4) {
        if (a.act_dtype == MNQ_FP16) MNQ_MID(MNQ_INT4, __half);
        else MNQ_MID(MNQ_INT4, __nv_bfloat16);
    } else {
        if (a.act_dtype == MNQ_FP16) MNQ_MID(MNQ_INT8, __half);
        else MNQ_MID(MNQ_INT8, __nv_bfloat16);
    }
#undef MNQ_MID
#undef MNQ_MID_WIDE
    if (rc || pl.num_chunks == 1) return rc;
    return launch_splitk_reduce(p.partial, a.out, p.M, p.N, a.ldc, pl.num_chunks, a.act_dtype, a.epi, a.stream);
}

// More than 32 tokens: the streaming plan (and its tensor map) does not exist, so the weight map is made here.
int launch_gemv_mid_wide(const MatmulArgs& a, const mnq_tuning* tuning)
{
    const int64_t row_bytes = a.quant == MNQ_INT4 ? a.K / 2 : a.K;
    CUtensorMap wmap;
    const int rc = encode_tensor_map_2d(&wmap, a.wq, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, static_cast<uint64_t>(row_bytes) / 4,
                                        static_cast<uint64_t>(a.N), static_cast<uint64_t>(row_bytes), kPieceBytes / 4, 16,
                                        CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    return launch_gemv_mid(a, tuning, wmap);
}

int read_mid_status(unsigned int* out, bool clear)
{
    unsigned int v = 0;
    int rc = check_cuda(cudaMemcpyFromSymbol(&v, g_mid_status, sizeof v), "cudaMemcpyFromSymbol(mid status)");
    if (rc) return rc;
    if (clear && v) {
        const unsigned int zero = 0;
        rc = check_cuda(cudaMemcpyToSymbol(g_mid_status, &zero, sizeof zero), "cudaMemcpyToSymbol(mid status)");
        if (rc) return rc;
    }
    *out = v;
    return MNQ_SUCCESS;
}

}  // namespace mnq
