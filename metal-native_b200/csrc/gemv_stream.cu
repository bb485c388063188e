// Decode-shaped fused dequantise + matmul, streaming variant: the kernel the benchmark
// shapes run.  Same arithmetic as gemv_mma_kernel (gemv.cu) - exact (q-8) / q integers
// into m16n8k16 warp MMAs with fp32 accumulators, per-group scale of the fp32 partial
// sums, zeros through per-group activation sums - but the packed weights reach the
// warps through shared memory:
//
//   * every warp owns a small ring of stages in shared memory; one stage holds a piece
//     of CH consecutive packed bytes of each of the warp's 16 weight rows;
//   * the warp fills its own stages with 16 bulk asynchronous copies (cp.async.bulk,
//     one per row, each a contiguous CH-byte read) that signal an mbarrier, so the
//     loads in flight are bounded by shared memory, not by registers or occupancy,
//     and DRAM sees long contiguous bursts;
//   * lanes then pick their MMA fragments out of the stage with conflict-free 128-bit
//     shared loads (row stride CH + 64 bytes).
//
// Requirements: packed row length a multiple of 16 bytes, 16-byte aligned base, group
// size a multiple of one step (128 k for int4, 64 k for int8) or a single group.
// Everything else runs gemv_mma_kernel or the any-shape kernel.
//
// Every wait on an mbarrier is bounded: if a copy never lands the warp records the
// fact in the status word (mnq_device_status) and leaves instead of spinning forever.
#include <limits.h>

#include "mnq_common.cuh"

namespace mnq {

__device__ unsigned int g_device_status = 0;  // bit 0: a bounded wait gave up

namespace {

constexpr int kStepBytes = 64;       // packed bytes of one row consumed per step (4 lanes x 16)
constexpr int kMaxSplitK = 32;
constexpr int kMaxSmem = 220 * 1024;
constexpr unsigned kSpinLimit = 1u << 24;

struct StreamParams {
    const void* x;
    const uint8_t* wq;
    const void* scales;
    const void* zeros;
    void* out;
    float* partial;          // [num_chunks][M][N]
    unsigned int* counters;  // [row blocks]
    int M, N, K;
    long long lda, ldc;
    int row_bytes;
    int group_size;       // INT_MAX: single group
    int steps_per_group;  // INT_MAX: single group
    int G;
    int scale_dtype;
    int steps_per_chunk;
    int total_steps;      // ceil(row_bytes / 64)
    int num_chunks;
    int segs;
    int xs_stride;
    int x_vec_ok;
    int rbw;              // row blocks per warp
    int piece_bytes;      // CH
    int stages;           // S
    int row_blocks;       // ceil(N / 16)
};

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
// Bounded wait; false if it gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
    for (unsigned i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <int QUANT, typename T, int NT>
__global__ void __launch_bounds__(512)
gemv_stream_kernel(const StreamParams p)
{
    constexpr int STEP = (QUANT == MNQ_INT4) ? 128 : 64;  // k per step

    extern __shared__ __align__(128) unsigned char smem[];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int warps = blockDim.x >> 5;
    const int chunk = blockIdx.y;
    const int r = lane >> 2;
    const int t = lane & 3;

    const int step_begin = chunk * p.steps_per_chunk;
    const int step_end = min(p.total_steps, step_begin + p.steps_per_chunk);
    const int nsteps = step_end - step_begin;
    const int k_begin = step_begin * STEP;
    const int byte_begin = step_begin * kStepBytes;
    const int byte_end = min(p.row_bytes, step_end * kStepBytes);
    const int seg0 = (p.group_size == INT_MAX) ? 0 : k_begin / p.group_size;
    const bool has_zero = (p.zeros != nullptr);

    // ---- shared memory carve-up ------------------------------------------------------
    const int CH = p.piece_bytes;
    const int RS = CH + 64;                      // row stride inside a stage
    const int stage_bytes = 16 * RS;
    const int ring_bytes = p.stages * stage_bytes;
    const int sc_elems = p.rbw * 16 * p.segs;    // per warp, per array (16-bit values)
    const int sc_bytes = ((sc_elems * 2 * (has_zero ? 2 : 1)) + 15) & ~15;
    unsigned char* xs = smem;                                         // [M][xs_stride]
    float* xsum = reinterpret_cast<float*>(xs + (size_t)p.M * p.xs_stride);   // [segs][NT*8]
    unsigned char* warp_base = reinterpret_cast<unsigned char*>(xsum + p.segs * NT * 8);
    warp_base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(warp_base) + 127) & ~uintptr_t(127));
    unsigned char* my = warp_base + (size_t)warp * (ring_bytes + sc_bytes + 64);
    unsigned char* ring = my;                                         // [stages][16][RS]
    unsigned short* ssc = reinterpret_cast<unsigned short*>(my + ring_bytes);   // [rbw][16][segs]
    unsigned short* szr = ssc + sc_elems;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(my + ring_bytes + sc_bytes);  // [stages] <= 8

    // ---- this warp's row blocks ----------------------------------------------------------
    const int rb_first = (blockIdx.x * warps + warp) * p.rbw;
    int nrb = min(p.rbw, p.row_blocks - rb_first);
    if (nrb < 0) nrb = 0;
    const int ppr = (byte_end - byte_begin + CH - 1) / CH;   // pieces per row block
    const int total_pieces = nrb * ppr;

    if (lane == 0) {
        for (int s = 0; s < p.stages; ++s) mbar_init(smem_u32(&bars[s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    auto issue_piece = [&](int j) {
        const int rbi = j / ppr;
        const int pc = j - rbi * ppr;
        const int stage = j % p.stages;
        const int b0 = byte_begin + pc * CH;
        const int bytes = min(CH, byte_end - b0);
        const uint32_t bar = smem_u32(&bars[stage]);
        if (lane == 0) mbar_expect_tx(bar, 16u * bytes);
        __syncwarp();
        if (lane < 16) {
            const int n = min((rb_first + rbi) * 16 + lane, p.N - 1);
            bulk_copy_g2s(smem_u32(ring + (size_t)stage * stage_bytes + lane * RS),
                          p.wq + (size_t)n * p.row_bytes + b0, bytes, bar);
        }
    };

    // ---- start streaming weights before anything else -----------------------------------
    for (int j = 0; j < p.stages && j < total_pieces; ++j) issue_piece(j);

    // ---- this warp's scales / zeros (raw 16-bit) -------------------------------------------
    for (int i = lane; i < nrb * 16 * p.segs; i += 32) {
        const int rr = i / p.segs;                 // rbi * 16 + row
        const int sg = i - rr * p.segs;
        const int n = rb_first * 16 + rr;
        const int g = seg0 + sg;
        unsigned short s = 0, z = 0;
        if (n < p.N && g < p.G) {
            s = __ldg(reinterpret_cast<const unsigned short*>(p.scales) + (size_t)n * p.G + g);
            if (has_zero) z = __ldg(reinterpret_cast<const unsigned short*>(p.zeros) + (size_t)n * p.G + g);
        }
        ssc[i] = s;
        if (has_zero) szr[i] = z;
    }

    // ---- stage activations (re-ordered for the MMA) and their group sums, CTA-wide -------
    if (has_zero) {
        for (int i = tid; i < p.segs * NT * 8; i += blockDim.x) xsum[i] = 0.f;
        __syncthreads();
    }
    {
        const int blocks_per_row = nsteps * (STEP / 8);
        const T* xg = static_cast<const T*>(p.x);
        for (int i = tid; i < p.M * blocks_per_row; i += blockDim.x) {
            const int m = i / blocks_per_row;
            const int b = i - m * blocks_per_row;
            const int k = k_begin + b * 8;
            uint32_t v[4];
            if (p.x_vec_ok && k + 8 <= p.K) {
                const uint4 q = __ldg(reinterpret_cast<const uint4*>(xg + (size_t)m * p.lda + k));
                v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
            } else {
                const unsigned short* xr = reinterpret_cast<const unsigned short*>(xg + (size_t)m * p.lda);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t lo = (k + 2 * e < p.K) ? xr[k + 2 * e] : 0u;
                    const uint32_t hi = (k + 2 * e + 1 < p.K) ? xr[k + 2 * e + 1] : 0u;
                    v[e] = lo | (hi << 16);
                }
            }
            if (has_zero) {
                float s = 0.f;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const unsigned short lo = static_cast<unsigned short>(v[e] & 0xFFFFu);
                    const unsigned short hi = static_cast<unsigned short>(v[e] >> 16);
                    s += F16Traits<T>::to_float(*reinterpret_cast<const T*>(&lo)) +
                         F16Traits<T>::to_float(*reinterpret_cast<const T*>(&hi));
                }
                const int seg = (p.group_size == INT_MAX) ? 0 : (k / p.group_size - seg0);
                atomicAdd(&xsum[seg * (NT * 8) + m], s);
            }
            int pos;
            uint4 o;
            if (QUANT == MNQ_INT4) {
                // inside a 128-k step: 8-blocks laid out [word j][lane t]; inside an 8-block the
                // order k+0,k+4,k+1,k+5,k+2,k+6,k+3,k+7 (the pairing UnpackInt4 produces)
                const int step = b >> 4;
                const int bl = b & 15;
                const int tt = bl >> 2;
                const int jj = bl & 3;
                pos = step * STEP + (jj * 4 + tt) * 8;
                o.x = prmt(v[0], v[2], 0x5410u);
                o.y = prmt(v[0], v[2], 0x7632u);
                o.z = prmt(v[1], v[3], 0x5410u);
                o.w = prmt(v[1], v[3], 0x7632u);
            } else {
                pos = b * 8;
                o.x = v[0]; o.y = v[1]; o.z = v[2]; o.w = v[3];
            }
            *reinterpret_cast<uint4*>(xs + (size_t)m * p.xs_stride + (size_t)pos * 2) = o;
        }
    }
    __syncthreads();

    // ---- main loop ----------------------------------------------------------------------------
    const unsigned char* xrow[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) xrow[nt] = xs + (size_t)min(nt * 8 + r, p.M - 1) * p.xs_stride;
    T* out = static_cast<T*>(p.out);
    bool gave_up = false;

    int j = 0;
    for (int rbi = 0; rbi < nrb && !gave_up; ++rbi) {
        float part[NT][2][4], tot[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) { part[nt][0][i] = 0.f; part[nt][1][i] = 0.f; tot[nt][i] = 0.f; }
        int steps_left = (p.steps_per_group == INT_MAX)
                             ? INT_MAX
                             : p.steps_per_group - (step_begin % p.steps_per_group);
        int seg = 0;
        const unsigned short* s0p = ssc + (rbi * 16 + r) * p.segs;
        const unsigned short* s1p = s0p + 8 * p.segs;
        const unsigned short* z0p = szr + (rbi * 16 + r) * p.segs;
        const unsigned short* z1p = z0p + 8 * p.segs;
        int s = 0;   // step index inside the chunk

        for (int pc = 0; pc < ppr; ++pc, ++j) {
            const int stage = j % p.stages;
            const uint32_t parity = (j / p.stages) & 1;
            if (!mbar_wait(smem_u32(&bars[stage]), parity)) { gave_up = true; break; }
            const int b0 = pc * CH;
            const int bytes = min(CH, byte_end - byte_begin - b0);
            const int psteps = (bytes + kStepBytes - 1) / kStepBytes;
            const unsigned char* st0 = ring + (size_t)stage * stage_bytes + r * RS + t * 16;
            const unsigned char* st1 = st0 + 8 * RS;
            for (int ps = 0; ps < psteps; ++ps, ++s) {
                const bool valid = (ps * kStepBytes + t * 16 + 16 <= bytes);
                uint4 wa = make_uint4(0, 0, 0, 0), wb = make_uint4(0, 0, 0, 0);
                if (valid) {
                    wa = *reinterpret_cast<const uint4*>(st0 + ps * kStepBytes);
                    wb = *reinterpret_cast<const uint4*>(st1 + ps * kStepBytes);
                }
                const uint32_t aw[4] = {wa.x, wa.y, wa.z, wa.w};
                const uint32_t bw[4] = {wb.x, wb.y, wb.z, wb.w};
                if (QUANT == MNQ_INT4) {
#pragma unroll
                    for (int jw = 0; jw < 4; ++jw) {
                        uint32_t A[4], B[4];
                        UnpackInt4<T>::run(aw[jw], A);
                        UnpackInt4<T>::run(bw[jw], B);
                        const int xoff = (s * STEP + (jw * 4 + t) * 8) * 2;
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const uint4 xv = *reinterpret_cast<const uint4*>(xrow[nt] + xoff);
                            mma_16x8x16<T>(part[nt][0], A[0], B[0], A[1], B[1], xv.x, xv.y);
                            mma_16x8x16<T>(part[nt][1], A[2], B[2], A[3], B[3], xv.z, xv.w);
                        }
                    }
                } else {
#pragma unroll
                    for (int jw = 0; jw < 4; jw += 2) {
                        uint32_t A0[2], B0[2], A1[2], B1[2];
                        UnpackInt8<T>::run(aw[jw], A0);
                        UnpackInt8<T>::run(bw[jw], B0);
                        UnpackInt8<T>::run(aw[jw + 1], A1);
                        UnpackInt8<T>::run(bw[jw + 1], B1);
                        const int xoff = (s * STEP + t * 16 + jw * 4) * 2;
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const uint4 xv = *reinterpret_cast<const uint4*>(xrow[nt] + xoff);
                            mma_16x8x16<T>(part[nt][0], A0[0], B0[0], A0[1], B0[1], xv.x, xv.y);
                            mma_16x8x16<T>(part[nt][1], A1[0], B1[0], A1[1], B1[1], xv.z, xv.w);
                        }
                    }
                }
                if (--steps_left == 0 || s == nsteps - 1) {
                    const float sc0 = (p.scale_dtype == MNQ_BF16)
                                          ? __uint_as_float((uint32_t)s0p[seg] << 16)
                                          : __half2float(__ushort_as_half(s0p[seg]));
                    const float sc1 = (p.scale_dtype == MNQ_BF16)
                                          ? __uint_as_float((uint32_t)s1p[seg] << 16)
                                          : __half2float(__ushort_as_half(s1p[seg]));
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        tot[nt][0] = fmaf(sc0, part[nt][0][0] + part[nt][1][0], tot[nt][0]);
                        tot[nt][1] = fmaf(sc0, part[nt][0][1] + part[nt][1][1], tot[nt][1]);
                        tot[nt][2] = fmaf(sc1, part[nt][0][2] + part[nt][1][2], tot[nt][2]);
                        tot[nt][3] = fmaf(sc1, part[nt][0][3] + part[nt][1][3], tot[nt][3]);
#pragma unroll
                        for (int i = 0; i < 4; ++i) { part[nt][0][i] = 0.f; part[nt][1][i] = 0.f; }
                    }
                    if (has_zero) {
                        const float z0 = (p.scale_dtype == MNQ_BF16)
                                             ? __uint_as_float((uint32_t)z0p[seg] << 16)
                                             : __half2float(__ushort_as_half(z0p[seg]));
                        const float z1 = (p.scale_dtype == MNQ_BF16)
                                             ? __uint_as_float((uint32_t)z1p[seg] << 16)
                                             : __half2float(__ushort_as_half(z1p[seg]));
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const float2 xsv =
                                *reinterpret_cast<const float2*>(&xsum[seg * (NT * 8) + nt * 8 + 2 * t]);
                            tot[nt][0] = fmaf(-z0, xsv.x, tot[nt][0]);
                            tot[nt][1] = fmaf(-z0, xsv.y, tot[nt][1]);
                            tot[nt][2] = fmaf(-z1, xsv.x, tot[nt][2]);
                            tot[nt][3] = fmaf(-z1, xsv.y, tot[nt][3]);
                        }
                    }
                    steps_left = p.steps_per_group;
                    ++seg;
                }
            }
            __syncwarp();   // every lane is done reading this stage
            if (j + p.stages < total_pieces) issue_piece(j + p.stages);
        }
        if (gave_up) break;

        // ---- epilogue of this row block ---------------------------------------------------
        const int rb = rb_first + rbi;
        const int n0 = rb * 16 + r;
        const int n1 = n0 + 8;
        if (p.num_chunks == 1) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int m = nt * 8 + 2 * t + (i & 1);
                    const int n = (i & 2) ? n1 : n0;
                    if (m < p.M && n < p.N) out[(size_t)m * p.ldc + n] = F16Traits<T>::from_float(tot[nt][i]);
                }
            continue;
        }
        float* mine = p.partial + (size_t)chunk * p.M * p.N;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int m = nt * 8 + 2 * t + (i & 1);
                const int n = (i & 2) ? n1 : n0;
                if (m < p.M && n < p.N) __stcg(&mine[(size_t)m * p.N + n], tot[nt][i]);
            }
        __threadfence();
        __syncwarp();
        unsigned int arrival = 0;
        if (lane == 0) arrival = atomicAdd(&p.counters[rb], 1u);
        arrival = __shfl_sync(0xffffffffu, arrival, 0);
        if (arrival != (unsigned int)(p.num_chunks - 1)) continue;
        __threadfence();
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int m = nt * 8 + 2 * t + (i & 1);
                const int n = (i & 2) ? n1 : n0;
                if (m < p.M && n < p.N) {
                    float v = 0.f;
                    for (int c = 0; c < p.num_chunks; ++c)
                        v += __ldcg(&p.partial[((size_t)c * p.M + m) * p.N + n]);
                    out[(size_t)m * p.ldc + n] = F16Traits<T>::from_float(v);
                }
            }
        __syncwarp();
        if (lane == 0) p.counters[rb] = 0u;   // leave the workspace ready for the next call
    }

    if (gave_up) {
        if (lane == 0) atomicOr(&g_device_status, 1u);
        // Copies already issued may still land in this CTA's shared memory: give each
        // outstanding stage one more bounded wait before the CTA exits.
        for (int jj = j; jj < total_pieces && jj < j + p.stages; ++jj)
            mbar_wait(smem_u32(&bars[jj % p.stages]), (jj / p.stages) & 1);
    }
}

struct StreamPlan {
    int nt, warps, rbw, num_chunks, steps_per_chunk, total_steps, segs, xs_stride, piece_bytes, stages;
    size_t smem;
    unsigned grid_x;
};

bool plan_stream(const MatmulArgs& a, const mnq_tuning* tuning, size_t workspace_bytes, StreamPlan* out)
{
    if (a.M < 1 || a.M > 32) return false;
    if (a.quant == MNQ_INT4 && (a.K & 1)) return false;
    if (a.K > (1 << 28) || a.N > (1 << 30)) return false;
    const int64_t row_bytes = a.quant == MNQ_INT4 ? a.K / 2 : a.K;
    if (row_bytes % 16 || reinterpret_cast<uintptr_t>(a.wq) % 16) return false;
    const int step = a.quant == MNQ_INT4 ? 128 : 64;
    if (a.group_size < a.K && a.group_size % step) return false;

    StreamPlan pl{};
    pl.nt = a.M <= 8 ? 1 : (a.M <= 16 ? 2 : 4);
    pl.total_steps = static_cast<int>((row_bytes + kStepBytes - 1) / kStepBytes);
    const int64_t row_blocks = (a.N + 15) / 16;
    const bool has_zero = a.zeros != nullptr;

    int warps = (tuning && tuning->warps_per_cta > 0) ? tuning->warps_per_cta : 8;
    if (warps > 16) warps = 16;
    while (warps > 1 && row_blocks < warps) warps >>= 1;
    pl.warps = warps;
    pl.piece_bytes = (tuning && tuning->piece_bytes > 0) ? tuning->piece_bytes : 256;
    pl.stages = (tuning && tuning->stages > 0) ? tuning->stages : 3;
    if (pl.stages > 8) pl.stages = 8;
    if (pl.piece_bytes % 64) return false;
    const int ctas_per_sm = (tuning && tuning->ctas_per_sm > 0) ? tuning->ctas_per_sm : 1;
    const int64_t slots = static_cast<int64_t>(a.sm_count) * ctas_per_sm * warps;

    int chunks = 1, rbw = 1;
    if (tuning && tuning->split_k > 0) {
        chunks = tuning->split_k;
    } else if (row_blocks < slots) {
        chunks = static_cast<int>((slots + row_blocks / 2) / row_blocks);
        const int min_steps = 4;
        if (chunks > pl.total_steps / min_steps) chunks = pl.total_steps / min_steps;
    }
    if (chunks > kMaxSplitK) chunks = kMaxSplitK;
    if (chunks > pl.total_steps) chunks = pl.total_steps;
    if (chunks < 1 || row_blocks > kMaxCounters) chunks = 1;

    for (;;) {
        pl.steps_per_chunk = (pl.total_steps + chunks - 1) / chunks;
        pl.num_chunks = (pl.total_steps + pl.steps_per_chunk - 1) / pl.steps_per_chunk;
        const int64_t units = row_blocks * pl.num_chunks;
        rbw = static_cast<int>((units + slots - 1) / slots);
        if (tuning && tuning->row_blocks_per_warp > 0) rbw = tuning->row_blocks_per_warp;
        if (rbw < 1) rbw = 1;
        pl.rbw = rbw;
        const int64_t chunk_k = static_cast<int64_t>(pl.steps_per_chunk) * step;
        pl.segs = (a.group_size >= a.K) ? 1 : static_cast<int>(chunk_k / a.group_size + 2);
        const int row_pad = (a.quant == MNQ_INT4) ? 64 : 16;
        pl.xs_stride = static_cast<int>(((chunk_k * 2 + 127) / 128) * 128 + row_pad);
        const size_t ring = static_cast<size_t>(pl.stages) * 16 * (pl.piece_bytes + 64);
        const size_t sc = ((static_cast<size_t>(rbw) * 16 * pl.segs * 2 * (has_zero ? 2 : 1)) + 15) & ~size_t(15);
        pl.smem = static_cast<size_t>(a.M) * pl.xs_stride + static_cast<size_t>(pl.segs) * pl.nt * 8 * 4 + 128 +
                  static_cast<size_t>(warps) * (ring + sc + 64);
        size_t need_ws = 0;
        if (pl.num_chunks > 1)
            need_ws = kCounterBytes + static_cast<size_t>(pl.num_chunks) * a.M * a.N * 4;
        const bool smem_ok = pl.smem <= kMaxSmem;
        const bool ws_ok = need_ws <= workspace_bytes;
        if (smem_ok && ws_ok) break;
        if (!smem_ok) {
            if (pl.stages > 2) { --pl.stages; continue; }
            if (chunks >= pl.total_steps || chunks >= kMaxSplitK) return false;
            ++chunks;
            continue;
        }
        if (chunks == 1) return false;
        --chunks;
    }
    pl.grid_x = static_cast<unsigned>((row_blocks + static_cast<int64_t>(warps) * rbw - 1) /
                                      (static_cast<int64_t>(warps) * rbw));
    *out = pl;
    return true;
}

template <int QUANT, typename T, int NT>
int launch_stream_one(const StreamParams& p, dim3 grid, int threads, size_t smem, cudaStream_t stream)
{
    auto* kern = &gemv_stream_kernel<QUANT, T, NT>;
    if (smem > 48 * 1024) {
        const int rc = check_cuda(
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem),
            "cudaFuncSetAttribute(gemv_stream)");
        if (rc) return rc;
    }
    kern<<<grid, threads, smem, stream>>>(p);
    return check_cuda(cudaGetLastError(), "gemv_stream launch");
}

template <int QUANT, typename T>
int launch_stream_nt(const StreamParams& p, int nt, dim3 grid, int threads, size_t smem, cudaStream_t stream)
{
    if (nt == 1) return launch_stream_one<QUANT, T, 1>(p, grid, threads, smem, stream);
    if (nt == 2) return launch_stream_one<QUANT, T, 2>(p, grid, threads, smem, stream);
    return launch_stream_one<QUANT, T, 4>(p, grid, threads, smem, stream);
}

}  // namespace

bool gemv_stream_supported(const MatmulArgs& a, const mnq_tuning* tuning)
{
    StreamPlan pl;
    return plan_stream(a, tuning, a.workspace ? a.workspace_bytes : 0, &pl);
}

int launch_gemv_stream(const MatmulArgs& a, const mnq_tuning* tuning)
{
    StreamPlan pl;
    if (!plan_stream(a, tuning, a.workspace ? a.workspace_bytes : 0, &pl))
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: no streaming GEMV plan for this problem");
    const int step = a.quant == MNQ_INT4 ? 128 : 64;
    StreamParams p{};
    p.x = a.x; p.wq = static_cast<const uint8_t*>(a.wq); p.scales = a.scales; p.zeros = a.zeros; p.out = a.out;
    p.M = static_cast<int>(a.M); p.N = static_cast<int>(a.N); p.K = static_cast<int>(a.K);
    p.lda = a.lda; p.ldc = a.ldc;
    p.row_bytes = static_cast<int>(a.quant == MNQ_INT4 ? a.K / 2 : a.K);
    const bool single_group = a.group_size >= a.K;
    p.group_size = single_group ? INT_MAX : a.group_size;
    p.steps_per_group = single_group ? INT_MAX : a.group_size / step;
    p.G = a.G; p.scale_dtype = a.scale_dtype;
    p.steps_per_chunk = pl.steps_per_chunk; p.total_steps = pl.total_steps; p.num_chunks = pl.num_chunks;
    p.segs = pl.segs; p.xs_stride = pl.xs_stride;
    p.x_vec_ok = (reinterpret_cast<uintptr_t>(a.x) % 16 == 0) && (a.lda % 8 == 0);
    p.rbw = pl.rbw; p.piece_bytes = pl.piece_bytes; p.stages = pl.stages;
    p.row_blocks = static_cast<int>((a.N + 15) / 16);
    if (pl.num_chunks > 1) {
        unsigned char* ws = static_cast<unsigned char*>(a.workspace);
        p.counters = reinterpret_cast<unsigned int*>(ws);
        p.partial = reinterpret_cast<float*>(ws + kCounterBytes);
    }
    dim3 grid(pl.grid_x, static_cast<unsigned>(pl.num_chunks), 1);
    const int threads = pl.warps * 32;
#define MNQ_GS(Q, T) return launch_stream_nt<Q, T>(p, pl.nt, grid, threads, pl.smem, a.stream)
    if (a.quant == MNQ_INT4) {
        if (a.act_dtype == MNQ_FP16) MNQ_GS(MNQ_INT4, __half);
        MNQ_GS(MNQ_INT4, __nv_bfloat16);
    }
    if (a.act_dtype == MNQ_FP16) MNQ_GS(MNQ_INT8, __half);
    MNQ_GS(MNQ_INT8, __nv_bfloat16);
#undef MNQ_GS
}

int read_device_status(unsigned int* out, bool clear)
{
    unsigned int v = 0;
    int rc = check_cuda(cudaMemcpyFromSymbol(&v, g_device_status, sizeof v), "cudaMemcpyFromSymbol(status)");
    if (rc) return rc;
    if (clear && v) {
        const unsigned int zero = 0;
        rc = check_cuda(cudaMemcpyToSymbol(g_device_status, &zero, sizeof zero), "cudaMemcpyToSymbol(status)");
        if (rc) return rc;
    }
    *out = v;
    return MNQ_SUCCESS;
}

}  // namespace mnq
