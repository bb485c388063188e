// Decode-shaped fused dequantise + matmul (M <= 32 activation rows), plus the
// any-shape guarded kernel.
//
// Replaces the reference's dequant_matmul_int{4,8}_vecmat_fp16
// (shaders/matmul_dequant_kernel.metal:229-345, 485-576), but computes every row
// m < M (the reference kernels only ever write row 0).
//
// The kernel is bound by HBM: each packed weight byte is read once with 128-bit
// no-L1-allocate loads, several loads in flight per lane.  A warp owns 16 output
// rows n.  The four lanes that share a row read 4 x LW consecutive bytes of it per
// step; the nibbles / bytes are turned into exact (q-8) / q values in registers
// (mnq_common.cuh) and multiplied against up to NT x 8 activation rows with
// m16n8k16 warp MMAs whose accumulators are fp32 - the K reduction happens inside
// the MMA (16 k per instruction, 4 lanes x 4 k) instead of a shuffle tree.  Scales
// are applied to the fp32 partial sum of each quantisation group and zeros via the
// per-group sum of activations:
//     out[m,n] = sum_g ( s[n,g] * sum_{k in g} (q-8) x[m,k]  -  z[n,g] * sum_{k in g} x[m,k] )
// so the integers entering the MMA are exact in fp16 and in bf16.
//
// When there are too few 16-row blocks to fill the GPU the K range is cut into
// chunks (grid.y); each CTA writes its fp32 partial tile to the workspace and the
// last CTA to arrive for a row tile adds the chunks in a fixed order (deterministic
// result), writes the output and clears the arrival counter.
#include <limits.h>

#include "mnq_common.cuh"

namespace mnq {
namespace {

constexpr int kMaxSplitK = 32;
constexpr int kMaxSmemBytes = 200 * 1024;

struct GemvParams {
    const void* x;
    const uint8_t* wq;
    const void* scales;
    const void* zeros;
    void* out;
    float* partial;          // [num_chunks][M][N] fp32 (split-K only)
    unsigned int* counters;  // [row tiles] arrival counters (split-K only)
    int M, N, K;
    long long lda, ldc;
    int row_bytes;        // packed bytes per weight row
    int group_size;       // INT_MAX when there is a single group per row
    int steps_per_group;  // group_size / STEP, INT_MAX for a single group
    int G;                // scale/zero columns
    int scale_dtype;
    Epilogue epi;         // applied to the fp32 result before the store
    int steps_per_chunk;  // chunk length in steps
    int total_steps;      // ceil(K / STEP)
    int num_chunks;
    int segs;             // upper bound of groups touched by one chunk
    int xs_stride;        // bytes between activation rows in shared memory
    int x_vec_ok;         // activations can be read with 16-byte loads
};

template <int WPL> struct Words { uint32_t w[WPL]; };

template <int LW>
__device__ __forceinline__ Words<LW / 4> load_words(const uint8_t* p, bool valid)
{
    Words<LW / 4> r;
    if (!valid) {
#pragma unroll
        for (int i = 0; i < LW / 4; ++i) r.w[i] = 0u;
        return r;
    }
    if (LW == 16) {
        const uint4 v = ldg_stream_16(p);
        r.w[0] = v.x; r.w[1 % (LW / 4)] = v.y; r.w[2 % (LW / 4)] = v.z; r.w[3 % (LW / 4)] = v.w;
    } else if (LW == 8) {
        const uint2 v = ldg_stream_8(p);
        r.w[0] = v.x; r.w[1 % (LW / 4)] = v.y;
    } else {
        r.w[0] = ldg_stream_4(p);
    }
    return r;
}

__device__ __forceinline__ float load16_as_float(const void* base, long long idx, int dtype)
{
    return widen16(base, static_cast<size_t>(idx), dtype);
}

// QUANT: MNQ_INT4 / MNQ_INT8.  T: __half / __nv_bfloat16 (activations and output).
// LW: bytes of one weight row a lane reads per step (16, 8 or 4).
// NT: activation rows handled = NT * 8.
template <int QUANT, typename T, int LW, int NT>
__global__ void __launch_bounds__(512)
gemv_mma_kernel(const GemvParams p)
{
    constexpr int WPL = LW / 4;                                  // 32-bit words per lane per step
    constexpr int STEP = (QUANT == MNQ_INT4) ? 8 * LW : 4 * LW;  // k per step (4 lanes x LW bytes)
    constexpr int STEP_BYTES = 4 * LW;                           // packed bytes of a row per step
    constexpr int U = 4;                                         // loads kept in flight per lane-row

    extern __shared__ __align__(16) unsigned char smem[];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int warps = blockDim.x >> 5;
    const int rows_per_cta = warps * 16;
    const int row_tile0 = blockIdx.x * rows_per_cta;
    const int chunk = blockIdx.y;

    const int step_begin = chunk * p.steps_per_chunk;
    const int step_end = min(p.total_steps, step_begin + p.steps_per_chunk);
    const int nsteps = step_end - step_begin;
    const int k_begin = step_begin * STEP;
    const int seg0 = (p.group_size == INT_MAX) ? 0 : k_begin / p.group_size;
    const bool has_zero = (p.zeros != nullptr);

    // ---- shared memory carve-up ------------------------------------------------
    unsigned char* xs = smem;                                                   // [M][xs_stride]
    float* ssc = reinterpret_cast<float*>(smem + (size_t)p.M * p.xs_stride);    // [rows][segs]
    float* szr = ssc + rows_per_cta * p.segs;                                   // [rows][segs]
    float* xsum = szr + (has_zero ? rows_per_cta * p.segs : 0);                 // [segs][NT*8]

    // ---- lane geometry -----------------------------------------------------------
    const int r = lane >> 2;  // row within the 16-row block (and r + 8); also the MMA column
    const int t = lane & 3;
    const int n0 = row_tile0 + warp * 16 + r;
    const int n1 = n0 + 8;
    const uint8_t* row0 = p.wq + (size_t)min(n0, p.N - 1) * p.row_bytes;
    const uint8_t* row1 = p.wq + (size_t)min(n1, p.N - 1) * p.row_bytes;
    const int lane_byte0 = step_begin * STEP_BYTES + t * LW;

    // ---- start streaming weights before anything else ---------------------------
    Words<WPL> wa[U], wb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int off = lane_byte0 + u * STEP_BYTES;
        const bool ok = (u < nsteps) && (off + LW <= p.row_bytes);
        wa[u] = load_words<LW>(row0 + off, ok);
        wb[u] = load_words<LW>(row1 + off, ok);
    }

    // ---- stage activations (re-ordered for the MMA), group sums, scales, zeros --
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
                    const T lo = *reinterpret_cast<const T*>(reinterpret_cast<const unsigned short*>(&v[e]));
                    const T hi = *reinterpret_cast<const T*>(reinterpret_cast<const unsigned short*>(&v[e]) + 1);
                    s += F16Traits<T>::to_float(lo) + F16Traits<T>::to_float(hi);
                }
                const int seg = (p.group_size == INT_MAX) ? 0 : (k / p.group_size - seg0);
                atomicAdd(&xsum[seg * (NT * 8) + m], s);
            }
            int pos;  // element position inside the staged row
            uint4 o;
            if (QUANT == MNQ_INT4) {
                // order inside an 8-block: k+0,k+4,k+1,k+5,k+2,k+6,k+3,k+7 (UnpackInt4 pairing);
                // blocks of one step are laid out [word j][lane t] so that the four lanes of a
                // row read 64 contiguous bytes.
                const int step = b / (STEP / 8);
                const int bl = b - step * (STEP / 8);
                const int tt = bl / WPL;
                const int jj = bl - tt * WPL;
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
        for (int i = tid; i < rows_per_cta * p.segs; i += blockDim.x) {
            const int rr = i / p.segs;
            const int sg = i - rr * p.segs;
            const int n = row_tile0 + rr;
            const int g = seg0 + sg;
            float s = 0.f, z = 0.f;
            if (n < p.N && g < p.G) {
                s = load16_as_float(p.scales, (long long)n * p.G + g, p.scale_dtype);
                if (has_zero) z = load16_as_float(p.zeros, (long long)n * p.G + g, p.scale_dtype);
            }
            ssc[i] = s;
            if (has_zero) szr[i] = z;
        }
    }
    __syncthreads();

    // ---- main loop -----------------------------------------------------------------
    float part[NT][4], tot[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) { part[nt][i] = 0.f; tot[nt][i] = 0.f; }

    // Activation row each MMA column reads.  Columns beyond M re-read row M-1: their
    // products land in accumulator columns that are never stored.
    const unsigned char* xrow[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) xrow[nt] = xs + (size_t)min(nt * 8 + r, p.M - 1) * p.xs_stride;

    int steps_left = (p.steps_per_group == INT_MAX)
                         ? INT_MAX
                         : p.steps_per_group - (step_begin % p.steps_per_group);
    int seg = 0;
    const float* my_s0 = ssc + (warp * 16 + r) * p.segs;
    const float* my_s1 = my_s0 + 8 * p.segs;
    const float* my_z0 = szr + (warp * 16 + r) * p.segs;
    const float* my_z1 = my_z0 + 8 * p.segs;

    for (int s0 = 0; s0 < nsteps; s0 += U) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = s0 + u;
            if (s < nsteps) {
                const Words<WPL> a = wa[u], bq = wb[u];
                {   // refill this slot with the load U steps ahead
                    const int sn = s + U;
                    const int off = lane_byte0 + sn * STEP_BYTES;
                    const bool ok = (sn < nsteps) && (off + LW <= p.row_bytes);
                    wa[u] = load_words<LW>(row0 + off, ok);
                    wb[u] = load_words<LW>(row1 + off, ok);
                }
                if (QUANT == MNQ_INT4) {
#pragma unroll
                    for (int j = 0; j < WPL; ++j) {
                        uint32_t A[4], B[4];
                        UnpackInt4<T>::run(a.w[j], A);
                        UnpackInt4<T>::run(bq.w[j], B);
                        const int xoff = (s * STEP + (j * 4 + t) * 8) * 2;
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const uint4 xv = *reinterpret_cast<const uint4*>(xrow[nt] + xoff);
                            mma_16x8x16<T>(part[nt], A[0], B[0], A[1], B[1], xv.x, xv.y);
                            mma_16x8x16<T>(part[nt], A[2], B[2], A[3], B[3], xv.z, xv.w);
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < WPL; ++j) {
                        uint32_t A[2], B[2];
                        UnpackInt8<T>::run(a.w[j], A);
                        UnpackInt8<T>::run(bq.w[j], B);
                        const int xoff = (s * STEP + t * LW + j * 4) * 2;
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const uint2 xv = *reinterpret_cast<const uint2*>(xrow[nt] + xoff);
                            mma_16x8x16<T>(part[nt], A[0], B[0], A[1], B[1], xv.x, xv.y);
                        }
                    }
                }
                // close the quantisation group: scale its fp32 partial sum
                if (--steps_left == 0 || s == nsteps - 1) {
                    const float sc0 = my_s0[seg], sc1 = my_s1[seg];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        tot[nt][0] = fmaf(sc0, part[nt][0], tot[nt][0]);
                        tot[nt][1] = fmaf(sc0, part[nt][1], tot[nt][1]);
                        tot[nt][2] = fmaf(sc1, part[nt][2], tot[nt][2]);
                        tot[nt][3] = fmaf(sc1, part[nt][3], tot[nt][3]);
                        part[nt][0] = part[nt][1] = part[nt][2] = part[nt][3] = 0.f;
                    }
                    if (has_zero) {
                        const float z0 = my_z0[seg], z1 = my_z1[seg];
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
        }
    }

    // ---- epilogue --------------------------------------------------------------------
    // Accumulator i of tile nt is output (m = nt*8 + 2t + (i&1), n = n0 or n1).
    if (p.num_chunks == 1) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int m = nt * 8 + 2 * t + (i & 1);
                const int n = (i & 2) ? n1 : n0;
                if (m < p.M && n < p.N) store_result<T>(p.epi, p.out, p.ldc, m, n, tot[nt][i]);
            }
        return;
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
    __syncthreads();
    __shared__ unsigned int arrival;
    if (tid == 0) arrival = atomicAdd(&p.counters[blockIdx.x], 1u);
    __syncthreads();
    if (arrival != (unsigned int)(p.num_chunks - 1)) return;
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
                store_result<T>(p.epi, p.out, p.ldc, m, n, v);
            }
        }
    if (tid == 0) p.counters[blockIdx.x] = 0u;  // leave the workspace ready for the next call
}

// ---------------------------------------------------------------------------
// Any-shape kernel: one warp per output column n, lanes stride over packed bytes,
// fp32 dequantise (product, then subtraction) and fp32 FMA, shuffle reduction.
// Handles odd tails, unaligned pointers, any group size, any M.
// ---------------------------------------------------------------------------
template <int QUANT, typename T>
__global__ void __launch_bounds__(256)
generic_kernel(const T* __restrict__ x, const uint8_t* __restrict__ wq, const void* __restrict__ scales,
               const void* __restrict__ zeros, void* __restrict__ out, int M, int N, int K, long long lda,
               long long ldc, int group_size, int G, int scale_dtype, const Epilogue epi)
{
    constexpr int MB = 4;
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int m0 = blockIdx.y * MB;
    if (n >= N) return;
    const int row_bytes = (QUANT == MNQ_INT4) ? ((K + 1) >> 1) : K;
    const uint8_t* row = wq + (size_t)n * row_bytes;
    float acc[MB] = {0.f, 0.f, 0.f, 0.f};
    constexpr int PER = (QUANT == MNQ_INT4) ? 2 : 1;
    for (int b = lane; b < row_bytes; b += 32) {
        const uint8_t byte = row[b];
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int k = b * PER + e;
            if (k >= K) break;
            int q;
            if (QUANT == MNQ_INT4) q = static_cast<int>(e ? (byte >> 4) : (byte & 0xF)) - 8;
            else q = static_cast<int>(static_cast<int8_t>(byte));
            const int g = (group_size >= K) ? 0 : k / group_size;
            const float s = widen16(scales, (size_t)n * G + g, scale_dtype);
            const float z = zeros ? widen16(zeros, (size_t)n * G + g, scale_dtype) : 0.f;
            const float w = __fsub_rn(__fmul_rn(static_cast<float>(q), s), z);
#pragma unroll
            for (int mm = 0; mm < MB; ++mm)
                if (m0 + mm < M)
                    acc[mm] = fmaf(F16Traits<T>::to_float(x[(size_t)(m0 + mm) * lda + k]), w, acc[mm]);
        }
    }
#pragma unroll
    for (int mm = 0; mm < MB; ++mm) {
        float v = acc[mm];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && m0 + mm < M) store_result<T>(epi, out, ldc, m0 + mm, n, v);
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
inline int step_k(int quant, int lw) { return quant == MNQ_INT4 ? 8 * lw : 4 * lw; }

int pick_lane_width(const MatmulArgs& a)
{
    if (a.M < 1 || a.M > 32) return 0;
    if (a.quant == MNQ_INT4 && (a.K & 1)) return 0;
    if (a.K > (1 << 28) || a.N > (1 << 30)) return 0;
    const int64_t row_bytes = a.quant == MNQ_INT4 ? a.K / 2 : a.K;
    const uintptr_t wp = reinterpret_cast<uintptr_t>(a.wq);
    const int lws[3] = {16, 8, 4};
    for (int lw : lws) {
        if (row_bytes % lw || wp % lw) continue;
        if (a.group_size < a.K && a.group_size % step_k(a.quant, lw)) continue;
        return lw;
    }
    return 0;
}

struct GemvPlan {
    int lw, nt, warps, num_chunks, steps_per_chunk, total_steps, segs, xs_stride;
    size_t smem;
};

bool plan_gemv(const MatmulArgs& a, const mnq_tuning* tuning, int lw, size_t workspace_bytes, GemvPlan* out)
{
    GemvPlan pl{};
    pl.lw = lw;
    pl.nt = a.M <= 8 ? 1 : (a.M <= 16 ? 2 : 4);
    const int step = step_k(a.quant, lw);
    pl.total_steps = static_cast<int>((a.K + step - 1) / step);
    const int64_t row_blocks = (a.N + 15) / 16;

    int warps = (tuning && tuning->warps_per_cta > 0) ? tuning->warps_per_cta : (pl.nt == 4 ? 16 : 8);
    if (warps > 16) warps = 16;
    while (warps > 1 && row_blocks < warps) warps >>= 1;
    pl.warps = warps;
    const int64_t row_tiles = (row_blocks + warps - 1) / warps;

    // K chunks: enough CTAs for ~2 per SM, bounded by the workspace and by steps.
    int chunks = 1;
    if (tuning && tuning->split_k > 0) {
        chunks = tuning->split_k;
    } else {
        const int64_t want = 2LL * a.sm_count;
        if (row_tiles < want) chunks = static_cast<int>((want + row_tiles / 2) / row_tiles);
        const int min_steps = 4;  // keep at least a few loads per lane per chunk
        if (chunks > pl.total_steps / min_steps) chunks = pl.total_steps / min_steps;
    }
    if (chunks > kMaxSplitK) chunks = kMaxSplitK;
    if (chunks > pl.total_steps) chunks = pl.total_steps;
    if (chunks < 1 || row_tiles > kMaxCounters) chunks = 1;

    const bool has_zero = a.zeros != nullptr;
    for (;; ) {
        pl.steps_per_chunk = (pl.total_steps + chunks - 1) / chunks;
        pl.num_chunks = (pl.total_steps + pl.steps_per_chunk - 1) / pl.steps_per_chunk;
        const int64_t chunk_k = static_cast<int64_t>(pl.steps_per_chunk) * step;
        pl.segs = (a.group_size >= a.K) ? 1 : static_cast<int>(chunk_k / a.group_size + 2);
        const int row_pad = (a.quant == MNQ_INT4) ? 64 : 16;
        pl.xs_stride = static_cast<int>(((chunk_k * 2 + 127) / 128) * 128 + row_pad);
        pl.smem = static_cast<size_t>(a.M) * pl.xs_stride +
                  static_cast<size_t>(warps) * 16 * pl.segs * 4 * (has_zero ? 2 : 1) +
                  (has_zero ? static_cast<size_t>(pl.segs) * pl.nt * 8 * 4 : 0);
        size_t need_ws = 0;
        if (pl.num_chunks > 1)
            need_ws = kCounterBytes + static_cast<size_t>(pl.num_chunks) * a.M * a.N * 4;
        const bool smem_ok = pl.smem <= kMaxSmemBytes;
        const bool ws_ok = need_ws <= workspace_bytes;
        if (smem_ok && ws_ok) break;
        if (!smem_ok) {  // shorter chunks
            if (chunks >= pl.total_steps || chunks >= kMaxSplitK) return false;
            ++chunks;
            continue;
        }
        // workspace too small: fewer chunks (1 chunk needs none)
        if (chunks == 1) return false;
        --chunks;
        // shrinking chunks may break the shared-memory bound; check on the next pass
        if (chunks == 1) {
            const int64_t ck = static_cast<int64_t>(pl.total_steps) * step;
            const size_t sm1 = static_cast<size_t>(a.M) * (((ck * 2 + 127) / 128) * 128 + row_pad);
            if (sm1 > kMaxSmemBytes) return false;
        }
    }
    *out = pl;
    return true;
}

template <int QUANT, typename T, int LW, int NT>
int launch_one(const GemvParams& p, dim3 grid, int threads, size_t smem, cudaStream_t stream)
{
    auto* kern = &gemv_mma_kernel<QUANT, T, LW, NT>;
    if (smem > 48 * 1024) {
        const int rc = check_cuda(
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemBytes),
            "cudaFuncSetAttribute(gemv)");
        if (rc) return rc;
    }
    kern<<<grid, threads, smem, stream>>>(p);
    return check_cuda(cudaGetLastError(), "gemv launch");
}

template <int QUANT, typename T, int LW>
int launch_nt(const GemvParams& p, int nt, dim3 grid, int threads, size_t smem, cudaStream_t stream)
{
    if (nt == 1) return launch_one<QUANT, T, LW, 1>(p, grid, threads, smem, stream);
    if (nt == 2) return launch_one<QUANT, T, LW, 2>(p, grid, threads, smem, stream);
    return launch_one<QUANT, T, LW, 4>(p, grid, threads, smem, stream);
}

template <int QUANT, typename T>
int launch_lw(const GemvParams& p, int lw, int nt, dim3 grid, int threads, size_t smem, cudaStream_t stream)
{
    if (lw == 16) return launch_nt<QUANT, T, 16>(p, nt, grid, threads, smem, stream);
    if (lw == 8) return launch_nt<QUANT, T, 8>(p, nt, grid, threads, smem, stream);
    return launch_nt<QUANT, T, 4>(p, nt, grid, threads, smem, stream);
}

}  // namespace

bool gemv_supported(const MatmulArgs& a)
{
    if (a.M > 32) return gemv_mid_supported(a, nullptr);   // 33 to 64 tokens: the batched-decode kernel, bf16 only
    if (gemv_stream_supported(a, nullptr)) return true;
    const int lw = pick_lane_width(a);
    if (!lw) return false;
    GemvPlan pl;
    return plan_gemv(a, nullptr, lw, a.workspace ? a.workspace_bytes : 0, &pl);
}

size_t gemv_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size, int32_t quant)
{
    if (M > 32) return gemv_mid_workspace_bytes(M, N, K, group_size, quant);   // (0 where that kernel does not apply)
    if (M < 1 || N < 1 || K < 1 || group_size < 1) return 0;
    // what the streaming kernel's plan asks for; at least room for a 2-way split so that a
    // caller can force one
    bool streaming = false;
    size_t need = gemv_stream_workspace_bytes(M, N, K, group_size, quant, &streaming);
    const size_t two_way = kCounterBytes + static_cast<size_t>(2) * M * N * 4;
    if (need < two_way) need = two_way;
    const size_t mid = gemv_mid_workspace_bytes(M, N, K, group_size, quant);   // 5-32 tokens: the prepared activations
    if (need < mid) need = mid;
    if (streaming) return need;
    // shapes only the register-prefetch kernel takes: bound of the chunk count plan_gemv picks
    // on its own (occupancy-driven with the fewest row tiles, or forced by the staged activations)
    constexpr int64_t kSmBound = 192;
    const int64_t row_blocks = (N + 15) / 16;
    const int64_t row_tiles_min = (row_blocks + 15) / 16;
    int64_t chunks = (2 * kSmBound + row_tiles_min / 2) / row_tiles_min;
    const int64_t by_smem = (K * 2 * M + 128 * 1024 - 1) / (128 * 1024);
    if (chunks < by_smem) chunks = by_smem;
    if (chunks < 2) chunks = 2;
    if (chunks > kMaxSplitK) chunks = kMaxSplitK;
    const size_t v1 = kCounterBytes + static_cast<size_t>(chunks) * M * N * 4;
    return v1 > need ? v1 : need;
}

int launch_gemv(const MatmulArgs& a, const mnq_tuning* tuning)
{
    const int variant = tuning ? tuning->gemv_variant : 0;
    if (a.M > 32) return launch_gemv_mid_wide(a, tuning);
    if (variant != 1 && gemv_stream_supported(a, tuning)) return launch_gemv_stream(a, tuning);
    if (variant == 2)
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: the streaming GEMV kernel cannot take this problem");
    const int lw = pick_lane_width(a);
    if (!lw) return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: shape/alignment not supported by the GEMV kernels");
    GemvPlan pl;
    if (!plan_gemv(a, tuning, lw, a.workspace ? a.workspace_bytes : 0, &pl))
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: no GEMV plan fits shared memory / workspace");

    const int step = step_k(a.quant, lw);
    GemvParams p{};
    p.x = a.x; p.wq = static_cast<const uint8_t*>(a.wq); p.scales = a.scales; p.zeros = a.zeros;
    p.out = a.out;
    p.M = static_cast<int>(a.M); p.N = static_cast<int>(a.N); p.K = static_cast<int>(a.K);
    p.lda = a.lda; p.ldc = a.ldc;
    p.row_bytes = static_cast<int>(a.quant == MNQ_INT4 ? a.K / 2 : a.K);
    const bool single_group = a.group_size >= a.K;
    p.group_size = single_group ? INT_MAX : a.group_size;
    p.steps_per_group = single_group ? INT_MAX : a.group_size / step;
    p.G = a.G; p.scale_dtype = a.scale_dtype;
    p.epi = a.epi;
    p.steps_per_chunk = pl.steps_per_chunk; p.total_steps = pl.total_steps; p.num_chunks = pl.num_chunks;
    p.segs = pl.segs; p.xs_stride = pl.xs_stride;
    p.x_vec_ok = (reinterpret_cast<uintptr_t>(a.x) % 16 == 0) && (a.lda % 8 == 0);
    const int64_t row_blocks = (a.N + 15) / 16;
    const int64_t row_tiles = (row_blocks + pl.warps - 1) / pl.warps;
    if (pl.num_chunks > 1) {
        unsigned char* ws = static_cast<unsigned char*>(a.workspace);
        p.counters = reinterpret_cast<unsigned int*>(ws);
        p.partial = reinterpret_cast<float*>(ws + kCounterBytes);
    }
    dim3 grid(static_cast<unsigned>(row_tiles), static_cast<unsigned>(pl.num_chunks), 1);
    const int threads = pl.warps * 32;
#define MNQ_GEMV(Q, T) return launch_lw<Q, T>(p, pl.lw, pl.nt, grid, threads, pl.smem, a.stream)
    if (a.quant == MNQ_INT4) {
        if (a.act_dtype == MNQ_FP16) MNQ_GEMV(MNQ_INT4, __half);
        MNQ_GEMV(MNQ_INT4, __nv_bfloat16);
    }
    if (a.act_dtype == MNQ_FP16) MNQ_GEMV(MNQ_INT8, __half);
    MNQ_GEMV(MNQ_INT8, __nv_bfloat16);
#undef MNQ_GEMV
}

int launch_generic(const MatmulArgs& a)
{
    if (a.N > INT_MAX - 16 || a.K > INT_MAX / 2 || a.M > 65535LL * 4)
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: problem too large for the generic kernel");
    const int warps = 8;
    dim3 grid(static_cast<unsigned>((a.N + warps - 1) / warps), static_cast<unsigned>((a.M + 3) / 4), 1);
#define MNQ_GEN(Q, T)                                                                              \
    generic_kernel<Q, T><<<grid, warps * 32, 0, a.stream>>>(                                       \
        static_cast<const T*>(a.x), static_cast<const uint8_t*>(a.wq), a.scales, a.zeros,          \
        a.out, (int)a.M, (int)a.N, (int)a.K, a.lda, a.ldc, a.group_size, a.G, a.scale_dtype,       \
        a.epi)
    if (a.quant == MNQ_INT4) {
        if (a.act_dtype == MNQ_FP16) MNQ_GEN(MNQ_INT4, __half); else MNQ_GEN(MNQ_INT4, __nv_bfloat16);
    } else {
        if (a.act_dtype == MNQ_FP16) MNQ_GEN(MNQ_INT8, __half); else MNQ_GEN(MNQ_INT8, __nv_bfloat16);
    }
#undef MNQ_GEN
    return check_cuda(cudaGetLastError(), "generic launch");
}

}  // namespace mnq
