// Decode-shaped fused dequantise + matmul, the compact kernel for the common case: at most 8
// tokens, every 64-byte step of a packed row a whole quantisation group (int4 group 128, int8
// group 64) or one group per row, rows a whole number of 256-byte pieces.  Same data movement
// and arithmetic as gemv_stream_kernel (gemv_stream.cu; replaces the reference's
// dequant_matmul_int{4,8}_vecmat_fp16, shaders/matmul_dequant_kernel.metal:229-345, 485-576):
// one TMA tile copy per 16-row x 256-byte piece into a per-warp ring, packed integers fed to
// m16n8k16 warp MMAs through exact encodings, scale and offset applied per group in fp32.
//
// Why a second kernel.  A launch on a Qwen2.5-7B projection lasts 12-16 microseconds, of which
// the weights stream for 6-12; the rest is what a freshly started SM spends between entry and its
// first MMA, and the last piece's arithmetic after the last byte has arrived.  This kernel keeps
// the path to the first MMA short: the first ring stage is requested by the first instructions
// (before the dependency wait if the weights are declared immutable; the second stage goes out
// behind the activation loads, which would otherwise wait for it), the activation block is staged by
// straight-line code without atomics (a group's activation sum is a shuffle reduction inside an
// aligned run of lanes), and the scales and zeros of a piece are four aligned 8-byte loads through
// pointers advanced per piece.  CTAs are small (8 warps, two per SM) so that a CTA of the next
// kernel in the stream sets up while its neighbour still streams, and row blocks are dealt out
// evenly over one wave of CTAs.
#include <cuda.h>
#include <limits.h>

#include <type_traits>

#include "gemv_mma_common.cuh"

namespace mnq {

__device__ unsigned int g_lean_status = 0;   // bit 0: a bounded wait for a weight tile gave up; bit 2: a wait for another rank


namespace {

constexpr int kPieceBytes = 256;
constexpr int kPieceSteps = kPieceBytes / kStepBytes;   // 4
constexpr int kLeanMaxSmem = 224 * 1024;
constexpr int kXPerThread = 8;                          // activation 8-blocks a thread may stage

struct LeanParams {
    const void* x;
    const unsigned short* scales;
    const unsigned short* zeros;   // may be null
    void* out;
    float* partial;                // [num_chunks][M][N]
    unsigned int* counters;        // [row blocks]
    long long lda, ldc;
    int M, N, K, G;
    int steps_per_chunk, total_steps, num_chunks;
    int stages, row_blocks;
    int scale_bf16;
    int xs_stride;                 // bytes between staged activation rows
    int xsum_bytes;                // bytes of the activation-sum area that follows the staged rows
    int weights_immutable;
    int early_pieces;              // ring stages requested before the dependency wait when the weights are immutable
    Epilogue epi;
    GatherArgs gather;             // world > 0: the result goes to every rank's gathered buffer (GATHER kernels)
    int gather_vec;                // the gathered buffers allow 16-byte stores at every row block this call writes
    int stage_rbs;                 // row blocks of output a CTA may stage before it stores them to the peers
    unsigned int spin_limit;       // polls a wait on another rank may take
};

// GROUPED: every step is one quantisation group (scale and offset applied per step); otherwise
// one group per row (applied once per row block).
// GATHER: column-sharded call (mnq_dequant_matmul_gather).  Finished row blocks are staged in shared
// memory as [token][column]; when the CTA's warps are done it stores them into every rank's gathered
// buffer through peer-mapped pointers (16-byte pieces) and reports in; the last CTA of the grid
// publishes this rank's call number in every rank's flag block and waits, bounded, for every rank's
// number to arrive here.  The protocol and the flag words are those of gemv_stream_kernel.
template <int QUANT, typename T, bool GROUPED, bool GATHER>
__global__ void __launch_bounds__(512)
gemv_lean_kernel(const __grid_constant__ LeanParams p, const __grid_constant__ CUtensorMap wmap)
{
    using MT = __half;                                     // MMA element type (see gemv_stream.cu)
    constexpr bool CONVERT_X = !std::is_same<T, __half>::value;
    constexpr int STEP = (QUANT == MNQ_INT4) ? 128 : 64;  // k per step
    constexpr int SEG = STEP / 8;                          // 8-blocks (= lanes) per step
    constexpr int STAGE_BYTES = 16 * kPieceBytes;

    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ unsigned int x_max_bits;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int warps = blockDim.x >> 5;
    const int r = lane >> 2;
    const int t = lane & 3;

    const int step_begin = blockIdx.y * p.steps_per_chunk;
    const int nsteps = min(p.total_steps, step_begin + p.steps_per_chunk) - step_begin;   // a multiple of 4
    const int ppr = nsteps / kPieceSteps;                  // pieces per row block
    // row blocks are dealt out evenly over the grid's warps: warp w of W takes [w R / W, (w + 1) R / W),
    // so with 1.5 row blocks per warp the warps of every SM get ones and twos in turn
    const long long gw = (long long)blockIdx.x * warps + warp, W = (long long)gridDim.x * warps;
    const int rb_first = static_cast<int>(gw * p.row_blocks / W);
    const int nrb = static_cast<int>((gw + 1) * p.row_blocks / W) - rb_first;
    const int rb_cta = static_cast<int>((long long)blockIdx.x * warps * p.row_blocks / W);          // the CTA's first row block
    const int nrb_cta = static_cast<int>(((long long)blockIdx.x + 1) * warps * p.row_blocks / W) - rb_cta;
    __shared__ int peers_ready_cta;   // GATHER: 1 every rank has begun this call, -1 the wait for that gave up
    const int total_pieces = nrb * ppr;

    unsigned char* xs = smem;                                                       // [M][xs_stride]
    float* xsum = reinterpret_cast<float*>(smem + p.M * p.xs_stride);               // GROUPED: [nsteps][8]; else [8] then [M][nsteps]
    // GATHER: [token][stage_rbs * 16] outputs, then one "staged" byte per row block
    T* ostage = reinterpret_cast<T*>(smem + p.M * p.xs_stride + p.xsum_bytes);
    unsigned char* staged = reinterpret_cast<unsigned char*>(ostage + (GATHER ? p.M * p.stage_rbs * 16 : 0));
    const int ostage_bytes = GATHER ? ((p.M * p.stage_rbs * 32 + p.stage_rbs + 15) & ~15) : 0;
    unsigned char* ring = smem + ((p.M * p.xs_stride + p.xsum_bytes + ostage_bytes + 1023) & ~1023) +
                          warp * (p.stages * STAGE_BYTES + 128);
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(ring + p.stages * STAGE_BYTES);

    // ---- the weight stream starts at once ------------------------------------------------------
    int iss_rbi = 0, iss_pc = 0, iss_stage = 0, iss_count = 0;
    auto issue_piece = [&]() {
        if (lane == 0) {
            const uint32_t bar = smem_u32(&bars[iss_stage]);
            mbar_expect_tx(bar, 16u * kPieceBytes);
            tma_load_2d(smem_u32(ring + iss_stage * STAGE_BYTES), &wmap, (step_begin * kStepBytes + iss_pc * kPieceBytes) >> 2,
                        (rb_first + iss_rbi) * 16, bar);
        }
        ++iss_count;
        if (++iss_stage == p.stages) iss_stage = 0;
        if (++iss_pc == ppr) { iss_pc = 0; ++iss_rbi; }
    };
    if (lane == 0) {
        for (int s = 0; s < p.stages; ++s) mbar_init(smem_u32(&bars[s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (CONVERT_X && tid == 0) x_max_bits = 0u;

    // scales and zeros of this lane's two rows (fragment rows r and r + 8): pointers to the current
    // row block's first group of this chunk, advanced by four groups per piece
    const unsigned short *sp0 = p.scales, *sp1 = p.scales, *zp0 = p.zeros, *zp1 = p.zeros;
    auto point_at = [&](int rbi) {   // (rows past N are clamped: their results are never stored)
        const int n0 = (rb_first + rbi) * 16 + r, n1 = n0 + 8;
        const size_t g0 = GROUPED ? (size_t)step_begin : 0;
        sp0 = p.scales + (size_t)min(n0, p.N - 1) * p.G + g0;
        sp1 = p.scales + (size_t)min(n1, p.N - 1) * p.G + g0;
        if (p.zeros) { zp0 = p.zeros + (size_t)min(n0, p.N - 1) * p.G + g0; zp1 = p.zeros + (size_t)min(n1, p.N - 1) * p.G + g0; }
    };
    struct ScaleRegs { uint2 s0, s1, z0, z1; };
    auto load_scales = [&](ScaleRegs& q) {   // the next four groups of both rows, then advance
        if (GROUPED) {
            q.s0 = __ldg(reinterpret_cast<const uint2*>(sp0)); q.s1 = __ldg(reinterpret_cast<const uint2*>(sp1));
            sp0 += kPieceSteps; sp1 += kPieceSteps;
            if (p.zeros) {
                q.z0 = __ldg(reinterpret_cast<const uint2*>(zp0)); q.z1 = __ldg(reinterpret_cast<const uint2*>(zp1));
                zp0 += kPieceSteps; zp1 += kPieceSteps;
            }
        } else {
            q.s0.x = __ldg(sp0); q.s1.x = __ldg(sp1);
            if (p.zeros) { q.z0.x = __ldg(zp0); q.z1.x = __ldg(zp1); }
        }
    };
    ScaleRegs sc_cur, sc_nxt;
    sc_cur.s0 = sc_cur.s1 = sc_cur.z0 = sc_cur.z1 = make_uint2(0u, 0u);
    sc_nxt = sc_cur;
    if (nrb > 0) point_at(0);
    const int early = p.weights_immutable ? p.early_pieces : 0;   // pieces requested before the dependency wait
    for (int j = 0; j < early && j < total_pieces; ++j) issue_piece();
    if (early > 0 && nrb > 0) load_scales(sc_cur);
    // Launched programmatically dependent: everything above touched only this CTA's shared memory
    // and, if the caller declared them immutable, weights, scales and zeros; every other global
    // access comes after the previous kernel in the stream has completed.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- activations: this CTA's K chunk of every token, as 8-blocks ----------------------------
    const int bpr = nsteps * SEG;                 // 8-blocks per token row
    const int x_count = p.M * bpr;                // <= kXPerThread * blockDim.x, a multiple of SEG
    const T* xg = static_cast<const T*>(p.x);
    uint4 xv[kXPerThread];
#pragma unroll
    for (int u = 0; u < kXPerThread; ++u) {
        const int i = tid + u * blockDim.x;
        if (i < x_count) {
            const int m = (p.M == 1) ? 0 : i / bpr;
            const int b = i - m * bpr;
            xv[u] = __ldg(reinterpret_cast<const uint4*>(xg + (size_t)m * p.lda + (size_t)step_begin * STEP + b * 8));
        }
    }
    for (int j = early; j < p.stages && j < total_pieces; ++j) issue_piece();   // the rest of the ring, behind the activation loads
    if (early == 0 && nrb > 0) load_scales(sc_cur);
    // Sharded call: number of this call (the same on every rank), and the announcement that this
    // rank has begun it: whatever read its gathered output of the previous call came earlier in
    // the stream, so peers may overwrite that buffer from now on.
    unsigned int call_no = 0;
    if (GATHER) {
        unsigned int* mine = p.gather.flag_peer[p.gather.rank];
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(call_no) : "l"(mine + kGatherEpochWord) : "memory");
        call_no += 1u;
        if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 0)
            for (int g = 0; g < p.gather.world; ++g)
                asm volatile("st.relaxed.sys.global.u32 [%0], %1;"
                             ::"l"(p.gather.flag_peer[g] + kGatherReadyBase + p.gather.rank), "r"(call_no) : "memory");
        if (tid == 0) peers_ready_cta = 0;
        for (int i = tid; i < p.stage_rbs; i += blockDim.x) staged[i] = 0;
    }
    float x_down = 1.f, x_up = 1.f;               // 2^-shift and 2^shift of the bf16 -> fp16 rescale
    if (CONVERT_X) {
        __syncthreads();                          // x_max_bits is zero
        unsigned int mx = 0;
#pragma unroll
        for (int u = 0; u < kXPerThread; ++u)
            if (tid + u * blockDim.x < x_count) {
                const uint32_t w[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
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
        x_up = __int_as_float((127 + sh) << 23);
    }
#pragma unroll
    for (int u = 0; u < kXPerThread; ++u) {
        const int i0 = u * blockDim.x + (tid & ~31);        // first block of this warp in this round
        if (i0 >= x_count) break;                            // (warp-uniform)
        const int i = tid + u * blockDim.x;
        const bool valid = i < x_count;                      // whole SEG-lane runs are valid or not
        const int m = (!valid || p.M == 1) ? 0 : i / bpr;
        const int b = valid ? i - m * bpr : 0;
        uint32_t v[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
        if (!valid) v[0] = v[1] = v[2] = v[3] = 0u;
        if (CONVERT_X) {   // bf16 -> fp16, times 2^-shift (exact unless the result is subnormal)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(v[e] << 16) * x_down;
                const float hi = __uint_as_float(v[e] & 0xFFFF0000u) * x_down;
                v[e] = h2_as_u32(__floats2half2_rn(lo, hi));
            }
        }
        // sum of the staged values of one step (= SEG consecutive lanes), the same bits in every lane
        float sum = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(u32_as_h2(v[e]));
            sum += f.x;
            sum += f.y;
        }
#pragma unroll
        for (int d = 1; d < SEG; d <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
        if (valid && (lane & (SEG - 1)) == 0) {
            if (GROUPED) xsum[(b / SEG) * 8 + m] = sum;
            else xsum[8 + m * nsteps + b / SEG] = sum;
        }
        if (!valid) continue;
        int pos;
        uint4 o;
        if (QUANT == MNQ_INT4) {
            // inside a 128-k step the 8-blocks are laid out [word j][lane t]; inside an 8-block the
            // order is k+0,k+4,k+2,k+6 | k+1,k+5,k+3,k+7 (low-nibble pairs, then high-nibble pairs, the
            // latter pre-multiplied by 1/16: see Enc<MNQ_INT4, __half>)
            const int step = b >> 4, bl = b & 15;
            pos = step * STEP + ((bl & 3) * 4 + (bl >> 2)) * 8;
            const __half2 k16 = __half2half2(__ushort_as_half(0x2C00));   // 1/16
            o.x = prmt(v[0], v[2], 0x5410u);
            o.y = prmt(v[1], v[3], 0x5410u);
            o.z = h2_as_u32(__hmul2(u32_as_h2(prmt(v[0], v[2], 0x7632u)), k16));
            o.w = h2_as_u32(__hmul2(u32_as_h2(prmt(v[1], v[3], 0x7632u)), k16));
        } else {
            pos = b * 8;
            o = make_uint4(v[0], v[1], v[2], v[3]);
        }
        *reinterpret_cast<uint4*>(xs + (size_t)m * p.xs_stride + (size_t)pos * 2) = o;
    }
    __syncthreads();
    if (!GROUPED) {
        // one group per row: the chunk's activation sum per token, steps added in index order
        if (warp < p.M) {
            float s = 0.f;
            for (int i = lane; i < nsteps; i += 32) s += xsum[8 + warp * nsteps + i];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
            if (lane == 0) xsum[warp] = s;
        }
        __syncthreads();
    }

    // ---- main loop ----------------------------------------------------------------------------------
    const unsigned char* xrow = xs + (size_t)min(r, p.M - 1) * p.xs_stride + ((QUANT == MNQ_INT4) ? t * 16 : t * 32);
    const bool scale_bf16 = p.scale_bf16 != 0;
    const bool has_zero = p.zeros != nullptr;
    // two 16-bit values of a register as floats
    auto widen2 = [&](uint32_t w, float& a, float& b) {
        if (scale_bf16) { a = __uint_as_float(w << 16); b = __uint_as_float(w & 0xFFFF0000u); }
        else { const float2 f = __half22float2(u32_as_h2(w)); a = f.x; b = f.y; }
    };
    // one finished output: stored (with the epilogue), or staged for the peers
    auto emit = [&](int m, int n, float v) {
        if (!GATHER) store_result<T>(p.epi, p.out, p.ldc, m, n, v);
        else ostage[(m * p.stage_rbs + (n >> 4) - rb_cta) * 16 + (n & 15)] = F16Traits<T>::from_float(v);
    };
    bool gave_up = false;
    int rb_arrived = 0;
    int stage = 0;
    uint32_t parity = 0;
    for (int rbi = 0; rbi < nrb && !gave_up; ++rbi) {
        if (!GROUPED && rbi + 1 < nrb) { point_at(rbi + 1); load_scales(sc_nxt); }   // the next row block's scale and zero
        float tot[1][4] = {{0.f, 0.f, 0.f, 0.f}};
        float acc[1][4] = {{0.f, 0.f, 0.f, 0.f}};     // !GROUPED: one chain over the whole chunk
        const float* Xp = xsum + 2 * t;
        int xoff = 0;
        for (int pc = 0; pc < ppr; ++pc) {
            if (GROUPED) {
                if (pc + 1 == ppr && rbi + 1 < nrb) point_at(rbi + 1);
                if (pc + 1 < ppr || rbi + 1 < nrb) load_scales(sc_nxt);
            }
            if (!mbar_wait(smem_u32(&bars[stage]), parity)) { gave_up = true; break; }
            const unsigned char* st0 = ring + stage * STAGE_BYTES + r * kPieceBytes + t * 16;
            const unsigned char* st1 = st0 + 8 * kPieceBytes;
            uint4 wa[kPieceSteps], wb[kPieceSteps];
#pragma unroll
            for (int ps = 0; ps < kPieceSteps; ++ps) {
                wa[ps] = *reinterpret_cast<const uint4*>(st0 + ps * kStepBytes);
                wb[ps] = *reinterpret_cast<const uint4*>(st1 + ps * kStepBytes);
            }
            if (GROUPED) {
                float sa[4], sb[4], za[4] = {0.f, 0.f, 0.f, 0.f}, zb[4] = {0.f, 0.f, 0.f, 0.f};
                widen2(sc_cur.s0.x, sa[0], sa[1]); widen2(sc_cur.s0.y, sa[2], sa[3]);
                widen2(sc_cur.s1.x, sb[0], sb[1]); widen2(sc_cur.s1.y, sb[2], sb[3]);
                if (has_zero) {
                    widen2(sc_cur.z0.x, za[0], za[1]); widen2(sc_cur.z0.y, za[2], za[3]);
                    widen2(sc_cur.z1.x, zb[0], zb[1]); widen2(sc_cur.z1.y, zb[2], zb[3]);
                }
#pragma unroll
                for (int ps = 0; ps < kPieceSteps; ++ps) {
                    const unsigned char* const xb[1] = {xrow + xoff + ps * STEP * 2};
                    float a4[1][4];
                    step_mma<QUANT, MT, 1, true>(wa[ps], wb[ps], xb, a4);
                    // S = s / alpha, Z = (beta + c) s + z (see Enc)
                    close_group<1>(tot, a4, sa[ps] * Enc<QUANT, MT>::inv_alpha, sb[ps] * Enc<QUANT, MT>::inv_alpha,
                                   fmaf(Enc<QUANT, MT>::offset, sa[ps], za[ps]), fmaf(Enc<QUANT, MT>::offset, sb[ps], zb[ps]),
                                   Xp + ps * 8);
                }
                Xp += kPieceSteps * 8;
                sc_cur = sc_nxt;
            } else {
#pragma unroll
                for (int ps = 0; ps < kPieceSteps; ++ps) {
                    const unsigned char* const xb[1] = {xrow + xoff + ps * STEP * 2};
                    step_mma<QUANT, MT, 1, false>(wa[ps], wb[ps], xb, acc);
                }
            }
            xoff += kPieceSteps * STEP * 2;
            __syncwarp();   // every lane is done reading this stage
            if (iss_count < total_pieces) issue_piece();
            if (++stage == p.stages) { stage = 0; parity ^= 1u; }
        }
        if (gave_up) break;
        if (!GROUPED) {
            float s0, s1, z0 = 0.f, z1 = 0.f, unused;
            widen2(sc_cur.s0.x, s0, unused); widen2(sc_cur.s1.x, s1, unused);
            if (has_zero) { widen2(sc_cur.z0.x, z0, unused); widen2(sc_cur.z1.x, z1, unused); }
            close_group<1>(tot, acc, s0 * Enc<QUANT, MT>::inv_alpha, s1 * Enc<QUANT, MT>::inv_alpha,
                           fmaf(Enc<QUANT, MT>::offset, s0, z0), fmaf(Enc<QUANT, MT>::offset, s1, z1), xsum + 2 * t);
            sc_cur = sc_nxt;
        }

        // ---- epilogue of this row block: accumulator i is output (m = 2t + (i & 1), n = n0 or n0 + 8)
        const int rb = rb_first + rbi;
        const int n0 = rb * 16 + r;
        if (p.num_chunks == 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int m = 2 * t + (i & 1);
                const int n = (i & 2) ? n0 + 8 : n0;
                if (m < p.M && n < p.N) emit(m, n, CONVERT_X ? tot[0][i] * x_up : tot[0][i]);
            }
            if (GATHER && lane == 0) staged[rb - rb_cta] = 1;
            continue;
        }
        float* mine = p.partial + (size_t)blockIdx.y * p.M * p.N;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int m = 2 * t + (i & 1);
            const int n = (i & 2) ? n0 + 8 : n0;
            if (m < p.M && n < p.N) __stcg(&mine[(size_t)m * p.N + n], CONVERT_X ? tot[0][i] * x_up : tot[0][i]);
        }
        __threadfence();
        __syncwarp();
        unsigned int arrival = 0;
        if (lane == 0) arrival = atomicAdd(&p.counters[rb], 1u);
        arrival = __shfl_sync(0xffffffffu, arrival, 0);
        rb_arrived = rbi + 1;
        if (arrival != (unsigned int)(p.num_chunks - 1)) continue;
        __threadfence();
        // last chunk to arrive: add the chunks in index order (deterministic), one output per lane
        // and pass with all of its loads in flight together
        for (int o = lane; o < 16 * p.M; o += 32) {
            const int m = o >> 4;
            const int n = rb * 16 + (o & 15);
            const float* src = p.partial + (size_t)m * p.N + min(n, p.N - 1);
            const size_t plane = (size_t)p.M * p.N;
            float v = 0.f;
            for (int c0 = 0; c0 < p.num_chunks; c0 += 8) {
                float part[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) part[c] = __ldcg(src + (size_t)min(c0 + c, p.num_chunks - 1) * plane);
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    if (c0 + c < p.num_chunks) v += part[c];
            }
            if (n < p.N) emit(m, n, v);
        }
        __syncwarp();
        if (lane == 0) p.counters[rb] = 0u;   // leave the counters ready for the next call
        if (GATHER && lane == 0) staged[rb - rb_cta] = 1;
    }

    if (GATHER) {
        __syncthreads();   // every warp's outputs are staged
        bool any = false;
        for (int i = 0; i < nrb_cta; ++i) any |= staged[i] != 0;
        if (tid == 0 && any) {
            // every rank has begun this call, i.e. none still reads the previous call's gathered output
            // (the words are written by the peers; nothing is read through them, so plain loads do)
            const volatile unsigned int* ready = p.gather.flag_peer[p.gather.rank] + kGatherReadyBase;
            int ok = 1;
            for (int g = 0; g < p.gather.world && ok > 0; ++g) {
                bool in = false;
                for (unsigned int spin = 0; spin < p.spin_limit && !in; ++spin) {
                    in = static_cast<int>(ready[g] - call_no) >= 0;
                    if (!in) __nanosleep(100);
                }
                if (!in) ok = -1;
            }
            peers_ready_cta = ok;
        }
        __syncthreads();
        if (any && peers_ready_cta > 0) {
            // (rank, row block, token, half of the block's 16 columns): one 16-byte store each
            const int per_rank = nrb_cta * p.M * 2;
            for (int idx = tid; idx < per_rank * p.gather.world; idx += blockDim.x) {
                const int g = idx / per_rank;
                int e = idx - g * per_rank;
                const int rbl = e / (p.M * 2);
                e -= rbl * p.M * 2;
                const int m = e >> 1, h = e & 1;
                if (!staged[rbl]) continue;
                const int n = (rb_cta + rbl) * 16 + h * 8;
                const T* src = ostage + (m * p.stage_rbs + rbl) * 16 + h * 8;
                T* dst = static_cast<T*>(p.gather.out_peer[g]) + (size_t)m * p.ldc + p.gather.n_offset + n;
                if (p.gather_vec && n + 8 <= p.N) {
                    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
                } else {
                    for (int k = 0; k < 8; ++k)
                        if (n + k < p.N) dst[k] = src[k];
                }
            }
        }
        // The thread that reports for the CTA orders every thread's peer stores (the barrier puts
        // them before it) ahead of its arrival with a device-scope fence; the last CTA to arrive has
        // thereby observed every CTA's stores, and its one system-scope fence (fences are cumulative)
        // orders them all ahead of the arrival words it sends out.  (A system-scope fence per CTA
        // cost 6-8 us per launch: three hundred of them queue behind each other.)  The last CTA then
        // waits, bounded, until every rank's word says the same here: the kernel's completion means
        // "the gathered output is complete here".
        __syncthreads();
        if (tid == 0) {
            if (any && peers_ready_cta < 0) atomicOr(&g_lean_status, 4u);
            __threadfence();
            unsigned int* mine = p.gather.flag_peer[p.gather.rank];
            const unsigned int total = gridDim.x * gridDim.y;
            if (atomicAdd(mine + kGatherCounterWord, 1u) == total - 1) {
                mine[kGatherCounterWord] = 0u;   // ready for the next call
                __threadfence_system();
                for (int g = 0; g < p.gather.world; ++g)
                    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.gather.flag_peer[g] + p.gather.rank),
                                 "r"(call_no) : "memory");
                bool all_in = true;
                for (int src = 0; src < p.gather.world && all_in; ++src) {
                    bool in = false;
                    for (unsigned int spin = 0; spin < p.spin_limit && !in; ++spin) {
                        unsigned int v;
                        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine + src) : "memory");
                        in = static_cast<int>(v - call_no) >= 0;
                        if (!in) __nanosleep(100);
                    }
                    all_in = in;
                }
                if (!all_in) atomicOr(&g_lean_status, 4u);   // a rank never reported: give up, do not hang
                asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(mine + kGatherEpochWord), "r"(call_no) : "memory");
            }
        }
    }

    if (gave_up) {
        if (lane == 0) atomicOr(&g_lean_status, 1u);
        // the arrival counters must still return to zero (the workspace is reused by later calls)
        if (p.num_chunks > 1 && lane == 0)
            for (int rbi = rb_arrived; rbi < nrb; ++rbi)
                if (atomicAdd(&p.counters[rb_first + rbi], 1u) == (unsigned int)(p.num_chunks - 1))
                    p.counters[rb_first + rbi] = 0u;
        // copies already requested may still land in this CTA's shared memory
        for (int k = 0; k < p.stages; ++k) {
            mbar_wait(smem_u32(&bars[stage]), parity);
            if (++stage == p.stages) { stage = 0; parity ^= 1u; }
        }
    }
}

template <int QUANT, typename T, bool GROUPED, bool GATHER>
int launch_lean_one(const LeanParams& p, const CUtensorMap& wmap, dim3 grid, int threads, size_t smem, cudaStream_t stream)
{
    auto* kern = &gemv_lean_kernel<QUANT, T, GROUPED, GATHER>;
    static std::atomic<uint64_t> attr_set{0};   // (one flag word per template instantiation)
    if (smem > 48 * 1024 && !attribute_done_on_device(attr_set)) {
        const int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kLeanMaxSmem),
                                  "cudaFuncSetAttribute(gemv_lean)");
        if (rc) return rc;
        mark_attribute_done_on_device(attr_set);
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, p, wmap), "gemv_lean launch");
}

// row blocks one CTA handles at most (they are dealt out evenly over one wave of CTAs)
int lean_grid_x(const MatmulArgs& a, const LeanShape& s)
{
    const int64_t row_blocks = (a.N + 15) / 16;
    const int64_t want = (row_blocks + s.warps - 1) / s.warps;
    const int64_t cap = s.resident_ctas / s.num_chunks > 0 ? s.resident_ctas / s.num_chunks : 1;
    return static_cast<int>(want < cap ? want : cap);
}

size_t lean_smem(const MatmulArgs& a, const LeanShape& s, int* xs_stride, int* xsum_bytes, int* stage_rbs_out = nullptr)
{
    const int step = a.quant == MNQ_INT4 ? 128 : 64;
    const bool grouped = a.group_size < a.K;
    const int64_t chunk_k = static_cast<int64_t>(s.steps_per_chunk) * step;
    *xs_stride = static_cast<int>(chunk_k * 2 + (a.quant == MNQ_INT4 ? 64 : 16));   // the pad staggers rows over banks
    *xsum_bytes = grouped ? s.steps_per_chunk * 8 * 4 : (8 + static_cast<int>(a.M) * s.steps_per_chunk) * 4;
    int stage_rbs = 0, ostage_bytes = 0;
    if (a.gather.world > 0) {
        const int64_t row_blocks = (a.N + 15) / 16;
        stage_rbs = static_cast<int>((row_blocks + lean_grid_x(a, s) - 1) / lean_grid_x(a, s)) + 1;
        ostage_bytes = (static_cast<int>(a.M) * stage_rbs * 32 + stage_rbs + 15) & ~15;
    }
    if (stage_rbs_out) *stage_rbs_out = stage_rbs;
    return ((static_cast<size_t>(a.M) * *xs_stride + *xsum_bytes + ostage_bytes + 1023) & ~size_t(1023)) +
           static_cast<size_t>(s.warps) * (static_cast<size_t>(s.stages) * 16 * kPieceBytes + 128);
}

}  // namespace

bool gemv_lean_supported(const MatmulArgs& a, const LeanShape& s)
{
    const int step = a.quant == MNQ_INT4 ? 128 : 64;
    if (a.M < 1 || a.M > 8 || a.swiglu_h > 0) return false;
    if (a.gather.world > 0 && (a.epi.kind != MNQ_EPI_NONE || a.epi.out_f32)) return false;
    if (a.K % step || s.total_steps % kPieceSteps) return false;                       // whole pieces only
    if (s.num_chunks > 1 && s.steps_per_chunk % kPieceSteps) return false;
    const bool grouped = a.group_size < a.K;
    if (grouped) {
        if (a.group_size != step || a.G % kPieceSteps) return false;                    // a step is a group; 8-byte scale loads
        if (reinterpret_cast<uintptr_t>(a.scales) % 8 || (a.zeros && reinterpret_cast<uintptr_t>(a.zeros) % 8)) return false;
    }
    if (reinterpret_cast<uintptr_t>(a.x) % 16 || a.lda % 8) return false;
    const int64_t blocks = a.M * static_cast<int64_t>(s.steps_per_chunk) * (step / 8);
    if (blocks > static_cast<int64_t>(kXPerThread) * s.warps * 32) return false;       // activation block staged in one go
    int xs_stride, xsum_bytes;
    return lean_smem(a, s, &xs_stride, &xsum_bytes) <= kLeanMaxSmem;
}

int launch_gemv_lean(const MatmulArgs& a, const LeanShape& s, const CUtensorMap& wmap)
{
    LeanParams p{};
    p.x = a.x;
    p.scales = static_cast<const unsigned short*>(a.scales);
    p.zeros = static_cast<const unsigned short*>(a.zeros);
    p.out = a.out;
    p.lda = a.lda; p.ldc = a.ldc;
    p.M = static_cast<int>(a.M); p.N = static_cast<int>(a.N); p.K = static_cast<int>(a.K); p.G = a.G;
    p.steps_per_chunk = s.steps_per_chunk; p.total_steps = s.total_steps; p.num_chunks = s.num_chunks;
    p.stages = s.stages;
    p.row_blocks = static_cast<int>((a.N + 15) / 16);
    p.scale_bf16 = a.scale_dtype == MNQ_BF16 ? 1 : 0;
    const size_t smem = lean_smem(a, s, &p.xs_stride, &p.xsum_bytes, &p.stage_rbs);
    p.gather = a.gather;
    p.spin_limit = static_cast<unsigned int>(option_value(MNQ_OPT_PEER_WAIT_POLLS));
    if (a.gather.world > 0) {   // 16-byte peer stores: every row block starts on a 16-byte boundary of every buffer
        bool ok = (a.ldc * 2) % 16 == 0 && (a.gather.n_offset * 2) % 16 == 0;
        for (int g = 0; g < a.gather.world; ++g) ok = ok && reinterpret_cast<uintptr_t>(a.gather.out_peer[g]) % 16 == 0;
        p.gather_vec = ok ? 1 : 0;
    }
    p.weights_immutable = option_value(MNQ_OPT_WEIGHTS_IMMUTABLE) != 0 ? 1 : 0;
    // One stage of the ring goes out before the dependency wait, the rest behind the activation loads: the
    // L2 serves requests in arrival order, so every early weight request delays the activations (measured on
    // the Qwen2.5-7B gate+up shape: 17.8 us per launch with none early, 14.8 with one stage, 15.7 with both).
    p.early_pieces = 1;
    p.epi = a.epi;
    if (s.num_chunks > 1) {
        unsigned char* ws = static_cast<unsigned char*>(a.workspace);
        p.counters = reinterpret_cast<unsigned int*>(ws);
        p.partial = reinterpret_cast<float*>(ws + kCounterBytes);
    }
    // one wave of CTAs at most: the rest is dealt out inside the kernel
    const dim3 grid(static_cast<unsigned>(lean_grid_x(a, s)), static_cast<unsigned>(s.num_chunks), 1);
    const int threads = s.warps * 32;
    const bool grouped = a.group_size < a.K;
    const bool gather = a.gather.world > 0;
#define MNQ_LEAN(Q, T)                                                                                  \
    return grouped ? (gather ? launch_lean_one<Q, T, true, true>(p, wmap, grid, threads, smem, a.stream)   \
                             : launch_lean_one<Q, T, true, false>(p, wmap, grid, threads, smem, a.stream)) \
                   : (gather ? launch_lean_one<Q, T, false, true>(p, wmap, grid, threads, smem, a.stream)  \
                             : launch_lean_one<Q, T, false, false>(p, wmap, grid, threads, smem, a.stream))
    if (a.quant == MNQ_INT4) {
        if (a.act_dtype == MNQ_FP16) MNQ_LEAN(MNQ_INT4, __half);
        MNQ_LEAN(MNQ_INT4, __nv_bfloat16);
    }
    if (a.act_dtype == MNQ_FP16) MNQ_LEAN(MNQ_INT8, __half);
    MNQ_LEAN(MNQ_INT8, __nv_bfloat16);
#undef MNQ_LEAN
}



int read_lean_status(unsigned int* out, bool clear)
{
    unsigned int v = 0;
    int rc = check_cuda(cudaMemcpyFromSymbol(&v, g_lean_status, sizeof v), "cudaMemcpyFromSymbol(lean status)");
    if (rc) return rc;
    if (clear && v) {
        const unsigned int zero = 0;
        rc = check_cuda(cudaMemcpyToSymbol(g_lean_status, &zero, sizeof zero), "cudaMemcpyToSymbol(lean status)");
        if (rc) return rc;
    }
    *out = v;
    return MNQ_SUCCESS;
}

}  // namespace mnq
