// Decode-shaped fused dequantise + matmul, the general streaming kernel (M <= 32).  Replaces the
// reference's dequant_matmul_int{4,8}_vecmat_fp16 (shaders/matmul_dequant_kernel.metal:229-345,
// 485-576), computing every row m < M.  The common case of at most 8 tokens runs the compact
// kernel of gemv_lean.cu, which shares this file's plan, and 5 to 32 tokens the batched kernel of
// gemv_mid.cu; this kernel takes groups that span several steps, ragged rows, the fused SwiGLU
// epilogue, the fused all-gather above 8 tokens and calls without a workspace.
//
// Data movement.  Every warp owns 16 consecutive weight rows at a time and a small
// ring of stages in shared memory; one stage holds a piece of 256 consecutive packed
// bytes of each of those rows.  One lane fills a stage with a single TMA tile copy
// (cp.async.bulk.tensor.2d over a [N, row_bytes] tensor map, box 16 rows x 256 bytes,
// out-of-range rows and bytes zero-filled) that signals an mbarrier, so the bytes in
// flight are bounded by shared memory rather than by registers or occupancy, the copy
// costs one instruction per 4 KB, and DRAM sees contiguous bursts.  Lanes pick their
// MMA fragments out of the stage with 128-bit shared loads.
//
// Arithmetic.  m16n8k16 warp MMAs with fp32 accumulators; A = 16 weight rows,
// B = up to NT x 8 activation rows.  The packed integers are fed to the MMA with (almost)
// no conversion work, using encodings that are exact in the MMA's input type:
//   int4, fp16:  a nibble masked in place is the fp16 subnormal  n * 2^-24  (low
//                nibble of a byte) or  n * 2^-20  (high nibble): 5 logic ops per 8 weights;
//   int8, fp16:  byte ^ 0x80 placed in the low mantissa bits is  (q + 128) * 2^-24;
//   int4, bf16:  0x4300 | n  =  128 + n;
//   int8, bf16:  q itself (through the fp32 2^23 trick).
// With a = alpha * (q + beta) entering the MMA, the fp32 partial sum P of one
// quantisation group gives
//     sum_k (q - c) * s * x - z * x  =  (s / alpha) * P  -  ((beta + c) * s + z) * X
// where c = 8 for int4 and 0 for int8, and X is the sum of the group's activations.
// A lane fetches the raw 16-bit scale and zero of its two rows for one piece (four steps)
// straight into registers, one piece ahead, and widens them when a group closes; X is computed
// once per CTA when the activations are staged.
//
// Start-up.  The first global accesses after the dependency wait are the activation loads; the
// ring is requested right behind them (or, when the caller has declared the weights immutable,
// before the wait).  Loads that are issued behind a ring of weight tiles come back only after
// the tiles: the L2 serves requests in arrival order and every SM asks for its ring at once.
//
// When there are too few 16-row blocks to fill the GPU the K range is cut into chunks
// (grid.y); each warp writes its fp32 partial block to the workspace and the last warp
// to arrive for a row block adds the chunks in a fixed order (deterministic), writes the
// output and clears the arrival counter.
//
// Requirements: packed row length a multiple of 16 bytes, 16-byte aligned base, group
// size a multiple of one step (128 k for int4, 64 k for int8) or a single group.
// Everything else runs gemv_mma_kernel or the any-shape kernel (gemv.cu).
//
// Every wait on an mbarrier is bounded: if a copy never lands the warp records the
// fact in the status word (mnq_device_status) and leaves instead of spinning forever.
#include <cuda.h>
#include <limits.h>

#include <type_traits>

#include "gemv_mma_common.cuh"
#include "mnq_common.cuh"

namespace mnq {

__device__ unsigned int g_device_status = 0;  // bit 0: a wait for a weight tile gave up; bit 2: a wait for another rank

namespace {

constexpr int kMaxSplitK = 32;
constexpr int kMaxSmem = 224 * 1024;

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
    int group_shift;      // log2(group_size) if it is a power of two, else -1
    int steps_per_group;  // INT_MAX: single group
    int G;
    int scale_dtype;
    int steps_per_chunk;
    int total_steps;      // ceil(row_bytes / 64)
    int num_chunks;
    int segs;             // groups touched by one chunk, padded to a multiple of 4
    int xs_stride;
    int x_vec_ok;
    int rbw;              // row blocks per warp
    int stages;
    int row_blocks;       // ceil(N / 16)
    GatherArgs gather;    // world > 0: store to every rank's gathered buffer, then wait for all slices
    int gather_vec;       // the gathered buffers allow 16-byte stores at every column this call writes
    int defer_reduce;     // K chunks are added by a reduce kernel launched after this one: only store the partial sums
    int scale_vec;        // scales / zeros of a piece's four groups can be fetched as one aligned 8-byte load per row
    int weights_immutable;  // weights, scales and zeros are not written by earlier work on the stream: prefetch them at once
    unsigned int spin_limit;   // polls a wait on another rank may take before it gives up
    Epilogue epi;         // bias / activation / residual applied before the store; fp32 output mode
    int swiglu_h;         // > 0: fused SwiGLU -- a 16-row tile is 8 gate rows (j) and the 8 up rows (H + j); out is [M, H]
};

// T is the activation / output type.  The MMAs always run in fp16: bf16 activations are
// converted while they are staged, multiplied by a power of two chosen per CTA so that the
// largest one lands below 2^15 (exact: a bf16 significand fits fp16's), and the accumulated
// result is multiplied back.  That gives bf16 callers the cheap fp16 encodings of the packed
// weights and keeps every product exact.
template <int QUANT, typename T, int NT, int CH>
__global__ void __launch_bounds__(NT >= 4 ? 256 : 512)
gemv_stream_kernel(const StreamParams p, const __grid_constant__ CUtensorMap wmap,
                   const __grid_constant__ CUtensorMap wmap8)
{
    using MT = __half;                                     // MMA element type
    constexpr bool CONVERT_X = !std::is_same<T, __half>::value;
    constexpr int STEP = (QUANT == MNQ_INT4) ? 128 : 64;  // k per step
    constexpr int RS = CH;                                 // row stride inside a stage (dense TMA box)
    constexpr int STAGE_BYTES = 16 * RS;
    constexpr int PSTEPS = CH / kStepBytes;                // steps in a full piece

    extern __shared__ __align__(128) unsigned char smem[];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int warps = blockDim.x >> 5;
    const int chunk = blockIdx.y;
    const int r = lane >> 2;
    const int t = lane & 3;
    // Fragment row r reads stage row wr (and wr + 8).  (A TMA box is dense, so rows are a
    // multiple of 128 bytes apart and the two rows a quarter-warp reads together collide on
    // banks: a 2-way conflict on 2 of the ~12 shared loads per step.)
    const int wr = r;

    const int step_begin = chunk * p.steps_per_chunk;
    const int step_end = min(p.total_steps, step_begin + p.steps_per_chunk);
    const int nsteps = step_end - step_begin;
    const int k_begin = step_begin * STEP;
    const int byte_begin = step_begin * kStepBytes;
    const int byte_end = min(p.row_bytes, step_end * kStepBytes);
    const int seg0 = (p.group_size == INT_MAX) ? 0 : k_begin / p.group_size;
    const bool has_zero = (p.zeros != nullptr);
    const bool group_is_step = (p.steps_per_group == 1);

    // ---- shared memory carve-up (offsets from the base, so every access stays a
    //      shared-space access) ---------------------------------------------------------
    const int ring_bytes = p.stages * STAGE_BYTES;
    const int xsum_off = p.M * p.xs_stride;
    const int xsumi_off = (xsum_off + p.segs * NT * 8 * 4 + 7) & ~7;
    const int warp0_off = (xsumi_off + p.segs * NT * 8 * 8 + 1023) & ~1023;
    const int per_warp = ring_bytes + 128;
    unsigned char* xs = smem;                                                  // [M][xs_stride]
    float* xsum = reinterpret_cast<float*>(smem + xsum_off);                   // [segs][NT*8]
    // the same sums in 2^-24 fixed point: integer adds commute, so the shared-memory atomics
    // below give the same bits whatever order the warps arrive in
    unsigned long long* xsumi = reinterpret_cast<unsigned long long*>(smem + xsumi_off);
    unsigned char* my = smem + warp0_off + warp * per_warp;
    unsigned char* ring = my;                                                  // [stages][16][CH]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(my + ring_bytes);  // [stages] <= 8

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

    // Producer state: next piece to request (row block, piece, stage).  One lane issues a
    // single TMA tile copy per piece; rows past N and bytes past the row end are zero-filled
    // by the TMA unit, so every piece is a full box.
    int iss_rbi = 0, iss_pc = 0, iss_stage = 0, iss_count = 0;
    auto issue_piece = [&]() {
        if (lane == 0) {
            const uint32_t bar = smem_u32(&bars[iss_stage]);
            mbar_expect_tx(bar, 16u * CH);
            if (p.swiglu_h > 0) {
                // stage rows 0..7: gate rows of this 8-row block; rows 8..15: the matching up rows
                const int j0 = (rb_first + iss_rbi) * 8;
                tma_load_2d(smem_u32(ring + iss_stage * STAGE_BYTES), &wmap8, (byte_begin + iss_pc * CH) >> 2, j0, bar);
                tma_load_2d(smem_u32(ring + iss_stage * STAGE_BYTES + 8 * RS), &wmap8, (byte_begin + iss_pc * CH) >> 2,
                            p.swiglu_h + j0, bar);
            } else {
                tma_load_2d(smem_u32(ring + iss_stage * STAGE_BYTES), &wmap, (byte_begin + iss_pc * CH) >> 2,
                            (rb_first + iss_rbi) * 16, bar);
            }
        }
        ++iss_count;
        if (++iss_stage == p.stages) iss_stage = 0;
        if (++iss_pc == ppr) { iss_pc = 0; ++iss_rbi; }
    };

    // ---- prologue ------------------------------------------------------------------------
    // Order matters for latency: the few small loads everything waits for (scales, zeros,
    // activations) are issued first, all of them before any is used, so they cost one
    // round trip and are not queued behind the bulk weight traffic; then the first weight
    // pieces are requested; only then are the small loads consumed.
    for (int i = tid; i < p.segs * NT * 8; i += blockDim.x) xsumi[i] = 0ull;
    __shared__ unsigned int x_max_bits;   // largest |activation| of this CTA's chunk, as bf16 bits
    __shared__ volatile int peers_ready_cta;   // sharded call: every rank has begun this call
    if (CONVERT_X && tid == 0) x_max_bits = 0u;
    float x_down = 1.f, x_up = 1.f;       // 2^-x_shift and 2^x_shift

    constexpr int XB = (NT == 1) ? 2 : 4;          // activation loads in flight per thread
    const int blocks_per_row = nsteps * (STEP / 8);
    const int x_count = p.M * blocks_per_row;
    const T* xg = static_cast<const T*>(p.x);
    const unsigned short* sc16 = static_cast<const unsigned short*>(p.scales);
    const unsigned short* zr16 = static_cast<const unsigned short*>(p.zeros);

    auto load_x_block = [&](int i, uint32_t (&v)[4], int& m, int& b, int& k) {
        m = (p.M == 1) ? 0 : i / blocks_per_row;
        b = i - m * blocks_per_row;
        k = k_begin + b * 8;
        if (p.x_vec_ok && k + 8 <= p.K) {
            const uint4 q = __ldg(reinterpret_cast<const uint4*>(xg + (size_t)m * p.lda + k));
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
        } else {
            const unsigned short* xr = reinterpret_cast<const unsigned short*>(xg + (size_t)m * p.lda);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t lo = (k + 2 * e < p.K) ? __ldg(xr + k + 2 * e) : 0u;
                const uint32_t hi = (k + 2 * e + 1 < p.K) ? __ldg(xr + k + 2 * e + 1) : 0u;
                v[e] = lo | (hi << 16);
            }
        }
    };
    // Called by all 32 lanes of a warp together; lanes without a block pass m = -1.
    auto store_x_block = [&](uint32_t (&v)[4], int m, int b, int k) {
        const bool valid = m >= 0;
        if (!valid) { v[0] = v[1] = v[2] = v[3] = 0u; m = 0; b = 0; k = k_begin; }
        if (CONVERT_X) {   // bf16 -> fp16, times 2^-x_shift (exact unless the result is subnormal)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(v[e] << 16) * x_down;
                const float hi = __uint_as_float(v[e] & 0xFFFF0000u) * x_down;
                v[e] = h2_as_u32(__floats2half2_rn(lo, hi));
            }
        }
        // Sum of the block's eight staged values, in a fixed order.
        float sum = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(u32_as_h2(v[e]));
            sum += f.x;
            sum += f.y;
        }
        const int sg = (p.group_size == INT_MAX) ? 0
                     : (p.group_shift >= 0 ? (k >> p.group_shift) : k / p.group_size) - seg0;
        // Lanes hold consecutive 8-blocks, so the blocks of one (group, token) sit in a run of
        // adjacent lanes: the run is added up with shuffles (a fixed tree, so the same bits every
        // time) and its first lane adds the total to the group's sum in shared memory.  Several
        // warps may contribute to one group; their totals are rounded to a 2^-24 grid and added
        // as 64-bit integers, which commute, so the result does not depend on arrival order.
        const int key = valid ? sg * (NT * 8) + m : -1;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const float other = __shfl_down_sync(0xffffffffu, sum, d);
            const int okey = __shfl_down_sync(0xffffffffu, key, d);
            if (lane + d < 32 && okey == key) sum += other;
        }
        const int pkey = __shfl_up_sync(0xffffffffu, key, 1);
        if (valid && (lane == 0 || pkey != key))
            atomicAdd(&xsumi[key], static_cast<unsigned long long>(__float2ll_rn(sum * 16777216.f)));
        if (!valid) return;
        int pos;
        uint4 o;
        if (QUANT == MNQ_INT4) {
            // inside a 128-k step the 8-blocks are laid out [word j][lane t]; inside an 8-block
            // the order is k+0,k+4,k+2,k+6 | k+1,k+5,k+3,k+7: first the pairs the low-nibble MMA
            // consumes, then the pairs of the high-nibble MMA
            const int step = b >> 4;
            const int bl = b & 15;
            pos = step * STEP + ((bl & 3) * 4 + (bl >> 2)) * 8;
            o.x = prmt(v[0], v[2], 0x5410u);   // (x0, x4)
            o.y = prmt(v[1], v[3], 0x5410u);   // (x2, x6)
            o.z = prmt(v[0], v[2], 0x7632u);   // (x1, x5)
            o.w = prmt(v[1], v[3], 0x7632u);   // (x3, x7)
            if (Enc<QUANT, MT>::hi_x_scale) {
                const __half2 k16 = __half2half2(__ushort_as_half(0x2C00));   // 1/16
                o.z = h2_as_u32(__hmul2(u32_as_h2(o.z), k16));
                o.w = h2_as_u32(__hmul2(u32_as_h2(o.w), k16));
            }
        } else {
            pos = b * 8;
            o.x = v[0]; o.y = v[1]; o.z = v[2]; o.w = v[3];
        }
        *reinterpret_cast<uint4*>(xs + (size_t)m * p.xs_stride + (size_t)pos * 2) = o;
    };
    // Scales and zeros are not staged: a lane fetches, straight into registers, the raw 16-bit
    // scale and zero of its two rows (fragment rows r and r + 8) for the PSTEPS steps of one
    // piece, one piece ahead of the piece it is multiplying, and widens them when a group closes.
    // When a step is a whole group and the rows are suitably aligned that is one 8-byte load per
    // row and array; otherwise one 16-bit load per step (steps of one group repeat its address).
    static_assert(PSTEPS == 4, "a piece's scales travel as four 16-bit values per row");
    struct ScaleRegs { uint2 s0, s1, z0, z1; };
    const bool scale_bf16 = (p.scale_dtype == MNQ_BF16);
    auto load_scales = [&](int rbi, int pc, ScaleRegs& q) {
        q.s0 = q.s1 = q.z0 = q.z1 = make_uint2(0u, 0u);
        int na, nb;
        bool oka, okb;
        if (p.swiglu_h > 0) {   // tile row -> weight row: 8 gate rows, then their 8 up rows
            const int j = (rb_first + rbi) * 8 + r;
            na = j; nb = p.swiglu_h + j;
            oka = okb = j < p.swiglu_h;
        } else {
            na = (rb_first + rbi) * 16 + r; nb = na + 8;
            oka = na < p.N; okb = nb < p.N;
        }
        const int s_abs = step_begin + pc * PSTEPS;   // first step of the piece, counted from the row start
        if (group_is_step && p.scale_vec && s_abs + PSTEPS <= p.G) {
            if (oka) {
                q.s0 = __ldg(reinterpret_cast<const uint2*>(sc16 + (size_t)na * p.G + s_abs));
                if (has_zero) q.z0 = __ldg(reinterpret_cast<const uint2*>(zr16 + (size_t)na * p.G + s_abs));
            }
            if (okb) {
                q.s1 = __ldg(reinterpret_cast<const uint2*>(sc16 + (size_t)nb * p.G + s_abs));
                if (has_zero) q.z1 = __ldg(reinterpret_cast<const uint2*>(zr16 + (size_t)nb * p.G + s_abs));
            }
            return;
        }
        uint32_t v[4][PSTEPS];
#pragma unroll
        for (int ps = 0; ps < PSTEPS; ++ps) {
            int g = (p.steps_per_group == INT_MAX) ? 0 : (group_is_step ? s_abs + ps : (s_abs + ps) / p.steps_per_group);
            g = min(g, p.G - 1);
            v[0][ps] = oka ? __ldg(sc16 + (size_t)na * p.G + g) : 0u;
            v[1][ps] = okb ? __ldg(sc16 + (size_t)nb * p.G + g) : 0u;
            v[2][ps] = (oka && has_zero) ? __ldg(zr16 + (size_t)na * p.G + g) : 0u;
            v[3][ps] = (okb && has_zero) ? __ldg(zr16 + (size_t)nb * p.G + g) : 0u;
        }
        q.s0 = make_uint2(v[0][0] | (v[0][1] << 16), v[0][2] | (v[0][3] << 16));
        q.s1 = make_uint2(v[1][0] | (v[1][1] << 16), v[1][2] | (v[1][3] << 16));
        q.z0 = make_uint2(v[2][0] | (v[2][1] << 16), v[2][2] | (v[2][3] << 16));
        q.z1 = make_uint2(v[3][0] | (v[3][1] << 16), v[3][2] | (v[3][3] << 16));
    };
    // folded scale and offset of step ps of a piece: S = s / alpha, Z = (beta + c) s + z
    auto fold = [&](const uint2& sv, const uint2& zv, int ps, float& S, float& Z) {
        const uint32_t sw = (ps & 2) ? sv.y : sv.x, zw = (ps & 2) ? zv.y : zv.x;
        const uint32_t sb = (ps & 1) ? (sw >> 16) : (sw & 0xFFFFu), zb = (ps & 1) ? (zw >> 16) : (zw & 0xFFFFu);
        float s0, z0;
        if (scale_bf16) {
            s0 = __uint_as_float(sb << 16);
            z0 = __uint_as_float(zb << 16);
        } else {
            s0 = __half2float(__ushort_as_half((unsigned short)sb));
            z0 = __half2float(__ushort_as_half((unsigned short)zb));
        }
        S = s0 * Enc<QUANT, MT>::inv_alpha;
        Z = fmaf(Enc<QUANT, MT>::offset, s0, z0);
    };

    // Immutable weights: the ring and the first scales are requested before the wait below, while
    // the previous kernel in the stream may still be running.
    ScaleRegs sc_cur, sc_nxt;
    sc_cur.s0 = sc_cur.s1 = sc_cur.z0 = sc_cur.z1 = make_uint2(0u, 0u);
    sc_nxt = sc_cur;
    // (one stage only: every early weight request delays the activation loads issued after the wait)
    const int early = p.weights_immutable ? 1 : 0;
    for (int j = 0; j < early && j < total_pieces; ++j) issue_piece();
    if (early > 0 && total_pieces > 0) load_scales(0, 0, sc_cur);
    // With a programmatic dependent launch this CTA may have started while the previous kernel
    // in the stream was still running.  Everything above touched only this CTA's shared memory
    // (and, if the caller declared them immutable, weights, scales and zeros); every other global
    // read comes after that kernel and its writes completed.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // the next kernel in the stream may be scheduled as soon as this one leaves room
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Sharded call: number of this call (the same on every rank), and the announcement that this
    // rank has begun it: whatever read its gathered output of the previous call came earlier
    // in the stream, so peers may overwrite that buffer from now on.
    unsigned int call_no = 0;
    bool peers_ready = false;
    if (p.gather.world > 0) {
        if (tid == 0) peers_ready_cta = 0;
        unsigned int* mine = p.gather.flag_peer[p.gather.rank];
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(call_no) : "l"(mine + kGatherEpochWord) : "memory");
        call_no += 1u;
        // (plain system-scope stores, all in flight together: nothing is published through this
        // word, it only has to come after the stream's earlier work, which the launch ensures)
        if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 0)
            for (int g = 0; g < p.gather.world; ++g)
                asm volatile("st.relaxed.sys.global.u32 [%0], %1;"
                             ::"l"(p.gather.flag_peer[g] + kGatherReadyBase + p.gather.rank), "r"(call_no) : "memory");
    }

    uint32_t xv[XB][4];
    int xm[XB], xb[XB], xk[XB];
#pragma unroll
    for (int u = 0; u < XB; ++u) {
        const int i = tid + u * blockDim.x;
        xm[u] = -1;
        if (i < x_count) load_x_block(i, xv[u], xm[u], xb[u], xk[u]);
    }

    // The activation loads go out ahead of the weight stream: a request issued behind a full ring
    // of weight tiles waits in the memory system until those tiles have been fetched.
    for (int j = early; j < p.stages && j < total_pieces; ++j) issue_piece();
    if (early == 0 && total_pieces > 0) load_scales(0, 0, sc_cur);
    __syncthreads();   // xsum (and x_max_bits) are zeroed

    if (CONVERT_X) {
        // largest |x| of the chunk -> power-of-two scale that puts it just below 2^15
        unsigned int mx = 0;
#pragma unroll
        for (int u = 0; u < XB; ++u)
            if (xm[u] >= 0) {
#pragma unroll
                for (int e = 0; e < 4; ++e) mx = max(mx, max(xv[u][e] & 0x7FFFu, (xv[u][e] >> 16) & 0x7FFFu));
            }
        // blocks beyond the first batch, eight loads in flight per thread (a clamped index
        // re-reads the last block, which leaves the maximum unchanged)
        for (int i0 = XB * blockDim.x + tid; i0 < x_count; i0 += 8 * blockDim.x) {
            uint32_t t4[8][4];
            int a, b, c;
#pragma unroll
            for (int u = 0; u < 8; ++u) load_x_block(min(i0 + u * (int)blockDim.x, x_count - 1), t4[u], a, b, c);
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
                for (int e = 0; e < 4; ++e) mx = max(mx, max(t4[u][e] & 0x7FFFu, (t4[u][e] >> 16) & 0x7FFFu));
        }
        mx = __reduce_max_sync(0xffffffffu, mx);
        if (lane == 0 && mx) atomicMax(&x_max_bits, mx);
        __syncthreads();
        const int E = static_cast<int>(x_max_bits >> 7);          // biased bf16 exponent of the maximum
        int sh = (E == 0) ? 0 : (E - 127) - 14;
        sh = max(-100, min(100, sh));
        x_down = __int_as_float((127 - sh) << 23);
        x_up = __int_as_float((127 + sh) << 23);
    }

    // consume the activation loads
#pragma unroll
    for (int u = 0; u < XB; ++u)
        if (__any_sync(0xffffffffu, xm[u] >= 0)) store_x_block(xv[u], xm[u], xb[u], xk[u]);
    // whatever did not fit in the first batch (M > 8)
    {
        constexpr int XB2 = 8;   // deeper batches for the bulk of a many-token activation block
        for (int i0 = XB * blockDim.x; i0 < x_count; i0 += XB2 * blockDim.x) {
            uint32_t yv[XB2][4];
            int ym[XB2], yb[XB2], yk[XB2];
#pragma unroll
            for (int u = 0; u < XB2; ++u) {
                const int i = i0 + tid + u * blockDim.x;
                load_x_block(min(i, x_count - 1), yv[u], ym[u], yb[u], yk[u]);
                if (i >= x_count) ym[u] = -1;
            }
#pragma unroll
            for (int u = 0; u < XB2; ++u)
                if (__any_sync(0xffffffffu, ym[u] >= 0)) store_x_block(yv[u], ym[u], yb[u], yk[u]);
        }
    }
    __syncthreads();
    for (int i = tid; i < p.segs * NT * 8; i += blockDim.x)
        xsum[i] = static_cast<float>(static_cast<long long>(xsumi[i])) * (1.f / 16777216.f);
    __syncthreads();

    // ---- main loop ----------------------------------------------------------------------------
    // this lane's position inside a staged activation row: 16 bytes per 8-block at lane t (int4),
    // 32 bytes at lane t (int8)
    const int x_lane_off = (QUANT == MNQ_INT4) ? t * 16 : t * 32;
    const unsigned char* xrow[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
        xrow[nt] = xs + (size_t)min(nt * 8 + r, p.M - 1) * p.xs_stride + x_lane_off;
    T* out = static_cast<T*>(p.out);
    bool gather_failed = false;
    // Every rank has begun this call, i.e. no rank still reads the previous call's gathered
    // output.  Looked up once per CTA (the first thread to need it polls the local flag words,
    // bounded; the words are written by the peers, nothing is read through them, so plain
    // volatile loads do) and remembered in shared memory for the rest.
    auto wait_peers_ready = [&]() -> bool {
        if (peers_ready) return true;
        if (gather_failed) return false;
        if (peers_ready_cta < 0) { gather_failed = true; return false; }   // another thread of the CTA already gave up
        if (!peers_ready_cta) {
            const volatile unsigned int* mine = p.gather.flag_peer[p.gather.rank] + kGatherReadyBase;
            for (int g = 0; g < p.gather.world; ++g) {
                bool in = false;
                for (unsigned int spin = 0; spin < p.spin_limit && !in; ++spin) {
                    in = static_cast<int>(mine[g] - call_no) >= 0;
                    if (!in) __nanosleep(100);
                }
                if (!in) { gather_failed = true; peers_ready_cta = -1; return false; }
            }
            peers_ready_cta = 1;
        }
        peers_ready = true;
        return true;
    };
    // Plain call: one store.  Sharded call: the same element goes to every rank's gathered buffer
    // (peer-mapped device pointers; the local rank is one of them).
    auto store_out = [&](int m, int n, float v32) {
        if (p.gather.world == 0) {
            store_result<T>(p.epi, p.out, p.ldc, m, n, v32);
        } else {
            if (!wait_peers_ready()) return;
            const T v = F16Traits<T>::from_float(v32);
            for (int g = 0; g < p.gather.world; ++g)
                static_cast<T*>(p.gather.out_peer[g])[(size_t)m * p.ldc + p.gather.n_offset + n] = v;
        }
    };
    bool gave_up = false;
    int rb_arrived = 0;   // row blocks of this warp whose arrival has been counted (K split in this kernel)

    int stage = 0;
    uint32_t parity = 0;
    // Sharded call, few tokens, no K split: a warp keeps the outputs of its (at most two) row
    // blocks in registers; after the loop the CTA lays them out as [token][column] in the
    // activation staging area and copies whole 16-byte pieces to every rank (one store
    // instruction covers 512 contiguous bytes of a peer's row instead of 16).
    const bool stage_out = (NT == 1) && p.gather.world > 0 && p.num_chunks == 1 && p.rbw <= 2 && p.gather_vec;
    float keep[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    for (int rbi = 0; rbi < nrb && !gave_up; ++rbi) {
        float acc[NT][4], tot[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) { acc[nt][i] = 0.f; tot[nt][i] = 0.f; }
        int steps_left = (p.steps_per_group == INT_MAX)
                             ? INT_MAX
                             : p.steps_per_group - (step_begin % p.steps_per_group);
        const float* Xp = xsum + 2 * t;   // advanced as groups close
        int s = 0;          // step index inside the chunk
        int xoff = 0;       // byte offset of step s in the staged activation rows
        int bytes_left = byte_end - byte_begin;

        for (int pc = 0; pc < ppr; ++pc) {
            // scales and zeros of the piece after this one (the next row block's first, at the end of a row)
            if (pc + 1 < ppr) load_scales(rbi, pc + 1, sc_nxt);
            else if (rbi + 1 < nrb) load_scales(rbi + 1, 0, sc_nxt);
            if (!mbar_wait(smem_u32(&bars[stage]), parity)) { gave_up = true; break; }
            const unsigned char* st0 = ring + stage * STAGE_BYTES + wr * RS + t * 16;
            const unsigned char* st1 = st0 + 8 * RS;
            if (bytes_left >= CH && group_is_step) {
                // full piece, one quantisation group per step: fully unrolled
                uint4 wa[PSTEPS], wb[PSTEPS];
#pragma unroll
                for (int ps = 0; ps < PSTEPS; ++ps) {
                    wa[ps] = *reinterpret_cast<const uint4*>(st0 + ps * kStepBytes);
                    wb[ps] = *reinterpret_cast<const uint4*>(st1 + ps * kStepBytes);
                }
                float Sa[PSTEPS], Sb[PSTEPS], Za[PSTEPS], Zb[PSTEPS];
#pragma unroll
                for (int ps = 0; ps < PSTEPS; ++ps) {
                    fold(sc_cur.s0, sc_cur.z0, ps, Sa[ps], Za[ps]);
                    fold(sc_cur.s1, sc_cur.z1, ps, Sb[ps], Zb[ps]);
                }
                const unsigned char* xb[NT];
#pragma unroll
                for (int ps = 0; ps < PSTEPS; ++ps) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) xb[nt] = xrow[nt] + xoff + ps * STEP * 2;
                    float a4[NT][4];
                    step_mma<QUANT, MT, NT, true>(wa[ps], wb[ps], xb, a4);
                    close_group<NT>(tot, a4, Sa[ps], Sb[ps], Za[ps], Zb[ps], Xp + ps * (NT * 8));
                }
                s += PSTEPS;
                xoff += PSTEPS * STEP * 2;
                Xp += PSTEPS * (NT * 8);
            } else {
                const int bytes = min(CH, bytes_left);
                const int psteps = (bytes + kStepBytes - 1) / kStepBytes;
                for (int ps = 0; ps < psteps; ++ps, ++s, xoff += STEP * 2) {
                    // bytes of this piece past the chunk end belong to the next chunk
                    const bool valid = (ps * kStepBytes + t * 16 + 16 <= bytes);
                    uint4 wa = make_uint4(0, 0, 0, 0), wb = make_uint4(0, 0, 0, 0);
                    if (valid) {
                        wa = *reinterpret_cast<const uint4*>(st0 + ps * kStepBytes);
                        wb = *reinterpret_cast<const uint4*>(st1 + ps * kStepBytes);
                    }
                    const unsigned char* xb[NT];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) xb[nt] = xrow[nt] + xoff;
                    step_mma<QUANT, MT, NT, false>(wa, wb, xb, acc);
                    if (--steps_left == 0 || s == nsteps - 1) {
                        float Sa, Sb, Za, Zb;
                        fold(sc_cur.s0, sc_cur.z0, ps, Sa, Za);
                        fold(sc_cur.s1, sc_cur.z1, ps, Sb, Zb);
                        close_group<NT>(tot, acc, Sa, Sb, Za, Zb, Xp);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
                        steps_left = p.steps_per_group;
                        Xp += NT * 8;
                    }
                }
            }
            bytes_left -= CH;
            sc_cur = sc_nxt;
            __syncwarp();   // every lane is done reading this stage
            if (iss_count < total_pieces) issue_piece();
            if (++stage == p.stages) { stage = 0; parity ^= 1u; }
        }
        if (gave_up) break;

        // ---- epilogue of this row block ---------------------------------------------------
        // Accumulator i of tile nt is output (m = nt*8 + 2t + (i&1), n = n0 or n1).
        const int rb = rb_first + rbi;
        const int n0 = rb * 16 + wr;
        const int n1 = n0 + 8;
        if (p.swiglu_h > 0) {
            // accumulators 0,1 are gate row j (tokens 2t, 2t+1), 2,3 the up row H + j: out = silu(gate) * up
            const int j = rb * 8 + wr;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int m = nt * 8 + 2 * t + i;
                    if (m < p.M && j < p.swiglu_h) {
                        const float gte = CONVERT_X ? tot[nt][i] * x_up : tot[nt][i];
                        const float upv = CONVERT_X ? tot[nt][i + 2] * x_up : tot[nt][i + 2];
                        out[(size_t)m * p.ldc + j] = F16Traits<T>::from_float(gte / (1.f + __expf(-gte)) * upv);
                    }
                }
            continue;
        }
        if (p.num_chunks == 1) {
            if (stage_out) {
#pragma unroll
                for (int i = 0; i < 4; ++i) keep[rbi & 1][i] = CONVERT_X ? tot[0][i] * x_up : tot[0][i];
                continue;
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int m = nt * 8 + 2 * t + (i & 1);
                    const int n = (i & 2) ? n1 : n0;
                    if (m < p.M && n < p.N)
                        store_out(m, n, CONVERT_X ? tot[nt][i] * x_up : tot[nt][i]);
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
                if (m < p.M && n < p.N) __stcg(&mine[(size_t)m * p.N + n], CONVERT_X ? tot[nt][i] * x_up : tot[nt][i]);
            }
        if (p.defer_reduce) continue;   // a second kernel adds the chunks
        __threadfence();
        __syncwarp();
        unsigned int arrival = 0;
        if (lane == 0) arrival = atomicAdd(&p.counters[rb], 1u);
        arrival = __shfl_sync(0xffffffffu, arrival, 0);
        rb_arrived = rbi + 1;
        if (arrival != (unsigned int)(p.num_chunks - 1)) continue;
        __threadfence();
        // Last chunk to arrive: add the chunks in index order (deterministic).  One output per
        // lane and pass, its loads issued together (indices past the last chunk are clamped and
        // their values dropped), so the whole reduction costs one round trip to L2 per pass.
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
            if (n < p.N) store_out(m, n, v);
        }
        __syncwarp();
        if (lane == 0) p.counters[rb] = 0u;   // leave the counters ready for the next call
    }

    if (p.gather.world > 0) {
        // Every CTA orders its peer stores before its arrival (device scope); the last CTA of the
        // grid tells every rank that this rank's slice of this call is complete and waits
        // (bounded) until every rank has said the same here, so that the kernel's completion
        // means "the gathered output is complete on this rank".
        if (stage_out) {
            __syncthreads();   // every warp is done reading the staged activations
            T* st = reinterpret_cast<T*>(xs);                       // [M][cols]
            const int cols = warps * p.rbw * 16;                    // columns of this CTA, contiguous in N
            for (int rbi = 0; rbi < nrb; ++rbi)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int m = 2 * t + (i & 1);
                    const int c = (warp * p.rbw + rbi) * 16 + ((i & 2) ? wr + 8 : wr);
                    if (m < p.M) st[m * cols + c] = F16Traits<T>::from_float(keep[rbi & 1][i]);
                }
            if (tid == 0) wait_peers_ready();
            __syncthreads();
            if (peers_ready_cta > 0) {
                const int n_cta = blockIdx.x * cols;
                const int vpr = cols / 8;                           // 16-byte pieces per token row
                const int per_rank = p.M * vpr;
                for (int idx = tid; idx < per_rank * p.gather.world; idx += blockDim.x) {
                    const int g = idx / per_rank;
                    const int r = idx - g * per_rank;
                    const int m = r / vpr;
                    const int v = r - m * vpr;
                    const int n = n_cta + v * 8;
                    T* dst = static_cast<T*>(p.gather.out_peer[g]) + (size_t)m * p.ldc + p.gather.n_offset + n;
                    if (n + 8 <= p.N) {
                        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(st + m * cols + v * 8);
                    } else {
                        for (int k = 0; k < 8; ++k)
                            if (n + k < p.N) dst[k] = st[m * cols + v * 8 + k];
                    }
                }
            }
        }
        if (gather_failed) atomicOr(&g_device_status, 4u);
        // The thread that reports for the CTA orders every thread's peer stores (the barrier puts
        // them before it) ahead of its arrival.
        __syncthreads();
        if (tid == 0) {
            __threadfence();   // device scope: the last CTA's system-scope fence below is cumulative
            unsigned int* mine = p.gather.flag_peer[p.gather.rank];
            const unsigned int total = gridDim.x * gridDim.y;
            if (atomicAdd(mine + kGatherCounterWord, 1u) == total - 1) {
                mine[kGatherCounterWord] = 0u;   // ready for the next call
                // one system-scope fence orders every CTA's peer stores (observed through the
                // device-scope arrivals above: fences are cumulative) before the arrival words, which
                // then go out together; the polls are acquire loads
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
                if (!all_in) atomicOr(&g_device_status, 4u);   // a rank never reported: give up, do not hang
                asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(mine + kGatherEpochWord), "r"(call_no) : "memory");
            }
        }
    }

    if (gave_up) {
        if (lane == 0) atomicOr(&g_device_status, 1u);
        // The arrival counters must still return to zero (the workspace is reused by later calls):
        // this warp reports for the row blocks it abandoned, and whoever arrives last clears the
        // counter.  Their outputs stay unwritten; the status word says so.
        if (p.num_chunks > 1 && !p.defer_reduce && p.swiglu_h == 0 && lane == 0)
            for (int rbi = rb_arrived; rbi < nrb; ++rbi)
                if (atomicAdd(&p.counters[rb_first + rbi], 1u) == (unsigned int)(p.num_chunks - 1))
                    p.counters[rb_first + rbi] = 0u;
        // Copies already requested may still land in this CTA's shared memory: give each
        // stage one more bounded wait before the CTA exits.
        for (int k = 0; k < p.stages; ++k) {
            mbar_wait(smem_u32(&bars[stage]), parity);
            if (++stage == p.stages) { stage = 0; parity ^= 1u; }
        }
    }
}

struct StreamPlan {
    int nt, warps, rbw, num_chunks, steps_per_chunk, total_steps, segs, xs_stride, piece_bytes, stages;
    size_t smem;
    unsigned grid_x;
    int resident_ctas;   // SMs x CTAs per SM the plan assumed
};

// One planning attempt for a given number of CTAs per SM; `smem_limit` is what one CTA may use so
// that this many are resident together.
bool plan_stream_at(const MatmulArgs& a, const mnq_tuning* tuning, size_t workspace_bytes, int ctas_per_sm,
                    size_t smem_limit, StreamPlan* out)
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
    // fused SwiGLU: a 16-row tile is 8 gate rows plus their 8 up rows, and K is never split (the
    // activation function needs the complete sums)
    const bool swiglu = a.swiglu_h > 0;
    const int64_t row_blocks = swiglu ? (a.swiglu_h + 7) / 8 : (a.N + 15) / 16;

    // 16 warps per CTA (measured: always better than 8 at equal work); the widest activation
    // tile is compiled for 256 threads
    // Up to 8 tokens: CTAs of 8 warps, two per SM (measured 1 us per launch better than one CTA of 16 on
    // the Qwen2.5-7B shapes: a CTA of the next kernel starts its set-up while its neighbour still streams)
    int warps = (tuning && tuning->warps_per_cta > 0) ? tuning->warps_per_cta
                                                       : ((pl.nt == 2 || (pl.nt == 1 && ctas_per_sm == 1)) ? 16 : 8);
    if (warps > 16) warps = 16;
    if (pl.nt >= 4 && warps > 8) warps = 8;
    while (warps > 1 && row_blocks < warps) warps >>= 1;
    pl.warps = warps;
    pl.piece_bytes = (tuning && tuning->piece_bytes > 0) ? tuning->piece_bytes : 256;
    if (pl.piece_bytes != 256) return false;   // one piece = four steps; its scales travel as four values per row
    // more than 8 tokens: chunks are short and there are fewer warps, so each warp keeps more
    // pieces in flight (the loop below takes stages away again if shared memory runs out)
    // Two pieces in flight per warp already keep HBM busy; a deeper ring only delays the activation
    // loads, which queue in L2 behind every SM's outstanding weight requests (measured: three stages
    // cost 1.5 us per launch on the Qwen2.5-7B gate+up shape).  With more than 8 tokens the chunks
    // are short and there are fewer warps, so each warp keeps more pieces in flight.
    pl.stages = (tuning && tuning->stages > 0) ? tuning->stages : (pl.nt >= 2 ? 4 : 2);
    if (pl.stages > 8) pl.stages = 8;
    if (pl.stages < 2) pl.stages = 2;
    const int64_t slots = static_cast<int64_t>(a.sm_count) * ctas_per_sm * warps;

    // K chunks.  A warp processes `rbw` units (row block x chunk) one after the other, so the
    // kernel lasts about rbw x (steps per chunk + a fixed per-unit cost); pick the chunk count
    // that minimises that, i.e. fills the warp slots without spilling into a nearly empty
    // second pass.
    int chunks = 1, rbw = 1;
    // More than 8 tokens: every CTA converts and stages its K chunk of the whole activation
    // block, which costs about 0.2 step-times per token and step and dwarfs the streaming if the
    // chunk is long.  Short chunks with many row blocks per warp stage little and reuse it a
    // lot, so the model below also charges the staging, and a warp may take up to 8 row blocks.
    const bool many_tokens = pl.nt >= 2;
    int rbw_cap = many_tokens ? 8 : 2;
    if (swiglu) {
        chunks = 1;
    } else if (tuning && tuning->split_k > 0) {
        chunks = tuning->split_k;
    } else if (row_blocks <= kMaxCounters) {
        double best_cost = 1e30;
        for (int c = 1; c <= kMaxSplitK && c <= pl.total_steps; ++c) {
            int spc = (pl.total_steps + c - 1) / c;
            if (c > 1 && spc < 4) break;
            if (c > 1) spc = (spc + 3) & ~3;   // whole 256-byte pieces: no partial piece at a chunk's end
            double cost;
            if (many_tokens) {
                const int64_t per_warp = (row_blocks * c + slots - 1) / slots;           // units per warp
                const int64_t waves = (per_warp + rbw_cap - 1) / rbw_cap;                // CTAs per SM, one after the other
                cost = static_cast<double>(per_warp) * (spc + 8) + static_cast<double>(waves) * 0.2 * a.M * spc +
                       (c > 1 ? 10.0 : 0.0);
            } else {
                const int64_t passes = (row_blocks * c + slots - 1) / slots;
                // cutting K at all costs the planes, a fence, an atomic and the last arriver's reads, about as
                // long as 20 steps take (Llama-3-8B gate/up, 896 row blocks and 32 steps: 10.8 us uncut, 11.6 us
                // cut in two)
                cost = static_cast<double>(passes) * (spc + 8) + (c > 1 ? 20.0 + 0.25 * c : 0.0);
            }
            if (cost < best_cost - 1e-9) { best_cost = cost; chunks = c; }
        }
    }
    if (chunks > kMaxSplitK) chunks = kMaxSplitK;
    if (chunks > pl.total_steps) chunks = pl.total_steps;
    if (chunks < 1 || row_blocks > kMaxCounters) chunks = 1;

    bool grew_for_smem = false;
    for (;;) {
        pl.steps_per_chunk = (pl.total_steps + chunks - 1) / chunks;
        if (chunks > 1) pl.steps_per_chunk = (pl.steps_per_chunk + 3) & ~3;
        pl.num_chunks = (pl.total_steps + pl.steps_per_chunk - 1) / pl.steps_per_chunk;
        const int64_t units = row_blocks * pl.num_chunks;
        // a warp takes at most rbw_cap consecutive row blocks (their scales are all staged up
        // front); beyond that the grid simply has more CTAs than SMs
        rbw = static_cast<int>((units + slots - 1) / slots);
        if (rbw > rbw_cap) rbw = rbw_cap;
        if (tuning && tuning->row_blocks_per_warp > 0) rbw = tuning->row_blocks_per_warp;
        if (rbw < 1) rbw = 1;
        pl.rbw = rbw;
        const int64_t chunk_k = static_cast<int64_t>(pl.steps_per_chunk) * step;
        int segs = (a.group_size >= a.K) ? 1 : static_cast<int>(chunk_k / a.group_size + 1);
        pl.segs = (segs + 3) & ~3;
        const int row_pad = (a.quant == MNQ_INT4) ? 64 : 16;
        pl.xs_stride = static_cast<int>(((chunk_k * 2 + 127) / 128) * 128 + row_pad);
        if (!(tuning && tuning->stages > 0)) {
            const int64_t pieces = static_cast<int64_t>(rbw) * ((static_cast<int64_t>(pl.steps_per_chunk) * kStepBytes +
                                                                   pl.piece_bytes - 1) / pl.piece_bytes);
            if (pl.stages > pieces) pl.stages = static_cast<int>(pieces < 2 ? 2 : pieces);
        }
        const size_t ring = static_cast<size_t>(pl.stages) * 16 * pl.piece_bytes;
        pl.smem = ((static_cast<size_t>(a.M) * pl.xs_stride + static_cast<size_t>(pl.segs) * pl.nt * 8 * 12 + 8 + 1023) &
                   ~size_t(1023)) + static_cast<size_t>(warps) * (ring + 128);
        size_t need_ws = 0;
        if (pl.num_chunks > 1) need_ws = kCounterBytes + static_cast<size_t>(pl.num_chunks) * a.M * a.N * 4;
        const bool smem_ok = pl.smem <= smem_limit;
        const bool ws_ok = need_ws <= workspace_bytes;
        const bool may_split = !swiglu && chunks < pl.total_steps && chunks < kMaxSplitK && row_blocks <= kMaxCounters &&
                               !(tuning && tuning->split_k > 0);
        // up to 8 tokens: the compact kernel stages at most kLeanMaxStaged activations per CTA; shorter
        // chunks, if the workspace has room for one more plane, keep the problem on it
        if (smem_ok && ws_ok && pl.nt == 1 && may_split && a.M * chunk_k > kLeanMaxStaged &&
            kCounterBytes + static_cast<size_t>(pl.num_chunks + 1) * a.M * a.N * 4 <= workspace_bytes) {
            ++chunks;
            continue;
        }
        if (smem_ok && ws_ok) break;
        if (!smem_ok) {
            // too much shared memory: fewer stages, then shorter chunks (less staged
            // activation), then fewer warps
            if (pl.stages > 2) { --pl.stages; continue; }
            if (many_tokens && rbw_cap > 1 && !(tuning && tuning->row_blocks_per_warp > 0)) { rbw_cap >>= 1; continue; }
            if (may_split) {
                ++chunks;
                grew_for_smem = true;
                continue;
            }
            if (warps > 4 && !(tuning && tuning->warps_per_cta > 0)) {
                warps >>= 1;
                pl.warps = warps;
                continue;   // `slots` keeps counting the original warps: rbw grows instead
            }
            return false;
        }
        if (chunks == 1 || grew_for_smem) return false;   // (shorter chunks were needed for shared memory)
        --chunks;
    }
    pl.resident_ctas = a.sm_count * ctas_per_sm;
    pl.grid_x = static_cast<unsigned>((row_blocks + static_cast<int64_t>(pl.warps) * rbw - 1) /
                                      (static_cast<int64_t>(pl.warps) * rbw));
    *out = pl;
    return true;
}

// Up to 8 tokens the kernels run two CTAs per SM: the plan must then leave room for both (an SM has
// 227 KB, of which every resident CTA reserves 1 KB), which with several tokens' activations staged
// means shorter K chunks; only if no such plan exists does a single CTA per SM take everything.
bool plan_stream(const MatmulArgs& a, const mnq_tuning* tuning, size_t workspace_bytes, StreamPlan* out)
{
    int ctas_per_sm = (tuning && tuning->ctas_per_sm > 0) ? tuning->ctas_per_sm : (a.M <= 8 ? 2 : 1);
    if (ctas_per_sm > 2) ctas_per_sm = 2;
    if (ctas_per_sm == 2 && plan_stream_at(a, tuning, workspace_bytes, 2, (227 * 1024) / 2 - 1024, out)) return true;
    return plan_stream_at(a, tuning, workspace_bytes, 1, kMaxSmem, out);
}

template <int QUANT, typename T, int NT, int CH>
int launch_stream_one(const StreamParams& p, const CUtensorMap& wmap, const CUtensorMap& wmap8, dim3 grid, int threads,
                      size_t smem, cudaStream_t stream)
{
    auto* kern = &gemv_stream_kernel<QUANT, T, NT, CH>;
    static std::atomic<uint64_t> attr_set{0};   // (one flag word per template instantiation)
    if (smem > 48 * 1024 && !attribute_done_on_device(attr_set)) {
        const int rc = check_cuda(
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem),
            "cudaFuncSetAttribute(gemv_stream)");
        if (rc) return rc;
        mark_attribute_done_on_device(attr_set);
    }
    // Programmatic dependent launch: the CTAs of this kernel may be scheduled while the previous
    // kernel in the stream is still draining (that hides the launch gap and the cold start);
    // they touch nothing but their own shared memory before `griddepcontrol.wait`.
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
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, p, wmap, wmap8), "gemv_stream launch");
}

template <int QUANT, typename T>
int launch_stream_nt(const StreamParams& p, const CUtensorMap& wmap, const CUtensorMap& wmap8, int nt, int ch, dim3 grid,
                     int threads, size_t smem, cudaStream_t stream)
{
    if (nt == 1) return launch_stream_one<QUANT, T, 1, 256>(p, wmap, wmap8, grid, threads, smem, stream);
    if (nt == 2) return launch_stream_one<QUANT, T, 2, 256>(p, wmap, wmap8, grid, threads, smem, stream);
    return launch_stream_one<QUANT, T, 4, 256>(p, wmap, wmap8, grid, threads, smem, stream);
}

}  // namespace

// Workspace the streaming plan wants for a problem on a 148-SM part with ideally aligned
// buffers and zeros present (the largest shared-memory footprint); 0 if K is not split, and
// `*supported` tells whether the streaming kernel takes the problem at all.
size_t gemv_stream_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size, int32_t quant, bool* supported)
{
    MatmulArgs a{};
    a.x = a.wq = a.scales = a.zeros = reinterpret_cast<const void*>(uintptr_t(4096));
    a.M = M; a.N = N; a.K = K; a.lda = K; a.ldc = N;
    a.group_size = group_size;
    a.G = K > 0 ? static_cast<int32_t>((K + group_size - 1) / group_size) : 0;
    a.quant = quant; a.act_dtype = MNQ_FP16; a.scale_dtype = MNQ_FP16;
    a.sm_count = 148;
    StreamPlan pl;
    *supported = plan_stream(a, nullptr, ~size_t(0), &pl);
    if (!*supported || pl.num_chunks <= 1) return 0;
    return kCounterBytes + static_cast<size_t>(pl.num_chunks) * M * N * 4;
}

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
    p.group_shift = -1;
    if (!single_group && (a.group_size & (a.group_size - 1)) == 0)
        for (int sh = 0; sh < 31; ++sh)
            if ((1 << sh) == a.group_size) p.group_shift = sh;
    p.G = a.G; p.scale_dtype = a.scale_dtype;
    p.steps_per_chunk = pl.steps_per_chunk; p.total_steps = pl.total_steps; p.num_chunks = pl.num_chunks;
    p.segs = pl.segs; p.xs_stride = pl.xs_stride;
    p.x_vec_ok = (reinterpret_cast<uintptr_t>(a.x) % 16 == 0) && (a.lda % 8 == 0);
    p.rbw = pl.rbw; p.stages = pl.stages;
    p.row_blocks = static_cast<int>(a.swiglu_h > 0 ? (a.swiglu_h + 7) / 8 : (a.N + 15) / 16);
    p.swiglu_h = static_cast<int>(a.swiglu_h);
    p.epi = a.epi;
    p.gather = a.gather;
    p.weights_immutable = option_value(MNQ_OPT_WEIGHTS_IMMUTABLE) != 0 ? 1 : 0;
    p.spin_limit = static_cast<unsigned int>(option_value(MNQ_OPT_PEER_WAIT_POLLS));
    // one aligned 8-byte load fetches a row's four scales of a piece: rows and chunk starts must
    // fall on 8-byte boundaries
    p.scale_vec = (a.G % 4 == 0) && (pl.num_chunks == 1 || pl.steps_per_chunk % 4 == 0) &&
                  reinterpret_cast<uintptr_t>(a.scales) % 8 == 0 &&
                  (a.zeros == nullptr || reinterpret_cast<uintptr_t>(a.zeros) % 8 == 0);
    // many tokens: the chunk planes are big and every unit would pay a fence and an atomic round
    // trip; a separate coalesced kernel adds them instead (not with the fused gather, whose peer
    // stores live in this kernel)
    p.defer_reduce = (pl.num_chunks > 1 && pl.nt >= 2 && a.gather.world == 0) ? 1 : 0;
    p.gather_vec = 0;
    if (a.gather.world > 0) {
        const size_t es = 2;   // fp16 / bf16 output
        bool ok = (a.ldc * es) % 16 == 0 && (a.gather.n_offset * es) % 16 == 0;
        for (int g = 0; g < a.gather.world; ++g) ok = ok && reinterpret_cast<uintptr_t>(a.gather.out_peer[g]) % 16 == 0;
        p.gather_vec = ok ? 1 : 0;
    }
    if (pl.num_chunks > 1) {
        unsigned char* ws = static_cast<unsigned char*>(a.workspace);
        p.counters = reinterpret_cast<unsigned int*>(ws);
        p.partial = reinterpret_cast<float*>(ws + kCounterBytes);
    }
    // packed weights as a [N, row_bytes / 4] tensor of 32-bit words; box = 16 rows x CH bytes
    CUtensorMap wmap;
    const int rc = encode_tensor_map_2d(&wmap, a.wq, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4,
                                        static_cast<uint64_t>(p.row_bytes) / 4, static_cast<uint64_t>(a.N),
                                        static_cast<uint64_t>(p.row_bytes), pl.piece_bytes / 4, 16,
                                        CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    // fused SwiGLU: the same tensor with 8-row boxes (a stage is filled by two copies)
    CUtensorMap wmap8 = wmap;
    if (a.swiglu_h > 0) {
        const int rc8 = encode_tensor_map_2d(&wmap8, a.wq, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4,
                                             static_cast<uint64_t>(p.row_bytes) / 4, static_cast<uint64_t>(a.N),
                                             static_cast<uint64_t>(p.row_bytes), pl.piece_bytes / 4, 8,
                                             CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc8) return rc8;
    }
    // 5 to 32 tokens: the kernel that reads activations prepared once per call (see gemv_mid.cu);
    // variants 3 and 4 leave it out, and so do small layers of few rows (of at least 4 MB: below that
    // every kernel takes the same 7-9 us) unless variant 9 asks for it
    const bool mid_pays = !(few_rows_small_layer(a) && packed_weight_bytes(a) >= (int64_t(4) << 20)) ||
                          (tuning && tuning->gemv_variant == 9);
    if (!(tuning && (tuning->gemv_variant == 3 || tuning->gemv_variant == 4)) && mid_pays && gemv_mid_supported(a, tuning))
        return launch_gemv_mid(a, tuning, wmap);
    // the compact kernel takes the common decode case (see gemv_lean.cu); variant 3 forces this one
    if (pl.nt == 1 && !(tuning && tuning->gemv_variant == 3)) {
        LeanShape ls{pl.warps, pl.num_chunks, pl.steps_per_chunk, pl.total_steps, pl.stages, pl.resident_ctas};
        if (gemv_lean_supported(a, ls)) return launch_gemv_lean(a, ls, wmap);
    }
    dim3 grid(pl.grid_x, static_cast<unsigned>(pl.num_chunks), 1);
    const int threads = pl.warps * 32;
#define MNQ_GS(Q, T) rcl = launch_stream_nt<Q, T>(p, wmap, wmap8, pl.nt, pl.piece_bytes, grid, threads, pl.smem, a.stream)
    int rcl;
    if (a.quant == MNQ_INT4) {
        if (a.act_dtype == MNQ_FP16) MNQ_GS(MNQ_INT4, __half);
        else MNQ_GS(MNQ_INT4, __nv_bfloat16);
    } else {
        if (a.act_dtype == MNQ_FP16) MNQ_GS(MNQ_INT8, __half);
        else MNQ_GS(MNQ_INT8, __nv_bfloat16);
    }
#undef MNQ_GS
    if (rcl || !p.defer_reduce) return rcl;
    return launch_splitk_reduce(p.partial, a.out, p.M, p.N, a.ldc, pl.num_chunks, a.act_dtype, a.epi, a.stream);
}

int read_gemm_status(unsigned int* out, bool clear);

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
    unsigned int g = 0, l = 0, md = 0;
    rc = read_gemm_status(&g, clear);
    if (rc) return rc;
    rc = read_lean_status(&l, clear);
    if (rc) return rc;
    rc = read_mid_status(&md, clear);
    if (rc) return rc;
    *out = v | g | l | md;
    return MNQ_SUCCESS;
}


}  // namespace mnq
