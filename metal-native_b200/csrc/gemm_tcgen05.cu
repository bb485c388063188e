// Prefill-shaped fused dequantise + matmul (M > 32) on the 5th-generation tensor cores.
// Replaces the reference's tiled kernels dequant_matmul_int4_fp16 / dequant_matmul_int8_fp16
// (shaders/matmul_dequant_kernel.metal:55-223, 351-479): dequantise a weight tile into
// shared memory, multiply, fp32 accumulate, 16-bit store.
//
// Orientation.  The MMA's 128-row operand A is the WEIGHT tile (128 output columns n x 64 k,
// K-major), its N-side operand B an ACTIVATION tile (<= 256 tokens x 64 k, K-major), so the
// accumulator in tensor memory is out^T: TMEM lane = n, TMEM column = token.  A CTA keeps one
// or two accumulators (up to 2 x 256 columns = all of tensor memory) and multiplies the same
// dequantised weight tile against one or two activation tiles, so each weight is dequantised
// once for up to 512 tokens.  Weight tiles and activation tiles travel in separate rings.
//
// Roles (352 threads):
//   warp 0      one lane issues the TMA loads of activation tiles (128-byte swizzle);
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (4 per 64-k block) and
//               tcgen05.commit, which frees the stage and finally publishes the accumulator;
//   warp 10     one lane issues the TMA loads of PACKED weight tiles (128 rows x 128 bytes,
//               128-byte swizzle) into a raw ring, so DRAM sees 128-byte row segments;
//   warps 2-9   (two threads per weight row) first copy the CTA's scales and zeros into a
//               shared-memory table (no global load may be in flight later: the proxy fence
//               they execute per tile would wait for it), then read the packed words from
//               the raw ring, dequantise to fp16 with one rounding
//               (fma(q-8, s, -z) on exact integers) and write the 128-byte-swizzled K-major
//               tile the MMA reads; afterwards they read the accumulator back with tcgen05.ld
//               and store out[m, n].
// bf16 activations: with one scale per row and no zeros the tile holds the exact integers and
// the scale is applied to the fp32 accumulator; otherwise every weight is kept as two bf16
// values (BSplit below) and every MMA is issued twice.
//
// Few tiles (a long-K, narrow-N layer) leave SMs idle, so K can be split over grid.z: every
// split writes its fp32 partial result to the workspace as [split][M][N], and a second small
// kernel on the same stream adds the splits in a fixed order and writes the output.  (Letting
// the last CTA to arrive do the addition inside the GEMM kernel left the whole reduction to a
// few hundred warps with a handful of loads in flight each; it took longer than the GEMM.)
//
// Every mbarrier wait is bounded; a wait that gives up sets bit 1 of the device status word
// and the CTA falls through to its teardown (tensor memory is always released).
#include <cuda.h>

#include <algorithm>
#include <type_traits>

#include "mnq_common.cuh"

namespace mnq {

// Own status word (device variables are per translation unit without relocatable device
// code); read_device_status() in gemv_stream.cu merges it through read_gemm_status().
__device__ unsigned int g_gemm_status = 0;


namespace {

constexpr int BN = 128;          // weight rows per CTA (MMA M)
constexpr int BK = 64;           // k per stage: one 128-byte swizzle row of 16-bit elements
constexpr int A_BYTES = BN * BK * 2;
// A waiting thread may stay suspended in hardware for up to kSuspendNs per try (it is woken
// when the phase completes), so a wait costs few instructions; kSpin tries bound the total.
constexpr unsigned kSpin = 1u << 22;
constexpr uint32_t kSuspendNs = 1000;

constexpr int kMaxSplits = 6;

struct GemmParams {
    const uint8_t* wq;
    const void* scales;
    const void* zeros;
    void* out;
    int M, N, K;
    long long ldc;
    int row_bytes;
    int group_size;     // >= K: one group
    int G;
    int scale_dtype;
    int tok;            // tokens per CTA tile = nh * tokh (<= 512)
    int tokh;           // tokens per accumulator / activation tile (multiple of 16, <= 256)
    int nh;             // accumulators per CTA (1 or 2)
    int stages;         // weight-tile (A) ring
    int b_stages;       // activation-tile (B) ring
    int tmem_cols;      // power of two >= max(32, tok)
    int tmem_a_col;     // weight tiles in tensor memory (TA kernels): first column of their ring, 32 columns per slot (64 with two tiles per k-block)
    int epilogue_scale; // 1: tile holds integers, scale applied to the accumulator
    int raw_stages;     // stages of the packed-weight ring
    int raw_segs;       // 128-byte-wide boxes per stage (consecutive along k)
    int commit_every;   // k-blocks per tcgen05.commit (1 or 2)
    int table_groups;   // quantisation groups per row held in the shared-memory scale table
    int splits;         // K splits (grid.z)
    int kb_per_split;   // 64-k blocks per split
    float* partial;     // [splits][M][N] fp32 (splits > 1)
    int vec_store;      // bit 0: out allows 16-byte stores, bit 1: the split-K planes do
    Epilogue epi;       // applied to the fp32 result before the store; fp32 output mode
    // raw-integer tiles (RawInt): per-token factor and activation sum, written by prep_activations_kernel
    const float* tok_scale;   // [M]: out column m is multiplied by it (undoes the activations' power-of-two rescale)
    const float* tok_sum;     // [M]: sum over k of the original activations of token m
    int offset_term;          // 1: this launch subtracts (128 s + z) * tok_sum (always; with K split, split 0 does)
    // Tail cut (single CTAs, no K split otherwise): the tiles along N from tail_from on -- the ones that would
    // run as a last, partly empty round of CTAs -- are cut tail_splits ways along K, tail_kb k-blocks each;
    // CTA x >= tail_from is part (x - tail_from) % tail_splits of tile tail_from + (x - tail_from) / tail_splits
    // and writes its fp32 result to plane [part][M][N - tail_from * 128] of tail_partial.  -1: none.
    int tail_from;
    int tail_splits;
    int tail_kb;
    float* tail_partial;
};

__device__ __forceinline__ uint32_t s_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool bar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(kSuspendNs) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity)
{
    for (unsigned i = 0; i < kSpin; ++i)
        if (bar_try(bar, parity)) return true;
    return false;
}
// ---- CTA pair (cluster of two) helpers ----
__device__ __forceinline__ uint32_t cluster_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// Arrival on a barrier of either CTA of the pair.  Default (CTA-scope) release: what the
// arrival publishes is this warp's dequantised tile, already pushed to the async proxy by
// fence.proxy.async, and it is read only by this SM's own tensor core; the barrier is merely
// where the leader learns of it.  (A cluster-scope release here costs ~0.4 us per k-block.)
__device__ __forceinline__ void bar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// wait that also acquires writes released by the peer CTA's threads
__device__ __forceinline__ bool bar_wait_cluster(uint32_t bar, uint32_t parity)
{
    for (unsigned i = 0; i < kSpin; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity), "r"(kSuspendNs) : "memory");
        if (ok) return true;
    }
    return false;
}
// hardware barrier over all threads of both CTAs (no spinning)
__device__ __forceinline__ void cluster_sync()
{
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA tile load whose completion may be signalled on a barrier of either CTA of the pair
// (`bar` is a shared::cluster address); the destination is this CTA's shared memory
__device__ __forceinline__ void tma_load_tile_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

__device__ __forceinline__ void tma_load_tile(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// K-major, 128-byte swizzle shared-memory matrix descriptor: rows of 128 bytes, 8-row
// groups 1024 bytes apart.  Start address, leading and stride byte offsets are in units
// of 16 bytes; bits 46-47 = 1 (descriptor version of this architecture); bits 61-63 = 2
// (128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr)
{
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: fp32 accumulate, A and B both K-major, M = rows (128, or
// 256 for a CTA pair), N = tok.
__device__ __forceinline__ uint32_t instr_desc(int tok, bool bf16, int rows)
{
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(tok >> 3) << 17) |
           (static_cast<uint32_t>(rows >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the weight tile (A) read from tensor memory: 128 lanes = rows, the 16 k of one MMA in 8
// consecutive 32-bit columns (two 16-bit values each) from a_tmem.
__device__ __forceinline__ void umma_ta(uint32_t tmem_d, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// 8 columns of this thread's tensor-memory lane from 8 registers (two 16-byte chunks of a tile row)
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint4& a, const uint4& b)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// CTA pair: one MMA over both CTAs' weight tiles (256 rows) and both halves of the activation tile
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar)
{
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(both) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v)
{
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// 8 consecutive k of one row -> one 16-byte chunk of 16-bit values in natural k order.
template <int QUANT, typename T> struct TileChunk;

template <> struct TileChunk<MNQ_INT4, __half> {
    static constexpr int WORDS = 1;   // packed 32-bit words per chunk
    static __device__ __forceinline__ uint4 run(const uint32_t* w, __half2 s2, __half2 nz2)
    {
        uint32_t P[4];
        UnpackInt4<__half>::run(w[0], P);   // (q0-8,q4-8) (q1-8,q5-8) (q2-8,q6-8) (q3-8,q7-8)
#pragma unroll
        for (int i = 0; i < 4; ++i) P[i] = h2_as_u32(__hfma2(u32_as_h2(P[i]), s2, nz2));
        uint4 o;
        o.x = prmt(P[0], P[1], 0x5410u);   // (w0, w1)
        o.y = prmt(P[2], P[3], 0x5410u);   // (w2, w3)
        o.z = prmt(P[0], P[1], 0x7632u);   // (w4, w5)
        o.w = prmt(P[2], P[3], 0x7632u);   // (w6, w7)
        return o;
    }
};
template <> struct TileChunk<MNQ_INT8, __half> {
    static constexpr int WORDS = 2;
    static __device__ __forceinline__ uint4 run(const uint32_t* w, __half2 s2, __half2 nz2)
    {
        uint32_t a[2], b[2];
        UnpackInt8<__half>::run(w[0], a);
        UnpackInt8<__half>::run(w[1], b);
        uint4 o;
        o.x = h2_as_u32(__hfma2(u32_as_h2(a[0]), s2, nz2));
        o.y = h2_as_u32(__hfma2(u32_as_h2(a[1]), s2, nz2));
        o.z = h2_as_u32(__hfma2(u32_as_h2(b[0]), s2, nz2));
        o.w = h2_as_u32(__hfma2(u32_as_h2(b[1]), s2, nz2));
        return o;
    }
};
// bf16: exact integers, no scale here
template <> struct TileChunk<MNQ_INT4, __nv_bfloat16> {
    static constexpr int WORDS = 1;
    static __device__ __forceinline__ uint4 run(const uint32_t* w, __half2, __half2)
    {
        uint32_t P[4];
        UnpackInt4<__nv_bfloat16>::run(w[0], P);
        uint4 o;
        o.x = prmt(P[0], P[1], 0x5410u);
        o.y = prmt(P[2], P[3], 0x5410u);
        o.z = prmt(P[0], P[1], 0x7632u);
        o.w = prmt(P[2], P[3], 0x7632u);
        return o;
    }
};
template <> struct TileChunk<MNQ_INT8, __nv_bfloat16> {
    static constexpr int WORDS = 2;
    static __device__ __forceinline__ uint4 run(const uint32_t* w, __half2, __half2)
    {
        uint32_t a[2], b[2];
        UnpackInt8<__nv_bfloat16>::run(w[0], a);
        UnpackInt8<__nv_bfloat16>::run(w[1], b);
        return make_uint4(a[0], a[1], b[0], b[1]);
    }
};

// Raw-integer tiles: int8 weights with one scale per row enter the tensor core as the exact fp16
// values (q + 128) * 2^-24 (byte ^ 0x80 in the low mantissa bits of an fp16 subnormal): one XOR per
// word and one byte permute per pair of weights instead of a convert, a multiply and an add.  The
// activations are fp16 (bf16 ones are converted once per call, prep_activations_kernel), and the
// epilogue turns the accumulator P of row n and token m into
//     s_n * 2^24 * c_m * P  -  (128 s_n + z_n) * X_m
// with c_m the token's power-of-two rescale and X_m the sum of its activations.
struct RawInt {};
template <> struct TileChunk<MNQ_INT8, RawInt> {
    static constexpr int WORDS = 2;
    static __device__ __forceinline__ uint4 run(const uint32_t* w, __half2, __half2)
    {
        const uint32_t u0 = w[0] ^ 0x80808080u, u1 = w[1] ^ 0x80808080u;
        return make_uint4(prmt(u0, 0u, 0x4140u), prmt(u0, 0u, 0x4342u), prmt(u1, 0u, 0x4140u), prmt(u1, 0u, 0x4342u));
    }
};
// bf16 activations with group-wise scales (or zeros): a dequantised weight does not fit bf16's
// 8 significant bits (rounding it would cost 1.6e-3 relative error by itself), and the MMA wants
// both operands in one format.  So the weight w = fma(q, s, -z), computed in fp32, is split into
// two bf16 values, hi = RN(w) and lo = RN(w - hi) (together good to 2^-16 relative), kept as
// two tiles, and every MMA is issued twice, once per tile, into the same accumulator.
struct BSplit {};
// bf16 activations with group-wise scales (or zeros), the faster and less exact way, for callers that opt in
// (MNQ_OPT_BF16_FP16_TILES) and whose workspace has room: the
// activations are converted once per call to fp16 times a per-token power of two (prep_activations_kernel,
// as for raw-integer tiles) and the weight tile is ONE fp16 tile, as for fp16 activations.  The scales
// and zeros of a row are divided by a power of two 2^E chosen per row and K split so that
// max(8 |s|, |z|) lands in [1, 2) (whatever 16-bit type they come in, they then fit fp16's range and keep
// their significand; groups 2^14 below the row's largest lose bits worth less than that), and the
// epilogue multiplies the accumulator by 2^E and the token's power of two.  Every weight is then rounded to
// fp16's 11 significant bits, as with fp16 activations (noise of about 2.8e-4 of the output RMS), where the
// two-tile path keeps 16.
struct HalfTile {};

template <int QUANT> struct SplitChunk;
template <> struct SplitChunk<MNQ_INT4> {
    static constexpr int WORDS = 1;
    // q - 8 of the chunk's eight weights as floats, in k order
    static __device__ __forceinline__ void ints(const uint32_t* w, float (&q)[8])
    {
        uint32_t P[4];
        UnpackInt4<__nv_bfloat16>::run(w[0], P);   // (q0,q4) (q1,q5) (q2,q6) (q3,q7) as exact bf16 pairs
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            q[i] = __uint_as_float(P[i] << 16);
            q[i + 4] = __uint_as_float(P[i] & 0xFFFF0000u);
        }
    }
};
template <> struct SplitChunk<MNQ_INT8> {
    static constexpr int WORDS = 2;
    static __device__ __forceinline__ void ints(const uint32_t* w, float (&q)[8])
    {
        constexpr float BIAS = 8388736.0f;   // 2^23 + 128
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t u = w[h] ^ 0x80808080u;
            q[4 * h + 0] = __uint_as_float(prmt(u, 0x4B000000u, 0x7440u)) - BIAS;
            q[4 * h + 1] = __uint_as_float(prmt(u, 0x4B000000u, 0x7441u)) - BIAS;
            q[4 * h + 2] = __uint_as_float(prmt(u, 0x4B000000u, 0x7442u)) - BIAS;
            q[4 * h + 3] = __uint_as_float(prmt(u, 0x4B000000u, 0x7443u)) - BIAS;
        }
    }
};
template <int QUANT>
__device__ __forceinline__ void split_chunk(const uint32_t* w, float s, float nz, uint4& hi, uint4& lo)
{
    float q[8];
    SplitChunk<QUANT>::ints(w, q);
    uint32_t H[4], L[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float a = fmaf(q[2 * i], s, nz), b = fmaf(q[2 * i + 1], s, nz);
        const __nv_bfloat162 h2 = __floats2bfloat162_rn(a, b);
        H[i] = b2_as_u32(h2);
        const float ra = a - __uint_as_float(H[i] << 16), rb = b - __uint_as_float(H[i] & 0xFFFF0000u);
        L[i] = b2_as_u32(__floats2bfloat162_rn(ra, rb));
    }
    hi = make_uint4(H[0], H[1], H[2], H[3]);
    lo = make_uint4(L[0], L[1], L[2], L[3]);
}

// Staged element stores for the epilogue.
template <typename E> struct StageIO;
template <> struct StageIO<float> {
    static __device__ __forceinline__ void put(uint32_t addr, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
    static __device__ __forceinline__ float get(uint32_t addr) { float v; asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr)); return v; }
    static __device__ __forceinline__ float from(float v) { return v; }
};
template <> struct StageIO<__half> {
    static __device__ __forceinline__ void put(uint32_t addr, __half v) { asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(__half_as_ushort(v)) : "memory"); }
    static __device__ __forceinline__ __half get(uint32_t addr) { unsigned short v; asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr)); return __ushort_as_half(v); }
    static __device__ __forceinline__ __half from(float v) { return __float2half_rn(v); }
};
template <> struct StageIO<__nv_bfloat16> {
    static __device__ __forceinline__ void put(uint32_t addr, __nv_bfloat16 v) { asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(__bfloat16_as_ushort(v)) : "memory"); }
    static __device__ __forceinline__ __nv_bfloat16 get(uint32_t addr) { unsigned short v; asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr)); return __ushort_as_bfloat16(v); }
    static __device__ __forceinline__ __nv_bfloat16 from(float v) { return __float2bfloat16_rn(v); }
};

// Epilogue of one CTA tile, run by the eight dequantise warps (256 threads, `e` = 0..255).
// Accumulator lane = weight row, columns = tokens, but the output is [token][row]: a thread
// storing its own accumulator elements writes 2 or 4 bytes per token row.  Instead the tile
// goes through shared memory in slabs of 64 tokens (two buffers, so one barrier per slab):
// each warp drops its 32 x 32 block as [token][row], then all threads copy the slab out as
// 16-byte pieces of whole 128-row lines.  `vec`: destination base and leading dimension allow
// 16-byte stores; otherwise the copy is element by element (still whole lines per warp).
// T: the activation type (what bias and residual hold).  FINAL: the values stored are the
// operator's result, so the epilogue is applied while they are staged; otherwise (a K split's
// fp32 plane) they are stored as they are.
// tok_scale / tok_sum / zterm: raw-integer tiles only (tok_scale == nullptr otherwise): the value of token m is
// acc * scale * tok_scale[m] - zterm * tok_sum[m].
template <typename E, typename T, bool FINAL>
__device__ __forceinline__ void epilogue_tile(uint32_t tmem_base, int quad, int half, int row, int e, int tok,
                                              uint32_t stage0, float scale, E* dst, size_t ld, int n0, int N, int m0,
                                              int M, bool vec, const Epilogue& epi, const float* tok_scale = nullptr,
                                              const float* tok_sum = nullptr, float zterm = 0.f)
{
    constexpr int RB = BN * (int)sizeof(E);    // bytes per staged token row
    constexpr int PPR = RB / 16;               // 16-byte pieces per row
    constexpr int RPS = 256 / PPR;             // rows per copy step
    constexpr int EPP = 16 / (int)sizeof(E);   // elements per piece
    const int slabs = (tok + 63) / 64;
    for (int j = 0; j < slabs; ++j) {
        const uint32_t stage = stage0 + (uint32_t)((j & 1) * 64 * RB);
        const int c0 = j * 64 + half * 32;     // this warp's 32 tokens of the slab
        if (c0 < tok) {
            uint32_t v[32];
            tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const uint32_t at = stage + (uint32_t)(half * 32 * RB) + (uint32_t)row * (uint32_t)sizeof(E);
            if (tok_scale) {
                const bool n_ok = n0 + row < N;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int m = min(m0 + c0 + i, M - 1);
                    float val = fmaf(-zterm, __ldg(tok_sum + m), __uint_as_float(v[i]) * scale * __ldg(tok_scale + m));
                    if (FINAL && n_ok && m0 + c0 + i < M) val = epilogue_value<T>(epi, val, m0 + c0 + i, n0 + row);
                    StageIO<E>::put(at + i * RB, StageIO<E>::from(val));
                }
            } else if (FINAL && epi.kind != MNQ_EPI_NONE) {
                const bool n_ok = n0 + row < N;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float val = __uint_as_float(v[i]) * scale;
                    if (n_ok && m0 + c0 + i < M) val = epilogue_value<T>(epi, val, m0 + c0 + i, n0 + row);
                    StageIO<E>::put(at + i * RB, StageIO<E>::from(val));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) StageIO<E>::put(at + i * RB, StageIO<E>::from(__uint_as_float(v[i]) * scale));
            }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (vec) {
            const int piece = e % PPR, rsub = e / PPR;
            const int n = n0 + piece * EPP;
#pragma unroll 4
            for (int r = rsub; r < 64; r += RPS) {
                const int c = j * 64 + r;
                const int m = m0 + c;
                if (c < tok && m < M) {
                    if (n + EPP <= N) {
                        const uint4 q = lds128(stage + (uint32_t)(r * RB + piece * 16));
                        __stcg(reinterpret_cast<uint4*>(dst + (size_t)m * ld + n), q);
                    } else {
                        for (int k = 0; k < EPP; ++k)
                            if (n + k < N)
                                dst[(size_t)m * ld + n + k] = StageIO<E>::get(stage + (uint32_t)(r * RB + (piece * EPP + k) * (int)sizeof(E)));
                    }
                }
            }
        } else {
            for (int idx = e; idx < 64 * BN; idx += 256) {
                const int r = idx / BN, nn = idx % BN;
                const int c = j * 64 + r;
                const int m = m0 + c;
                if (c < tok && m < M && n0 + nn < N)
                    dst[(size_t)m * ld + n0 + nn] = StageIO<E>::get(stage + (uint32_t)(r * RB + nn * (int)sizeof(E)));
            }
        }
    }
}

// PAIR: launched as clusters of two CTAs along x.  Each CTA still owns 128 weight rows and its
// own accumulators, but one `cta_group::2` MMA, issued by the even CTA (the leader), covers
// both: every CTA loads only half of each activation tile (tokh / 2 tokens) and the tensor
// cores read the other half from the peer's shared memory, which halves the L2 -> SM traffic
// of activation tiles.  Both CTAs run the same stage sequence; "tile ready" barriers live in
// the leader (the peer's dequantise warps and TMA signal them remotely), "tile free" barriers
// in each CTA (the leader commits to both).
// T: activation and output type.  TT: what the weight ring holds -- T itself (fp16: scale and zero
// folded in; bf16: the exact integers, one scale per row applied to the accumulator), or BSplit
// (bf16 activations, group-wise scales: two bf16 tiles per k-block, see above).
// OCC2: tiles of at most 256 tokens leave half of the SM's shared memory, tensor memory and
// registers unused, and a CTA of this kernel spends most of its time waiting (on loads, on the
// MMA, on its own barriers): two CTAs per SM, each planned for half the shared memory.
// TA (tiles of at most 128 tokens, single CTAs): the dequantise warps write the weight tile into
// TENSOR memory (tcgen05.st, a thread's row of 64 values = 32 columns of its lane; the two tiles of
// BSplit side by side in a 64-column slot) and the MMA takes its A operand from there.  A 128 x 64 tile then never passes through shared memory
// (16 KB written and 16 KB read per k-block otherwise, most of the shared-memory traffic of a CTA that
// multiplies few tokens, which is what bounds such a CTA), and its ring lives in the tensor-memory
// columns the accumulator leaves free.
template <int QUANT, typename T, typename TT, bool PAIR, bool OCC2, bool TA = false>
__global__ void __launch_bounds__(352, OCC2 ? 2 : 1)
gemm_tcgen05_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap,
                    const __grid_constant__ CUtensorMap wmap)
{
    constexpr int WPK = (QUANT == MNQ_INT4) ? 1 : 2;   // 16-byte packed chunks per 32 k of one row
    constexpr int KB_BYTES = WPK * 32;                  // packed bytes per row per k-block
    constexpr int KPR = 128 / KB_BYTES;                 // k-blocks covered by one raw stage (128 packed bytes per row)
    constexpr int RAW_BYTES = BN * 128;
    constexpr bool IS_BF16 = std::is_same<T, __nv_bfloat16>::value;
    constexpr bool SPLIT = std::is_same<TT, BSplit>::value;
    constexpr bool RAW = std::is_same<TT, RawInt>::value;      // fp16 tiles of raw integers, fp16 activations whatever T is
    constexpr bool HALF_T = std::is_same<TT, HalfTile>::value; // fp16 tiles and fp16 copies of bf16 activations
    constexpr bool MMA_BF16 = IS_BF16 && !RAW && !HALF_T;
    using TileT = typename std::conditional<RAW, RawInt, typename std::conditional<HALF_T, __half, T>::type>::type;
    constexpr int A_STAGE = TA ? 0 : (SPLIT ? 2 * A_BYTES : A_BYTES);   // shared-memory bytes of one weight-ring slot
    static_assert(!TA || !PAIR, "weight tiles in tensor memory: single CTAs");
    constexpr int A_COLS = SPLIT ? 64 : 32;   // tensor-memory columns of one weight-ring slot (TA): the high halves, then the low ones

    extern __shared__ unsigned char smem_raw[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ float row_up[HALF_T ? BN : 1];   // HalfTile: 2^E of every weight row of the tile
    // ready[8], done[8], accum, raw_full[4], raw_empty[4]
    __shared__ __align__(8) unsigned long long bars[2 * 8 + 1 + 2 * 4];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    int tile_x = blockIdx.x, part = blockIdx.z, kb_per_part = p.kb_per_split;
    bool cut = p.splits > 1;   // this CTA's result is one of several partial sums over K
    if (!PAIR && p.tail_from >= 0 && (int)blockIdx.x >= p.tail_from) {
        const int t = (int)blockIdx.x - p.tail_from;
        tile_x = p.tail_from + t / p.tail_splits;
        part = t % p.tail_splits;
        kb_per_part = p.tail_kb;
        cut = true;
    }
    const bool in_tail = !PAIR && p.tail_from >= 0 && tile_x >= p.tail_from;
    const int n0 = tile_x * BN;
    const int m0 = blockIdx.y * p.tok;
    const int kb_begin = part * kb_per_part;
    const int num_kb = min(p.K / BK, kb_begin + kb_per_part) - kb_begin;   // k-blocks of this part
    // Rings: S weight tiles, SB activation stages (one stage = the nh tiles of one k-block).
    // Synchronisation is per k-block, on D = max(S, SB) barrier pairs indexed kb % D:
    // ready[kb % D] completes when the k-block's weight tile is dequantised (one arrival per
    // dequantise warp that works on it: four per CTA) and its activation tiles have landed (one arrival with the byte count);
    // done[(kb / CE) % (D / CE)] completes when the MMAs of the CE consecutive k-blocks around kb have
    // read their operands: with CE = 2 there is one commit per pair of k-blocks, because a commit
    // costs the issuing thread a few hundred cycles and at small token counts that thread sets the
    // pace.  A producer refilling ring slot kb % S (or kb % SB) waits for the barrier that covers
    // k-block kb - S (kb - SB).  So the MMA thread does one wait per k-block and one commit per CE.
    const int S = p.stages, SB = p.b_stages, D = max(S, SB);
    const int CE = p.commit_every;   // k-blocks per commit: 2 when both rings are deep enough (then S, SB are even), else 1
    const int H = D / CE;            // `done` barriers
    const uint32_t rank = PAIR ? cluster_rank() : 0u;   // 0: leader (issues the MMAs), 1: peer
    const int b_rows = PAIR ? p.tokh / 2 : p.tokh;       // tokens of each activation tile this CTA loads
    const int b_bytes = b_rows * 128;
    const uint32_t tiles = (s_u32(smem_raw) + 1023u) & ~1023u;   // 1024-byte aligned: weight-tile ring
    const uint32_t btiles = tiles + S * A_STAGE;                  // activation-tile ring
    const uint32_t raw0 = btiles + SB * p.nh * b_bytes;           // packed-weight ring
    const int R = p.raw_stages;
    const int NSEG = p.raw_segs;
    const uint32_t tbl0 = raw0 + R * NSEG * RAW_BYTES;                   // [group][row] scale | zero << 16
    const int KPS = KPR * NSEG;                                   // k-blocks per packed stage
    const int num_raw = (num_kb + KPS - 1) / KPS;
    // Every CTA (pair) walks its k-blocks in a rotated order, starting at a different packed
    // stage: CTAs launched together would otherwise all ask L2 for the same activation lines
    // at the same moment.  Sequence index i -> k-block (i + k_rot) mod num_kb.
    const int st = (int)((blockIdx.x >> 1) % (unsigned)num_raw);
    const int k_rot = st * KPS;
    const uint32_t ready0 = s_u32(&bars[0]), done0 = s_u32(&bars[8]), accum = s_u32(&bars[16]);
    const uint32_t rfull0 = s_u32(&bars[17]), rempty0 = s_u32(&bars[21]);

    if (tid == 0) {
        // ready: the dequantise warps of every CTA feeding the MMA, plus the thread that announces the bytes
        for (int d = 0; d < D; ++d) bar_init(ready0 + 8 * d, (PAIR ? 8 : 4) + 1);
        for (int h = 0; h < H; ++h) bar_init(done0 + 8 * h, 1);
        bar_init(accum, 1);
        for (int r = 0; r < R; ++r) { bar_init(rfull0 + 8 * r, 1); bar_init(rempty0 + 8 * r, 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {   // one warp of each CTA of the pair
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(s_u32(&tmem_base_slot)), "r"((uint32_t)p.tmem_cols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(s_u32(&tmem_base_slot)), "r"((uint32_t)p.tmem_cols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (PAIR) cluster_sync();   // the peer's barriers are initialised before anything signals them
    else __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    bool failed = false;
    // Launched programmatically dependent: the set-up above may have run while the previous
    // kernel in the stream was finishing; nothing global is read or written before it is done.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // and the next kernel in the stream may begin its own set-up
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ---------------- activation tiles by TMA ----------------
        if (lane == 0) {
            const uint32_t ready_at = PAIR ? map_to_rank(ready0, 0) : ready0;   // the leader's barriers
            const uint32_t stage_bytes = (uint32_t)(p.nh * b_bytes);
            int sb = 0, d = 0;
            int wd = 0; uint32_t wph = 0;   // pair barrier of k-block i - SB and its phase
            for (int i = 0; i < num_kb; ++i) {
                const int kb = i + k_rot < num_kb ? i + k_rot : i + k_rot - num_kb;
                if (i >= SB && (CE == 1 || !((i - SB) & 1))) {   // CE = 2: the second k-block of a pair is free with the first
                    if (!bar_wait(done0 + 8 * wd, wph)) { failed = true; break; }
                    if (++wd == H) { wd = 0; wph ^= 1u; }
                }
                // one arrival announcing all the bytes of the k-block (both CTAs' halves for a pair)
                if (rank == 0) bar_expect_tx(ready0 + 8 * d, PAIR ? 2u * stage_bytes : stage_bytes);
                for (int h = 0; h < p.nh; ++h) {
                    const uint32_t dst = btiles + (uint32_t)(sb * p.nh + h) * (uint32_t)b_bytes;
                    if (PAIR)
                        tma_load_tile_pair(dst, &xmap, (kb_begin + kb) * BK, m0 + h * p.tokh + (int)rank * b_rows,
                                           ready_at + 8 * d);
                    else
                        tma_load_tile(dst, &xmap, (kb_begin + kb) * BK, m0 + h * p.tokh, ready0 + 8 * d);
                }
                if (++sb == SB) sb = 0;
                if (++d == D) d = 0;
            }
        }
    } else if (warp == 10) {
        // ---------------- packed weight tiles by TMA ----------------
        if (lane == 0) {
            int r = 0; uint32_t ph = 0;
            for (int j = 0; j < num_raw; ++j) {
                if (!bar_wait(rempty0 + 8 * r, ph ^ 1u)) { failed = true; break; }
                // NSEG boxes side by side along k: each row's 128-byte pieces are adjacent in memory
                // and requested back to back (boxes past the end of K are zero-filled)
                bar_expect_tx(rfull0 + 8 * r, (uint32_t)(NSEG * RAW_BYTES));
                const int jj = st + j < num_raw ? st + j : st + j - num_raw;
                for (int u = 0; u < NSEG; ++u)
                    tma_load_tile(raw0 + (r * NSEG + u) * RAW_BYTES, &wmap,
                                  (((kb_begin + (jj * NSEG + u) * KPR) * KB_BYTES) >> 2), n0, rfull0 + 8 * r);
                if (++r == R) { r = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        // The whole warp walks the k-blocks (uniform control flow and operand addresses) and one
        // elected lane issues: with the loop inside an `if (lane == 0)` every tcgen05.mma cost the
        // issuing thread about 47 cycles of its own (measured on static operands), ten times what
        // it costs from convergent code, and at few tokens that thread sets the pace.
        if (rank == 0) {
            uint32_t elected;
            asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(elected));
            const uint32_t idesc = instr_desc(p.tokh, MMA_BF16, PAIR ? 2 * BN : BN);
            int s = 0, sb = 0, d = 0; uint32_t dph = 0;
            int hp = 0;                             // pair barrier of this k-block
            for (int kb = 0; kb < num_kb; ++kb) {   // kb: position in this CTA's k order
                const bool landed = PAIR ? bar_wait_cluster(ready0 + 8 * d, dph) : bar_wait(ready0 + 8 * d, dph);
                if (!__all_sync(0xffffffffu, landed)) { failed = true; break; }   // the lanes leave together
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t adesc = smem_desc_sw128(tiles + s * A_STAGE);
                const uint64_t adesc_lo = smem_desc_sw128(tiles + s * A_STAGE + A_BYTES);   // SPLIT only
                const bool commit_now = CE == 1 || (kb & 1) || kb == num_kb - 1;
                if (elected) {
                for (int h = 0; h < p.nh; ++h) {
                    const uint64_t bdesc = smem_desc_sw128(btiles + (uint32_t)(sb * p.nh + h) * (uint32_t)b_bytes);
                    const uint32_t acc = tmem_base + (uint32_t)(h * p.tokh);
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j) {   // 32 bytes along k = 2 descriptor address units
                        if (TA) umma_ta(acc, tmem_base + (uint32_t)(p.tmem_a_col + s * A_COLS + 8 * j), bdesc + 2 * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                        else if (PAIR) umma_pair(acc, adesc + 2 * j, bdesc + 2 * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                        else umma(acc, adesc + 2 * j, bdesc + 2 * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                        if (SPLIT) {   // the low halves of the weights, same activations, same accumulator
                            if (TA) umma_ta(acc, tmem_base + (uint32_t)(p.tmem_a_col + s * A_COLS + 32 + 8 * j), bdesc + 2 * j, idesc, 1u);
                            else if (PAIR) umma_pair(acc, adesc_lo + 2 * j, bdesc + 2 * j, idesc, 1u);
                            else umma(acc, adesc_lo + 2 * j, bdesc + 2 * j, idesc, 1u);
                        }
                    }
                }
                // operands of this k-block are free once these MMAs have read them
                if (commit_now) {
                    if (PAIR) umma_commit_pair(done0 + 8 * hp);
                    else umma_commit(done0 + 8 * hp);
                }
                }
                __syncwarp();
                if (commit_now && ++hp == H) hp = 0;
                if (++s == S) s = 0;
                if (++sb == SB) sb = 0;
                if (++d == D) { d = 0; dph ^= 1u; }
            }
            if (elected) {
                if (PAIR) umma_commit_pair(accum);   // accumulators complete, in both CTAs
                else umma_commit(accum);
            }
            __syncwarp();
        }
    } else {
        // ---------------- dequantise weight tiles, then epilogue ----------------
        const int quad = warp & 3;             // tensor-memory lane quadrant this warp may read
        const int half = (warp - 2) >> 2;      // parity of the k-blocks this warp dequantises / which columns in the epilogue
        const int row = quad * 32 + lane;      // row of the tile = TMEM lane
        const int n = n0 + row;
        const size_t sc_row = (size_t)min(n, p.N - 1) * p.G;
        // byte offset of 16-byte chunk c inside this row's 128-byte line, after the 128-byte swizzle
        uint32_t xoff[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) xoff[c] = (uint32_t)((c ^ (row & 7)) << 4);
        // k-blocks per quantisation group as a shift when it is a power of two (it almost always is)
        const int kbg = (p.group_size >= p.K) ? 1 : p.group_size / BK;
        const int kbg_shift = (kbg & (kbg - 1)) == 0 ? 31 - __clz(kbg) : -1;
        const bool one_group = p.group_size >= p.K;
        const int g_first = one_group ? 0 : (kb_begin * BK) / p.group_size;
        if (!RAW) {   // scale | zero << 16 of every (row, group) this CTA touches, [group][row]
            const unsigned short* sc16 = static_cast<const unsigned short*>(p.scales);
            const unsigned short* zr16 = static_cast<const unsigned short*>(p.zeros);
            const int g_last = one_group ? 0 : ((kb_begin + num_kb) * BK - 1) / p.group_size;
            const int gc = g_last - g_first + 1;          // <= p.table_groups
            // eight entries per thread and pass, all loads issued before the first store: the whole
            // table costs one or two global round trips instead of one per entry
            // Two threads per weight row, each taking half of the row's groups as one contiguous
            // run: sixteen groups per pass with every load issued before the first store, so the
            // table costs a global round trip or two.  Indices past the end are clamped (the load
            // is harmless, the store is skipped): no branch separates the loads.
            constexpr int TU = 16;
            const int rr = (tid - 64) >> 1, hp = (tid - 64) & 1;
            const int gh = (gc + 1) >> 1;
            const int gbeg = hp * gh, gend = min(gc, gbeg + gh);
            const size_t rowsrc = (size_t)min(n0 + rr, p.N - 1) * p.G + g_first;
            const unsigned short* zsrc = zr16 ? zr16 : sc16;
            float down = 1.f;   // HalfTile: 2^-E of this row
            if (HALF_T) {
                // largest of 8 |s| and |z| over the row's groups of this split (both threads of the row)
                const bool sbf = p.scale_dtype == MNQ_BF16;
                auto mag = [&](uint32_t bits) {
                    return sbf ? fabsf(__uint_as_float(bits << 16)) : fabsf(__half2float(__ushort_as_half((unsigned short)bits)));
                };
                float mx = 0.f;
                for (int g0 = gbeg; g0 < gend; g0 += TU) {
                    uint32_t sv[TU], zv[TU];
#pragma unroll
                    for (int u = 0; u < TU; ++u) {
                        const int g = min(g0 + u, gend - 1);
                        sv[u] = __ldg(sc16 + rowsrc + g);
                        zv[u] = __ldg(zsrc + rowsrc + g);
                    }
#pragma unroll
                    for (int u = 0; u < TU; ++u) mx = fmaxf(mx, fmaxf(8.f * mag(sv[u]), zr16 ? mag(zv[u]) : 0.f));
                }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                // E = floor(log2(mx)) from the exponent field (zero, subnormal, inf or nan rows: E = 0)
                const int ex = static_cast<int>((__float_as_uint(mx) >> 23) & 0xFFu);
                const int E = (ex == 0 || ex == 255) ? 0 : max(-100, min(100, ex - 127));
                down = __int_as_float(static_cast<uint32_t>(127 - E) << 23);
                if (hp == 0) row_up[rr] = __int_as_float(static_cast<uint32_t>(127 + E) << 23);
            }
            for (int g0 = gbeg; g0 < gend; g0 += TU) {
                uint32_t sv[TU], zv[TU];
#pragma unroll
                for (int u = 0; u < TU; ++u) {
                    const int g = min(g0 + u, gend - 1);
                    sv[u] = __ldg(sc16 + rowsrc + g);
                    zv[u] = __ldg(zsrc + rowsrc + g);
                }
                if (HALF_T) {   // to fp16 bits, divided by the row's power of two (exact unless the result is subnormal)
                    const bool sbf = p.scale_dtype == MNQ_BF16;
#pragma unroll
                    for (int u = 0; u < TU; ++u) {
                        const float sf = sbf ? __uint_as_float(sv[u] << 16) : __half2float(__ushort_as_half((unsigned short)sv[u]));
                        const float zf = sbf ? __uint_as_float(zv[u] << 16) : __half2float(__ushort_as_half((unsigned short)zv[u]));
                        sv[u] = __half_as_ushort(__float2half_rn(sf * down));
                        zv[u] = __half_as_ushort(__float2half_rn(zf * down));
                    }
                }
#pragma unroll
                for (int u = 0; u < TU; ++u)
                    if (g0 + u < gend)
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(tbl0 + (uint32_t)(((g0 + u) * BN + rr) * 4)),
                                     "r"(sv[u] | (zr16 ? zv[u] << 16 : 0u)) : "memory");
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight dequantise warps only
        }

        const uint32_t ready_at = PAIR ? map_to_rank(ready0, 0) : ready0;   // the leader's barriers
        // This warp takes every other k-block of the CTA's k order (whole 64-k rows of its 32 weight rows),
        // so it pays for the barrier traffic of a k-block only every other k-block.
        int s = half, d = half;                 // kb % S and kb % D of this warp's next k-block (S, D >= 2)
        // barrier covering k-block i - S, and its phase, from this warp's first i >= S: the warp takes
        // every other k-block, so it meets every pair barrier once (CE = 2) or every other barrier (CE = 1)
        int wd = CE == 1 ? ((S ^ half) & 1) : 0; uint32_t wph = 0;
        const int wstep = CE == 1 ? 2 : 1;
        int r = 0; uint32_t rph = 0;
        int seq = 0;                            // position of the next k-block in this CTA's k order
        for (int j = 0; j < num_raw && !failed; ++j) {
            if (!bar_wait(rfull0 + 8 * r, rph)) { failed = true; break; }
            const int jj = st + j < num_raw ? st + j : st + j - num_raw;
            for (int u = 0; u < NSEG && !failed; ++u) {
            const uint32_t raw_row = raw0 + (r * NSEG + u) * RAW_BYTES + row * 128;
#pragma unroll
            for (int q = 0; q < KPR; ++q) {
                const int kb = (jj * NSEG + u) * KPR + q;
                if (kb >= num_kb || failed) break;
                const int i = seq++;
                if ((i & 1) != half) continue;
                uint32_t w[WPK * 8];
#pragma unroll
                for (int i = 0; i < 2 * WPK; ++i) {
                    const int chunk = q * (8 / KPR) + i;   // 16-byte chunk of the 128-byte raw row
                    const uint4 pk = lds128(raw_row + xoff[chunk]);
                    w[4 * i] = pk.x; w[4 * i + 1] = pk.y; w[4 * i + 2] = pk.z; w[4 * i + 3] = pk.w;
                }
                const int gi = one_group ? 0
                               : (kbg_shift >= 0 ? (kb_begin + kb) >> kbg_shift : (kb_begin + kb) / kbg) - g_first;
                const uint32_t sz = RAW ? 0u : lds32(tbl0 + (uint32_t)(gi * BN + row) * 4u);
                __half2 s2 = __half2half2(__ushort_as_half((unsigned short)(sz & 0xFFFFu)));
                // -z with the sign flipped in place (exact)
                __half2 nz2 = __half2half2(__ushort_as_half((unsigned short)((sz >> 16) ^ 0x8000u)));
                if (i >= S) {   // the MMAs that read this ring slot S k-blocks ago are done
                    if (!bar_wait(done0 + 8 * wd, wph)) { failed = true; break; }
                    wd += wstep;
                    if (wd >= H) { wd -= H; wph ^= 1u; }
                }
                const uint32_t a_row = tiles + s * A_STAGE + row * 128;
                if constexpr (SPLIT) {
                    // scale and -zero as fp32, from whichever 16-bit type the table holds
                    float s32, nz32;
                    if (p.scale_dtype == MNQ_BF16) {
                        s32 = __uint_as_float(sz << 16);
                        nz32 = -__uint_as_float(sz & 0xFFFF0000u);
                    } else {
                        s32 = __half2float(__ushort_as_half((unsigned short)(sz & 0xFFFFu)));
                        nz32 = -__half2float(__ushort_as_half((unsigned short)(sz >> 16)));
                    }
                    if constexpr (TA) {
                        // this thread's row of both tiles: 32 + 32 columns of its tensor-memory lane
                        const uint32_t a_t = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(p.tmem_a_col + s * A_COLS);
#pragma unroll
                        for (int c = 0; c < 8; c += 2) {
                            uint4 hi0, lo0, hi1, lo1;
                            split_chunk<QUANT>(&w[c * SplitChunk<QUANT>::WORDS], s32, nz32, hi0, lo0);
                            split_chunk<QUANT>(&w[(c + 1) * SplitChunk<QUANT>::WORDS], s32, nz32, hi1, lo1);
                            tmem_st8(a_t + 4 * c, hi0, hi1);
                            tmem_st8(a_t + 32 + 4 * c, lo0, lo1);
                        }
                        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    } else {
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            uint4 hi, lo;
                            split_chunk<QUANT>(&w[c * SplitChunk<QUANT>::WORDS], s32, nz32, hi, lo);
                            sts128(a_row + xoff[c], hi);
                            sts128(a_row + A_BYTES + xoff[c], lo);
                        }
                    }
                } else if constexpr (TA) {
                    // this thread's row of the tile: 32 columns of its tensor-memory lane, 8 at a time
                    using Chunk = TileChunk<QUANT, TileT>;
                    const uint32_t a_t = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(p.tmem_a_col + s * A_COLS);
#pragma unroll
                    for (int c = 0; c < 8; c += 2) {
                        const uint4 o0 = Chunk::run(&w[c * Chunk::WORDS], s2, nz2);
                        const uint4 o1 = Chunk::run(&w[(c + 1) * Chunk::WORDS], s2, nz2);
                        tmem_st8(a_t + 4 * c, o0, o1);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                } else {
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        using Chunk = TileChunk<QUANT, TileT>;
                        const uint4 o = Chunk::run(&w[c * Chunk::WORDS], s2, nz2);
                        sts128(a_row + xoff[c], o);
                    }
                }
                if (!TA) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) bar_arrive_cluster(ready_at + 8 * d);   // the leader waits for both CTAs' tiles
                    else bar_arrive(ready0 + 8 * d);
                }
                s += 2;
                if (s >= S) s -= S;
                d += 2;
                if (d >= D) d -= D;
            }
            }
            __syncwarp();
            if (lane == 0) bar_arrive(rempty0 + 8 * r);   // this warp is done with the raw stage
            if (++r == R) { r = 0; rph ^= 1u; }
        }

        // epilogue: accumulator row `row` holds out[m0 .. m0+tok, n]; this warp takes the
        // 32-column chunks with chunk index % 2 == half
        if (!failed && !bar_wait(accum, 0)) failed = true;
        // The epilogue synchronises the eight warps with each other, so they all take it or none
        // does: every thread arrives here, failed or not, and learns whether any of them failed.
        {
            uint32_t any;
            asm volatile(
                "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\t"
                "bar.red.or.pred p, 1, 256, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(any) : "r"((uint32_t)failed) : "memory");
            if (any && !failed) failed = true;
        }
        if (!failed) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float scale = 1.f, zterm = 0.f;
            if (p.epilogue_scale) scale = widen16(p.scales, sc_row, p.scale_dtype);
            const float* tscale = nullptr;
            if (HALF_T) {   // the tile was built from scales and zeros divided by the row's 2^E
                scale = row_up[row];
                tscale = p.tok_scale;
            }
            if (RAW) {
                const float s_n = scale;
                scale = s_n * 16777216.f;
                if (p.offset_term && (!cut || part == 0))
                    zterm = fmaf(128.f, s_n, p.zeros ? widen16(p.zeros, sc_row, p.scale_dtype) : 0.f);
                tscale = p.tok_scale;
            }
            // with K split, this CTA's result goes to its [M][N] plane of the workspace instead;
            // the rings are idle now (every MMA has completed), so their memory stages the tile
            if (in_tail) {   // plane `part` of the tail's own planes, Nt = N - tail_from * 128 columns wide; indexed by the global n
                const size_t Nt = (size_t)(p.N - p.tail_from * BN);
                epilogue_tile<float, T, false>(tmem_base, quad, half, row, tid - 64, p.tok, tiles, scale,
                                               p.tail_partial + (size_t)part * p.M * Nt - (size_t)p.tail_from * BN, Nt, n0, p.N, m0, p.M,
                                               (p.vec_store & 2) != 0, p.epi, tscale, p.tok_sum, zterm);
            } else if (cut)
                epilogue_tile<float, T, false>(tmem_base, quad, half, row, tid - 64, p.tok, tiles, scale,
                                               p.partial + (size_t)part * p.M * p.N, (size_t)p.N, n0, p.N, m0, p.M,
                                               (p.vec_store & 2) != 0, p.epi, tscale, p.tok_sum, zterm);
            else if (p.epi.out_f32)
                epilogue_tile<float, T, true>(tmem_base, quad, half, row, tid - 64, p.tok, tiles, scale,
                                              static_cast<float*>(p.out), (size_t)p.ldc, n0, p.N, m0, p.M,
                                              (p.vec_store & 4) != 0, p.epi, tscale, p.tok_sum, zterm);
            else
                epilogue_tile<T, T, true>(tmem_base, quad, half, row, tid - 64, p.tok, tiles, scale, static_cast<T*>(p.out),
                                          (size_t)p.ldc, n0, p.N, m0, p.M, (p.vec_store & 1) != 0, p.epi, tscale, p.tok_sum, zterm);
        }
    }
    if (failed && lane == 0) atomicOr(&g_gemm_status, 2u);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    // a pair releases its tensor memory, and lets go of each other's shared memory, together
    if (PAIR) cluster_sync();
    else __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols)
                         : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols)
                         : "memory");
    }
}

// out[m, n] = sum over splits of partial[z][m][n], splits added in index order (deterministic).
// VEC: eight consecutive n per thread as two 16-byte loads per split and one 16-byte store.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, void* __restrict__ out_v, int M,
                                                            int N, int64_t ldc, int splits, const Epilogue epi)
{
    T* out = static_cast<T*>(out_v);   // (VEC is never chosen with the fp32 output mode)
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the planes are the previous kernel's output
    const size_t plane = (size_t)M * N;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    if (VEC) {
        const size_t total = plane / 8;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
            const size_t e = i * 8;
            // planes in batches of six: every load of a batch is issued before the first add
            // (indices past the last plane are clamped and their values dropped)
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
            for (int z0 = 0; z0 < splits; z0 += 6) {
                float4 lo[6], hi[6];
#pragma unroll
                for (int z = 0; z < 6; ++z) {
                    const size_t at = (size_t)min(z0 + z, splits - 1) * plane + e;
                    lo[z] = __ldcs(reinterpret_cast<const float4*>(partial + at));
                    hi[z] = __ldcs(reinterpret_cast<const float4*>(partial + at + 4));
                }
#pragma unroll
                for (int z = 0; z < 6; ++z)
                    if (z0 + z < splits) {
                        a.x += lo[z].x; a.y += lo[z].y; a.z += lo[z].z; a.w += lo[z].w;
                        b.x += hi[z].x; b.y += hi[z].y; b.z += hi[z].z; b.w += hi[z].w;
                    }
            }
            const size_t m = e / N, n = e % N;
            if (epi.kind != MNQ_EPI_NONE) {
                a.x = epilogue_value<T>(epi, a.x, (int)m, (int)n);     a.y = epilogue_value<T>(epi, a.y, (int)m, (int)n + 1);
                a.z = epilogue_value<T>(epi, a.z, (int)m, (int)n + 2); a.w = epilogue_value<T>(epi, a.w, (int)m, (int)n + 3);
                b.x = epilogue_value<T>(epi, b.x, (int)m, (int)n + 4); b.y = epilogue_value<T>(epi, b.y, (int)m, (int)n + 5);
                b.z = epilogue_value<T>(epi, b.z, (int)m, (int)n + 6); b.w = epilogue_value<T>(epi, b.w, (int)m, (int)n + 7);
            }
            union { T h[8]; uint4 u; } pk;
            pk.h[0] = F16Traits<T>::from_float(a.x); pk.h[1] = F16Traits<T>::from_float(a.y);
            pk.h[2] = F16Traits<T>::from_float(a.z); pk.h[3] = F16Traits<T>::from_float(a.w);
            pk.h[4] = F16Traits<T>::from_float(b.x); pk.h[5] = F16Traits<T>::from_float(b.y);
            pk.h[6] = F16Traits<T>::from_float(b.z); pk.h[7] = F16Traits<T>::from_float(b.w);
            *reinterpret_cast<uint4*>(out + m * ldc + n) = pk.u;
        }
    } else {
        for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < plane; e += stride) {
            float acc = __ldcs(partial + e);
            for (int z = 1; z < splits; ++z) acc += __ldcs(partial + z * plane + e);
            store_result<T>(epi, out_v, ldc, (int)(e / N), (int)(e % N), acc);
        }
    }
}

// Prepares the activations for raw-integer tiles, one CTA per token row: the row's sum X_m (fp32,
// threads stride over the row, then a fixed tree: the same bits every time), and for bf16 rows an
// fp16 copy multiplied by the power of two c_m^-1 that puts the row's largest magnitude just below
// 2^15 (exact: a bf16 significand fits fp16's; only values 2^29 below the row's maximum are flushed).
// fp16 rows are used as they are (c_m = 1).
template <typename T>
__global__ void __launch_bounds__(256) prep_activations_kernel(const T* __restrict__ x, long long lda, int K,
                                                               __half* __restrict__ x16, float* __restrict__ tok_scale,
                                                               float* __restrict__ tok_sum)
{
    constexpr bool CONVERT = std::is_same<T, __nv_bfloat16>::value;
    __shared__ float warp_sum[8];
    __shared__ unsigned int warp_max[8];
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the activations may be the previous kernel's output
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int m = blockIdx.x;
    const uint4* row = reinterpret_cast<const uint4*>(x + (size_t)m * lda);
    const int n8 = K / 8;   // K is a multiple of 64
    float down = 1.f, up = 1.f;
    if (CONVERT) {
        unsigned int mx = 0;
        for (int i = threadIdx.x; i < n8; i += 256) {
            const uint4 q = __ldg(row + i);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) mx = max(mx, max(w[e] & 0x7FFFu, (w[e] >> 16) & 0x7FFFu));
        }
        mx = __reduce_max_sync(0xffffffffu, mx);
        if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = mx;
        __syncthreads();
        mx = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) mx = max(mx, warp_max[w]);
        const int E = static_cast<int>(mx >> 7);           // biased bf16 exponent of the maximum
        int sh = (E == 0) ? 0 : (E - 127) - 14;
        sh = max(-100, min(100, sh));
        down = __int_as_float((127 - sh) << 23);
        up = __int_as_float((127 + sh) << 23);
    }
    float sum = 0.f;
    for (int i = threadIdx.x; i < n8; i += 256) {
        const uint4 q = __ldg(row + i);
        uint32_t w[4] = {q.x, q.y, q.z, q.w};
        if (CONVERT) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xFFFF0000u);
                sum += lo;
                sum += hi;
                w[e] = h2_as_u32(__floats2half2_rn(lo * down, hi * down));
            }
            reinterpret_cast<uint4*>(x16 + (size_t)m * K)[i] = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(u32_as_h2(w[e]));
                sum += f.x;
                sum += f.y;
            }
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += warp_sum[w];
        tok_sum[m] = t;
        tok_scale[m] = up;
    }
}

struct GemmPlan {
    int tok, tokh, nh, tiles_m, stages, b_stages, raw_stages, raw_segs, commit_every, table_groups, tmem_cols, splits, kb_per_split;
    int pair;       // 1: clusters of two CTAs sharing each activation tile
    int occ2;       // 1: planned for two CTAs per SM (at most half the shared memory, <= 256 tensor-memory columns)
    int tiles_n;    // CTAs along N (even when pair)
    int raw;        // 1: raw-integer tiles (int8, one scale per row): activations prepared in the workspace first
    int half;       // 1: bf16 activations through fp16 tiles (HalfTile): activations prepared in the workspace first
    int ta;         // 1: weight tiles in tensor memory, from column tmem_a_col on
    int tmem_a_col;
    int tail_from, tail_splits, tail_kb;   // tail cut (see GemmParams): -1 / 1 / 0 when there is none
    size_t tail_offset;                    // of the tail's planes in the workspace
    size_t smem;
};

constexpr int kMaxTableGroups = 64;   // 32 KB of scale table at most

// K splits: the count that minimises waves x (k-blocks per split + fixed per-CTA cost) plus
// the cost of writing and re-reading one fp32 result plane per split and of the second
// launch (about 12 k-block times plus the plane traffic), all in units of one k-block time
// (around half a microsecond).
int choose_splits(int64_t tiles, int num_kb, int sm_count, double plane_bytes, int ctas_per_sm = 1,
                  double* cost_out = nullptr)
{
    // two CTAs sharing an SM each run slower (about 1.35x: together they get ~1.5x the throughput)
    const double slow = ctas_per_sm > 1 ? 1.35 : 1.0;
    int best = 1;
    double best_cost = 1e30;
    for (int sp = 1; sp <= kMaxSplits && sp <= num_kb; ++sp) {
        const int64_t waves = (tiles * sp + static_cast<int64_t>(sm_count) * ctas_per_sm - 1) /
                              (static_cast<int64_t>(sm_count) * ctas_per_sm);
        const double cost = static_cast<double>(waves) * ((num_kb + sp - 1) / sp + 8) * slow +
                            (sp > 1 ? 12.0 + sp * plane_bytes / 2.5e6 : 0.0);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = sp; }
    }
    if (cost_out) *cost_out = best_cost;
    return best;
}

// One or two CTAs per SM, and how many K splits: whichever the model above makes cheaper.
int choose_occupancy_and_splits(bool occ2_ok, int64_t tiles, int num_kb, int sm_count, double plane_bytes, int* occ2)
{
    double c1 = 0, c2 = 0;
    const int s1 = choose_splits(tiles, num_kb, sm_count, plane_bytes, 1, &c1);
    *occ2 = 0;
    if (!occ2_ok) return s1;
    const int s2 = choose_splits(tiles, num_kb, sm_count, plane_bytes, 2, &c2);
    if (c2 < c1) { *occ2 = 1; return s2; }
    return s1;
}

inline size_t split_workspace_bytes(int splits, int64_t M, int64_t N)
{
    return kCounterBytes + static_cast<size_t>(splits) * static_cast<size_t>(M) * static_cast<size_t>(N) * 4;
}

// Raw-integer tiles: int8 weights with one scale per row, up to kRawMaxTokens tokens (beyond that the
// kernel is bound by the tensor pipe and the dequantise work hides behind it, while preparing the
// activations would cost a pass over them).  The workspace then also holds, after the K-split planes,
// the per-token factors and sums and (bf16 activations) their fp16 copy.
constexpr int64_t kRawMaxTokens = 256;
inline bool raw_applicable(int64_t M, int64_t K, int32_t group_size, int32_t quant)
{
    return quant == MNQ_INT8 && group_size >= K && M <= kRawMaxTokens;
}
inline size_t raw_region_offset(int splits, int64_t M, int64_t N)
{
    const size_t planes = splits > 1 ? static_cast<size_t>(splits) * static_cast<size_t>(M) * static_cast<size_t>(N) * 4 : 0;
    return (kCounterBytes + planes + 255) & ~size_t(255);
}
inline size_t raw_region_bytes(int64_t M, int64_t K, bool convert)
{
    const size_t tok = ((static_cast<size_t>(M) * 8 + 255) & ~size_t(255));   // scale and sum per token
    return tok + (convert ? static_cast<size_t>(M) * static_cast<size_t>(K) * 2 : 0);
}

// Tail cut.  `tiles` CTAs on `slots` resident CTAs run as full rounds plus a last round of `rem` CTAs that
// takes as long as a full one; cut `ts` ways along K, those tiles make ceil(rem * ts / slots) rounds of
// 1 / ts the length (plus the fixed cost of a CTA, about 8 k-block times).  Returns the number of parts (1: no
// cut) and the first tile of the tail.
int choose_tail(int64_t tiles, int num_kb, int64_t slots, int64_t M, int* from)
{
    *from = -1;
    if (tiles <= slots || num_kb < 32) return 1;
    const int64_t rem = tiles % slots;
    if (rem == 0) return 1;
    int best_ts = 1;
    double best = num_kb + 8.0;
    for (int ts = 2; ts <= 4; ++ts) {
        const int64_t rounds = (rem * ts + slots - 1) / slots;
        // (+ the second launch and the planes' traffic, as for K splits)
        const double cost = rounds * ((num_kb + ts - 1) / ts + 8.0) + 6.0 + ts * (4.0 * M * rem * BN) / 2.5e6;
        if (cost < best * 0.9) { best = cost; best_ts = ts; }
    }
    if (best_ts > 1) *from = static_cast<int>(tiles - rem);
    return best_ts;
}
inline size_t tail_bytes(int ts, int64_t M, int64_t N, int from)
{
    return static_cast<size_t>(ts) * static_cast<size_t>(M) * static_cast<size_t>(N - static_cast<int64_t>(from) * BN) * 4;
}

// Token tiling and CTA pairing: up to 512 tokens per CTA as two accumulators of up to 256;
// CTA pairs (variant 0: for tiles of more than 256 tokens, where activation tiles dominate the
// L2 -> SM traffic and no longer fit three stages deep otherwise; 1: never; 2: always).
bool tile_plan(int64_t M, int64_t N, int variant, GemmPlan* out)
{
    GemmPlan& pl = *out;
    pl.tiles_m = static_cast<int>((M + 511) / 512);
    const int64_t per_tile = (M + pl.tiles_m - 1) / pl.tiles_m;
    if (per_tile > 256) {
        pl.nh = 2;
        pl.tokh = static_cast<int>((((per_tile + 1) / 2 + 31) / 32) * 32);
    } else {
        pl.nh = 1;
        pl.tokh = static_cast<int>(((per_tile + 15) / 16) * 16);
    }
    if (pl.tokh > 256) pl.tokh = 256;
    pl.tok = pl.nh * pl.tokh;
    pl.tiles_m = static_cast<int>((M + pl.tok - 1) / pl.tok);
    if (pl.tiles_m > 65535) return false;
    int cols = 32;
    while (cols < pl.tok) cols <<= 1;
    pl.tmem_cols = cols;
    pl.pair = variant == 1 ? 0 : variant == 2 ? 1 : (pl.tok > 256 && N > BN);
    pl.tiles_n = static_cast<int>((N + BN - 1) / BN);
    if (pl.pair) pl.tiles_n = (pl.tiles_n + 1) & ~1;
    return true;
}

bool plan_gemm(const MatmulArgs& a, const mnq_tuning* tuning, GemmPlan* out)
{
    if (a.M < 1 || a.N < 1 || a.K < BK || a.K % BK) return false;
    if (a.K > (1 << 28) || a.N > (1 << 30) || a.M > (1 << 24)) return false;
    if (reinterpret_cast<uintptr_t>(a.wq) % 16 || reinterpret_cast<uintptr_t>(a.x) % 16 || a.lda % 8) return false;
    if (a.group_size < a.K && a.group_size % BK) return false;
    if (a.act_dtype == MNQ_FP16 && a.scale_dtype != MNQ_FP16 && !raw_applicable(a.M, a.K, a.group_size, a.quant))
        return false;   // the fp16 tile math is fp16 x fp16
    // int8 with one scale per row, few tokens: raw-integer tiles (variant 5 forbids them); their workspace
    // need is checked once the K split is known
    bool raw = raw_applicable(a.M, a.K, a.group_size, a.quant) && !(tuning && tuning->gemv_variant == 5) &&
               (a.act_dtype == MNQ_BF16 || a.scale_dtype == MNQ_FP16 || a.scale_dtype == MNQ_BF16);
    // bf16 activations otherwise: integer tile when one scale per row and no zeros, else two bf16 tiles per k-block
    bool split_tiles = !raw && a.act_dtype == MNQ_BF16 && (a.group_size < a.K || a.zeros != nullptr);
    // ... or, if the caller opted in (MNQ_OPT_BF16_FP16_TILES) and the workspace can hold an fp16 copy of the
    // activations, one fp16 tile (HalfTile; variant 8 forbids it); checked again once the K split is known
    bool half_tiles = split_tiles && option_value(MNQ_OPT_BF16_FP16_TILES) != 0 && !(tuning && tuning->gemv_variant == 8) &&
                      a.workspace &&
                      a.workspace_bytes >= raw_region_offset(1, a.M, a.N) + raw_region_bytes(a.M, a.K, true);
    if (half_tiles) split_tiles = false;
    size_t a_stage = split_tiles ? 2 * A_BYTES : A_BYTES;
    GemmPlan pl{};
    if (!tile_plan(a.M, a.N, tuning ? tuning->gemv_variant : 0, &pl)) return false;

    const int num_kb = static_cast<int>(a.K / BK);
    const int64_t tiles = static_cast<int64_t>(pl.tiles_n) * pl.tiles_m;
    // two CTAs per SM where a CTA needs at most half of everything (variant 3 forbids it)
    const bool occ2_ok = !pl.pair && pl.tmem_cols <= 256 && !split_tiles && !(tuning && tuning->gemv_variant == 3);
    int want_occ2 = 0;
    int best = choose_occupancy_and_splits(occ2_ok, tiles, num_kb, a.sm_count, 4.0 * a.M * a.N, &want_occ2);
    if (tuning && tuning->split_k > 0) best = tuning->split_k;
    if (tuning && tuning->gemv_variant == 4) want_occ2 = occ2_ok ? 1 : 0;   // variant 4: two CTAs per SM whenever possible
    if (best > kMaxSplits) best = kMaxSplits;
    if (best > num_kb) best = num_kb;
    while (best > 1 && split_workspace_bytes(best, a.M, a.N) > (a.workspace ? a.workspace_bytes : 0))
        --best;   // not enough workspace: fewer splits (one split needs none)
    // the scale table holds at most kMaxTableGroups groups per row: split K further if needed
    const int64_t total_groups = a.group_size >= a.K ? 1 : (a.K + a.group_size - 1) / a.group_size;
    const int min_splits = static_cast<int>((total_groups + kMaxTableGroups - 1) / kMaxTableGroups);
    if (best < min_splits) best = min_splits;
    if (best > kMaxSplits || best > num_kb) return false;
    if (best > 1 && split_workspace_bytes(best, a.M, a.N) > (a.workspace ? a.workspace_bytes : 0)) return false;
    pl.kb_per_split = (num_kb + best - 1) / best;
    pl.splits = (num_kb + pl.kb_per_split - 1) / pl.kb_per_split;
    if (raw && raw_region_offset(pl.splits, a.M, a.N) + raw_region_bytes(a.M, a.K, a.act_dtype == MNQ_BF16) >
                   (a.workspace ? a.workspace_bytes : 0)) {
        // not enough workspace for the prepared activations: the dequantising tile path
        raw = false;
        if (a.act_dtype == MNQ_FP16 && a.scale_dtype != MNQ_FP16) return false;
        split_tiles = a.act_dtype == MNQ_BF16 && (a.group_size < a.K || a.zeros != nullptr);
        a_stage = split_tiles ? 2 * A_BYTES : A_BYTES;
    }
    if (half_tiles && raw_region_offset(pl.splits, a.M, a.N) + raw_region_bytes(a.M, a.K, true) > a.workspace_bytes) {
        // the K split's planes left no room for the fp16 copy: two bf16 tiles per k-block after all
        half_tiles = false;
        split_tiles = true;
        a_stage = 2 * A_BYTES;
        want_occ2 = 0;
    }
    pl.raw = raw ? 1 : 0;
    pl.half = half_tiles ? 1 : 0;
    pl.table_groups = a.group_size >= a.K
                          ? 1
                          : static_cast<int>((static_cast<int64_t>(pl.kb_per_split) * BK + a.group_size - 1) / a.group_size + 1);

    // shared memory: packed ring, scale table, then activation stages (one stage = the nh tiles
    // of a k-block; about 60 % of what is left, they have the longer latency to hide) and weight tiles
    const size_t b_stage = static_cast<size_t>(pl.nh) * (pl.pair ? pl.tokh / 2 : pl.tokh) * 128;
    pl.raw_segs = 1;
    const size_t epilogue_min = 1024 + 2 * 64 * BN * 4;   // the epilogue stages two 64-token slabs of fp32
    // weight tiles in tensor memory (see the kernel): tiles of at most 128 tokens (variant 6 forbids it)
    // (two bf16 tiles per k-block take a 64-column slot)
    const bool ta_ok = !pl.pair && pl.nh == 1 && pl.tok <= 128 && !(tuning && tuning->gemv_variant == 6);
    const int slot_cols = split_tiles ? 64 : 32;
    const int accum_cols = pl.tmem_cols;
    auto size_rings = [&](size_t total, int tmem_budget) -> bool {
        size_t ring = 0, budget = 0;
        int bst = 0;
        if (ta_ok) {
            int slots = (tmem_budget - accum_cols) / slot_cols;
            if (slots > 8) slots = 8;
            pl.raw_stages = 3;
            ring = static_cast<size_t>(pl.raw_stages) * pl.raw_segs * BN * 128 + static_cast<size_t>(pl.table_groups) * BN * 4;
            if (slots >= 2 && ring + 1024 + 2 * b_stage <= total) {
                budget = total - 1024 - ring;
                bst = static_cast<int>(budget / b_stage);
                if (bst > 8) bst = 8;
                int ast = slots;
                pl.commit_every = 1;
                if (bst >= 4 && ast >= 4) {
                    pl.commit_every = 2;
                    bst &= ~1;
                    ast &= ~1;
                }
                pl.b_stages = bst;
                pl.stages = ast;
                pl.ta = 1;
                pl.tmem_a_col = accum_cols;
                pl.tmem_cols = tmem_budget;
                pl.smem = 1024 + ring + b_stage * bst;
                if (pl.smem < epilogue_min) pl.smem = epilogue_min;
                return pl.smem <= total;
            }
        }
        pl.ta = 0;
        pl.tmem_cols = accum_cols;
        // big activation stages leave room for two packed stages (8 k-blocks of int4 ahead), small ones for three
        for (pl.raw_stages = b_stage >= 24 * 1024 ? 2 : 3; pl.raw_stages >= 1; --pl.raw_stages) {
            ring = static_cast<size_t>(pl.raw_stages) * pl.raw_segs * BN * 128 + static_cast<size_t>(pl.table_groups) * BN * 4;
            if (ring + 1024 + 2 * a_stage + 2 * b_stage > total) continue;
            budget = total - 1024 - ring;
            bst = static_cast<int>(budget * 6 / 10 / b_stage);
            if (bst < 2) bst = 2;
            if (bst > 8) bst = 8;
            if (budget >= b_stage * bst + 2 * a_stage) break;
        }
        if (pl.raw_stages < 1) return false;
        int ast = static_cast<int>((budget - b_stage * bst) / a_stage);
        if (ast > 8) ast = 8;
        if (raw) {
            // Few tokens: the kernel streams weights and a k-block in flight needs a weight tile and an
            // activation tile alike, so both rings get the same depth (the 60 % rule above leaves two
            // weight tiles at 64 tokens, and a CTA then waits on its own MMAs every other k-block).
            int n = static_cast<int>(budget / (a_stage + b_stage));
            if (n > 8) n = 8;
            if (n >= 2) {
                ast = n;
                bst = static_cast<int>((budget - a_stage * n) / b_stage);
                if (bst > 8) bst = 8;
            }
        }
        // deep rings: release operands a pair of k-blocks at a time (needs even stage counts)
        pl.commit_every = 1;
        if (bst >= 4 && ast >= 4) {
            pl.commit_every = 2;
            bst &= ~1;
            ast &= ~1;
        }
        pl.b_stages = bst;
        pl.stages = ast;
        pl.smem = 1024 + ring + b_stage * bst + static_cast<size_t>(ast) * a_stage;
        if (pl.smem < epilogue_min) pl.smem = epilogue_min;
        return pl.smem <= total;
    };
    pl.occ2 = 0;
    if (want_occ2 && size_rings(112 * 1024, 256)) pl.occ2 = 1;
    else if (!size_rings(226 * 1024, 512)) return false;
    // a last, partly empty round of CTAs: cut those tiles along K (variant 7 forbids it)
    pl.tail_from = -1; pl.tail_splits = 1; pl.tail_kb = 0; pl.tail_offset = 0;
    if (!pl.pair && pl.splits == 1 && pl.tiles_m == 1 && !(tuning && tuning->gemv_variant == 7)) {
        int from = -1;
        const int ts = choose_tail(tiles, num_kb, static_cast<int64_t>(a.sm_count) * (pl.occ2 ? 2 : 1), a.M, &from);
        if (ts > 1) {
            const bool prepared = pl.raw || pl.half;
            const size_t at = prepared ? ((raw_region_offset(1, a.M, a.N) + raw_region_bytes(a.M, a.K, a.act_dtype == MNQ_BF16) + 255) & ~size_t(255))
                                       : ((kCounterBytes + 255) & ~size_t(255));
            if (a.workspace && a.workspace_bytes >= at + tail_bytes(ts, a.M, a.N, from)) {
                pl.tail_from = from; pl.tail_splits = ts; pl.tail_kb = (num_kb + ts - 1) / ts; pl.tail_offset = at;
            }
        }
    }
    *out = pl;
    return true;
}

template <int QUANT, typename T, typename TT>
int launch_gemm_one(const GemmParams& p, const CUtensorMap& xmap, const CUtensorMap& wmap, dim3 grid, size_t smem,
                    bool pair, bool occ2, bool ta, cudaStream_t stream)
{
    auto* kern = pair ? &gemm_tcgen05_kernel<QUANT, T, TT, true, false> : &gemm_tcgen05_kernel<QUANT, T, TT, false, false>;
    if constexpr (!std::is_same<TT, BSplit>::value) {
        if (occ2 && !pair) kern = &gemm_tcgen05_kernel<QUANT, T, TT, false, true>;
        if (ta && !pair) kern = occ2 ? &gemm_tcgen05_kernel<QUANT, T, TT, false, true, true> : &gemm_tcgen05_kernel<QUANT, T, TT, false, false, true>;
    } else {
        if (ta && !pair) kern = &gemm_tcgen05_kernel<QUANT, T, TT, false, false, true>;
    }
    // per kernel of this instantiation: CTA pairs, single CTAs, two CTAs per SM, and the two with weight tiles in tensor memory
    static std::atomic<uint64_t> attr_set[5];
    std::atomic<uint64_t>& attr_flags = attr_set[pair ? 0 : (ta ? (occ2 ? 4 : 3) : (occ2 ? 2 : 1))];
    if (smem > 48 * 1024 && !attribute_done_on_device(attr_flags)) {
        const int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024),
                                  "cudaFuncSetAttribute(gemm_tcgen05)");
        if (rc) return rc;
        mark_attribute_done_on_device(attr_flags);
    }
    {
        // programmatic dependent launch (see the kernel); CTA pairs are clusters of two along x
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(352);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 2;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pair ? 2 : 1;
        const int rcl = check_cuda(cudaLaunchKernelEx(&cfg, kern, p, xmap, wmap), "gemm_tcgen05 launch");
        if (rcl) return rcl;
    }
    const int rc = check_cuda(cudaGetLastError(), "gemm_tcgen05 launch");
    if (!rc && p.tail_from >= 0) {
        // second launch: add the tail's planes and write those columns of the output
        const int64_t n_at = static_cast<int64_t>(p.tail_from) * BN;
        Epilogue epi = p.epi;
        const size_t esz = 2;   // bias and residual hold the activation type
        if (epi.bias) epi.bias = static_cast<const unsigned char*>(epi.bias) + n_at * esz;
        if (epi.residual) epi.residual = static_cast<const unsigned char*>(epi.residual) + n_at * esz;
        void* out_at = static_cast<unsigned char*>(p.out) + n_at * (epi.out_f32 ? 4 : 2);
        return launch_splitk_reduce(p.tail_partial, out_at, p.M, static_cast<int>(p.N - n_at), p.ldc, p.tail_splits,
                                    std::is_same<T, __nv_bfloat16>::value ? MNQ_BF16 : MNQ_FP16, epi, stream);
    }
    if (rc || p.splits <= 1) return rc;
    // second launch: add the splits' planes and write the output
    return launch_splitk_reduce(p.partial, p.out, p.M, p.N, p.ldc, p.splits,
                                std::is_same<T, __nv_bfloat16>::value ? MNQ_BF16 : MNQ_FP16, p.epi, stream);
}

}  // namespace

template <typename T>
static int launch_reduce_t(const float* partial, void* out, int M, int N, int64_t ldc, int splits, const Epilogue& epi,
                           cudaStream_t stream)
{
    const bool vec = N % 8 == 0 && ldc % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 && !epi.out_f32;
    const size_t work = vec ? (size_t)M * N / 8 : (size_t)M * N;
    size_t blocks = (work + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    auto* red = vec ? &splitk_reduce_kernel<T, true> : &splitk_reduce_kernel<T, false>;
    return check_cuda(cudaLaunchKernelEx(&cfg, red, partial, out, M, N, (long long)ldc, splits, epi), "splitk_reduce launch");
}

int launch_splitk_reduce(const float* partial, void* out, int M, int N, int64_t ldc, int splits, int32_t act_dtype,
                         const Epilogue& epi, cudaStream_t stream)
{
    if (act_dtype == MNQ_BF16) return launch_reduce_t<__nv_bfloat16>(partial, out, M, N, ldc, splits, epi, stream);
    return launch_reduce_t<__half>(partial, out, M, N, ldc, splits, epi, stream);
}

int read_gemm_status(unsigned int* out, bool clear)
{
    unsigned int v = 0;
    int rc = check_cuda(cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof v), "cudaMemcpyFromSymbol(gemm status)");
    if (rc) return rc;
    if (clear && v) {
        const unsigned int zero = 0;
        rc = check_cuda(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof zero), "cudaMemcpyToSymbol(gemm status)");
        if (rc) return rc;
    }
    *out = v;
    return MNQ_SUCCESS;
}

bool gemm_supported(const MatmulArgs& a)
{
    GemmPlan pl;
    return plan_gemm(a, nullptr, &pl);
}

size_t gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size, int32_t quant)
{
    const size_t base = gemm_split_workspace_bytes(M, N, K, group_size);
    if (M < 1 || N < 1 || K < BK || K % BK) return base;
    // room for the prepared activations (raw-integer tiles; fp16 tiles for bf16 activations if the caller opted
    // in): per-token factor and sum and, sized for bf16 activations, their fp16 copy
    // the tail cut's planes (whichever occupancy the plan ends up with), after the prepared activations if any
    size_t tail = 0;
    {
        GemmPlan pl{};
        if (base <= kCounterBytes && tile_plan(M, N, 0, &pl) && !pl.pair && pl.tiles_m == 1)
            for (int per_sm = 1; per_sm <= 2; ++per_sm) {
                int from = -1;
                const int ts = choose_tail(pl.tiles_n, static_cast<int>(K / BK), 148 * per_sm, M, &from);
                if (ts > 1) tail = std::max(tail, tail_bytes(ts, M, N, from) + 256);
            }
    }
    if (!raw_applicable(M, K, group_size, quant) && option_value(MNQ_OPT_BF16_FP16_TILES) == 0)
        return tail ? ((std::max(base, kCounterBytes) + 255) & ~size_t(255)) + tail : base;
    const int splits = base > kCounterBytes ? static_cast<int>((base - kCounterBytes) / (static_cast<size_t>(M) * N * 4)) : 1;
    return ((raw_region_offset(splits, M, N) + raw_region_bytes(M, K, true) + 255) & ~size_t(255)) + tail;
}

size_t gemm_split_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t group_size)
{
    // What plan_gemm asks for on a 148-SM part (B200).  On a device where it would split
    // further, the plan falls back to the number of splits the given workspace can hold.
    if (M < 1 || N < 1 || K < BK || K % BK) return 0;
    GemmPlan pl{};
    if (!tile_plan(M, N, 0, &pl)) return 0;
    const int64_t tiles = static_cast<int64_t>(pl.tiles_n) * pl.tiles_m;
    int occ2 = 0;   // as plan_gemm
    int splits = choose_occupancy_and_splits(!pl.pair && pl.tmem_cols <= 256, tiles, static_cast<int>(K / BK), 148,
                                             4.0 * M * N, &occ2);
    const int64_t total_groups = group_size >= K ? 1 : (K + group_size - 1) / group_size;
    const int min_splits = static_cast<int>((total_groups + kMaxTableGroups - 1) / kMaxTableGroups);
    if (splits < min_splits) splits = min_splits;
    if (splits <= 1 || splits > kMaxSplits) return 0;
    return split_workspace_bytes(splits, M, N);
}

int launch_gemm(const MatmulArgs& a, const mnq_tuning* tuning)
{
    GemmPlan pl;
    if (!plan_gemm(a, tuning, &pl))
        return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul: the tensor-core kernel cannot take this problem "
                                          "(needs K % 64 == 0, 16-byte aligned operands, group_size % 64 == 0 or >= K, "
                                          "fp16 scales with fp16 activations)");
    GemmParams p{};
    p.wq = static_cast<const uint8_t*>(a.wq); p.scales = a.scales; p.zeros = a.zeros; p.out = a.out;
    p.M = static_cast<int>(a.M); p.N = static_cast<int>(a.N); p.K = static_cast<int>(a.K);
    p.ldc = a.ldc;
    p.row_bytes = static_cast<int>(a.quant == MNQ_INT4 ? a.K / 2 : a.K);
    p.group_size = a.group_size; p.G = a.G; p.scale_dtype = a.scale_dtype;
    p.tok = pl.tok; p.tokh = pl.tokh; p.nh = pl.nh; p.stages = pl.stages; p.b_stages = pl.b_stages;
    p.raw_stages = pl.raw_stages; p.raw_segs = pl.raw_segs; p.commit_every = pl.commit_every; p.table_groups = pl.table_groups; p.tmem_cols = pl.tmem_cols;
    p.tmem_a_col = pl.tmem_a_col;
    const bool split_tiles = !pl.raw && !pl.half && a.act_dtype == MNQ_BF16 && (a.group_size < a.K || a.zeros != nullptr);
    p.epilogue_scale = (a.act_dtype == MNQ_BF16 && !split_tiles && !pl.half) ? 1 : 0;
    p.splits = pl.splits; p.kb_per_split = pl.kb_per_split;
    p.vec_store = ((reinterpret_cast<uintptr_t>(a.out) % 16 == 0 && a.ldc % 8 == 0) ? 1 : 0) | ((a.N % 4 == 0) ? 2 : 0) |
                  ((reinterpret_cast<uintptr_t>(a.out) % 16 == 0 && a.ldc % 4 == 0) ? 4 : 0);
    p.epi = a.epi;
    p.tail_from = pl.tail_from; p.tail_splits = pl.tail_splits; p.tail_kb = pl.tail_kb;
    if (pl.tail_from >= 0) p.tail_partial = reinterpret_cast<float*>(static_cast<unsigned char*>(a.workspace) + pl.tail_offset);
    if (pl.splits > 1) {
        unsigned char* ws = static_cast<unsigned char*>(a.workspace);
        p.partial = reinterpret_cast<float*>(ws + kCounterBytes);
    }

    // raw-integer tiles, fp16 tiles for bf16 activations: per-token factors and sums (and the fp16 copy of bf16
    // activations) first
    const void* x_for_tiles = a.x;
    int64_t lda_tiles = a.lda;
    bool x_is_bf16 = a.act_dtype == MNQ_BF16;
    if (pl.raw || pl.half) {
        unsigned char* region = static_cast<unsigned char*>(a.workspace) + raw_region_offset(pl.splits, a.M, a.N);
        float* tok_scale = reinterpret_cast<float*>(region);
        float* tok_sum = tok_scale + a.M;
        __half* x16 = reinterpret_cast<__half*>(region + ((static_cast<size_t>(a.M) * 8 + 255) & ~size_t(255)));
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(static_cast<unsigned>(a.M));
        cfg.blockDim = dim3(256);
        cfg.stream = a.stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int rcp;
        if (x_is_bf16)
            rcp = check_cuda(cudaLaunchKernelEx(&cfg, &prep_activations_kernel<__nv_bfloat16>, static_cast<const __nv_bfloat16*>(a.x),
                                                (long long)a.lda, (int)a.K, x16, tok_scale, tok_sum), "prep_activations launch");
        else
            rcp = check_cuda(cudaLaunchKernelEx(&cfg, &prep_activations_kernel<__half>, static_cast<const __half*>(a.x),
                                                (long long)a.lda, (int)a.K, x16, tok_scale, tok_sum), "prep_activations launch");
        if (rcp) return rcp;
        p.tok_scale = tok_scale;
        p.tok_sum = tok_sum;
        p.offset_term = pl.raw ? 1 : 0;
        p.epilogue_scale = pl.raw ? 1 : 0;
        if (x_is_bf16) { x_for_tiles = x16; lda_tiles = a.K; x_is_bf16 = false; }
    }
    // activations as a [M, K] tensor of 16-bit elements; box = 64 k x the tokens one CTA loads, 128-byte swizzle
    CUtensorMap xmap;
    const int rc = encode_tensor_map_2d(&xmap, x_for_tiles, x_is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                        2, static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.M),
                                        static_cast<uint64_t>(lda_tiles) * 2, BK,
                                        static_cast<uint32_t>(pl.pair ? pl.tokh / 2 : pl.tokh),
                                        CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    // packed weights as a [N, row_bytes / 4] tensor of 32-bit words; box = 128 bytes x 128 rows,
    // 128-byte swizzle so that 32 threads reading 32 different rows do not collide on banks
    CUtensorMap wmap;
    const int rc2 = encode_tensor_map_2d(&wmap, a.wq, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4,
                                         static_cast<uint64_t>(p.row_bytes) / 4, static_cast<uint64_t>(a.N),
                                         static_cast<uint64_t>(p.row_bytes), 32, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc2) return rc2;
    dim3 grid(static_cast<unsigned>(pl.tail_from >= 0 ? pl.tail_from + (pl.tiles_n - pl.tail_from) * pl.tail_splits : pl.tiles_n),
              static_cast<unsigned>(pl.tiles_m), static_cast<unsigned>(pl.splits));
    const bool pair = pl.pair != 0;
    if (pl.raw) {   // int8 only (plan_gemm)
        if (a.act_dtype == MNQ_FP16) return launch_gemm_one<MNQ_INT8, __half, RawInt>(p, xmap, wmap, grid, pl.smem, pair, pl.occ2 != 0, pl.ta != 0, a.stream);
        return launch_gemm_one<MNQ_INT8, __nv_bfloat16, RawInt>(p, xmap, wmap, grid, pl.smem, pair, pl.occ2 != 0, pl.ta != 0, a.stream);
    }
    if (pl.half) {   // bf16 activations only (plan_gemm)
        if (a.quant == MNQ_INT4) return launch_gemm_one<MNQ_INT4, __nv_bfloat16, HalfTile>(p, xmap, wmap, grid, pl.smem, pair, pl.occ2 != 0, pl.ta != 0, a.stream);
        return launch_gemm_one<MNQ_INT8, __nv_bfloat16, HalfTile>(p, xmap, wmap, grid, pl.smem, pair, pl.occ2 != 0, pl.ta != 0, a.stream);
    }
    if (a.quant == MNQ_INT4) {
        if (a.act_dtype == MNQ_FP16) return launch_gemm_one<MNQ_INT4, __half, __half>(p, xmap, wmap, grid, pl.smem, pair, pl.occ2 != 0, pl.ta != 0, a.stream);
        if (split_tiles) return launch_gemm_one<MNQ_INT4, __nv_bfloat16, BSplit>(p, xmap, wmap, grid, pl.smem, pair, pl.occ2 != 0, pl.ta != 0, a.stream);
        return launch_gemm_one<MNQ_INT4, __nv_bfloat16, __nv_bfloat16>(p, xmap, wmap, grid, pl.smem, pair, pl.occ2 != 0, pl.ta != 0, a.stream);
    }
    if (a.act_dtype == MNQ_FP16) return launch_gemm_one<MNQ_INT8, __half, __half>(p, xmap, wmap, grid, pl.smem, pair, pl.occ2 != 0, pl.ta != 0, a.stream);
    if (split_tiles) return launch_gemm_one<MNQ_INT8, __nv_bfloat16, BSplit>(p, xmap, wmap, grid, pl.smem, pair, pl.occ2 != 0, pl.ta != 0, a.stream);
    return launch_gemm_one<MNQ_INT8, __nv_bfloat16, __nv_bfloat16>(p, xmap, wmap, grid, pl.smem, pair, pl.occ2 != 0, pl.ta != 0, a.stream);
}

}  // namespace mnq

