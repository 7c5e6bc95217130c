// Fused decode attention over the packed block-32 cache, head_dim 128: tensor-core kernels.
//
// Why tensor cores on an HBM-bound scan: at 70 % of HBM bandwidth a B200 streams ~8e12 packed
// codes per second, and every code meets one FMA per query head of the GQA group (x2 for K and
// V).  On the SIMT pipes that is more lane-instructions than the chip can issue, so the
// QK^T and PV contractions go through mma.sync.m16n8k16 (f16 in, f32 accumulate) and the SIMT
// pipes only unpack codes.  tcgen05 is not used: its operands must be staged in shared memory,
// which would cost a shared-memory write per dequantized value, and the per-(token, block) V scale
// leaves its P V product only 8 useful rows of a 64-row MMA; mma.sync takes the unpacked codes
// straight from registers.
//
// Layout of one warp step (16 tokens t0..t0+15, lane = 4*n + j):
//   S = K~ Q~^T :  M = 16 tokens (rows n and n + 8), N = 8 columns of rotated queries (group <= 4: the f16
//       hi parts of heads 0..3, then their lo parts; else 8 heads, hi and lo in two MMAs), K = 16 dims of
//       ONE 32-block.  Lane (n, j) supplies, for tokens t0+n and t0+8+n and block b, the eight codes
//       j*8..j*8+7 of the block; two MMAs per block cover all 16 tokens.  Because each MMA stays inside one
//       block, the per-block scale |s| is applied to the f32 accumulator (one FMA per token and column),
//       not to the elements.  Softmax runs on (token n / n + 8, two heads per lane); the row maximum is
//       reduced over the 8 lane groups n.
//   O^T = V^T P' :  M = 16 dims of ONE block, N = 8 columns (as above), K = 16 tokens.  The probabilities
//       (times the V scale, P' = p |s_v|) are transposed from (token rows, head columns) to the B fragment
//       (tokens 2j, 2j+1 of column n) by movmatrix, one instruction per 8 x 8 block.
//
// Code -> f16:
//   4-bit MaxNorm grid (codebooks.rs:63-73): centroid i = (2R/15)(i - 7.5).  A nibble masked into
//   mantissa bits 1..4 (5..8) of 0x6400 reads 1024 + 2i (1024 + 32i); one HFMA2 with exactly
//   representable constants turns it into the exact f16 value i - 7.5 (see nibbles_to_half2).
//   3-bit (any codebook of 8 entries, or 4 entries stored at 3-bit width): a 64-entry half2 table
//   indexed by two codes, replicated once per bank (entry e of lane l at word 32*e + l) so that
//   every lookup is conflict-free.  The table holds centroid / kappa, where the f32 factor kappa
//   is chosen so that all table values are (almost) exactly representable in f16.
// Both the rotated query and P' are split into f16 hi + lo parts, so every product entering the
// f32 accumulators is exact up to the (tiny) table error of the 3-bit path.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <float.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <type_traits>

#include "tqb_common.cuh"
#include "tqb_merge.cuh"
#include "tqb_pqo_quant.cuh"

namespace tqb {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kD = 128;
constexpr int kGroup = 16;             // tokens per warp step
constexpr float kNegBig = -1.0e30f;    // finite stand-in for -inf (keeps exp2 arguments NaN-free)
constexpr int kStages = 4;

struct MmaArgs {
    const void* q;
    const uint8_t* kb;    // K indices, [hkv, kv_stride, 16*BITS]
    const uint16_t* ks;   // [hkv, kv_stride, 4]
    const uint8_t* vb;
    const uint16_t* vs;
    float* partial_out;
    float* partial_max;
    float* partial_sum;
    int hq, hkv, g, kv_len, kv_stride, num_partitions, part_size;
    float qk_const;   // softmax_scale * log2(e) * (grid step | kappa)
    float v_const;    // grid step | kappa
    float sign_mag;
    float lut[8];     // 3-bit path: centroid / kappa
    // fused merge: the CTA that finishes a KV head last combines its partitions (counters == nullptr: off)
    unsigned* counters;   // [hq] (one per KV head used) then [hkv][merge_groups(P)]: zero before the launch; left zero by it
    float* group_out;     // two-level merge: group partials [hq][merge_groups(P)][128], max and sum [hq][merge_groups(P)]
    float* group_max;
    float* group_sum;
    void* out;
    float* lse_out;
    int out_dtype;
    // fused append: the new token's K / V vectors [hkv, 128] of the query dtype (nullptr: off).  The CTA whose
    // partition holds token kv_len - 1 quantizes them into row kv_len - 1 before it starts streaming.
    const void* app_k;
    const void* app_v;
    float outer_centroid;
    // reference entry point: the kernel runs only if *gate == gate_want (nullptr: always)
    const int* gate;
    int gate_want;
    const float* dev_signs;   // with a gate: the caller's sign pattern (its magnitude replaces sign_mag)
    // causal chunk: "KV head" x of the grid is query position x / alias_heads on cache head x % alias_heads and
    // sees kv_len0 + x / alias_heads tokens (0: off, every head has its own rows and kv_len tokens)
    int alias_heads, kv_len0;
    // QJL correction of the scores (tq_attention_kernel.cu:197-231): sign sketch words [hkv, kv_stride, 4], residual
    // norms [hkv, kv_stride] (f16 bits), projected queries [hq, 128]; qjl_const = sqrt(pi/2) / sqrt(128) * softmax_scale * log2(e)
    const uint32_t* qjl_signs;
    const uint16_t* qjl_norms;
    const float* rq;
    float qjl_const;
    // sequence-parallel decode: the merging CTA of a KV head pushes the head group's record to every rank (world == 0: off)
    PeerPush peer;
    // host side only: launch with programmatic stream serialization (TQB_DECODE_OVERLAP)
    int overlap;
};

__device__ __forceinline__ void st_relaxed_sys(unsigned* p, unsigned v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    // not volatile: a pure function of its register operands, free to be scheduled between loads
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// m16n8k32, signed 8-bit operands, 32-bit integer result; the addend is zero (a fresh accumulator per call).
__device__ __forceinline__ void imma16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ void imma16832_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
    return d;
}
__device__ __forceinline__ uint32_t bit_select(uint32_t a, uint32_t b, uint32_t mask) {
    return (a & mask) | (b & ~mask);   // one LOP3
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Eight 4-bit codes of one word -> four half2 registers holding the exact values code - 7.5:
//   x[0] = (c0, c4), x[1] = (c1, c5), x[2] = (c2, c6), x[3] = (c3, c7).
// A nibble moved to mantissa bits 1..4 of 0x6400 reads 1024 + 2c, at bits 5..8 it reads 1024 + 32c;
// one HFMA2 with constants that f16 holds exactly (0.5, -519.5 | 1/32, -39.5) turns either into c - 7.5.
__device__ __forceinline__ void nibbles_to_half2(uint32_t w, uint32_t (&x)[4]) {
    const uint32_t kMagic = 0x64006400u;                       // half2(1024, 1024)
    const __half2 kHalf = u32_as_h2(0x38003800u);              // 0.5
    const __half2 kM519 = u32_as_h2(0xE00FE00Fu);              // -519.5
    const __half2 k32nd = u32_as_h2(0x28002800u);              // 1/32
    const __half2 kM39 = u32_as_h2(0xD0F0D0F0u);               // -39.5
    const uint32_t w1 = w << 1, w7 = w >> 7;
    x[0] = h2_as_u32(__hfma2(u32_as_h2(lop3_and_or(w1, 0x001e001eu, kMagic)), kHalf, kM519));
    x[1] = h2_as_u32(__hfma2(u32_as_h2(lop3_and_or(w1, 0x01e001e0u, kMagic)), k32nd, kM39));
    x[2] = h2_as_u32(__hfma2(u32_as_h2(lop3_and_or(w7, 0x001e001eu, kMagic)), kHalf, kM519));
    x[3] = h2_as_u32(__hfma2(u32_as_h2(lop3_and_or(w7, 0x01e001e0u, kMagic)), k32nd, kM39));
}

__device__ __forceinline__ uint32_t pack_hi(float a, float b) { return h2_as_u32(__floats2half2_rn(a, b)); }
__device__ __forceinline__ uint32_t pack_lo(float a, float b) {
    const __half2 hi = __floats2half2_rn(a, b);
    const float2 hf = __half22float2(hi);
    return h2_as_u32(__floats2half2_rn(a - hf.x, b - hf.y));
}

__device__ __forceinline__ float wht32_lane(float v, int lane) {
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
        float other = __shfl_xor_sync(0xffffffffu, v, h);
        v = (lane & h) ? (other - v) : (v + other);
    }
    return v;
}

// ---- per-warp asynchronous staging -------------------------------------------------------
// Each warp owns a ring of kStages stages in shared memory; one stage holds the packed bytes of
// 16 consecutive tokens of one KV head: K indices [16][ROWB], V indices [16][ROWB], K scales
// [16][8 B], V scales [16][8 B] (ROWB = 64 for 4-bit, 48 for 3-bit).  Lanes fill a stage with
// cp.async (16-byte pieces for the indices, 8-byte pieces for the scales) and track completion
// with commit/wait groups, so no thread ever spins on a flag.
// 4-bit: the 16-byte piece c of token row t is stored at piece c ^ ((t >> 1) & 3); with that XOR
// the K pattern (8 tokens x word j) and the V pattern (4 tokens x half-word n) both touch 32
// distinct banks.  3-bit rows are 12 words long, which already spreads both patterns over the
// banks, so they are stored densely.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(dst), "l"(src) : "memory");
}
// The same with immediate offsets folded into the address operands (no address arithmetic in registers).
template <int DOFF, int SOFF>
__device__ __forceinline__ void cp_async16_o(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0+%2], [%1+%3], 16;\n" ::"r"(dst), "l"(src), "n"(DOFF), "n"(SOFF) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// ---- TMA staging (used when asked for and the cache layout allows it) ---------------------------
// A stage holds one 64-token tile of the CTA (16 tokens per warp).  One thread arms the stage's "full"
// mbarrier with the byte count and issues four tensor copies: the K and V index tiles (2-D maps [row bytes,
// all token rows], box = 64 rows; 64-byte swizzle for 4-bit rows) and the K and V scale rows (1-D maps of
// 8-byte elements, box = 64).  Rows past the end of the arrays are zero-filled by the hardware.  Each warp
// arrives on the stage's "empty" mbarrier when it is done with its rows; the producer waits for the four
// arrivals before it refills the stage.  Every wait polls a phase parity with a bound.
struct alignas(64) TmaMaps {
    CUtensorMap k, v, ks, vs;
};
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P1;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, P1;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: try_wait itself sleeps up to a hardware time limit per call.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < (1 << 16); ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_1d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x) {
    asm volatile("cp.async.bulk.tensor.1d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3}], [%2];\n"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
template <int BITS>
__device__ __forceinline__ void tma_tile_fill(const TmaMaps& m, uint32_t tile, uint32_t bar, int row);

__device__ unsigned g_stage_timeouts = 0;   // staging waits that ran out (never expected)

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr) : "memory");   // ordered against other memory operations only
    return v;
}
template <int OFF>
__device__ __forceinline__ uint32_t lds32_o(uint32_t base) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1+%2];\n" : "=r"(v) : "r"(base), "n"(OFF) : "memory");
    return v;
}
template <int OFF>
__device__ __forceinline__ uint2 lds64_o(uint32_t base) {
    uint2 v;
    asm("ld.shared.v2.u32 {%0,%1}, [%2+%3];\n" : "=r"(v.x), "=r"(v.y) : "r"(base), "n"(OFF) : "memory");
    return v;
}
template <int OFF>
__device__ __forceinline__ uint4 lds128_volatile_o(uint32_t base) {
    uint4 v;   // volatile: re-read where it is used instead of being kept in registers across the loop
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(base), "n"(OFF));
    return v;
}

// Four 8x8 matrices of 16-bit elements; lane l supplies the address of row l & 7 of matrix l >> 3.
// Plain: lane (n, j) receives elements 2j, 2j+1 of row n (one 32-bit word).  Transposed: it receives
// element n of rows 2j and 2j+1.
template <int OFF>
__device__ __forceinline__ void ldsm4_o(uint32_t base, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4+%5];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(base), "n"(OFF) : "memory");
}
template <int OFF>
__device__ __forceinline__ void ldsm4t_o(uint32_t base, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4+%5];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(base), "n"(OFF) : "memory");
}

// Transpose of an 8x8 matrix of 16-bit elements held one row per lane group: lane (n, j) gives elements
// (2j, 2j+1) of row n and receives elements (2j, 2j+1) of column n.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}

// Compile-time loop: f(std::integral_constant<int, I>) for I = 0..N-1 (lets loop indices be immediate operands).
template <int I, int N, typename F>
__device__ __forceinline__ void static_for(F&& f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_for<I + 1, N>(f);
    }
}

template <int BITS>
struct Geo {
    static constexpr int kRowB = 16 * BITS;            // packed bytes per token row
    static constexpr int kIdxB = kGroup * kRowB;       // one index array of a stage
    // + K and V scales; 4-bit stages are padded to a multiple of 512 bytes so that the XOR pattern below
    // (bits 4..5 of an address ^ bits 7..8) is the same in every stage - it is TMA's 64-byte swizzle
    static constexpr int kStageB = BITS == 4 ? (2 * kIdxB + 256 + 511) / 512 * 512 : 2 * kIdxB + 256;
    static constexpr int kRingB = kStages * kStageB;
    static constexpr int kTileB = kWarps * (2 * kIdxB + 256);   // TMA staging: one 64-token tile of the CTA
    static constexpr int kPieces = kIdxB / 16;         // 16-byte pieces per index array (64 | 48)
};

// Tile layout: [K rows of warps 0..3][V rows of warps 0..3][K scale rows][V scale rows].
template <int BITS>
__device__ __forceinline__ void tma_tile_fill(const TmaMaps& m, uint32_t tile, uint32_t bar, int row) {
    using G = Geo<BITS>;
    mbar_expect_tx(bar, G::kTileB);
    tma_load_2d(tile, &m.k, bar, 0, row);
    tma_load_2d(tile + kWarps * G::kIdxB, &m.v, bar, 0, row);
    tma_load_1d(tile + 2 * kWarps * G::kIdxB, &m.ks, bar, row);
    tma_load_1d(tile + 2 * kWarps * G::kIdxB + kWarps * 128, &m.vs, bar, row);
}

// Per-lane copy plan of one stage: up to two 16-byte index pieces of K and of V, and one 8-byte
// scale row (K for lanes 0..15, V for lanes 16..31).  The 16 token rows of a stage are contiguous in
// global memory, so piece c of the stage sits at (stage start) + 16 c: the plan keeps running pointers
// to the lane's first piece (the second is 512 bytes further) and to its scale row.
struct FillPlan {
    const uint8_t* k;     // lane's piece of the stage that is filled next
    const uint8_t* v;
    const uint16_t* sc;
    uint32_t dst0, dst1, dsts;   // shared-memory offsets inside a stage
    int t0, t1, ts;       // token rows (inside the group) of the two pieces and of the scale row
    bool has1;
};

template <int BITS>
__device__ __forceinline__ FillPlan make_plan(const MmaArgs& a, size_t row0, int first, int lane) {
    using G = Geo<BITS>;
    FillPlan f;
    constexpr int ppr = G::kRowB / 16;       // pieces per row: 4 | 3
    const int c0 = lane, c1 = lane + 32;
    f.t0 = c0 / ppr;
    f.t1 = c1 / ppr;
    const int pc0 = c0 - f.t0 * ppr, pc1 = c1 - f.t1 * ppr;
    f.has1 = c1 < G::kPieces;
    f.k = a.kb + (row0 + first) * G::kRowB + c0 * 16;
    f.v = a.vb + (row0 + first) * G::kRowB + c0 * 16;
    if (BITS == 4) {
        f.dst0 = f.t0 * 64 + ((pc0 ^ ((f.t0 >> 1) & 3)) << 4);
        f.dst1 = f.t1 * 64 + ((pc1 ^ ((f.t1 >> 1) & 3)) << 4);
    } else {
        f.dst0 = c0 * 16;
        f.dst1 = c1 * 16;
    }
    f.ts = lane & 15;
    f.sc = (lane < 16 ? a.ks : a.vs) + (row0 + first + f.ts) * 4;
    f.dsts = 2 * G::kIdxB + (lane < 16 ? 0 : 128) + f.ts * 8;
    return f;
}

// Issues the copies of the 16 tokens starting at `gs` (where the plan's pointers stand) into the stage at
// shared address `st`, then moves the pointers on by `stride` tokens.  In the final group of a sequence rows
// past the last valid token re-read the last token (they are masked later).
template <int BITS>
__device__ __forceinline__ void stage_fill(FillPlan& f, bool issue, bool ragged, int stride, int gs, int last, uint32_t st) {
    using G = Geo<BITS>;
    const bool has1 = BITS == 4 || f.has1;   // 64 pieces of a 4-bit stage: two per lane
    if (issue) {
        if (!ragged) {
            // the lane's second piece sits 512 bytes further, in global memory and (the swizzle of row t + 8
            // equals that of row t) in the stage
            const uint32_t d0 = st + f.dst0;
            cp_async16_o<0, 0>(d0, f.k);
            cp_async16_o<G::kIdxB, 0>(d0, f.v);
            if (has1) {
                cp_async16_o<512, 512>(d0, f.k);
                cp_async16_o<G::kIdxB + 512, 512>(d0, f.v);
            }
            cp_async8(st + f.dsts, f.sc);
        } else {
            const long long b0 = (long long)(min(gs + f.t0, last) - (gs + f.t0)) * G::kRowB;
            const long long b1 = (long long)(min(gs + f.t1, last) - (gs + f.t1)) * G::kRowB;
            const long long bs = (long long)(min(gs + f.ts, last) - (gs + f.ts)) * 4;
            cp_async16(st + f.dst0, f.k + b0);
            cp_async16(st + G::kIdxB + f.dst0, f.v + b0);
            if (has1) {
                cp_async16(st + f.dst1, f.k + 512 + b1);
                cp_async16(st + G::kIdxB + f.dst1, f.v + 512 + b1);
            }
            cp_async8(st + f.dsts, f.sc + bs);
        }
    }
    f.k += (size_t)stride * G::kRowB;
    f.v += (size_t)stride * G::kRowB;
    f.sc += (size_t)stride * 4;
}

// Grid (kv heads, partitions), 4 warps; each warp walks its partition in steps of 16 tokens and
// keeps its own online-softmax state; the four states are merged through shared memory at the
// end and written as one split-K partial.
//
// NSPLIT = true (GQA group <= 4): MMA columns 2h and 2h + 1 carry the f16 "hi" and "lo" part of head h - of
// the rotated query in S = K~ Q~^T, of P' in O^T = V^T P' - so one MMA delivers the split-precision product.  NSPLIT = false (group 5..8): 8 heads per MMA, hi and lo take one MMA each.
//
// TMA = true: stages are filled by the tensor copy engine (one thread per CTA issues them); otherwise by
// per-lane cp.async.  Both deliver the same bytes in the same swizzled layout.  Measured at 512 KV heads x
// 8192 tokens: cp.async 181-184 us per launch, TMA 191-195 us (4-bit); 230 vs 236-239 us (3-bit).  A first
// TMA version with one 16-token box set per warp (four small copies per warp and step) was slower still
// (193-196 us).  The per-warp cp.async rings let the four warps drift apart freely and keep the copy issue
// off any single warp's critical path; the shared tile ring couples them through its barriers.  So cp.async
// is the default and TMA is opt-in (TQB_DECODE_TMA).
//
// QJL = true (3-bit, cp.async staging): the score of every token gets the correction of the reference's kernel
// (tq_attention_kernel.cu:197-231), norm_t * sqrt(pi/2) / sqrt(128) * sum_d rq[h, d] * (+-1 by the token's sign
// sketch), computed on the integer tensor-core path: the 128 sign bits of a token enter as 0 / 1 bytes (one shift and
// one AND per four of them), the projected query rq as a 20-bit integer in three base-256 digits, and
// sum rq (2 bit - 1) = 2 sum rq bit - sum rq.  The sketch words and norms are fetched straight from global memory one
// step ahead of their use (16 + 2 bytes per token; they are not staged).
template <typename QT, int BITS, bool NSPLIT, bool TMA, bool QJL = false>
__global__ void __launch_bounds__(kThreads, 4) decode_mma_kernel(MmaArgs a, const __grid_constant__ TmaMaps maps,
                                                                 const __grid_constant__ Codebook app_cb) {
    if (a.gate != nullptr && *a.gate != a.gate_want) return;   // the caller's tables are not the ones this kernel decodes
    using G = Geo<BITS>;
    // Dynamic shared memory: [3-bit only: lookup table at an 8 KB-aligned address, so that a table address
    // is formed by OR-ing (index << 7) into the lane's base with one LOP3][stage rings, 1 KB-aligned].
    extern __shared__ unsigned char s_dyn[];
    __shared__ __align__(8) unsigned long long s_bar[2][kStages];   // TMA staging: full / empty barriers of the stages
    __shared__ float s_q[8 * kD];   // rotated queries (prologue only)
    __shared__ __align__(16) uint4 s_qfr[8][32];   // MMA fragments of the rotated queries, [operand set * 4 + block][lane]
    __shared__ float s_qinv[8], s_qsc[8];          // integer operands: per head, value -> 20-bit integer and back (see below)
    __shared__ __align__(16) uint4 s_rqfr[QJL ? (NSPLIT ? 4 : 8) : 1][32];   // QJL: digit fragments of the projected queries
    __shared__ int s_rqsum[8];                     // QJL: per head, the sum of the integer projected query
    const uint32_t dyn_base = (uint32_t)__cvta_generic_to_shared(s_dyn);
    const uint32_t lut_base = BITS == 3 ? ((dyn_base + 8191u) & ~8191u) : 0u;
    const uint32_t rings_base = BITS == 3 ? lut_base + 8192u : ((dyn_base + 1023u) & ~1023u);
    unsigned char* s_raw = s_dyn + (rings_base - dyn_base);
    // epilogue view of the ring memory (the rings are idle then)
    float (*s_o)[8][kD] = reinterpret_cast<float (*)[8][kD]>(s_raw);                 // [kWarps][8][128]
    float (*s_m)[8] = reinterpret_cast<float (*)[8]>(s_raw + kWarps * 8 * kD * 4);   // [kWarps][8]
    float (*s_l)[8] = s_m + kWarps;
    static_assert(kWarps * G::kRingB >= kWarps * 8 * kD * 4 + kWarps * 8 * 4 * 2 + kWarps * 8 * 4 * 4, "ring too small");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = lane >> 2, j = lane & 3;     // n: MMA column / row group, j: position in the quad
    const int kvh = blockIdx.x, part = blockIdx.y;
    const int g = a.g;

    // ---- the queries first: eight small loads per thread that are in flight ahead of the bulk copies started next,
    // instead of queueing behind them (one (head, block) unit per load; consumed after the copies are issued) ----
    float qpre[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int u = warp + kWarps * i, hh = u >> 2, b = u & 3;
        qpre[i] = hh < g ? to_f32<QT>(reinterpret_cast<const QT*>(a.q)[(size_t)(kvh * g + hh) * kD + b * 32 + lane]) : 0.0f;
    }
    // ---- start streaming the first stages: the copies do not depend on q ----
    int kv_len = a.kv_len, cache_head = kvh;
    if (a.alias_heads > 0) {
        const int pos = kvh / a.alias_heads;
        cache_head = kvh - pos * a.alias_heads;
        kv_len = a.kv_len0 + pos;
    }
    const int t_begin = part * a.part_size;
    const int t_end = min(t_begin + a.part_size, kv_len);
    const size_t row0 = (size_t)cache_head * a.kv_stride;
    const int last = kv_len - 1;
    const int first = t_begin + warp * kGroup;
    const int stride = kWarps * kGroup;
    const int ngroups = first < t_end ? (t_end - first + stride - 1) / stride : 0;
    if (a.app_k != nullptr && last >= t_begin && last < t_end) {
        // Fused append.  Only this CTA ever reads row `last` of this KV head, so a block-wide barrier after
        // the stores is all the ordering needed.  One thread per 32-block: warp w takes block w of K (lane 0)
        // and of V (lane 1); same code, same bits as block_quantize_pqo_kernel.
        if (lane < 2) {
            const bool is_v = lane == 1;
            const QT* src = reinterpret_cast<const QT*>(is_v ? a.app_v : a.app_k) + (size_t)kvh * kD + warp * 32;
            uint32_t w[4];
            const float scale = pqo_quantize_block<QT, BITS>(src, app_cb, a.outer_centroid, w);
            const size_t row = row0 + last;
            uint8_t* bp = const_cast<uint8_t*>(is_v ? a.vb : a.kb) + row * G::kRowB + warp * (4 * BITS);
            if (BITS == 4) {
                *reinterpret_cast<uint4*>(bp) = make_uint4(w[0], w[1], w[2], w[3]);
            } else {
                uint32_t* wp = reinterpret_cast<uint32_t*>(bp);
                wp[0] = w[0]; wp[1] = w[1]; wp[2] = w[2];
            }
            const_cast<uint16_t*>(is_v ? a.vs : a.ks)[row * 4 + warp] = f32_to_f16_bits(-scale);   // outlier blocks store -scale
        }
        __threadfence();   // device-wide: a later launch that starts early (below) reads these rows
        if (TMA) asm volatile("fence.proxy.async;\n" ::: "memory");   // the tensor copies read through the async proxy
        __syncthreads();
    }
    // Programmatic dependent launch.  From here on the next kernel on the stream may start on the SMs this grid leaves
    // free, IF it was launched with programmatic stream serialization (TQB_DECODE_OVERLAP): its streaming pass then
    // overlaps this grid's tail and merge.  Such a launch reads q, the appended vectors and the cache early, and
    // waits for this grid's completion (griddepcontrol.wait, further down) before it touches what the two share: the
    // split-K scratch, the tickets and the outputs.  The appended row was stored and fenced above.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    // cp.async: every warp owns a ring of 16-token stages.  TMA: the CTA owns a ring of 64-token tiles and
    // `ring` / `st` address this warp's K rows inside a tile.
    constexpr uint32_t kPitch = TMA ? G::kTileB : G::kStageB;           // distance between stages
    constexpr uint32_t kVD = TMA ? kWarps * G::kIdxB : G::kIdxB;        // from a warp's K rows to its V rows
    constexpr uint32_t kSD = TMA ? kWarps * 128 : 128;                  // from its K scale rows to its V scale rows
    const uint32_t ring = TMA ? rings_base + warp * G::kIdxB : rings_base + warp * G::kRingB;
    const uint32_t sdelta = TMA ? 2 * kWarps * G::kIdxB - warp * (G::kIdxB - 128) : 2 * G::kIdxB;   // K rows -> K scale rows
    FillPlan plan = TMA ? FillPlan{} : make_plan<BITS>(a, row0, first, lane);
    const uint32_t full0 = (uint32_t)__cvta_generic_to_shared(&s_bar[0][0]);
    const uint32_t empty0 = (uint32_t)__cvta_generic_to_shared(&s_bar[1][0]);
    const int ntiles = t_begin < t_end ? (t_end - t_begin + stride - 1) / stride : 0;   // 64-token tiles of the CTA
    const int nsteps = TMA ? ntiles : ngroups;
    const int trow0 = (int)row0 + t_begin;                     // TMA: token row of tile 0 in the whole array
    const bool producer = TMA && tid == 0;
    if (TMA) {
        if (producer) {
#pragma unroll
            for (int i = 0; i < kStages; ++i) {
                mbar_init(full0 + 8 * i, 1);
                mbar_init(empty0 + 8 * i, kWarps);
            }
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
#pragma unroll
            for (int i = 0; i < kStages - 1; ++i)
                if (i < ntiles) tma_tile_fill<BITS>(maps, rings_base + i * G::kTileB, full0 + 8 * i, trow0 + i * stride);
        }
        // the other threads first touch a barrier after the block-wide barriers of the query prologue
    } else {
#pragma unroll
        for (int i = 0; i < kStages - 1; ++i) {
            stage_fill<BITS>(plan, i < ngroups, first + i * stride + kGroup > last + 1, stride, first + i * stride, last, ring + i * G::kStageB);
            cp_async_commit();
        }
    }
    uint32_t st = ring;                                        // stage being consumed (this warp's K rows)
    uint32_t st_fill = TMA ? rings_base + (kStages - 1) * G::kTileB : ring + (kStages - 1) * G::kStageB;   // stage being refilled
    // TMA: barrier offset (8 x stage) of st / of st_fill, phase of st's full barrier, phase of st_fill's empty barrier
    uint32_t boff = 0, boff_fill = 8 * (kStages - 1), parity = 0, eparity = 1;
    bool stage_ok = true;

    // per-thread shared-memory offsets inside a stage; every load of the token loop is one of three or four
    // per-step base registers (stage + offset) plus an immediate
    uint32_t offK0, offK1, offV = 0, offVh = 0;      // 4-bit: ldmatrix rows of blocks (0,1) / (2,3); 3-bit: first / second word
    uint32_t ksh = 0, vsh = 0;                       // 3-bit: funnel shifts
    if (BITS == 4) {
        // ldmatrix row addresses: lane l supplies row l & 7 of matrix l >> 3.  Matrix m covers the token
        // octet m & 1 and the block 2 * pair + (m >> 1); a row is the 16-byte piece of one token.
        const int tok = 8 * ((lane >> 3) & 1) + (lane & 7), blk = lane >> 4;
        offK0 = tok * 64 + ((blk ^ ((tok >> 1) & 3)) << 4);
        offK1 = offK0 ^ 32;                          // blocks 2, 3: piece index ^ 2
    } else {
        // K: the 24 bits at byte 3j of block b of token n;  V: the 12 bits at bit 12n of block b of token 2j
        const int kw0 = (3 * j) >> 2;
        const int vw0 = (12 * n) >> 5;
        ksh = ((3 * j) & 3) * 8;
        vsh = (12 * n) & 31;
        offK0 = n * 48 + 4 * kw0;                    // + 12 b, + 8 rows per octet
        offK1 = offK0 + ((kw0 < 2) ? 4 : 0);
        offV = kVD + (2 * j) * 48 + 4 * vw0;         // + 12 b, + 48 per token, + 8 rows per octet
        offVh = offV + ((vsh + 12 > 32) ? 4 : 0);
    }
    constexpr uint32_t kOct = 8 * G::kRowB;                                     // 8 token rows
    constexpr uint32_t kRow = G::kRowB;
    const uint32_t offS = sdelta + n * 8;                                       // K scale row of token n (+64: token n + 8)
    const uint32_t lut = lut_base + lane * 4;

    if (BITS == 3) {
        // entry e = c0 | c1 << 3 -> half2(lut[c0], lut[c1]), one copy per bank
        for (int i = tid; i < 64 * 32; i += kThreads) {
            const int e = i >> 5;
            const uint32_t v = pack_hi(a.lut[e & 7], a.lut[e >> 3]);
            asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(lut_base + i * 4), "r"(v) : "memory");
        }
    }
    // ---- rotate the g queries of this KV head once: q~ = sigma .* H32(q_b) / sqrt(32), constants folded ----
    {
        const uint32_t neg = 0xB1A6D4B2u;  // src/cache/precomputed/rotation.rs:16-20
        const float mag = a.dev_signs != nullptr ? fabsf(a.dev_signs[0]) : a.sign_mag;
        const float sign = ((neg >> lane) & 1u) ? -mag : mag;
        const float inv_sqrt = 1.0f / sqrtf(32.0f);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int u = warp + kWarps * i, hh = u >> 2, b = u & 3;
            const float v = wht32_lane(qpre[i], lane);
            s_q[hh * kD + b * 32 + lane] = ((v * inv_sqrt) * sign) * a.qk_const;
        }
    }
    __syncthreads();
    // Scores are computed as S = K~ Q~^T: the A operand is the unpacked K tile (M = 16 tokens of one block), the B
    // operand holds the rotated queries (N = 8 columns).
    // 3-bit (f16 MMA, K = 16 dims): NSPLIT (group <= 4): columns 2h and 2h + 1 are the f16 hi and lo parts of q~ of
    // head h, so one MMA gives the split-precision product and both parts of a head land in the same lane; else two
    // operand sets (hi, lo) of 8 heads.  For block b and half m the k-slots (2j, 2j+1 | 2j+8, 2j+9) hold the dims
    // 32b + 8j + 4m + (0, 1 | 2, 3) that the code unpacker delivers; s_qfr[set * 4 + b][lane] = (b0, b1 of half 0,
    // b0, b1 of half 1) of the lane's column n.
    // 4-bit (integer MMA, K = 32 dims = the whole block): k-slots 4j .. 4j+3 hold dims 32b + 8j + (0, 2, 4, 6) (the even
    // nibbles of word j), k-slots 16 + 4j .. hold dims 32b + 8j + (1, 3, 5, 7) (the odd nibbles).
    if (BITS == 4) {
        // 4-bit: the scores run on the integer tensor-core path (mma.sync m16n8k32, s8 x s8 -> s32).  A code c enters
        // as the byte 16 (c - 7.5) (two logic operations per four codes, see the token loop); the rotated query of a
        // head enters as a 20-bit integer v = round(q~ 2^19 / max |q~|) split into three balanced base-256 digits
        // v = 65536 D2 + 256 D1 + D0, one MMA column per digit.  All integer arithmetic is exact, |sum| < 2^31 (32 dims
        // x 120 x 2^19), and q~ is represented to 2^-20 of the head's largest component.
        for (int hh = warp; hh < 8; hh += kWarps) {
            float m = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) m = fmaxf(m, fabsf(s_q[hh * kD + lane + 32 * i]));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            if (lane == 0) {
                const bool ok = m > 0.0f && m < 3.0e38f;
                s_qinv[hh] = ok ? 524287.0f / m : 0.0f;
                s_qsc[hh] = ok ? m / (524287.0f * 16.0f) : 0.0f;
            }
        }
        __syncthreads();
        const int b = warp;   // one block per warp
        const int head = NSPLIT ? (n >> 1) : n;
        const float* sq = s_q + head * kD;
        const float inv = s_qinv[head];
        uint32_t dg[3][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}};   // [digit 0 = D0 (low)][k half: dims 8j + even | 8j + odd]
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int v = __float2int_rn(sq[32 * b + 8 * j + 2 * i + half] * inv);
                const int d0 = (int)(signed char)(v & 0xFF);
                const int v1 = (v - d0) >> 8;
                const int d1 = (int)(signed char)(v1 & 0xFF);
                const int d2 = (v1 - d1) >> 8;
                dg[0][half] |= (uint32_t)(d0 & 0xFF) << (8 * i);
                dg[1][half] |= (uint32_t)(d1 & 0xFF) << (8 * i);
                dg[2][half] |= (uint32_t)(d2 & 0xFF) << (8 * i);
            }
        if (NSPLIT) {
            // columns 2h, 2h + 1 of the first MMA: digits D2, D1 of head h; of the second MMA: D0 and an empty column
            const bool odd = n & 1;
            s_qfr[b][lane] = make_uint4(odd ? dg[1][0] : dg[2][0], odd ? dg[1][1] : dg[2][1], odd ? 0u : dg[0][0], odd ? 0u : dg[0][1]);
        } else {
            // column h of three MMAs: digits D2, D1, D0 of head h
            s_qfr[b][lane] = make_uint4(dg[2][0], dg[2][1], dg[1][0], dg[1][1]);
            s_qfr[4 + b][lane] = make_uint4(dg[0][0], dg[0][1], 0u, 0u);
        }
    } else {
        const float* sq = s_q + (NSPLIT ? (n >> 1) : n) * kD;
        const int b = warp;   // one block per warp
#pragma unroll
        for (int set = 0; set < (NSPLIT ? 1 : 2); ++set) {
            const bool lo_part = NSPLIT ? (n & 1) : (set == 1);
            uint32_t r[4];
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const int d0 = 32 * b + 8 * j + 4 * m;
                const float qa = sq[d0], qb = sq[d0 + 1];
                const float qc = sq[d0 + 2], qd = sq[d0 + 3];
                r[2 * m] = lo_part ? pack_lo(qa, qb) : pack_hi(qa, qb);
                r[2 * m + 1] = lo_part ? pack_lo(qc, qd) : pack_hi(qc, qd);
            }
            s_qfr[set * 4 + b][lane] = make_uint4(r[0], r[1], r[2], r[3]);
        }
    }
    __syncthreads();
    if constexpr (QJL) {
        // The projected queries rq of the g heads replace the rotated queries in s_q (those live in their fragments
        // by now), are scaled to 20-bit integers per head like the 4-bit path's queries, and laid out as B fragments:
        // MMA number m (0..3) contracts, in lane quad position j, the dims 32j + 2m + 8i (k-slots 4j + i) and
        // 32j + 2m + 1 + 8i (k-slots 16 + 4j + i), i = 0..3 - the order in which the sign bits are peeled off a word.
        for (int i = tid; i < 8 * kD; i += kThreads) {
            const int hh = i >> 7;
            s_q[i] = hh < g ? a.rq[(size_t)(kvh * g + hh) * kD + (i & 127)] : 0.0f;
        }
        __syncthreads();
        for (int hh = warp; hh < 8; hh += kWarps) {
            float m = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) m = fmaxf(m, fabsf(s_q[hh * kD + lane + 32 * i]));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            const bool ok = m > 0.0f && m < 3.0e38f;
            const float inv = ok ? 524287.0f / m : 0.0f;
            int sum = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) sum += __float2int_rn(s_q[hh * kD + lane + 32 * i] * inv);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (lane == 0) {
                s_qinv[hh] = inv;
                s_qsc[hh] = ok ? m / 524287.0f : 0.0f;
                s_rqsum[hh] = sum;
            }
        }
        __syncthreads();
        {
            const int m4 = warp;   // one of the four MMAs per warp
            const int head = NSPLIT ? (n >> 1) : n;
            const float inv = s_qinv[head];
            uint32_t dg[3][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}};
#pragma unroll
            for (int half = 0; half < 2; ++half)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int v = __float2int_rn(s_q[head * kD + 32 * j + 2 * m4 + half + 8 * i] * inv);
                    const int d0 = (int)(signed char)(v & 0xFF);
                    const int v1 = (v - d0) >> 8;
                    const int d1 = (int)(signed char)(v1 & 0xFF);
                    const int d2 = (v1 - d1) >> 8;
                    dg[0][half] |= (uint32_t)(d0 & 0xFF) << (8 * i);
                    dg[1][half] |= (uint32_t)(d1 & 0xFF) << (8 * i);
                    dg[2][half] |= (uint32_t)(d2 & 0xFF) << (8 * i);
                }
            if (NSPLIT) {
                const bool odd = n & 1;
                s_rqfr[m4][lane] = make_uint4(odd ? dg[1][0] : dg[2][0], odd ? dg[1][1] : dg[2][1], odd ? 0u : dg[0][0], odd ? 0u : dg[0][1]);
            } else {
                s_rqfr[m4][lane] = make_uint4(dg[2][0], dg[2][1], dg[1][0], dg[1][1]);
                s_rqfr[4 + m4][lane] = make_uint4(dg[0][0], dg[0][1], 0u, 0u);
            }
        }
        __syncthreads();
    }
    const uint32_t qfr_base = (uint32_t)__cvta_generic_to_shared(&s_qfr[0][lane]);
    const uint32_t rqfr_base = (uint32_t)__cvta_generic_to_shared(&s_rqfr[0][lane]);
    // After the scores, lane (n, j) holds tokens n and n + 8 of the step and kE heads:
    //   NSPLIT: head j (its hi and lo columns 2j, 2j+1 are summed in the lane)  |  otherwise heads 2j, 2j+1.
    constexpr int kE = NSPLIT ? 1 : 2;
    float qsc[kE];                // 4-bit: integer score -> log2-domain score of the lane's head(s)
#pragma unroll
    for (int e = 0; e < kE; ++e) qsc[e] = BITS == 4 ? s_qsc[NSPLIT ? j : 2 * j + e] : 1.0f;
    float rqc[kE];                // QJL: integer correction -> log2-domain score, without the token's residual norm
    int rqsum[kE];
#pragma unroll
    for (int e = 0; e < kE; ++e) {
        rqc[e] = QJL ? s_qsc[NSPLIT ? j : 2 * j + e] * a.qjl_const : 0.0f;
        rqsum[e] = QJL ? s_rqsum[NSPLIT ? j : 2 * j + e] : 0;
    }
    // QJL: sketch word j and residual norm of tokens n and n + 8 of the step, fetched two steps ahead (tokens past
    // the end re-read the last token; they are masked later)
    uint32_t sgw[2] = {0u, 0u};
    uint32_t nrw[2] = {0u, 0u};
    auto qjl_fetch = [&](int it, uint32_t (&sg)[2], uint32_t (&nr)[2]) {
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const size_t row = row0 + (size_t)min(first + it * stride + n + 8 * t, last);
            sg[t] = __ldg(a.qjl_signs + row * 4 + j);
            nr[t] = __ldg(a.qjl_norms + row);
        }
    };
    // (two steps ahead: one step is shorter than a trip to HBM)
    uint32_t sg1[2] = {0u, 0u};
    uint32_t nr1[2] = {0u, 0u};
    if (QJL && nsteps > 0) qjl_fetch(0, sgw, nrw);
    if (QJL && nsteps > 1) qjl_fetch(1, sg1, nr1);
    float m_run[kE], l_run[kE];   // per head; l_run: this lane's tokens only
#pragma unroll
    for (int e = 0; e < kE; ++e) {
        m_run[e] = kNegBig;
        l_run[e] = 0.0f;
    }
    float o[4][2][4];
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[b][m][i] = 0.0f;

    // Loop control in terms of iteration numbers fixed before the loop: the last step that still refills a
    // stage, the step whose refill is the (only possibly) ragged last group, and the first step with tokens to mask.
    const int fill_end = ngroups - (kStages - 1);                                    // refill while it < fill_end
    const int rag_fill_it = (first + (ngroups - 1) * stride + kGroup > last + 1) ? fill_end - 1 : -1;
    const int rag_from = (t_end - kGroup - first < 0) ? 0 : (t_end - kGroup - first) / stride + 1;
    uint32_t st_prev = ring + (kStages - 1) * kPitch;   // cp.async: the stage consumed one step ago is the one refilled now
#pragma unroll 2
    for (int it = 0; it < nsteps; ++it) {
        if (TMA) {
            // A warp whose 16 rows of the tile lie past the end of the partition runs the step on them all
            // the same: every such token is masked below and contributes exactly nothing.
            if (producer && it + kStages - 1 < ntiles) {
                // refill the stage of tile it - 1 once all four warps have released it
                if (it >= 1 && !mbar_wait(empty0 + boff_fill, eparity)) stage_ok = false;
                else tma_tile_fill<BITS>(maps, st_fill, full0 + boff_fill, trow0 + (it + kStages - 1) * stride);
            }
            __syncwarp();
            if (boff_fill + 8 == 8 * kStages) { boff_fill = 0; eparity ^= 1u; } else boff_fill += 8;
            st_fill = (st_fill + kPitch == rings_base + kStages * kPitch) ? rings_base : st_fill + kPitch;
            if (!mbar_wait(full0 + boff, parity)) {   // never expected: give up on this partition and say so
                stage_ok = false;
                break;
            }
        } else {
            stage_fill<BITS>(plan, it < fill_end, it == rag_fill_it, stride, first + (it + kStages - 1) * stride, last, st_prev);
            cp_async_commit();
            cp_async_wait<kStages - 1>();
            __syncwarp();
        }

        const uint32_t bK0 = st + offK0, bK1 = st + offK1, bS = st + offS;
        // ---- S = K~ Q~^T : rows = tokens (n, n + 8), columns = heads ----
        uint32_t kw[2][4];   // 4-bit: [block pair][octet | block parity << 1] -> word j of token n of the octet
        if (BITS == 4) {
            ldsm4_o<0>(bK0, kw[0]);
            ldsm4_o<0>(bK1, kw[1]);
        }
        float s[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};   // [token n | n + 8][head h(e)]
        {
            const uint2 sca = lds64_o<0>(bS), scb = lds64_o<64>(bS);   // scale rows of the two tokens
            static_for<0, 4>([&](auto b_) {
                constexpr int b = decltype(b_)::value;
                const __half2 pa = u32_as_h2(b < 2 ? sca.x : sca.y), pb = u32_as_h2(b < 2 ? scb.x : scb.y);
                const float ka = fabsf((b & 1) ? __high2float(pa) : __low2float(pa));
                const float kb = fabsf((b & 1) ? __high2float(pb) : __low2float(pb));
                if constexpr (BITS == 4) {
                    // Codes -> signed bytes 16 (c - 7.5) = 8 (2c - 15): flip the top bit of every nibble (c ^ 8 is the
                    // 4-bit two's complement of c - 8), move the nibble to the top of a byte and set bit 3 below it.
                    // Even nibbles (dims 8j + 0, 2, 4, 6) fill k-slots 4j .. 4j+3, odd nibbles k-slots 16 + 4j ..
                    const uint32_t u0 = kw[b >> 1][2 * (b & 1)] ^ 0x88888888u;        // token n
                    const uint32_t u1 = kw[b >> 1][2 * (b & 1) + 1] ^ 0x88888888u;    // token n + 8
                    const uint32_t a0 = lop3_and_or(u0 << 4, 0xF0F0F0F0u, 0x08080808u), a2 = lop3_and_or(u0, 0xF0F0F0F0u, 0x08080808u);
                    const uint32_t a1 = lop3_and_or(u1 << 4, 0xF0F0F0F0u, 0x08080808u), a3 = lop3_and_or(u1, 0xF0F0F0F0u, 0x08080808u);
                    const uint4 q4 = lds128_volatile_o<b * 512>(qfr_base);
                    int hi[4], lo[4];
                    imma16832(hi, a0, a1, a2, a3, q4.x, q4.y);
                    imma16832(lo, a0, a1, a2, a3, q4.z, q4.w);
                    if (NSPLIT) {   // hi: columns (D2, D1) of head j, lo: columns (D0, -)
                        const int i0 = (int)((uint32_t)hi[0] * 65536u + (uint32_t)hi[1] * 256u + (uint32_t)lo[0]);
                        const int i1 = (int)((uint32_t)hi[2] * 65536u + (uint32_t)hi[3] * 256u + (uint32_t)lo[2]);
                        s[0][0] = fmaf(ka, (float)i0, s[0][0]);
                        s[1][0] = fmaf(kb, (float)i1, s[1][0]);
                    } else {        // hi: digit D2 of heads 2j, 2j+1, lo: digit D1, third MMA: digit D0
                        const uint2 q2 = lds64_o<(4 + b) * 512>(qfr_base);
                        int l0[4];
                        imma16832(l0, a0, a1, a2, a3, q2.x, q2.y);
                        int iv[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) iv[i] = (int)((uint32_t)hi[i] * 65536u + (uint32_t)lo[i] * 256u + (uint32_t)l0[i]);
                        s[0][0] = fmaf(ka, (float)iv[0], s[0][0]);
                        s[0][1] = fmaf(ka, (float)iv[1], s[0][1]);
                        s[1][0] = fmaf(kb, (float)iv[2], s[1][0]);
                        s[1][1] = fmaf(kb, (float)iv[3], s[1][1]);
                    }
                } else {
                    uint32_t x[2][4];   // [token n | n + 8]: codes 8j..8j+7 of block b as four half2
                    static_for<0, 2>([&](auto t_) {
                        constexpr int t = decltype(t_)::value;
                        const uint32_t lo = lds32_o<12 * b + t * kOct>(bK0), hi = lds32_o<12 * b + t * kOct>(bK1);
                        const uint32_t w = __funnelshift_r(lo, hi, ksh);          // codes 8j..8j+7 in bits 0..23
                        x[t][0] = lds32(lop3_and_or(w << 7, 0x1F80u, lut));
                        x[t][1] = lds32(lop3_and_or(w << 1, 0x1F80u, lut));
                        x[t][2] = lds32(lop3_and_or(w >> 5, 0x1F80u, lut));
                        x[t][3] = lds32(lop3_and_or(w >> 11, 0x1F80u, lut));
                    });
                    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    static_for<0, (NSPLIT ? 1 : 2)>([&](auto set_) {
                        constexpr int set = decltype(set_)::value;
                        const uint4 q4 = lds128_volatile_o<(set * 4 + b) * 512>(qfr_base);
                        mma16816(acc, x[0][0], x[1][0], x[0][1], x[1][1], q4.x, q4.y);
                        mma16816(acc, x[0][2], x[1][2], x[0][3], x[1][3], q4.z, q4.w);
                    });
                    if (NSPLIT) {   // columns 2j, 2j+1 are the hi and lo part of one head: one running sum per token
                        s[0][0] = fmaf(ka, acc[1], fmaf(ka, acc[0], s[0][0]));
                        s[1][0] = fmaf(kb, acc[3], fmaf(kb, acc[2], s[1][0]));
                    } else {
                        s[0][0] = fmaf(ka, acc[0], s[0][0]);
                        s[0][1] = fmaf(ka, acc[1], s[0][1]);
                        s[1][0] = fmaf(kb, acc[2], s[1][0]);
                        s[1][1] = fmaf(kb, acc[3], s[1][1]);
                    }
                }
            });
        }
        float sc[2][kE];   // scores [token n | n + 8][head]
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int e = 0; e < kE; ++e) sc[t][e] = BITS == 4 ? s[t][e] * qsc[e] : s[t][e];
        if constexpr (QJL) {
            uint32_t sgn[2] = {0u, 0u}, nrn[2] = {0u, 0u};
            if (it + 2 < nsteps) qjl_fetch(it + 2, sgn, nrn);   // the sketch words of the step after next, in flight for two steps
            int ca[4] = {0, 0, 0, 0}, cb[4] = {0, 0, 0, 0}, cc[4] = {0, 0, 0, 0};
            static_for<0, 4>([&](auto m_) {
                constexpr int m4 = decltype(m_)::value;
                // bytes i of the four operands: sign bits 2 m4 + 8 i (and 2 m4 + 1 + 8 i) of the two tokens' words
                const uint32_t a0 = (sgw[0] >> (2 * m4)) & 0x01010101u, a1 = (sgw[1] >> (2 * m4)) & 0x01010101u;
                const uint32_t a2 = (sgw[0] >> (2 * m4 + 1)) & 0x01010101u, a3 = (sgw[1] >> (2 * m4 + 1)) & 0x01010101u;
                const uint4 r4 = lds128_volatile_o<m4 * 512>(rqfr_base);
                imma16832_acc(ca, a0, a1, a2, a3, r4.x, r4.y);
                imma16832_acc(cb, a0, a1, a2, a3, r4.z, r4.w);
                if (!NSPLIT) {
                    const uint2 r2 = lds64_o<(4 + m4) * 512>(rqfr_base);
                    imma16832_acc(cc, a0, a1, a2, a3, r2.x, r2.y);
                }
            });
            const float n0 = __half2float(__ushort_as_half((unsigned short)nrw[0]));
            const float n1 = __half2float(__ushort_as_half((unsigned short)nrw[1]));
            if (NSPLIT) {   // ca: columns (D2, D1) of head j, cb: (D0, -)
                const int i0 = (int)((uint32_t)ca[0] * 65536u + (uint32_t)ca[1] * 256u + (uint32_t)cb[0]);
                const int i1 = (int)((uint32_t)ca[2] * 65536u + (uint32_t)ca[3] * 256u + (uint32_t)cb[2]);
                sc[0][0] = fmaf((float)(2 * i0 - rqsum[0]), n0 * rqc[0], sc[0][0]);
                sc[1][0] = fmaf((float)(2 * i1 - rqsum[0]), n1 * rqc[0], sc[1][0]);
            } else {        // ca / cb / cc: digits D2 / D1 / D0 of heads 2j, 2j+1
                int iv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) iv[i] = (int)((uint32_t)ca[i] * 65536u + (uint32_t)cb[i] * 256u + (uint32_t)cc[i]);
                sc[0][0] = fmaf((float)(2 * iv[0] - rqsum[0]), n0 * rqc[0], sc[0][0]);
                sc[0][1] = fmaf((float)(2 * iv[1] - rqsum[1]), n0 * rqc[1], sc[0][1]);
                sc[1][0] = fmaf((float)(2 * iv[2] - rqsum[0]), n1 * rqc[0], sc[1][0]);
                sc[1][1] = fmaf((float)(2 * iv[3] - rqsum[1]), n1 * rqc[1], sc[1][1]);
            }
            sgw[0] = sg1[0]; sgw[1] = sg1[1]; nrw[0] = nr1[0]; nrw[1] = nr1[1];
            sg1[0] = sgn[0]; sg1[1] = sgn[1]; nr1[0] = nrn[0]; nr1[1] = nrn[1];
        }
        if (it >= rag_from) {   // ragged tail: tokens past the end (of the sequence, or of the partition) get zero weight
            const int gs = first + it * stride;
            if (TMA) {
                // the tensor copies brought whatever lies behind the last token: clear those scale rows, so
                // that a zero probability never meets an Inf or NaN scale
                const int t = lane & 15;
                if (gs + t >= t_end)
                    asm volatile("st.shared.v2.u32 [%0], {%1, %1};\n" ::"r"(st + sdelta + (lane >> 4) * kSD + t * 8), "r"(0u) : "memory");
                __syncwarp();
            }
#pragma unroll
            for (int t = 0; t < 2; ++t)
                if (gs + n + 8 * t >= t_end) {
#pragma unroll
                    for (int e = 0; e < kE; ++e) sc[t][e] = kNegBig;
                }
        }
        // ---- online softmax: the 16 tokens of a head are spread over the 8 lane groups n ----
        // The reference value m_run is only raised when the step's maximum exceeds it by more than kLazy
        // (in log2 units): any common reference gives the same result, p stays below 2^kLazy, and the
        // rescaling of the 32 accumulators becomes rare.
        constexpr float kLazy = 6.0f;
        float resc[kE], p[2][kE];
        bool changed = false;
#pragma unroll
        for (int e = 0; e < kE; ++e) {
            float mx = fmaxf(sc[0][e], sc[1][e]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = (mx - m_run[e] > kLazy) ? mx : m_run[e];
            resc[e] = ex2(m_run[e] - m_new);
            changed |= resc[e] != 1.0f;
            m_run[e] = m_new;
            p[0][e] = ex2(sc[0][e] - m_new);
            p[1][e] = ex2(sc[1][e] - m_new);
            l_run[e] = l_run[e] * resc[e] + (p[0][e] + p[1][e]);
        }
        if (__any_sync(0xffffffffu, changed)) {
            // columns (2j, 2j+1) of O^T: NSPLIT the hi and lo column of head j, otherwise heads 2j and 2j+1
            const float r0 = resc[0], r1 = resc[kE - 1];
#pragma unroll
            for (int b = 0; b < 4; ++b)
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    o[b][m][0] *= r0; o[b][m][1] *= r1; o[b][m][2] *= r0; o[b][m][3] *= r1;
                }
        }
        // ---- P' = p |s_v| as an exact f16 pair, in half2 arithmetic, then transposed for the next MMA ----
        // p = ph + pl (f16 each).  hi = rn(ph s) and ph s - hi are both f16 values (the product of two 11-bit
        // significands has 22 bits), so hi + lo with lo = fma(pl, s, fma(ph, s, -hi)) equals p s up to 2^-22
        // relative.  movmatrix takes registers holding the lane's two columns of one token row - NSPLIT: (hi, lo)
        // of head j, otherwise the hi (or lo) parts of heads 2j, 2j+1 - and turns each 8 x 8 matrix (token rows,
        // columns) into the B fragment (tokens 2j, 2j+1 of column n) of O^T = V^T P'.
        uint32_t pq[NSPLIT ? 1 : 2][4][2];   // [hi | lo][block][octet]
        if (NSPLIT) {
            // one head per lane: the half2 lanes run over the two tokens (n, n + 8); three instructions per
            // block give (hi', hi') and (lo', lo') of both tokens, two PRMTs re-pair them per token
            const __half2 ph = u32_as_h2(pack_hi(p[0][0], p[1][0])), pl = u32_as_h2(pack_lo(p[0][0], p[1][0]));
            const uint2 vs0 = lds64_o<kSD>(bS), vs1 = lds64_o<kSD + 64>(bS);   // V scale rows of tokens n, n + 8
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const __half2 sv = __habs2(u32_as_h2(__byte_perm(b < 2 ? vs0.x : vs0.y, b < 2 ? vs1.x : vs1.y, (b & 1) ? 0x7632 : 0x5410)));
                const __half2 hi = __hmul2(ph, sv);
                const __half2 lo = __hfma2(pl, sv, __hfma2(ph, sv, __hneg2(hi)));
                pq[0][b][0] = movmatrix_trans(__byte_perm(h2_as_u32(hi), h2_as_u32(lo), 0x5410));   // token n: (hi', lo') of head j
                pq[0][b][1] = movmatrix_trans(__byte_perm(h2_as_u32(hi), h2_as_u32(lo), 0x7632));   // token n + 8
            }
        } else {
            static_for<0, 2>([&](auto t_) {
                constexpr int t = decltype(t_)::value;
                const __half2 ph = u32_as_h2(pack_hi(p[t][0], p[t][kE - 1]));
                const __half2 pl = u32_as_h2(pack_lo(p[t][0], p[t][kE - 1]));
                const uint2 vsr = lds64_o<kSD + t * 64>(bS);   // V scale row of token n + 8t
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const __half2 svw = u32_as_h2(b < 2 ? vsr.x : vsr.y);
                    const __half2 sv = __habs2((b & 1) ? __high2half2(svw) : __low2half2(svw));   // (s, s)
                    const __half2 hi = __hmul2(ph, sv);
                    const __half2 lo = __hfma2(pl, sv, __hfma2(ph, sv, __hneg2(hi)));
                    pq[0][b][t] = movmatrix_trans(h2_as_u32(hi));
                    pq[NSPLIT ? 0 : 1][b][t] = movmatrix_trans(h2_as_u32(lo));
                }
            });
        }
        // ---- O^T += V^T P' ----
        uint32_t vw[2][4];   // 4-bit: codes 4n..4n+3 of (token 2j | token 2j+1 << 16), indexed like kw
        if (BITS == 4) {
            ldsm4t_o<kVD>(bK0, vw[0]);
            ldsm4t_o<kVD>(bK1, vw[1]);
        }
        const uint32_t bV = st + offV, bVh = st + offVh;   // 3-bit only
        static_for<0, 4>([&](auto b_) {
            constexpr int b = decltype(b_)::value;
            // codes 4n..4n+3 of block b of the four tokens, paired (token 2j, token 2j+1)
            uint32_t xab[4], xcd[4];
            if (BITS == 4) {
                nibbles_to_half2(vw[b >> 1][2 * (b & 1)], xab);
                nibbles_to_half2(vw[b >> 1][2 * (b & 1) + 1], xcd);
            } else {
                static_for<0, 2>([&](auto o_) {
                    constexpr int o8 = decltype(o_)::value;
                    constexpr int off = 12 * b + o8 * kOct;
                    const uint32_t xa = __funnelshift_r(lds32_o<off>(bV), lds32_o<off>(bVh), vsh);                // token 2j
                    const uint32_t xb = __funnelshift_r(lds32_o<off + kRow>(bV), lds32_o<off + kRow>(bVh), vsh);  // token 2j+1
                    // 6-bit fields (code of token 2j | code of token 2j+1 << 3): codes 0, 2 in z0, codes 1, 3 in z1
                    const uint32_t z0 = bit_select(xa, xb << 3, 0x1C7u);
                    const uint32_t z1 = bit_select(xa >> 3, xb, 0x1C7u);
                    uint32_t* xo = o8 == 0 ? xab : xcd;
                    xo[0] = lds32(lop3_and_or(z0 << 7, 0x1F80u, lut));
                    xo[2] = lds32(lop3_and_or(z0 << 1, 0x1F80u, lut));
                    xo[1] = lds32(lop3_and_or(z1 << 7, 0x1F80u, lut));
                    xo[3] = lds32(lop3_and_or(z1 << 1, 0x1F80u, lut));
                });
            }
#pragma unroll
            for (int ps = 0; ps < (NSPLIT ? 1 : 2); ++ps) {
                mma16816(o[b][0], xab[0], xab[1], xcd[0], xcd[1], pq[ps][b][0], pq[ps][b][1]);
                mma16816(o[b][1], xab[2], xab[3], xcd[2], xcd[3], pq[ps][b][0], pq[ps][b][1]);
            }
        });
        __syncwarp();   // every lane is done with this stage before it is refilled
        st_prev = st;
        st = (st + kPitch == ring + kStages * kPitch) ? ring : st + kPitch;
        if (TMA) {
            if (lane == 0) mbar_arrive(empty0 + boff);   // this warp releases its rows of the tile
            if (boff + 8 == 8 * kStages) { boff = 0; parity ^= 1u; } else boff += 8;
        }
    }
    bool gave_up = false;
    if (TMA) {
        if (!stage_ok && lane == 0) atomicAdd(&g_stage_timeouts, 1u);
        // a wait on a staged tile ran out in some warp: the whole partition is dropped (it merges as an empty
        // partition: weight 0) rather than merged half done; the count above tells the host
        gave_up = __syncthreads_or(stage_ok ? 0 : 1) != 0;
    } else {
        cp_async_wait<0>();
        __syncthreads();    // all rings idle: the memory is reused for the merge
    }
    if (gave_up) {
#pragma unroll
        for (int e = 0; e < kE; ++e) { m_run[e] = kNegBig; l_run[e] = 0.0f; }
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int i = 0; i < 4; ++i) o[b][m][i] = 0.0f;
    }

    // ---- merge the four warps (scores are in log2 units; partials are stored in natural units) ----
#pragma unroll
    for (int e = 0; e < kE; ++e) {
        float l = l_run[e];   // sum over the lane groups n (each holds two tokens per step)
        l += __shfl_xor_sync(0xffffffffu, l, 4);
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        if (n == 0) {
            const int h = NSPLIT ? j : 2 * j + e;
            s_m[warp][h] = m_run[e];
            s_l[warp][h] = l;
        }
    }
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            const int d0 = 32 * b + 4 * n + 2 * m;   // rows n / n+8 of the MMA hold dims d0 / d0+1
            s_o[warp][2 * j][d0] = o[b][m][0];
            s_o[warp][2 * j + 1][d0] = o[b][m][1];
            s_o[warp][2 * j][d0 + 1] = o[b][m][2];
            s_o[warp][2 * j + 1][d0 + 1] = o[b][m][3];
        }
    __syncthreads();
    // everything below writes memory that the previous launch on the stream may still use (scratch, tickets, outputs):
    // wait for it to complete (returns at once unless this launch was allowed to start early)
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    {
        const int d = tid;
        for (int hh = 0; hh < g; ++hh) {
            float M = kNegBig;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w][hh]);
            float L = 0.0f, O = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float e = ex2(s_m[w][hh] - M);
                L = fmaf(s_l[w][hh], e, L);
                const float ov = NSPLIT ? s_o[w][2 * hh][d] + s_o[w][2 * hh + 1][d] : s_o[w][hh][d];
                O = fmaf(ov, e, O);
            }
            const size_t pi = (size_t)(kvh * g + hh) * a.num_partitions + part;
            a.partial_out[pi * kD + d] = O * a.v_const;
            if (d == 0) {
                a.partial_max[pi] = (M <= kNegBig) ? -FLT_MAX : M * 0.6931471805599453f;
                a.partial_sum[pi] = L;
            }
        }
    }
    if (a.counters != nullptr) {
        // Last-arriver merge: every CTA publishes its partial (fence), then takes a ticket; the CTA that draws the last
        // ticket sees all partials it merges.  Up to 2 kMergeGroup partitions: one level, the last CTA of the KV head
        // merges them.  More: the last CTA of each group of kMergeGroup partitions merges its group into one more
        // partial, then takes a ticket of the KV head, and the last of those merges the group results.
        __shared__ int s_last;
        const int P = a.num_partitions;
        const int ngroups = merge_groups(P);
        MergeArgs m;
        m.partial_out = a.partial_out; m.partial_max = a.partial_max; m.partial_sum = a.partial_sum;
        m.dev_signs = nullptr; m.out = a.out; m.lse_out = a.lse_out;
        m.head_dim = kD; m.nblk = kD / 32; m.num_partitions = P; m.rotate = 1;
        m.out_dtype = a.out_dtype; m.sign_mag = a.sign_mag;
        m.num_copies = a.peer.world; m.num_q_heads = a.hq;
#pragma unroll
        for (int c = 0; c < kMaxPeers; ++c) m.copy_rec[c] = a.peer.rec[c];
        m.group_out = a.group_out; m.group_max = a.group_max; m.group_sum = a.group_sum;
        float* s_work = reinterpret_cast<float*>(s_raw);   // the ring memory is idle by now
        bool merged = false;
        __threadfence();
        __syncthreads();
        if (ngroups == 0) {
            if (tid == 0) s_last = atomicAdd(a.counters + kvh, 1u) == (unsigned)(P - 1) ? 1 : 0;
            __syncthreads();
            if (s_last) {
                __threadfence();
                merge_group128<false>(m, kvh * g, g, tid, s_work, 0, P, P);
                if (tid == 0) a.counters[kvh] = 0u;   // ready for the next launch
                merged = true;
            }
        } else {
            const int grp = part / kMergeGroup;
            const int gsize = min(kMergeGroup, P - grp * kMergeGroup);
            unsigned* c1 = a.counters + a.hq + kvh * ngroups + grp;
            if (tid == 0) s_last = atomicAdd(c1, 1u) == (unsigned)(gsize - 1) ? 1 : 0;
            __syncthreads();
            if (s_last) {
                __threadfence();
                merge_group128<true>(m, kvh * g, g, tid, s_work, grp * kMergeGroup, gsize, P, grp, ngroups);
                if (tid == 0) *c1 = 0u;
                __threadfence();
                __syncthreads();
                if (tid == 0) s_last = atomicAdd(a.counters + kvh, 1u) == (unsigned)(ngroups - 1) ? 1 : 0;
                __syncthreads();
                if (s_last) {
                    __threadfence();
                    m.partial_out = a.group_out; m.partial_max = a.group_max; m.partial_sum = a.group_sum;
                    merge_group128<false>(m, kvh * g, g, tid, s_work, 0, ngroups, ngroups);
                    if (tid == 0) a.counters[kvh] = 0u;
                    merged = true;
                }
            }
        }
        if (merged && a.peer.world > 0) {
            // the records are in the peers' memory: make them visible system-wide, then release this KV head's flag
            // on every rank (plain stores over NVLink; nobody is waited for here)
            __threadfence_system();
            __syncthreads();
            // Lane c of the first warp releases rank c's flag: ONE system-scope fence for the warp, then eight stores
            // that travel side by side.  (A release-store per rank, one after the other, paid a fence - a round trip
            // over NVLink - per rank: 26 us at eight ranks.)  The pointer is picked by selects: a run-time index
            // into the argument block would move it to local memory.
            if (tid < kMaxPeers) {
                unsigned* f = nullptr;
#pragma unroll
                for (int c = 0; c < kMaxPeers; ++c)
                    if (tid == c && c < a.peer.world) f = a.peer.flag[c];
                __threadfence_system();
                if (f != nullptr) st_relaxed_sys(f + kvh, a.peer.seq);
            }
        }
    }
}

// kappa in [1, 2) such that every centroid / kappa is as close as possible to an f16 value.
float best_kappa(const float* c, int n) {
    float best = 1.0f;
    double best_err = 1e9;
    for (int i = 0; i < (1 << 18); ++i) {
        const float kappa = 1.0f + (float)i / (float)(1 << 18);
        double err = 0.0;
        for (int k = 0; k < n; ++k) {
            if (c[k] == 0.0f) continue;
            const float v = c[k] / kappa;
            const float r = __half2float(__float2half_rn(v));
            err = fmax(err, fabs((double)r * kappa - c[k]) / fabs((double)c[k]));
        }
        if (err < best_err) { best_err = err; best = kappa; }
    }
    return best;
}

struct LutCache {
    bool valid = false;
    float kappa = 1.0f;
    float lut[8];
};
std::mutex g_lut_mutex;
LutCache g_lut_cache[2][2];   // [norm_mode][all_outlier]

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
PFN_cuTensorMapEncodeTiled tensor_map_encoder() {
    static PFN_cuTensorMapEncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
    }();
    return fn;
}

// Tensor maps over the packed cache of one launch.  Index arrays: 2-D [row bytes, token rows of all KV
// heads], box = one 64-token tile, 64-byte swizzle for 64-byte rows.  Scale arrays: 1-D, one 8-byte
// element per token row.  False when the layout does not meet the copy engine's alignment rules: a copy
// starts at token row kvh * kv_stride + 64 k, which must be a multiple of 16 bytes in the scale array.
template <int BITS>
bool make_tma_maps(const MmaArgs& a, TmaMaps& m) {
    using G = Geo<BITS>;
    PFN_cuTensorMapEncodeTiled enc = tensor_map_encoder();
    if (!enc) return false;
    const unsigned long long rows = (unsigned long long)a.hkv * (unsigned long long)a.kv_stride;
    if ((a.kv_stride & 1) || rows >= (1ull << 31)) return false;
    if (((uintptr_t)a.kb % 16) || ((uintptr_t)a.vb % 16) || ((uintptr_t)a.ks % 16) || ((uintptr_t)a.vs % 16)) return false;
    const cuuint64_t idx_dim[2] = {(cuuint64_t)G::kRowB, rows};
    const cuuint64_t idx_stride[1] = {(cuuint64_t)G::kRowB};
    const cuuint32_t idx_box[2] = {(cuuint32_t)G::kRowB, (cuuint32_t)(kWarps * kGroup)};
    const cuuint32_t ones[2] = {1, 1};
    const CUtensorMapSwizzle sw = BITS == 4 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE;
    const cuuint64_t sc_dim[1] = {rows};
    const cuuint32_t sc_box[1] = {(cuuint32_t)(kWarps * kGroup)};
    bool ok = true;
    ok = ok && enc(&m.k, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(a.kb), idx_dim, idx_stride, idx_box, ones,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    ok = ok && enc(&m.v, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(a.vb), idx_dim, idx_stride, idx_box, ones,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    ok = ok && enc(&m.ks, CU_TENSOR_MAP_DATA_TYPE_UINT64, 1, const_cast<uint16_t*>(a.ks), sc_dim, idx_stride, sc_box, ones,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    ok = ok && enc(&m.vs, CU_TENSOR_MAP_DATA_TYPE_UINT64, 1, const_cast<uint16_t*>(a.vs), sc_dim, idx_stride, sc_box, ones,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    return ok;
}

template <typename QT, int BITS, bool NSPLIT, bool TMA, bool QJL>
int launch_one(const MmaArgs& a, const TmaMaps& maps, const Codebook& app_cb, dim3 grid, cudaStream_t s) {
    using G = Geo<BITS>;
    // dynamic shared memory: the stage rings (1 KB alignment slack), for 3-bit after the 8 KB table and its slack
    const size_t dyn = BITS == 3 ? 16384 + kWarps * G::kRingB : 1024 + kWarps * G::kRingB;
    // the opt-in to more than 48 KB of dynamic shared memory is a per-device property of the kernel: set it once
    // per device and instantiation, not on every launch
    static std::atomic<unsigned long long> configured{0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
    if (dev < 0 || !((configured.load(std::memory_order_acquire) >> dev) & 1ull)) {
        cudaError_t e = cudaFuncSetAttribute(decode_mma_kernel<QT, BITS, NSPLIT, TMA, QJL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
        if (e != cudaSuccess) { set_cuda_error(e); return TQB_ERR_CUDA; }
        if (dev >= 0) configured.fetch_or(1ull << dev, std::memory_order_release);
    }
    if (a.overlap) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = dyn;
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, decode_mma_kernel<QT, BITS, NSPLIT, TMA, QJL>, a, maps, app_cb);
        if (e != cudaSuccess) { set_cuda_error(e); return TQB_ERR_CUDA; }
        return check_launch(s);
    }
    decode_mma_kernel<QT, BITS, NSPLIT, TMA, QJL><<<grid, kThreads, dyn, s>>>(a, maps, app_cb);
    return check_launch(s);
}

template <int BITS>
int launch(const MmaArgs& a, int g, int q_dtype, bool allow_tma, const Codebook& app_cb, dim3 grid, cudaStream_t s) {
    TmaMaps maps;
    memset(&maps, 0, sizeof(maps));
    const bool qjl = a.qjl_signs != nullptr;
    const bool tma = allow_tma && !qjl && make_tma_maps<BITS>(a, maps);
#define TQB_LAUNCH_MMA(QT)                                                                               \
    do {                                                                                                 \
        if constexpr (BITS == 3) {                                                                       \
            if (qjl) return g <= 4 ? launch_one<QT, BITS, true, false, true>(a, maps, app_cb, grid, s)   \
                                   : launch_one<QT, BITS, false, false, true>(a, maps, app_cb, grid, s); \
        }                                                                                                \
        if (g <= 4) return tma ? launch_one<QT, BITS, true, true, false>(a, maps, app_cb, grid, s)       \
                               : launch_one<QT, BITS, true, false, false>(a, maps, app_cb, grid, s);     \
        return tma ? launch_one<QT, BITS, false, true, false>(a, maps, app_cb, grid, s)                  \
                   : launch_one<QT, BITS, false, false, false>(a, maps, app_cb, grid, s);                \
    } while (0)
    if (q_dtype == TQB_F32) TQB_LAUNCH_MMA(float);
    else if (q_dtype == TQB_F16) TQB_LAUNCH_MMA(__half);
    else TQB_LAUNCH_MMA(__nv_bfloat16);
#undef TQB_LAUNCH_MMA
}

}  // namespace

// Returns TQB_ERR_UNSUPPORTED when the shape is outside what the tensor-core kernels cover;
// the caller then uses the general kernel.
// `counters` != nullptr fuses the merge into the kernel: [num_kv_heads] tickets, zeroed here unless the
// caller vouches for them (counters_clean).
int launch_decode_mma(const tqb_decode_params* p, int num_partitions, float* partial_out, float* partial_max,
                      float* partial_sum, float sign_mag, unsigned* counters, bool counters_clean, cudaStream_t s,
                      const int* gate, int gate_want, const float* dev_signs, int alias_heads, const PeerPush* peer,
                      float* group_area) {
    const int g = p->num_q_heads / p->num_kv_heads;
    const int nblk = p->head_dim / kBlock;
    const bool all_outlier = p->outlier_blocks < 0 || p->outlier_blocks >= nblk;
    const bool all_normal = p->outlier_blocks == 0;
    if (p->head_dim != kD || g > 8 || p->kv_len <= 0) return TQB_ERR_UNSUPPORTED;
    const bool pqo4 = p->bits == 4 && p->norm_mode == TQB_MAXNORM && all_outlier;
    const bool lut3 = p->bits == 3 && (all_outlier || all_normal);
    if (!pqo4 && !lut3) return TQB_ERR_UNSUPPORTED;
    if (p->qjl_enabled && !lut3) return TQB_ERR_UNSUPPORTED;   // the in-kernel QJL correction exists for the 3-bit kernels
    if (((uintptr_t)p->k_scales % 8) || ((uintptr_t)p->v_scales % 8)) return TQB_ERR_UNSUPPORTED;
    if (((uintptr_t)p->k_indices % 16) || ((uintptr_t)p->v_indices % 16)) return TQB_ERR_UNSUPPORTED;
    MmaArgs a{};
    a.q = p->q;
    a.kb = p->k_indices;
    a.ks = p->k_scales;
    a.vb = p->v_indices;
    a.vs = p->v_scales;
    a.partial_out = partial_out;
    a.partial_max = partial_max;
    a.partial_sum = partial_sum;
    a.hq = p->num_q_heads; a.hkv = p->num_kv_heads; a.g = g;
    a.kv_len = p->kv_len; a.kv_stride = p->kv_stride; a.num_partitions = num_partitions;
    const int step = kWarps * kGroup;
    a.part_size = ((p->kv_len + num_partitions - 1) / num_partitions + step - 1) / step * step;
    a.sign_mag = sign_mag;
    // fused append: the one-thread-per-block quantizer covers the all-outlier MaxNorm format
    Codebook app_cb{};
    if (p->append_k != nullptr) {
        if (!(p->norm_mode == TQB_MAXNORM && all_outlier) || !block_codebook(p->bits, p->norm_mode, app_cb)) return TQB_ERR_UNSUPPORTED;
        if (((uintptr_t)p->append_k % 16) || ((uintptr_t)p->append_v % 16)) return TQB_ERR_UNSUPPORTED;
        a.app_k = p->append_k;
        a.app_v = p->append_v;
        a.outer_centroid = app_cb.c[app_cb.n - 1];   // precomputed/mod.rs:78
    }
    a.gate = gate;
    a.gate_want = gate_want;
    a.dev_signs = dev_signs;
    if (p->qjl_enabled) {
        if (((uintptr_t)p->qjl_signs % 4) || ((uintptr_t)p->rq % 4)) return TQB_ERR_UNSUPPORTED;
        a.qjl_signs = reinterpret_cast<const uint32_t*>(p->qjl_signs);
        a.qjl_norms = p->qjl_norms;
        a.rq = p->rq;
        a.qjl_const = (1.2533141f * (1.0f / sqrtf((float)kD))) * p->softmax_scale * 1.4426950408889634f;   // tq_attention_kernel.cu:225
    }
    a.alias_heads = alias_heads;
    a.kv_len0 = alias_heads > 0 ? p->kv_len - p->num_kv_heads / alias_heads + 1 : p->kv_len;
    if (alias_heads > 0 && p->append_k != nullptr) return TQB_ERR_UNSUPPORTED;
    if (peer != nullptr && peer->world > 0) {
        if (counters == nullptr || peer->world > kMaxPeers || p->num_kv_heads > kPeerFlagHeads) return TQB_ERR_UNSUPPORTED;
        a.peer = *peer;
    }
    // early start only for the plain fused launch: no gate written by a check kernel, no memset between the launches
    a.overlap = ((p->flags & TQB_DECODE_OVERLAP) != 0 && gate == nullptr && counters != nullptr && counters_clean) ? 1 : 0;
    a.counters = counters;
    a.out = p->out;
    a.lse_out = p->lse_out;
    a.out_dtype = p->out_dtype;
    const int ngroups = merge_groups(num_partitions);
    if (counters != nullptr && ngroups > 0) {
        if (group_area == nullptr) return TQB_ERR_INVALID_ARGUMENT;
        a.group_out = group_area;
        a.group_max = group_area + (size_t)p->num_q_heads * ngroups * kD;
        a.group_sum = a.group_max + (size_t)p->num_q_heads * ngroups;
    }
    if (counters != nullptr && !counters_clean) {
        cudaError_t e = cudaMemsetAsync(counters, 0, sizeof(unsigned) * (size_t)p->num_q_heads * (1 + ngroups), s);
        if (e != cudaSuccess) { set_cuda_error(e); return TQB_ERR_CUDA; }
    }
    dim3 grid(p->num_kv_heads, num_partitions);
    const bool allow_tma = (p->flags & TQB_DECODE_TMA) != 0 && alias_heads == 0;   // the tensor maps assume one row range per grid head
    const float log2e = 1.4426950408889634f;
    if (pqo4) {
        const float R = 2.1573f;
        const float grid_step = (2.0f * R) / 15.0f;   // codebooks.rs:64-67
        a.qk_const = p->softmax_scale * log2e * grid_step;
        a.v_const = grid_step;
        return launch<4>(a, g, p->q_dtype, allow_tma, app_cb, grid, s);
    }
    {
        std::lock_guard<std::mutex> lock(g_lut_mutex);
        LutCache& lc = g_lut_cache[p->norm_mode == TQB_L2NORM ? 1 : 0][all_outlier ? 1 : 0];
        if (!lc.valid) {
            Codebook cb;
            if (!block_codebook(all_outlier ? 3 : 2, p->norm_mode, cb)) return TQB_ERR_UNSUPPORTED;
            float c[8];
            for (int i = 0; i < 8; ++i) c[i] = cb.c[i < cb.n ? i : cb.n - 1];   // codes past a 4-entry book clamp (quantize_tensor.rs:245)
            lc.kappa = best_kappa(c, 8);
            for (int i = 0; i < 8; ++i) lc.lut[i] = c[i] / lc.kappa;
            lc.valid = true;
        }
        a.qk_const = p->softmax_scale * log2e * lc.kappa;
        a.v_const = lc.kappa;
        for (int i = 0; i < 8; ++i) a.lut[i] = lc.lut[i];
    }
    return launch<3>(a, g, p->q_dtype, allow_tma, app_cb, grid, s);
}

}  // namespace tqb

extern "C" long long tqb_decode_stage_timeouts(void) {
    unsigned v = 0;
    if (cudaMemcpyFromSymbol(&v, tqb::g_stage_timeouts, sizeof(v)) != cudaSuccess) return -1;
    return (long long)v;
}
