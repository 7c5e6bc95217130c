// Causal attention of a prefill chunk over the packed block-32 cache on the 5th-generation tensor cores
// (tcgen05.mma, operands in shared memory, accumulators in tensor memory).  No counterpart kernel in the reference:
// its prefill dequantizes the whole cache and hands it to the engine (src/cache/pqo.rs:184-200, src/cache/common.rs:16-62).
//
// One CTA owns 128 query rows - 128 / g consecutive query tokens times the g query heads of one KV head - and walks the
// cache in tiles of 64 tokens.  Each K / V tile is unpacked ONCE per CTA (the decode kernels, run once per query token,
// unpack it once per token) and feeds M = 128 MMAs:
//   S  = Q~ K~^T         K~ = |s_k| (c - 7.5) (4-bit grid; |s_k| centroid / kappa for 3-bit) and the rotated, pre-scaled
//                        query, each rounded once to f16.  The scores are taken 128 tokens (two tiles) at a time: eight
//                        MMAs (16 dims each, N = 128) into a 128 x 128 f32 accumulator in tensor memory,
//                        double-buffered, so the tensor cores score step j + 1 while the softmax threads work on step j.
//   O_G += P V           P = exp2(s - m) as f16, handed to the tensor cores through TENSOR MEMORY: a softmax thread
//                        overwrites the first 32 of the 64 score columns it has just read with its row of P (two f16
//                        per column) and the MMA takes its A operand from there (no shared-memory round trip); V
//                        dequantized with its scale to f16 (MN-major B operand in shared memory), N = 128 dims, one
//                        128 x 128 f32 accumulator per softmax group G.
// Two softmax groups of four warps each: group G takes tile 2 j + G of every step (columns 64 G .. 64 G + 63 of the
// step's scores) with its own running (max, sum), P buffer and O accumulator - two independent online softmaxes over
// the even and the odd tiles, merged once at the end like two split-K partitions.  Thread r of a group owns query
// row r = tensor-memory lane r, so the online softmax needs no shuffles; the output is rotated back in registers
// (one 32-point butterfly per block) at the end.
// The f16 roundings of Q~, K~, P and V are this kernel's error budget (a few 1e-4 of the value range on the outputs;
// the decode kernels, which keep the query in f32 or as 20-bit integers, stay below 1e-5).
//
// Warp roles: warps 0-3 / 4-7 softmax group 0 / 1 (correction, epilogue), warps 8-9 load and unpack K tiles, warps
// 10-13 V tiles (two stages each), warp 14 issues the MMAs.  All hand-offs go through mbarriers; every wait is
// bounded and a wait that runs out sets a flag, drains and returns (tqb_chunk_umma_timeouts).
#include <cuda.h>
#include <float.h>

#include <atomic>

#include "tqb_common.cuh"

namespace tqb {
namespace {

constexpr int kRows = 128;          // query rows per CTA
constexpr int kTile = 64;           // cache tokens per step
constexpr int kD = 128;
constexpr int kThreads = 15 * 32;
// P = exp2(s - m) goes to the tensor cores through tensor memory: a softmax thread overwrites the first 32 columns of
// the 64 score columns it has just read with its row of P (two f16 per column), and the P V product takes its A operand
// from there.  (false: through shared memory, as a K-major swizzled tile.)
constexpr bool kPTmem = true;
constexpr float kNegBig = -1.0e30f;

// shared-memory map (bytes from a 1024-aligned base)
constexpr int kOffQ = 0;                         // [2 atoms][128 rows][128 B]
constexpr int kOffK = 32768;                     // [2 stages][2 atoms][128 tokens = two tiles][128 B]
constexpr int kOffV = kOffK + 2 * 32768;         // [2 stages][2 dim halves][8 token groups][8 tokens][128 B]
constexpr int kOffP = kOffV + 2 * 16384;         // [2 buffers][128 rows][128 B]
constexpr int kOffLut = kOffP + 2 * 16384;       // 3-bit: 64 half2
constexpr int kOffBar = kOffLut + 256;           // mbarriers
constexpr int kOffMl = kOffBar + 128;            // (max, sum) of every row of both softmax groups, for the final merge
constexpr int kSmemBytes = kOffMl + 2048 + 1024; // + alignment slack
constexpr uint32_t kTmemCols = 512;              // S buffers (128 columns: two tiles) at 0 and 128; O of group 0 at 256, of group 1 at 384

struct ChunkArgs {
    const void* q;        // [q_len, hq, 128]
    void* out;            // [q_len, hq, 128]
    float* lse_out;       // nullptr or [q_len, hq, 2]
    const uint8_t* kb;
    const uint16_t* ks;
    const uint8_t* vb;
    const uint16_t* vs;
    int hq, hkv, g, q_len, kv_len, kv_stride, out_dtype;
    float qk_const, v_const, sign_mag;
    float lut[8];
    unsigned* timeouts;
};

__device__ unsigned g_chunk_timeouts = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
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
// Bounded wait: false when the phase has not completed within about a quarter of a second (2^29 clock cycles).
// The first wait that runs out leaves a note of who waited for what: (role << 24) | (barrier << 16) | tile.
__device__ unsigned g_chunk_first_timeout = 0;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned note = 0) {
    // try_wait suspends the thread in hardware for a short while when the phase is not complete, so this loop does
    // not spin hot; the clock (a special-register read) is looked at only every 256th poll.
    long long t0 = 0;
    for (unsigned n = 1;; ++n) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((n & 255u) == 0u) {
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > (1ll << 29)) {
                atomicCAS(&g_chunk_first_timeout, 0u, note | 0x80000000u);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// Shared-memory matrix descriptor (tcgen05): start address, leading / stride byte offsets (all >> 4), version 1,
// 128-byte swizzle.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;      // descriptor version of this architecture
    d |= (uint64_t)2 << 61;      // SWIZZLE_128B
    return d;
}
// Instruction descriptor, kind::f16: f32 accumulate, f16 A and B, A K-major, M = 128.
__host__ __device__ constexpr uint32_t umma_idesc(int n, bool b_mn_major) {
    return (1u << 4) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// The same with the A operand in tensor memory: lane = row, one 32-bit column holds two consecutive K elements, so a
// K = 16 step reads 8 columns starting at a_tmem.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Eight 4-bit codes of a word -> four half2 of exact values code - 7.5, in the order (c0, c4), (c1, c5), (c2, c6), (c3, c7).
__device__ __forceinline__ void nibbles_to_half2(uint32_t w, uint32_t (&x)[4]) {
    const uint32_t kMagic = 0x64006400u;
    const __half2 kHalf = u32_as_h2(0x38003800u), kM519 = u32_as_h2(0xE00FE00Fu);
    const __half2 k32nd = u32_as_h2(0x28002800u), kM39 = u32_as_h2(0xD0F0D0F0u);
    const uint32_t w1 = w << 1, w7 = w >> 7;
    x[0] = h2_as_u32(__hfma2(u32_as_h2(lop3_and_or(w1, 0x001e001eu, kMagic)), kHalf, kM519));
    x[1] = h2_as_u32(__hfma2(u32_as_h2(lop3_and_or(w1, 0x01e001e0u, kMagic)), k32nd, kM39));
    x[2] = h2_as_u32(__hfma2(u32_as_h2(lop3_and_or(w7, 0x001e001eu, kMagic)), kHalf, kM519));
    x[3] = h2_as_u32(__hfma2(u32_as_h2(lop3_and_or(w7, 0x01e001e0u, kMagic)), k32nd, kM39));
}
// Position p (0..7) inside a group of eight unpacked 4-bit codes holds code kPerm4[p] of the word.
__device__ __forceinline__ int perm4(int p) { return (p >> 1) + 4 * (p & 1); }

__device__ __forceinline__ float wht32_lane(float v, int lane) {
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
        float other = __shfl_xor_sync(0xffffffffu, v, h);
        v = (lane & h) ? (other - v) : (v + other);
    }
    return v;
}

// 16 consecutive bytes of a swizzled 128-byte row: chunk c of row `row` of a tile whose rows are 128 bytes apart
__device__ __forceinline__ uint32_t sw128(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// ---- load + unpack role: IS_K ? warps 8-9 (K tiles, four pieces per thread) : warps 10-13 (V tiles, two pieces) ----
// A piece is one (token, block): 32 codes and their scale.  Eight consecutive lanes take the eight tokens of one token
// group (eight distinct swizzle phases, so the 16-byte stores of a quarter-warp fall into eight different bank
// groups), the four lane octets take the four blocks.  The packed pieces are fetched two tiles ahead of their use
// (two register sets), so that the trip to L2 / HBM is never waited for.
// K tiles 2 j and 2 j + 1 fill the two halves of K stage j % 2 (the scores are taken 128 tokens at a time); V tile i
// goes to V stage i % 2.
template <int BITS, bool IS_K>
__device__ __forceinline__ bool unpack_role(const ChunkArgs& a, unsigned char* sm, uint32_t bar_full, uint32_t bar_empty, int w2, int lane,
                                            size_t row0, int kv_hi, int ntiles) {
    constexpr int NP = IS_K ? 4 : 2;             // pieces per thread and tile
    constexpr int TSTEP = kTile / NP;            // token distance between a thread's pieces
    const int tl = 8 * w2 + (lane & 7), b = lane >> 3;
    const uint8_t* src_b = IS_K ? a.kb : a.vb;
    const uint16_t* src_s = IS_K ? a.ks : a.vs;
    uint4 pq[2][NP];
    uint32_t sr[2][NP];
    auto fetch = [&](int i, uint4 (&pqs)[NP], uint32_t (&srs)[NP]) {
#pragma unroll
        for (int h = 0; h < NP; ++h) {
            const size_t row = row0 + (size_t)min(i * kTile + tl + TSTEP * h, kv_hi - 1);
            if (BITS == 4) {
                pqs[h] = __ldg(reinterpret_cast<const uint4*>(src_b + row * 64) + b);
            } else {
                const uint32_t* pp = reinterpret_cast<const uint32_t*>(src_b + row * 48) + 3 * b;
                pqs[h] = make_uint4(__ldg(pp), __ldg(pp + 1), __ldg(pp + 2), 0u);
            }
            srs[h] = (uint32_t)__ldg(src_s + row * 4 + b);
        }
    };
    if (ntiles > 0) fetch(0, pq[0], sr[0]);
    if (ntiles > 1) fetch(1, pq[1], sr[1]);
    auto unpack_tile = [&](int i, uint4 (&pqc)[NP], uint32_t (&src)[NP]) -> bool {
        const int use = IS_K ? (i >> 1) : i;      // the use-th filling of the stage ring (two stages)
        const int st = use & 1;
        if (use >= 2 && !mbar_wait(bar_empty + 8 * st, ((use >> 1) - 1) & 1, (1u << 24) | ((IS_K ? 2u : 3u) << 16) | (unsigned)i)) return false;
        unsigned char* dst = sm + (IS_K ? kOffK + st * 32768 : kOffV + st * 16384);
#pragma unroll
        for (int h = 0; h < NP; ++h) {
            const int t = tl + TSTEP * h;
            const uint32_t w[4] = {pqc[h].x, pqc[h].y, pqc[h].z, pqc[h].w};
            const __half2 sc2 = __half2half2(__habs(__ushort_as_half((unsigned short)src[h])));
            // K: atom b / 2 (16 KB apart), row 64 (i % 2) + t, chunks 4 (b % 2) + j;
            // V: dim half b / 2 (8 KB apart), token group t / 8, row t % 8, same chunks
            const uint32_t off = IS_K ? (uint32_t)(b >> 1) * 16384u + (uint32_t)(i & 1) * 8192u
                                      : (uint32_t)(b >> 1) * 8192u + (uint32_t)(t >> 3) * 1024u;
            const int row = IS_K ? t : (t & 7);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t x[4];
                if (BITS == 4) {
                    nibbles_to_half2(w[j], x);
                } else {
                    // codes 8j .. 8j+7 of the block: bits 24j .. 24j+23 of the 96-bit stream, natural order
                    const int bit = 24 * j, wi = bit >> 5, sh = bit & 31;
                    const uint32_t cc = __funnelshift_r(w[wi], w[min(wi + 1, 2)], sh);
                    const uint32_t* lut = reinterpret_cast<const uint32_t*>(sm + kOffLut);
#pragma unroll
                    for (int e = 0; e < 4; ++e) x[e] = lut[(cc >> (6 * e)) & 63u];
                }
                // value = |scale| * code value, one rounding to f16
#pragma unroll
                for (int e = 0; e < 4; ++e) x[e] = h2_as_u32(__hmul2(u32_as_h2(x[e]), sc2));
                *reinterpret_cast<uint4*>(dst + off + sw128(row, 4 * (b & 1) + j)) = make_uint4(x[0], x[1], x[2], x[3]);
            }
        }
        if (i + 2 < ntiles) fetch(i + 2, pqc, src);
        fence_async_smem();
        mbar_arrive(bar_full + 8 * st);
        return true;
    };
    bool ok = true;
    for (int i = 0; i < ntiles && ok; i += 2) {     // ntiles is even
        ok = unpack_tile(i, pq[0], sr[0]);
        if (ok) ok = unpack_tile(i + 1, pq[1], sr[1]);
    }
    return ok;
}

template <typename QT, int BITS>
__global__ void __launch_bounds__(kThreads, 1) chunk_umma_kernel(ChunkArgs a) {
    extern __shared__ unsigned char s_dyn[];
    const uint32_t base = (smem_u32(s_dyn) + 1023u) & ~1023u;
    unsigned char* sm = s_dyn + (base - smem_u32(s_dyn));
    __shared__ uint32_t s_tmem;
    __shared__ int s_fail;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = a.g, TQ = kRows / g;
    const int mt = blockIdx.x, kvh = blockIdx.y;
    const int tok0 = mt * TQ;                                   // first query token of the tile
    const int ntok = min(TQ, a.q_len - tok0);                   // valid query tokens in the tile
    const int past = a.kv_len - a.q_len;                        // tokens before the chunk
    const int kv_hi = past + tok0 + ntok;                       // cache tokens visible to the tile's last query token
    const int npairs = (kv_hi + 2 * kTile - 1) / (2 * kTile);   // steps of two tiles (128 tokens); a tile past the end is
    const int ntiles = 2 * npairs;                              // unpacked from clamped rows and fully masked
    const size_t row0 = (size_t)kvh * a.kv_stride;

    // barriers (8 bytes each, indexed by stage / buffer / softmax group): K and V tiles are handed over separately, so
    // that the scores of a later step never wait for the P V product of an earlier one
    const uint32_t bar = base + kOffBar;
    constexpr uint32_t kKFull = 0, kKEmpty = 16, kVFull = 32, kVEmpty = 48, kSFull = 64, kPFull = 80, kOFull = 96;
    if (tid == 0) {
        s_fail = 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar + kKFull + 8 * i, 128);    // 64 threads, two tiles per stage
            mbar_init(bar + kKEmpty + 8 * i, 1);
            mbar_init(bar + kSFull + 8 * i, 1);
            mbar_init(bar + kVFull + 8 * i, 128);
            mbar_init(bar + kVEmpty + 8 * i, 1);
            mbar_init(bar + kPFull + 8 * i, 128);
        }
        mbar_init(bar + kOFull, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (BITS == 3) {
        for (int e = tid; e < 64; e += kThreads)
            reinterpret_cast<__half2*>(sm + kOffLut)[e] = __floats2half2_rn(a.lut[e & 7], a.lut[e >> 3]);
    }
    // ---- rotated queries -> Q tile (K-major, 128-byte swizzle, two atoms of 64 dims), rounded to f16 ----
    {
        const uint32_t neg = 0xB1A6D4B2u;   // src/cache/precomputed/rotation.rs:16-20
        const float sign = ((neg >> lane) & 1u) ? -a.sign_mag : a.sign_mag;
        const float inv_sqrt = 1.0f / sqrtf(32.0f);
        for (int u = warp; u < kRows * 4; u += kThreads / 32) {
            const int r = u >> 2, b = u & 3;
            const int tq = r / g, hh = r - tq * g;
            float v = 0.0f;
            if (tq < ntok)
                v = to_f32<QT>(reinterpret_cast<const QT*>(a.q)[((size_t)(tok0 + tq) * a.hq + kvh * g + hh) * kD + b * 32 + lane]);
            v = wht32_lane(v, lane);
            v = ((v * inv_sqrt) * sign) * a.qk_const;
            // position of dim (b, lane) inside the K tile's element order
            int pos = lane;
            if (BITS == 4) {   // word j = lane / 8 holds codes in the order c0, c4, c1, c5, ...: code k sits at position
                const int k = lane & 7;
                pos = (lane & ~7) | ((k & 3) * 2 + (k >> 2));
            }
            const int d = b * 32 + pos;
            const uint32_t off = (uint32_t)(d >> 6) * 16384u + sw128(r, (d & 63) >> 3) + (uint32_t)(d & 7) * 2u;
            *reinterpret_cast<__half*>(sm + kOffQ + off) = __float2half_rn(v);
        }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t tmemS = tmem, tmemO = tmem + 256;   // S buffer b at columns 128 b; O of softmax group G at 256 + 128 G

    if (warp >= 8 && warp < 10) {
        if (!unpack_role<BITS, true>(a, sm, bar + kKFull, bar + kKEmpty, warp - 8, lane, row0, kv_hi, ntiles)) atomicExch(&s_fail, 1);
    } else if (warp >= 10 && warp < 14) {
        if (!unpack_role<BITS, false>(a, sm, bar + kVFull, bar + kVEmpty, warp - 10, lane, row0, kv_hi, ntiles)) atomicExch(&s_fail, 1);
    } else if (warp == 14) {
        // ================= MMA issue (one lane) =================
        if (lane == 0) {
            constexpr uint32_t idescS = umma_idesc(2 * kTile, false), idescO = umma_idesc(kD, true);
            bool ok = true;
            // Descriptors are built once: inside the loops a descriptor is its base plus a compile-time offset in the
            // address field (bytes >> 4), so that the one issuing thread spends a handful of instructions per MMA.
            const uint64_t dQ = umma_desc(base + kOffQ, 16, 1024), dK = umma_desc(base + kOffK, 16, 1024);
            const uint64_t dP = umma_desc(base + kOffP, 16, 1024), dV = umma_desc(base + kOffV, 8192, 1024);
            // S(j) = Q~ K~^T for the 128 tokens of step j: 8 k-steps of 16 dims (atom = 64 dims = 16 KB, 32 bytes per
            // k-step), N = 128
            auto score = [&](int j) -> bool {
                const int st = j & 1;
                if (!mbar_wait(bar + kKFull + 8 * st, (j >> 1) & 1, (2u << 24) | (0u << 16) | (unsigned)j)) return false;
                tc_fence_after();
                const uint64_t kk0 = dK + (uint64_t)(st * (32768 >> 4));
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint64_t off = (uint64_t)(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
                    umma_f16(tmemS + st * 2 * kTile, dQ + off, kk0 + off, idescS, kk ? 1u : 0u);
                }
                umma_commit(bar + kSFull + 8 * st);
                umma_commit(bar + kKEmpty + 8 * st);   // the K stage is free when these MMAs are done
                return true;
            };
            // The scores run one step (two tiles) ahead of the softmax groups: S(j + 1) is issued before the P V products
            // of step j, into the buffer that both groups finished reading in step j - 1 (their p_full arrivals were
            // waited for one iteration earlier).
            if (npairs > 0) ok = score(0);
            for (int j = 0; j < npairs && ok; ++j) {
                if (j + 1 < npairs && !score(j + 1)) { ok = false; break; }
#pragma unroll
                for (int G = 0; G < 2; ++G) {
                    if (!mbar_wait(bar + kPFull + 8 * G, j & 1, (2u << 24) | (5u << 16) | (unsigned)j)) { ok = false; break; }
                    if (!mbar_wait(bar + kVFull + 8 * G, j & 1, (2u << 24) | (1u << 16) | (unsigned)j)) { ok = false; break; }
                    tc_fence_after();
                    // O_G += P V : four k-steps of 16 tokens
                    const uint64_t pv = dP + (uint64_t)(G * (16384 >> 4)), vv = dV + (uint64_t)(G * (16384 >> 4));
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        if (kPTmem)
                            umma_f16_ts(tmemO + G * kD, tmemS + (j & 1) * 2 * kTile + G * kTile + kk * 8, vv + (uint64_t)((kk * 2048) >> 4),
                                        idescO, (j | kk) ? 1u : 0u);
                        else
                            umma_f16(tmemO + G * kD, pv + (uint64_t)((kk * 32) >> 4), vv + (uint64_t)((kk * 2048) >> 4), idescO, (j | kk) ? 1u : 0u);
                    }
                    umma_commit(bar + kVEmpty + 8 * G);      // frees this V stage and P buffer when the MMAs issued so far are done
                }
            }
            if (ok) umma_commit(bar + kOFull);           // everything issued so far has completed when this arrives
            else atomicExch(&s_fail, 1);
        }
        __syncwarp();
    } else {
        // ================= softmax, correction, epilogue: two groups of four warps, thread = query row =================
        // Group G takes tile 2 j + G of every step j (columns 64 G .. 64 G + 63 of the step's scores), with its own
        // running (max, sum), P buffer and O accumulator: two independent online softmaxes over the even and the odd
        // tiles, merged once at the end like two split-K partitions.
        const int G = warp >> 2;
        const int r = tid & 127;
        const int tq = r / g, hh = r - tq * g;
        const bool row_valid = tq < ntok;
        const int limit = past + tok0 + tq + 1;                 // visible cache tokens of this row
        const int limit_min = past + tok0 + 1;                  // ... of the tile's first row
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tmemOG = tmemO + G * kD;
        float m_run = kNegBig, l_run = 0.0f;
        bool ok = true;
        for (int j = 0; j < npairs && ok; ++j) {
            const int i = 2 * j + G, sb = j & 1;
            // (the tensor-memory accesses below are warp-collective: the whole warp goes on, or none of it)
            if (!__all_sync(0xffffffffu, mbar_wait(bar + kSFull + 8 * sb, (j >> 1) & 1, (3u << 24) | (4u << 16) | (unsigned)j))) { ok = false; break; }
            tc_fence_after();
            float p[kTile];
            {
                uint32_t v0[32], v1[32];
                tmem_ld32(tmemS + lane_base + sb * 2 * kTile + G * kTile, v0);
                tmem_ld32(tmemS + lane_base + sb * 2 * kTile + G * kTile + 32, v1);
                tmem_wait_ld();
                if ((i + 1) * kTile <= limit_min) {
                    // every token of the tile is visible to every row (all tiles but the last few)
#pragma unroll
                    for (int t = 0; t < 32; ++t) {
                        p[t] = __uint_as_float(v0[t]);
                        p[32 + t] = __uint_as_float(v1[t]);
                    }
                } else {
#pragma unroll
                    for (int t = 0; t < 32; ++t) {
                        const int tok = i * kTile + t;
                        p[t] = (row_valid && tok < limit) ? __uint_as_float(v0[t]) : kNegBig;
                        p[32 + t] = (row_valid && tok + 32 < limit) ? __uint_as_float(v1[t]) : kNegBig;
                    }
                }
            }
            // four interleaved partial maxima / sums keep the dependency chains short
            float mx4[4] = {kNegBig, kNegBig, kNegBig, kNegBig};
#pragma unroll
            for (int t = 0; t < kTile; ++t) mx4[t & 3] = fmaxf(mx4[t & 3], p[t]);
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // lazy maximum: raise the reference only when this tile exceeds it by more than 2^6.  A row that has seen no
            // visible token yet keeps the sentinel; the floor below then turns its masked scores into exp2(-huge) = 0.
            const float m_new = (mx - m_run > 6.0f) ? mx : m_run;
            const float resc = ex2(m_run - m_new);
            const float m_use = fmaxf(m_new, -1.0e29f);
            m_run = m_new;
            float ls4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int t = 0; t < kTile; ++t) {
                p[t] = ex2(p[t] - m_use);
                ls4[t & 3] += p[t];
            }
            l_run = l_run * resc + ((ls4[0] + ls4[1]) + (ls4[2] + ls4[3]));
            // The group's P V product of the previous step must be done: it wrote the O accumulator rescaled here (and,
            // with P in shared memory, read the P buffer written below).  The wait is also the flow control of the
            // p_full barrier: without it a group could arrive for steps j and j + 1 before the issuing thread has looked
            // at step j, and a parity wait cannot tell a phase from the one two later (seen as bounded waits running
            // out when it was made conditional on a rescale).
            const bool rescale = j > 0 && __any_sync(0xffffffffu, resc != 1.0f);
            if (j > 0 && !__all_sync(0xffffffffu, mbar_wait(bar + kVEmpty + 8 * G, (j - 1) & 1, (3u << 24) | (3u << 16) | (unsigned)j))) { ok = false; break; }
            if (rescale) {
                // rescale this row of O (warp-collective tensor-memory accesses: every lane takes part with its own factor)
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t v[32];
                    tmem_ld32(tmemOG + lane_base + c * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int t = 0; t < 32; ++t) v[t] = __float_as_uint(__uint_as_float(v[t]) * resc);
                    tmem_st32(tmemOG + lane_base + c * 32, v);
                }
                tmem_wait_st();
            }
            if (kPTmem) {
                // P -> tensor memory: column c of the row holds tokens 2c (low half) and 2c + 1
                uint32_t w[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) w[c] = h2_as_u32(__floats2half2_rn(p[2 * c], p[2 * c + 1]));
                tmem_st32(tmemS + lane_base + sb * 2 * kTile + G * kTile, w);
                tmem_wait_st();
            } else {
                // P -> shared memory (K-major A operand: row r, 64 tokens = 128 bytes, swizzled 16-byte chunks)
                unsigned char* pt = sm + kOffP + G * 16384;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) w[e] = h2_as_u32(__floats2half2_rn(p[8 * c + 2 * e], p[8 * c + 2 * e + 1]));
                    *reinterpret_cast<uint4*>(pt + sw128(r, c)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                fence_async_smem();
            }
            tc_fence_before();
            mbar_arrive(bar + kPFull + 8 * G);
        }
        if (ok && npairs > 0 && !__all_sync(0xffffffffu, mbar_wait(bar + kOFull, 0, (3u << 24) | (6u << 16)))) ok = false;
        if (!ok) atomicExch(&s_fail, 1);
        tc_fence_after();
        // ---- merge of the two groups: exchange (max, sum) through shared memory; all eight warps meet here ----
        float2* ml = reinterpret_cast<float2*>(sm + kOffMl);
        ml[G * kRows + r] = make_float2(m_run, l_run);
        asm volatile("bar.sync 1, 256;\n" ::: "memory");
        if (ok && npairs > 0) {
            const float2 other = ml[(G ^ 1) * kRows + r];
            const float M = fmaxf(m_run, other.x);
            const float w_self = ex2(fmaxf(m_run - M, -200.0f)), w_other = ex2(fmaxf(other.x - M, -200.0f));
            const float w0 = G == 0 ? w_self : w_other, w1 = G == 0 ? w_other : w_self;
            const float l_tot = l_run * w_self + other.y * w_other;
            // ---- epilogue: group G takes blocks 2 G and 2 G + 1 of the row: O = w0 O_0 + w1 O_1, rotate the 32-block
            // back, normalise, store (every lane reads its row: the tensor-memory loads are warp-collective; rows past
            // the chunk's end are just not stored) ----
            const float inv_l = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
            const float inv_sqrt = 1.0f / sqrtf(32.0f);
            const uint32_t neg = 0xB1A6D4B2u;
            const size_t orow = ((size_t)(tok0 + tq) * a.hq + kvh * g + hh) * kD;
#pragma unroll 1
            for (int b = 2 * G; b < 2 * G + 2; ++b) {
                uint32_t va[32], vb[32];
                tmem_ld32(tmemO + lane_base + b * 32, va);
                tmem_ld32(tmemO + kD + lane_base + b * 32, vb);
                tmem_wait_ld();
                float x[32];
#pragma unroll
                for (int pz = 0; pz < 32; ++pz) {
                    const int d = BITS == 4 ? ((pz & ~7) | perm4(pz & 7)) : pz;   // column pz of the block holds dim d
                    const float sgn = ((neg >> d) & 1u) ? -a.sign_mag : a.sign_mag;
                    const float o = __uint_as_float(va[pz]) * w0 + __uint_as_float(vb[pz]) * w1;
                    x[d] = (o * a.v_const) * sgn;
                }
#pragma unroll
                for (int h = 1; h < 32; h <<= 1)
#pragma unroll
                    for (int i0 = 0; i0 < 32; i0 += 2 * h)
#pragma unroll
                        for (int jx = i0; jx < i0 + h; ++jx) {
                            const float xa = x[jx], xb = x[jx + h];
                            x[jx] = xa + xb;
                            x[jx + h] = xa - xb;
                        }
#pragma unroll
                for (int d = 0; d < 32; ++d) {
                    float o = x[d] * inv_sqrt;
                    if (a.lse_out == nullptr) o *= inv_l;
                    const size_t idx = orow + b * 32 + d;
                    if (!row_valid) continue;
                    if (a.out_dtype == TQB_F32) reinterpret_cast<float*>(a.out)[idx] = o;
                    else if (a.out_dtype == TQB_F16) reinterpret_cast<__half*>(a.out)[idx] = __float2half_rn(o);
                    else reinterpret_cast<__nv_bfloat16*>(a.out)[idx] = __float2bfloat16_rn(o);
                }
            }
            if (a.lse_out != nullptr && row_valid && G == 0) {
                float* lse = a.lse_out + ((size_t)(tok0 + tq) * a.hq + kvh * g + hh) * 2;
                lse[0] = M * 0.6931471805599453f;
                lse[1] = l_tot;
            }
        }
    }
    // ---- common exit: every wait above is bounded, so every thread gets here ----
    tc_fence_before();
    __syncthreads();
    if (s_fail && tid == 0) atomicAdd(a.timeouts, 1u);
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

float best_kappa3(const float* c, int n) {
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

template <typename QT, int BITS>
int launch_chunk(const ChunkArgs& a, dim3 grid, cudaStream_t s) {
    static std::atomic<unsigned long long> configured{0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
    if (dev < 0 || !((configured.load(std::memory_order_acquire) >> dev) & 1ull)) {
        cudaError_t e = cudaFuncSetAttribute(chunk_umma_kernel<QT, BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) { set_cuda_error(e); return TQB_ERR_CUDA; }
        if (dev >= 0) configured.fetch_or(1ull << dev, std::memory_order_release);
    }
    chunk_umma_kernel<QT, BITS><<<grid, kThreads, kSmemBytes, s>>>(a);
    return check_launch(s);
}

}  // namespace

// TQB_ERR_UNSUPPORTED when the shape is outside what this kernel covers (the caller then folds the chunk into decode launches).
int launch_chunk_umma(const tqb_decode_params* p, int q_len, cudaStream_t s) {
    const int nblk = p->head_dim / kBlock;
    const int g = p->num_kv_heads > 0 ? p->num_q_heads / p->num_kv_heads : 0;
    const bool all_outlier = p->outlier_blocks < 0 || p->outlier_blocks >= nblk;
    const bool all_normal = p->outlier_blocks == 0;
    if (p->head_dim != kD || p->qjl_enabled || p->kv_len <= 0 || q_len <= 0) return TQB_ERR_UNSUPPORTED;
    if (g != 1 && g != 2 && g != 4 && g != 8) return TQB_ERR_UNSUPPORTED;
    const bool pqo4 = p->bits == 4 && p->norm_mode == TQB_MAXNORM && all_outlier;
    const bool lut3 = p->bits == 3 && (all_outlier || all_normal);
    if (!pqo4 && !lut3) return TQB_ERR_UNSUPPORTED;
    if (((uintptr_t)p->k_indices % 16) || ((uintptr_t)p->v_indices % 16) || ((uintptr_t)p->k_scales % 8) || ((uintptr_t)p->v_scales % 8))
        return TQB_ERR_UNSUPPORTED;
    if (p->lse_out && p->out_dtype != TQB_F32) return TQB_ERR_INVALID_ARGUMENT;
    ChunkArgs a{};
    a.q = p->q; a.out = p->out; a.lse_out = p->lse_out;
    a.kb = p->k_indices; a.ks = p->k_scales; a.vb = p->v_indices; a.vs = p->v_scales;
    a.hq = p->num_q_heads; a.hkv = p->num_kv_heads; a.g = g; a.q_len = q_len; a.kv_len = p->kv_len; a.kv_stride = p->kv_stride;
    a.out_dtype = p->out_dtype;
    volatile float inv = 1.0f / sqrtf(32.0f);
    volatile float sq = sqrtf(32.0f);
    a.sign_mag = inv * sq;   // the reference's sign pattern: (1 / sqrt(32)) * sqrt(32) in f32
    const float log2e = 1.4426950408889634f;
    if (pqo4) {
        const float step = (2.0f * 2.1573f) / 15.0f;   // src/cache/precomputed/codebooks.rs:64-67
        a.qk_const = p->softmax_scale * log2e * step;
        a.v_const = step;
    } else {
        static std::atomic<int> ready[2][2];
        static float kappa_cache[2][2], lut_cache[2][2][8];
        const int m = p->norm_mode == TQB_L2NORM ? 1 : 0, o = all_outlier ? 1 : 0;
        if (ready[m][o].load(std::memory_order_acquire) != 2) {
            int expect = 0;
            if (ready[m][o].compare_exchange_strong(expect, 1)) {
                Codebook cb;
                if (!block_codebook(all_outlier ? 3 : 2, p->norm_mode, cb)) { ready[m][o].store(0); return TQB_ERR_UNSUPPORTED; }
                float c[8];
                for (int i = 0; i < 8; ++i) c[i] = cb.c[i < cb.n ? i : cb.n - 1];   // codes past a 4-entry book clamp (quantize_tensor.rs:245)
                const float kappa = best_kappa3(c, 8);
                kappa_cache[m][o] = kappa;
                for (int i = 0; i < 8; ++i) lut_cache[m][o][i] = c[i] / kappa;
                ready[m][o].store(2, std::memory_order_release);
            } else {
                while (ready[m][o].load(std::memory_order_acquire) == 1) {}
                if (ready[m][o].load(std::memory_order_acquire) != 2) return TQB_ERR_UNSUPPORTED;
            }
        }
        a.qk_const = p->softmax_scale * log2e * kappa_cache[m][o];
        a.v_const = kappa_cache[m][o];
        for (int i = 0; i < 8; ++i) a.lut[i] = lut_cache[m][o][i];
    }
    void* tptr = nullptr;
    if (cudaGetSymbolAddress(&tptr, g_chunk_timeouts) != cudaSuccess) return TQB_ERR_CUDA;
    a.timeouts = static_cast<unsigned*>(tptr);
    const int TQ = kRows / g;
    dim3 grid((q_len + TQ - 1) / TQ, p->num_kv_heads);
#define TQB_LAUNCH_CHUNK(QT) (p->bits == 4 ? launch_chunk<QT, 4>(a, grid, s) : launch_chunk<QT, 3>(a, grid, s))
    if (p->q_dtype == TQB_F32) return TQB_LAUNCH_CHUNK(float);
    if (p->q_dtype == TQB_F16) return TQB_LAUNCH_CHUNK(__half);
    return TQB_LAUNCH_CHUNK(__nv_bfloat16);
#undef TQB_LAUNCH_CHUNK
}

}  // namespace tqb

// Diagnostic: the note left by the first bounded wait that ran out (0: none): bit 31 set, role in bits 24..30
// (1 unpack, 2 MMA issue, 3 softmax), barrier in bits 16..23, tile in the low bits.
extern "C" unsigned tqb_chunk_umma_first_timeout(void) {
    unsigned v = 0;
    if (cudaMemcpyFromSymbol(&v, tqb::g_chunk_first_timeout, sizeof(v)) != cudaSuccess) return 0xFFFFFFFFu;
    return v;
}

extern "C" long long tqb_chunk_umma_timeouts(void) {
    unsigned v = 0;
    if (cudaMemcpyFromSymbol(&v, tqb::g_chunk_timeouts, sizeof(v)) != cudaSuccess) return -1;
    return (long long)v;
}
