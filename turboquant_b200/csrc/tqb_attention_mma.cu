// Fused decode attention over the packed block-32 cache, head_dim 128: tensor-core kernels.
//
// Why tensor cores on an HBM-bound scan: at 70 % of HBM bandwidth a B200 streams ~8e12 packed
// codes per second, and every code meets one FMA per query head of the GQA group (x2 for K and
// V).  On the SIMT pipes that is more lane-instructions than the chip can issue, so the
// QK^T and PV contractions go through mma.sync.m16n8k16 (f16 in, f32 accumulate) and the SIMT
// pipes only unpack codes.  tcgen05 is not used: its operands must be staged in shared memory,
// which would cost a shared-memory write per dequantized value, while mma.sync takes the
// unpacked codes straight from registers.
//
// Layout of one warp step (16 tokens t0..t0+15, lane = 4*n + j):
//   S^T = Q~ K^T :  M = query heads (rows 0..7 used), N = 8 tokens, K = 16 dims of ONE 32-block.
//       Lane (n, j) supplies, for token t0+8o+n and block b, the eight codes of word j of the
//       block; two MMAs per (octet o, block b).  Because each MMA stays inside one block, the
//       per-block scale |s| is applied to the f32 accumulator (2 FMAs), not to the elements.
//   O^T = V^T P  :  M = 16 dims of ONE block, N = 8 heads, K = 16 tokens.  The accumulator
//       fragment of S^T (head n, tokens 2j, 2j+1) is exactly the B fragment of this MMA, so the
//       probabilities never leave registers; the V scale is folded into them (P' = p |s_v|).
//
// Exactness (4-bit MaxNorm grid, codebooks.rs:63-73): centroid i = (2R/15)(i - 7.5).  Codes are
// converted to the exact f16 integers i - 8 (magic-number trick: (w & 0x000f000f) | 0x64006400
// is the half2 (1024 + i, 1024 + i')), the 0.5 offset is carried separately in f32, and both
// the rotated query and P' are split into f16 hi + lo parts, so every product entering the
// f32 accumulators is exact: the result matches an f32 evaluation to rounding noise.
#include <float.h>

#include "tqb_common.cuh"

namespace tqb {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kD = 128;
constexpr int kGroup = 16;             // tokens per warp step
constexpr float kNegBig = -1.0e30f;    // finite stand-in for -inf (keeps exp2 arguments NaN-free)

struct MmaArgs {
    const void* q;
    const uint32_t* kw;   // K indices as words, [hkv, kv_stride, 16]
    const uint16_t* ks;   // [hkv, kv_stride, 4]
    const uint32_t* vw;
    const uint16_t* vs;
    float* partial_out;
    float* partial_max;
    float* partial_sum;
    const float* dev_signs;
    int hq, hkv, g, kv_len, kv_stride, num_partitions, part_size;
    float qk_const;   // softmax_scale * log2(e) * (2R/15)
    float v_const;    // 2R/15
    float sign_mag;
};

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
    return d;
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Eight 4-bit codes of one word -> four half2 registers holding the exact integers code - 8:
//   x[0] = (c0, c4), x[1] = (c1, c5), x[2] = (c2, c6), x[3] = (c3, c7).
__device__ __forceinline__ void nibbles_to_half2(uint32_t w, uint32_t (&x)[4]) {
    const uint32_t kMagic = 0x64006400u;                       // half2(1024, 1024)
    const __half2 k1032 = u32_as_h2(0x64086408u);              // 1024 + 8
    const __half2 kSixteenth = u32_as_h2(0x2C002C00u);         // 1/16
    const __half2 kM72 = u32_as_h2(0xD480D480u);               // -(1024/16 + 8)
    const uint32_t w8 = w >> 8;
    x[0] = h2_as_u32(__hsub2(u32_as_h2(lop3_and_or(w, 0x000f000fu, kMagic)), k1032));
    x[1] = h2_as_u32(__hfma2(u32_as_h2(lop3_and_or(w, 0x00f000f0u, kMagic)), kSixteenth, kM72));
    x[2] = h2_as_u32(__hsub2(u32_as_h2(lop3_and_or(w8, 0x000f000fu, kMagic)), k1032));
    x[3] = h2_as_u32(__hfma2(u32_as_h2(lop3_and_or(w8, 0x00f000f0u, kMagic)), kSixteenth, kM72));
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
// 16 consecutive tokens of one KV head: K indices [16][64 B], V indices [16][64 B], K scales
// [16][8 B], V scales [16][8 B].  Lanes fill a stage with cp.async (16-byte pieces for the
// indices, 8-byte pieces for the scales) and track completion with commit/wait groups, so no
// thread ever spins on a flag.  The 16-byte piece c of token row t is stored at piece
// c ^ ((t >> 1) & 3): with that XOR both access patterns below touch 32 distinct banks.
constexpr int kStages = 4;
constexpr int kStageBytes = 1024 + 1024 + 128 + 128;
constexpr int kRingBytes = kStages * kStageBytes;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// Per-lane copy plan of one stage: two 16-byte index pieces (rows t0, t0 + 8) of K and of V,
// and one 8-byte scale row (K for lanes 0..15, V for lanes 16..31).
struct FillPlan {
    const uint8_t* k;     // K piece of row t0 of group 0
    const uint8_t* v;
    const uint16_t* sc;
    uint32_t dst0, dst1, dsts;
    int t0, ts;
};

__device__ __forceinline__ FillPlan make_plan(const MmaArgs& a, size_t row0, int first, int lane) {
    FillPlan f;
    f.t0 = lane >> 2;                // pieces lane and lane + 32 belong to rows t0 and t0 + 8
    const int pc = lane & 3;
    const uint8_t* kb = reinterpret_cast<const uint8_t*>(a.kw);
    const uint8_t* vb = reinterpret_cast<const uint8_t*>(a.vw);
    f.k = kb + (row0 + first + f.t0) * 64 + pc * 16;
    f.v = vb + (row0 + first + f.t0) * 64 + pc * 16;
    f.dst0 = f.t0 * 64 + ((pc ^ ((f.t0 >> 1) & 3)) << 4);
    f.dst1 = f.dst0 + 512;           // row t0 + 8 has the same (t >> 1) & 3
    f.ts = lane & 15;
    f.sc = (lane < 16 ? a.ks : a.vs) + (row0 + first + f.ts) * 4;
    f.dsts = 2048 + (lane < 16 ? 0 : 128) + f.ts * 8;
    return f;
}

// Issues the copies of the 16 tokens starting at `gs` = first + byte_off / 64 into the stage at
// shared address `st`.  Rows past the last valid token re-read the last token (they are masked
// later), which only happens in the final group of a sequence.
__device__ __forceinline__ void stage_fill(const FillPlan& f, size_t byte_off, int gs, int last, uint32_t st) {
    if (gs + 16 <= last + 1) {
        cp_async16(st + f.dst0, f.k + byte_off);
        cp_async16(st + f.dst1, f.k + byte_off + 512);
        cp_async16(st + 1024 + f.dst0, f.v + byte_off);
        cp_async16(st + 1024 + f.dst1, f.v + byte_off + 512);
        cp_async8(st + f.dsts, f.sc + (byte_off >> 4));
    } else {
        const long long b0 = (long long)(min(gs + f.t0, last) - (gs + f.t0)) * 64;
        const long long b1 = (long long)(min(gs + f.t0 + 8, last) - (gs + f.t0 + 8)) * 64;
        const long long bs = (long long)(min(gs + f.ts, last) - (gs + f.ts)) * 4;
        cp_async16(st + f.dst0, f.k + byte_off + b0);
        cp_async16(st + f.dst1, f.k + byte_off + 512 + b1);
        cp_async16(st + 1024 + f.dst0, f.v + byte_off + b0);
        cp_async16(st + 1024 + f.dst1, f.v + byte_off + 512 + b1);
        cp_async8(st + f.dsts, f.sc + (byte_off >> 4) + bs);
    }
}

// 4-bit MaxNorm ("PQO4") kernel.  Grid (kv heads, partitions), 4 warps; each warp walks its
// partition in steps of 16 tokens and keeps its own online-softmax state; the four states are
// merged through shared memory at the end and written as one split-K partial.
//
// NSPLIT = true (GQA group <= 4): the MMA columns 0..3 of O^T = V^T P' carry the f16 "hi" part of
// P' for heads 0..3 and columns 4..7 the "lo" part, so one MMA delivers the split-precision
// product.  NSPLIT = false (group 5..8): hi and lo take one MMA each.
// The query is split the same way along the 16 MMA rows of S^T = Q~ K^T: rows 0..7 hold the
// hi parts of the (up to) 8 heads, rows 8..15 the lo parts.
template <typename QT, bool NSPLIT>
__global__ void __launch_bounds__(kThreads, 3) decode_pqo4_mma_kernel(MmaArgs a) {
    __shared__ __align__(1024) unsigned char s_raw[kWarps * kRingBytes];
    __shared__ float s_q[8 * kD];   // rotated queries (prologue only)
    // epilogue view of the ring memory (the rings are idle then)
    float (*s_o)[8][kD] = reinterpret_cast<float (*)[8][kD]>(s_raw);                 // [kWarps][8][128]
    float (*s_m)[8] = reinterpret_cast<float (*)[8]>(s_raw + kWarps * 8 * kD * 4);   // [kWarps][8]
    float (*s_l)[8] = s_m + kWarps;
    float (*s_z)[8][4] = reinterpret_cast<float (*)[8][4]>(s_l + kWarps);
    __shared__ float s_sign[32];
    static_assert(kWarps * kRingBytes >= kWarps * 8 * kD * 4 + kWarps * 8 * 4 * 2 + kWarps * 8 * 4 * 4, "ring too small");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = lane >> 2, j = lane & 3;     // n: MMA column / row group, j: position in the quad
    const int kvh = blockIdx.x, part = blockIdx.y;
    const int g = a.g;

    // ---- start streaming the first stages before anything else: the copies do not depend on q ----
    float m_run = kNegBig, l_run = 0.0f;
    float z[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float o[4][2][4];
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[b][m][i] = 0.0f;

    const int t_begin = part * a.part_size;
    const int t_end = min(t_begin + a.part_size, a.kv_len);
    const size_t row0 = (size_t)kvh * a.kv_stride;
    const int last = a.kv_len - 1;
    const int first = t_begin + warp * kGroup;
    const int stride = kWarps * kGroup;
    const int ngroups = first < t_end ? (t_end - first + stride - 1) / stride : 0;

    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(s_raw) + warp * kRingBytes;
    // per-thread shared-memory offsets inside a stage
    uint32_t koff[4], voff[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        koff[b] = n * 64 + ((b ^ ((n >> 1) & 3)) << 4) + j * 4;                 // token n (+8o: +512), word j of block b
        voff[b] = 1024 + (2 * j) * 64 + ((b ^ j) << 4) + (n >> 1) * 4;          // token 2j (+e: +64, +8o: +512), word n/2
    }
    const uint32_t scoff = 2048 + (2 * j) * 8;                                   // scales of token 2j (+e: +8, +8o: +64)
    const uint32_t vsel = (n & 1) ? 0x7632u : 0x5410u;

    const FillPlan plan = make_plan(a, row0, first, lane);
    const size_t group_bytes = (size_t)stride * 64;   // K/V index bytes between consecutive groups of this warp
#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) {
        if (i < ngroups) stage_fill(plan, i * group_bytes, first + i * stride, last, ring + i * kStageBytes);
        cp_async_commit();
    }
    uint32_t st = ring;                                        // stage being consumed
    uint32_t st_fill = ring + (kStages - 1) * kStageBytes;     // stage being refilled
    size_t fill_off = (kStages - 1) * group_bytes;


    if (tid < 32) {
        const uint32_t neg = 0xB1A6D4B2u;  // src/cache/precomputed/rotation.rs:16-20
        s_sign[tid] = a.dev_signs ? a.dev_signs[tid] : (((neg >> tid) & 1u) ? -a.sign_mag : a.sign_mag);
    }
    __syncthreads();
    // ---- rotate the g queries of this KV head once: q~ = sigma .* H32(q_b) / sqrt(32), constants folded ----
    {
        const float inv_sqrt = 1.0f / sqrtf(32.0f);
        for (int u = warp; u < 8 * 4; u += kWarps) {
            const int hh = u >> 2, b = u & 3;
            float v = 0.0f;
            if (hh < g) v = to_f32<QT>(reinterpret_cast<const QT*>(a.q)[(size_t)(kvh * g + hh) * kD + b * 32 + lane]);
            v = wht32_lane(v, lane);
            s_q[hh * kD + b * 32 + lane] = ((v * inv_sqrt) * s_sign[lane]) * a.qk_const;
        }
    }
    __syncthreads();
    // A fragments: rows 0..7 = hi(q~) of head n, rows 8..15 = lo(q~) of head n.  For block b and
    // half m the k-slots (2j, 2j+1 | 2j+8, 2j+9) hold dims 32b + 8j + 2m + (0, 4 | 1, 5).
    uint32_t afr[4][2][4];
    float qbar[4];
    {
        const float* sq = s_q + n * kD;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            float s = 0.0f;
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const int d0 = 32 * b + 8 * j + 2 * m;
                const float q0 = sq[d0], q4 = sq[d0 + 4], q1 = sq[d0 + 1], q5 = sq[d0 + 5];
                afr[b][m][0] = pack_hi(q0, q4);
                afr[b][m][1] = pack_lo(q0, q4);
                afr[b][m][2] = pack_hi(q1, q5);
                afr[b][m][3] = pack_lo(q1, q5);
                s += (q0 + q4) + (q1 + q5);
            }
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            qbar[b] = 0.5f * s;   // the +0.5 of (i - 7.5) = (i - 8) + 0.5, summed over the block
        }
    }

    for (int it = 0; it < ngroups; ++it) {
        const int gs = first + it * stride;
        if (it + kStages - 1 < ngroups) stage_fill(plan, fill_off, gs + (kStages - 1) * stride, last, st_fill);
        cp_async_commit();
        fill_off += group_bytes;
        st_fill = (st_fill + kStageBytes == ring + kRingBytes) ? ring : st_fill + kStageBytes;
        cp_async_wait<kStages - 1>();
        __syncwarp();

        // ---- S^T = Q~ K^T ----
        float s[2][2];
#pragma unroll
        for (int o8 = 0; o8 < 2; ++o8) {
            s[o8][0] = 0.0f;
            s[o8][1] = 0.0f;
            const uint2 sc0 = lds64(st + scoff + o8 * 64), sc1 = lds64(st + scoff + o8 * 64 + 8);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                uint32_t x[4];
                nibbles_to_half2(lds32(st + koff[b] + o8 * 512), x);
                float acc[4] = {qbar[b], qbar[b], 0.0f, 0.0f};
                mma16816(acc, afr[b][0][0], afr[b][0][1], afr[b][0][2], afr[b][0][3], x[0], x[1]);
                mma16816(acc, afr[b][1][0], afr[b][1][1], afr[b][1][2], afr[b][1][3], x[2], x[3]);
                const __half2 p0 = u32_as_h2(b < 2 ? sc0.x : sc0.y), p1 = u32_as_h2(b < 2 ? sc1.x : sc1.y);
                const float k0 = fabsf((b & 1) ? __high2float(p0) : __low2float(p0));
                const float k1 = fabsf((b & 1) ? __high2float(p1) : __low2float(p1));
                s[o8][0] = fmaf(k0, acc[0] + acc[2], s[o8][0]);
                s[o8][1] = fmaf(k1, acc[1] + acc[3], s[o8][1]);
            }
        }
        if (gs + kGroup > a.kv_len) {   // ragged tail: tokens past the end get zero weight
#pragma unroll
            for (int o8 = 0; o8 < 2; ++o8)
#pragma unroll
                for (int e = 0; e < 2; ++e)
                    if (gs + 8 * o8 + 2 * j + e > last) s[o8][e] = kNegBig;
        }
        // ---- online softmax for head n (the quad holds its 16 tokens) ----
        float mx = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float resc = ex2(m_run - m_new);
        m_run = m_new;
        float p[2][2];
#pragma unroll
        for (int o8 = 0; o8 < 2; ++o8)
#pragma unroll
            for (int e = 0; e < 2; ++e) p[o8][e] = ex2(s[o8][e] - m_new);
        l_run = l_run * resc + ((p[0][0] + p[0][1]) + (p[1][0] + p[1][1]));
        if (__any_sync(0xffffffffu, resc != 1.0f)) {
            // column c of O^T belongs to head c (NSPLIT: head c & 3)
            const int h0 = NSPLIT ? ((2 * j) & 3) : 2 * j, h1 = NSPLIT ? ((2 * j + 1) & 3) : 2 * j + 1;
            const float r0 = __shfl_sync(0xffffffffu, resc, 4 * h0);
            const float r1 = __shfl_sync(0xffffffffu, resc, 4 * h1);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                z[b] *= resc;
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    o[b][m][0] *= r0; o[b][m][1] *= r1; o[b][m][2] *= r0; o[b][m][3] *= r1;
                }
            }
        }
        if (NSPLIT) {
            // lanes of rows 4..7 take over the probabilities of heads 0..3 and will supply the lo parts
#pragma unroll
            for (int o8 = 0; o8 < 2; ++o8)
#pragma unroll
                for (int e = 0; e < 2; ++e) p[o8][e] = __shfl_sync(0xffffffffu, p[o8][e], lane & 15);
        }
        // ---- O^T += V^T P' ----
        uint2 vs[2][2];
#pragma unroll
        for (int o8 = 0; o8 < 2; ++o8)
#pragma unroll
            for (int e = 0; e < 2; ++e) vs[o8][e] = lds64(st + 128 + scoff + o8 * 64 + e * 8);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            float pf[2][2];
#pragma unroll
            for (int o8 = 0; o8 < 2; ++o8)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const __half2 pr = u32_as_h2(b < 2 ? vs[o8][e].x : vs[o8][e].y);
                    pf[o8][e] = p[o8][e] * fabsf((b & 1) ? __high2float(pr) : __low2float(pr));
                }
            z[b] += (pf[0][0] + pf[0][1]) + (pf[1][0] + pf[1][1]);
            const uint32_t b0h = pack_hi(pf[0][0], pf[0][1]), b1h = pack_hi(pf[1][0], pf[1][1]);
            const uint32_t b0l = pack_lo(pf[0][0], pf[0][1]), b1l = pack_lo(pf[1][0], pf[1][1]);
            // half-word n of block b of the four tokens, paired (token 2j, token 2j+1)
            uint32_t xab[4], xcd[4];
            nibbles_to_half2(__byte_perm(lds32(st + voff[b]), lds32(st + voff[b] + 64), vsel), xab);
            nibbles_to_half2(__byte_perm(lds32(st + voff[b] + 512), lds32(st + voff[b] + 576), vsel), xcd);
            if (NSPLIT) {
                const uint32_t b0 = n < 4 ? b0h : b0l, b1 = n < 4 ? b1h : b1l;
                mma16816(o[b][0], xab[0], xab[1], xcd[0], xcd[1], b0, b1);
                mma16816(o[b][1], xab[2], xab[3], xcd[2], xcd[3], b0, b1);
            } else {
                mma16816(o[b][0], xab[0], xab[1], xcd[0], xcd[1], b0h, b1h);
                mma16816(o[b][0], xab[0], xab[1], xcd[0], xcd[1], b0l, b1l);
                mma16816(o[b][1], xab[2], xab[3], xcd[2], xcd[3], b0h, b1h);
                mma16816(o[b][1], xab[2], xab[3], xcd[2], xcd[3], b0l, b1l);
            }
        }
        __syncwarp();   // every lane is done with this stage before it is refilled
        st = (st + kStageBytes == ring + kRingBytes) ? ring : st + kStageBytes;
    }
    cp_async_wait<0>();
    __syncthreads();    // all rings idle: the memory is reused for the merge

    // ---- merge the four warps (scores are in log2 units; partials are stored in natural units) ----
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        z[b] += __shfl_xor_sync(0xffffffffu, z[b], 1);
        z[b] += __shfl_xor_sync(0xffffffffu, z[b], 2);
    }
    if (j == 0 && (!NSPLIT || n < 4)) {
        s_m[warp][n] = m_run;
        s_l[warp][n] = l_run;
#pragma unroll
        for (int b = 0; b < 4; ++b) s_z[warp][n][b] = z[b];
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
    {
        const int d = tid, b = d >> 5;
        for (int hh = 0; hh < g; ++hh) {
            float M = kNegBig;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w][hh]);
            float L = 0.0f, O = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float e = ex2(s_m[w][hh] - M);
                L = fmaf(s_l[w][hh], e, L);
                float ov = s_o[w][hh][d];
                if (NSPLIT) ov += s_o[w][hh + 4][d];
                O = fmaf(ov + 0.5f * s_z[w][hh][b], e, O);
            }
            const size_t pi = (size_t)(kvh * g + hh) * a.num_partitions + part;
            a.partial_out[pi * kD + d] = O * a.v_const;
            if (d == 0) {
                a.partial_max[pi] = (M <= kNegBig) ? -FLT_MAX : M * 0.6931471805599453f;
                a.partial_sum[pi] = L;
            }
        }
    }
}

}  // namespace

// Returns TQB_ERR_UNSUPPORTED when the shape is outside what the tensor-core kernels cover;
// the caller then uses the general kernel.
int launch_decode_mma(const tqb_decode_params* p, int num_partitions, float* partial_out, float* partial_max,
                      float* partial_sum, float sign_mag, cudaStream_t s) {
    const int g = p->num_q_heads / p->num_kv_heads;
    const int nblk = p->head_dim / kBlock;
    const bool all_outlier = p->outlier_blocks < 0 || p->outlier_blocks >= nblk;
    if (p->head_dim != kD || g > 8 || p->qjl_enabled) return TQB_ERR_UNSUPPORTED;
    if (!(p->bits == 4 && p->norm_mode == TQB_MAXNORM && all_outlier)) return TQB_ERR_UNSUPPORTED;
    if (((uintptr_t)p->k_scales % 8) || ((uintptr_t)p->v_scales % 8)) return TQB_ERR_UNSUPPORTED;
    if (((uintptr_t)p->k_indices % 16) || ((uintptr_t)p->v_indices % 16)) return TQB_ERR_UNSUPPORTED;
    if (p->kv_len <= 0) return TQB_ERR_UNSUPPORTED;
    MmaArgs a{};
    a.q = p->q;
    a.kw = reinterpret_cast<const uint32_t*>(p->k_indices);
    a.ks = p->k_scales;
    a.vw = reinterpret_cast<const uint32_t*>(p->v_indices);
    a.vs = p->v_scales;
    a.partial_out = partial_out;
    a.partial_max = partial_max;
    a.partial_sum = partial_sum;
    a.dev_signs = nullptr;
    a.hq = p->num_q_heads; a.hkv = p->num_kv_heads; a.g = g;
    a.kv_len = p->kv_len; a.kv_stride = p->kv_stride; a.num_partitions = num_partitions;
    const int step = kWarps * kGroup;
    a.part_size = ((p->kv_len + num_partitions - 1) / num_partitions + step - 1) / step * step;
    const float R = 2.1573f;
    const float grid_step = (2.0f * R) / 15.0f;   // codebooks.rs:64-67
    a.qk_const = p->softmax_scale * 1.4426950408889634f * grid_step;
    a.v_const = grid_step;
    a.sign_mag = sign_mag;
    dim3 grid(p->num_kv_heads, num_partitions);
#define TQB_LAUNCH_PQO4(QT)                                                              \
    do {                                                                                 \
        if (g <= 4) decode_pqo4_mma_kernel<QT, true><<<grid, kThreads, 0, s>>>(a);       \
        else decode_pqo4_mma_kernel<QT, false><<<grid, kThreads, 0, s>>>(a);             \
    } while (0)
    if (p->q_dtype == TQB_F32) TQB_LAUNCH_PQO4(float);
    else if (p->q_dtype == TQB_F16) TQB_LAUNCH_PQO4(__half);
    else TQB_LAUNCH_PQO4(__nv_bfloat16);
#undef TQB_LAUNCH_PQO4
    return check_launch(s);
}

}  // namespace tqb
