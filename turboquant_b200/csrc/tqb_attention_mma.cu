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

// 4-bit MaxNorm ("PQO4") kernel.  Grid (kv heads, partitions), 4 warps; each warp walks its
// partition in steps of 16 tokens and keeps its own online-softmax state; the four states are
// merged through shared memory at the end and written as one split-K partial.
template <typename QT>
__global__ void __launch_bounds__(kThreads, 3) decode_pqo4_mma_kernel(MmaArgs a) {
    __shared__ float s_o[kWarps][8][kD];   // prologue: rotated queries [8][128] live in s_o[0]
    __shared__ float s_m[kWarps][8], s_l[kWarps][8], s_z[kWarps][8][4];
    __shared__ float s_sign[32];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = lane >> 2, j = lane & 3;     // n: MMA column / row group, j: position in the quad
    const int kvh = blockIdx.x, part = blockIdx.y;
    const int g = a.g;

    if (tid < 32) {
        const uint32_t neg = 0xB1A6D4B2u;  // src/cache/precomputed/rotation.rs:16-20
        s_sign[tid] = a.dev_signs ? a.dev_signs[tid] : (((neg >> tid) & 1u) ? -a.sign_mag : a.sign_mag);
    }
    __syncthreads();
    // ---- rotate the g queries of this KV head once: q~ = sigma .* H32(q_b) / sqrt(32), constants folded ----
    {
        float* s_q = &s_o[0][0][0];
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
    // A fragments (rows = heads; only rows 0..7 are populated): for block b and half m the k-slots
    // (2j, 2j+1 | 2j+8, 2j+9) hold dims 32b + 8j + 2m + (0, 4 | 1, 5), matching nibbles_to_half2.
    uint32_t ahi[4][2][2], alo[4][2][2];
    float qbar[4];
    {
        const float* s_q = &s_o[0][0][0] + n * kD;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const int d0 = 32 * b + 8 * j + 2 * m;
                ahi[b][m][0] = pack_hi(s_q[d0], s_q[d0 + 4]);
                alo[b][m][0] = pack_lo(s_q[d0], s_q[d0 + 4]);
                ahi[b][m][1] = pack_hi(s_q[d0 + 1], s_q[d0 + 5]);
                alo[b][m][1] = pack_lo(s_q[d0 + 1], s_q[d0 + 5]);
            }
            float s = 0.0f;
            for (int i = 0; i < 32; ++i) s += s_q[32 * b + i];
            qbar[b] = 0.5f * s;   // the +0.5 of (i - 7.5) = (i - 8) + 0.5
        }
    }
    __syncthreads();   // s_o is reused by the epilogue

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

    for (int gs = t_begin + warp * kGroup; gs < t_end; gs += kWarps * kGroup) {
        // ---- loads: K words (token gs+8o+n, word j of each block), scales of tokens gs+8o+2j+e ----
        uint32_t kwv[2][4], vwv[2][2][4];
        uint2 ksc[2][2], vsc[2][2];
#pragma unroll
        for (int o8 = 0; o8 < 2; ++o8) {
            const size_t rk = (row0 + min(gs + 8 * o8 + n, last)) * 16;
#pragma unroll
            for (int b = 0; b < 4; ++b) kwv[o8][b] = __ldg(a.kw + rk + b * 4 + j);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const size_t rt = row0 + min(gs + 8 * o8 + 2 * j + e, last);
                ksc[o8][e] = __ldg(reinterpret_cast<const uint2*>(a.ks + rt * 4));
                vsc[o8][e] = __ldg(reinterpret_cast<const uint2*>(a.vs + rt * 4));
#pragma unroll
                for (int b = 0; b < 4; ++b) vwv[o8][e][b] = __ldg(a.vw + rt * 16 + b * 4 + (n >> 1));
            }
        }
        // ---- S^T = Q~ K^T ----
        float s[2][2];
#pragma unroll
        for (int o8 = 0; o8 < 2; ++o8) {
            s[o8][0] = 0.0f;
            s[o8][1] = 0.0f;
            const __half2 sc01[2] = {u32_as_h2(ksc[o8][0].x), u32_as_h2(ksc[o8][1].x)};
            const __half2 sc23[2] = {u32_as_h2(ksc[o8][0].y), u32_as_h2(ksc[o8][1].y)};
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                uint32_t x[4];
                nibbles_to_half2(kwv[o8][b], x);
                float acc[4] = {qbar[b], qbar[b], 0.0f, 0.0f};
                mma16816(acc, ahi[b][0][0], 0u, ahi[b][0][1], 0u, x[0], x[1]);
                mma16816(acc, alo[b][0][0], 0u, alo[b][0][1], 0u, x[0], x[1]);
                mma16816(acc, ahi[b][1][0], 0u, ahi[b][1][1], 0u, x[2], x[3]);
                mma16816(acc, alo[b][1][0], 0u, alo[b][1][1], 0u, x[2], x[3]);
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const __half2 pr = (b < 2) ? sc01[e] : sc23[e];
                    const float sk = fabsf((b & 1) ? __high2float(pr) : __low2float(pr));
                    s[o8][e] = fmaf(sk, acc[e], s[o8][e]);
                }
            }
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
            const float r0 = __shfl_sync(0xffffffffu, resc, 8 * j);        // head 2j
            const float r1 = __shfl_sync(0xffffffffu, resc, 8 * j + 4);    // head 2j+1
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                z[b] *= resc;
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    o[b][m][0] *= r0; o[b][m][1] *= r1; o[b][m][2] *= r0; o[b][m][3] *= r1;
                }
            }
        }
        // ---- O^T += V^T P' ----
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            float pf[2][2];
#pragma unroll
            for (int o8 = 0; o8 < 2; ++o8)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint32_t w = (b < 2) ? vsc[o8][e].x : vsc[o8][e].y;
                    const __half2 pr = u32_as_h2(w);
                    pf[o8][e] = p[o8][e] * fabsf((b & 1) ? __high2float(pr) : __low2float(pr));
                }
            z[b] += (pf[0][0] + pf[0][1]) + (pf[1][0] + pf[1][1]);
            const uint32_t b0h = pack_hi(pf[0][0], pf[0][1]), b1h = pack_hi(pf[1][0], pf[1][1]);
            const uint32_t b0l = pack_lo(pf[0][0], pf[0][1]), b1l = pack_lo(pf[1][0], pf[1][1]);
            // half-word n of block b of the four tokens, paired (token 2j, token 2j+1)
            const uint32_t sel = (n & 1) ? 0x7632u : 0x5410u;
            uint32_t xab[4], xcd[4];
            nibbles_to_half2(__byte_perm(vwv[0][0][b], vwv[0][1][b], sel), xab);
            nibbles_to_half2(__byte_perm(vwv[1][0][b], vwv[1][1][b], sel), xcd);
            mma16816(o[b][0], xab[0], xab[1], xcd[0], xcd[1], b0h, b1h);
            mma16816(o[b][0], xab[0], xab[1], xcd[0], xcd[1], b0l, b1l);
            mma16816(o[b][1], xab[2], xab[3], xcd[2], xcd[3], b0h, b1h);
            mma16816(o[b][1], xab[2], xab[3], xcd[2], xcd[3], b0l, b1l);
        }
    }

    // ---- merge the four warps (scores are in log2 units; partials are stored in natural units) ----
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        z[b] += __shfl_xor_sync(0xffffffffu, z[b], 1);
        z[b] += __shfl_xor_sync(0xffffffffu, z[b], 2);
    }
    if (j == 0) {
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
                O = fmaf(s_o[w][hh][d] + 0.5f * s_z[w][hh][b], e, O);
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
    if (p->q_dtype == TQB_F32) decode_pqo4_mma_kernel<float><<<grid, kThreads, 0, s>>>(a);
    else if (p->q_dtype == TQB_F16) decode_pqo4_mma_kernel<__half><<<grid, kThreads, 0, s>>>(a);
    else decode_pqo4_mma_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(a);
    return check_launch(s);
}

}  // namespace tqb
