// One 32-block of the all-outlier MaxNorm cache format quantized by ONE thread (in-register butterfly):
// the body of block_quantize_pqo_kernel, shared with the decode kernel, which appends the new token's K and
// V rows itself.  polar_quantize (src/cache/quantize_tensor.rs:40-176) with the scalar arithmetic of
// src/cache/cuda/kernels/tq_quant_kernel.cu:216-259; results are bit-identical to the general kernel.
#pragma once
#include "tqb_common.cuh"

namespace tqb {

template <typename T>
__device__ __forceinline__ void load32(const T* p, float (&v)[32]);
template <>
__device__ __forceinline__ void load32<float>(const float* p, float (&v)[32]) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float4 a = __ldg(reinterpret_cast<const float4*>(p) + k);
        v[4 * k] = a.x; v[4 * k + 1] = a.y; v[4 * k + 2] = a.z; v[4 * k + 3] = a.w;
    }
}
template <>
__device__ __forceinline__ void load32<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[32]) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint4 r = __ldg(reinterpret_cast<const uint4*>(p) + k);
        uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[8 * k + 2 * i] = __uint_as_float(w[i] << 16);
            v[8 * k + 2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
}
template <>
__device__ __forceinline__ void load32<__half>(const __half* p, float (&v)[32]) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint4 r = __ldg(reinterpret_cast<const uint4*>(p) + k);
        const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(h[i]);
            v[8 * k + 2 * i] = f.x;
            v[8 * k + 2 * i + 1] = f.y;
        }
    }
}

__device__ __forceinline__ void butterfly32_regs(float (&v)[32]) {
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if ((i & h) == 0) {
                float x = v[i], y = v[i + h];
                v[i] = x + y;
                v[i + h] = x - y;
            }
        }
    }
}

constexpr uint32_t kSignMask = 0xB1A6D4B2u;   // bit j set <=> sign j is -1 (precomputed/rotation.rs:16-20)


// Cell table for the 3-bit boundary search: cell c = round(t * kCellScale + kCellHalf); the 256 cells are far narrower
// than the gap between two boundaries, so a cell (widened by kCellSlop on both sides to absorb the rounding
// of the cell index) holds at most one boundary:  code = below + (t > bnd), exactly the count of
// boundaries below t.  .x = that boundary (FLT_MAX when the cell has none), .y = bit pattern of the number
// of boundaries under the cell.  |t| <= outer centroid (2.1520 for the 3-bit table) < 2.2 by construction
// of the MaxNorm scale, so the index never leaves the table.
constexpr float kCellScale = 58.0f;
constexpr float kCellHalf = 128.0f;   // an integer, so that kCellHalf + 1.5 * 2^23 is exact
constexpr float kCellSlop = 1e-3f;
__device__ __forceinline__ void build_cell_table(const Codebook& cb, int n_bnd, float2* lut, int tid, int nthreads) {
    for (int c = tid; c < 256; c += nthreads) {
        const float lo = ((float)c - 0.5f - kCellHalf) / kCellScale - kCellSlop;
        const float hi = ((float)c + 0.5f - kCellHalf) / kCellScale + kCellSlop;
        float bnd = 3.0e38f;
        unsigned below = 0;
        for (int k = 0; k < n_bnd; ++k) {
            const float b = cb.b[k];
            if (b < lo) ++below;
            else if (b <= hi) bnd = b;
        }
        lut[c] = make_float2(bnd, __uint_as_float(below));
    }
}

// x: the block's 32 input values (16-byte aligned).  w: packed codes (4 * BITS bytes, LSB-first), returns the
// f32 scale (before the outlier sign).  cb: the outlier codebook of BITS bits.  lut: the 3-bit cell table in
// shared memory (build_cell_table), or nullptr for the register bisection.  TABLE: the codebook is not the
// 4-bit uniform grid even when BITS = 4 (codes of a narrower codebook stored at BITS width); needs lut.
template <typename T, int BITS, bool TABLE = false>
__device__ __forceinline__ float pqo_quantize_block(const T* x, const Codebook& cb, float outer_centroid, uint32_t (&w)[4],
                                                    const float2* lut = nullptr) {
    const float inv_sqrt = 1.0f / sqrtf((float)kBlock);
    const float R = cb.c[(1 << BITS) - 1];
    const float inv_step = 15.0f / (2.0f * R);
    float v[32];
    load32<T>(x, v);
    butterfly32_regs(v);
    float amax_w = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax_w = fmaxf(amax_w, fabsf(v[i]));
    const float amax = amax_w * inv_sqrt;          // rounding is monotone: equals max_i |W_i * inv_sqrt|
    const float raw = __fdiv_rn(amax, outer_centroid);
    const float scale = raw > kMinNorm ? raw : kMinNorm;
    const float r = __frcp_rn(scale);
    w[0] = w[1] = w[2] = w[3] = 0u;
    if (BITS == 4 && !TABLE) {
        const float cpos = (inv_sqrt * r) * inv_step, cneg = -cpos;
        const float kMagic = 12582912.0f;          // 1.5 * 2^23
        bool near = false;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const float u = fmaf(v[i], ((kSignMask >> i) & 1u) ? cneg : cpos, 7.5f);
            const float y = u + kMagic;
            const float d = u - (y - kMagic);
            near |= fabsf(d) > 0.49998f;
            w[i >> 3] += (__float_as_uint(y) & 15u) << (4 * (i & 7));
        }
        if (near) {   // rare: exact division and the f32 boundary table
            w[0] = w[1] = w[2] = w[3] = 0u;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float rot = (v[i] * inv_sqrt) * (((kSignMask >> i) & 1u) ? -1.0f : 1.0f);
                const float t = __fdiv_rn(rot, scale);
                unsigned c = 0;
#pragma unroll
                for (int k = 0; k < 15; ++k) c += (t > cb.b[k]) ? 1u : 0u;
                w[i >> 3] += c << (4 * (i & 7));
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const float rot = v[i] * (((kSignMask >> i) & 1u) ? -inv_sqrt : inv_sqrt);
            const float q = rot * r;
            const float rem = fmaf(-q, scale, rot);
            const float t = fmaf(rem, r, q);           // == rot / scale, correctly rounded
            unsigned c;
            if (lut != nullptr) {
                const float y = fmaf(q, kCellScale, kCellHalf + 12582912.0f);   // round to nearest cell
                const float2 e = lut[__float_as_uint(y) & 255u];
                c = __float_as_uint(e.y) + (t > e.x ? 1u : 0u);
            } else {
                // bisection over the 7 boundaries (constant bank operands)
                const bool p1 = t > cb.b[3];
                const bool p2 = t > (p1 ? cb.b[5] : cb.b[1]);
                const float t3 = p1 ? (p2 ? cb.b[6] : cb.b[4]) : (p2 ? cb.b[2] : cb.b[0]);
                const bool p3 = t > t3;
                c = (p1 ? 4u : 0u) + (p2 ? 2u : 0u) + (p3 ? 1u : 0u);
            }
            const int bit = BITS * i;
            w[bit >> 5] += c << (bit & 31);
            if ((bit & 31) + BITS > 32) w[(bit >> 5) + 1] += c >> (32 - (bit & 31));
        }
    }
    return scale;
}

}  // namespace tqb
