// Split-K merge of decode attention: combines the per-partition (max, sum, un-normalised output)
// partials of one query head and applies the inverse rotation of the output.  Used by the stand-alone
// merge kernel and by the last CTA of a KV head inside the tensor-core decode kernel, so both produce
// identical bits.  Follows tq_fused_attention_reduce (src/cache/cuda/kernels/tq_attention_kernel.cu:299-332),
// with the inverse block rotation (src/cache/wht_tensor.rs:27-65) applied once per output block.
#pragma once
#include <float.h>

#include "tqb_common.cuh"

namespace tqb {

struct MergeArgs {
    const float* partial_out;   // [hq, P, D]
    const float* partial_max;   // [hq, P]  natural-log units
    const float* partial_sum;   // [hq, P]
    const float* dev_signs;     // legacy entry point (else nullptr)
    void* out;
    float* lse_out;             // nullptr, or [hq, 2]: out stays un-normalised and (max, sum) go here
    int head_dim, nblk, num_partitions, rotate;
    int out_dtype;
    float sign_mag;
};

namespace merge_detail {
__device__ __forceinline__ float sum32(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float wht32(float v, int lane) {
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
        float other = __shfl_xor_sync(0xffffffffu, v, h);
        v = (lane & h) ? (other - v) : (v + other);
    }
    return v;
}
__device__ __forceinline__ void store_out(void* out, int dtype, size_t i, float v) {
    if (dtype == TQB_F32) reinterpret_cast<float*>(out)[i] = v;
    else if (dtype == TQB_F16) reinterpret_cast<__half*>(out)[i] = __float2half_rn(v);
    else reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
}
}  // namespace merge_detail

// All threads of a CTA of `nwarps` warps call this for one query head; warp w handles output blocks
// w, w + nwarps, ...; lane = element of the block.  Partials are read past L1 (they may have been
// written by other CTAs of the same launch).
__device__ __forceinline__ void merge_head(const MergeArgs& a, int head, int lane, int warp, int nwarps) {
    using namespace merge_detail;
    const int D = a.head_dim, P = a.num_partitions;
    const float* pm = a.partial_max + (size_t)head * P;
    const float* ps = a.partial_sum + (size_t)head * P;
    // Lane p keeps (max, sum) of partition p; both loads are issued before either is used, and the partial
    // outputs below are fetched eight at a time, so the merge costs a few trips to L2, not one per partition.
    float pmv = -FLT_MAX, psv = 0.0f;
    if (lane < P) {
        pmv = __ldcg(pm + lane);
        psv = __ldcg(ps + lane);
    }
    float M = pmv;
    for (int p = lane + 32; p < P; p += 32) M = fmaxf(M, __ldcg(pm + p));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float wl = lane < P ? expf(pmv - M) : 0.0f;   // weight of partition `lane`
    float L = lane < P ? psv * wl : 0.0f;
    for (int p = lane + 32; p < P; p += 32) L += __ldcg(ps + p) * expf(__ldcg(pm + p) - M);
    L = sum32(L);
    const float inv_sqrt = 1.0f / sqrtf((float)kBlock);
    const uint32_t neg = 0xB1A6D4B2u;   // src/cache/precomputed/rotation.rs:16-20
    const float sg = a.dev_signs ? a.dev_signs[lane] : (((neg >> lane) & 1u) ? -a.sign_mag : a.sign_mag);
    const float inv_l = L > 0.0f ? 1.0f / L : 0.0f;
    for (int b = warp; b < a.nblk; b += nwarps) {
        const float* po = a.partial_out + (size_t)head * P * D + b * 32 + lane;
        float acc = 0.0f;   // sum over partitions in ascending order
        if (P <= 32) {
            for (int p0 = 0; p0 < P; p0 += 8) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = p0 + i < P ? __ldcg(po + (size_t)(p0 + i) * D) : 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (p0 + i < P) acc = fmaf(v[i], __shfl_sync(0xffffffffu, wl, p0 + i), acc);
            }
        } else {
            for (int p = 0; p < P; ++p) acc = fmaf(__ldcg(po + (size_t)p * D), expf(__ldcg(pm + p) - M), acc);
        }
        if (a.rotate) acc = wht32(acc * sg, lane) * inv_sqrt;
        if (a.lse_out == nullptr) acc *= inv_l;
        store_out(a.out, a.out_dtype, (size_t)head * D + b * 32 + lane, acc);
    }
    if (a.lse_out != nullptr && lane == 0 && warp == 0) {
        a.lse_out[head * 2] = M;
        a.lse_out[head * 2 + 1] = L;
    }
}

}  // namespace tqb
