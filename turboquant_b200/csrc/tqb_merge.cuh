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
    // merge_group128 only: when num_copies > 0 the un-normalised f32 result and the (max, sum) pairs go to these
    // record buffers ([num_q_heads, 128] floats, then [num_q_heads, 2]) instead of out / lse_out
    int num_copies, num_q_heads;
    float* copy_rec[kMaxPeers];
    // merge_group128<GROUP = true> only: where an intermediate partial goes
    float* group_out;
    float* group_max;
    float* group_sum;
};

// Two-level merge of the tensor-core decode kernels: partitions are merged in groups of kMergeGroup by the CTA that
// finishes a group, the group results by the CTA that finishes the last group of a KV head.  With P > 16 partitions the
// serial tail is two merges of about kMergeGroup and P / kMergeGroup slots instead of one of P slots by one CTA.
constexpr int kMergeGroup = 8;
__host__ __device__ inline int merge_groups(int num_partitions) {
    // up to two chunks of eight a single merge is shorter than two levels with their extra ticket round
    return num_partitions <= 2 * kMergeGroup ? 0 : (num_partitions + kMergeGroup - 1) / kMergeGroup;
}

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

// The same merge for ALL g query heads of one KV head by one CTA of 128 threads, head_dim 128: thread d owns output
// element d of every head (warp = 32-block, lane = element).  The slot weights exp(max_s - M) of all heads are
// tabulated in shared memory, and each thread walks the slots eight at a time with the loads of all heads in flight
// together, so a merge of S slots costs about S / 8 trips to L2 (merge_head makes one trip per slot, block and head).
//
// Source: slots [first, first + count) of arrays laid out [head][head_stride][...] (a.partial_*).
// Destination, GROUP = true: one more partial - un-normalised sum, max and sum of slot `gslot` of the group arrays
// (a.group_*, [head][group_stride][...]), still in the rotated domain.  GROUP = false: the final result as merge_head
// writes it (or, with num_copies > 0, the record copies).  Sums run over the slots in ascending order.
// `s_work`: shared memory, at least (16 + g * count) floats; all 128 threads must call.
template <bool GROUP>
__device__ __forceinline__ void merge_group128(const MergeArgs& a, int head0, int g, int tid, float* s_work, int first, int count,
                                               int head_stride, int gslot = 0, int group_stride = 0) {
    using namespace merge_detail;
    const int lane = tid & 31, warp = tid >> 5;
    constexpr int D = 128;
    float* s_M = s_work;          // [8]
    float* s_L = s_work + 8;      // [8]
    float* s_w = s_work + 16;     // [g][count]
    // A dependent trip to L2 costs more than a microsecond on this part, so the loads of a merge are issued together:
    // the first eight slots of the un-normalised outputs of all heads (up to 64 loads per thread) go out before the
    // (max, sum) pairs are even looked at, and each warp fetches the pairs of both of its heads in one go.
    const float* po = a.partial_out + ((size_t)head0 * head_stride + first) * D + tid;
    float v[8][8];
#pragma unroll
    for (int hh = 0; hh < 8; ++hh)
#pragma unroll
        for (int i = 0; i < 8; ++i)
            v[hh][i] = (hh < g && i < count) ? __ldcg(po + ((size_t)hh * head_stride + i) * D) : 0.0f;
    {
        const float* pm[2];
        const float* ps[2];
        float pmv[2] = {-FLT_MAX, -FLT_MAX}, psv[2] = {0.0f, 0.0f};
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int hh = warp + 4 * t;
            pm[t] = a.partial_max + (size_t)(head0 + hh) * head_stride + first;
            ps[t] = a.partial_sum + (size_t)(head0 + hh) * head_stride + first;
            if (hh < g && lane < count) {
                pmv[t] = __ldcg(pm[t] + lane);
                psv[t] = __ldcg(ps[t] + lane);
            }
        }
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int hh = warp + 4 * t;
            if (hh >= g) continue;
            float M = pmv[t];
            for (int p = lane + 32; p < count; p += 32) M = fmaxf(M, __ldcg(pm[t] + p));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
            const float wl = lane < count ? expf(pmv[t] - M) : 0.0f;
            if (lane < count) s_w[hh * count + lane] = wl;
            float L = lane < count ? psv[t] * wl : 0.0f;
            for (int p = lane + 32; p < count; p += 32) {
                const float wp = expf(__ldcg(pm[t] + p) - M);
                s_w[hh * count + p] = wp;
                L += __ldcg(ps[t] + p) * wp;
            }
            L = sum32(L);
            if (lane == 0) {
                s_M[hh] = M;
                s_L[hh] = L;
            }
        }
    }
    __syncthreads();
    float acc[8];
#pragma unroll
    for (int hh = 0; hh < 8; ++hh) acc[hh] = 0.0f;
    for (int p0 = 0; p0 < count; p0 += 8) {
        if (p0 > 0) {
#pragma unroll
            for (int hh = 0; hh < 8; ++hh)
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    v[hh][i] = (hh < g && p0 + i < count) ? __ldcg(po + ((size_t)hh * head_stride + p0 + i) * D) : 0.0f;
        }
#pragma unroll
        for (int hh = 0; hh < 8; ++hh)
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (hh < g && p0 + i < count) acc[hh] = fmaf(v[hh][i], s_w[hh * count + p0 + i], acc[hh]);
    }
    const float inv_sqrt = 1.0f / sqrtf((float)kBlock);
    const uint32_t neg = 0xB1A6D4B2u;   // src/cache/precomputed/rotation.rs:16-20
    const float sg = a.dev_signs ? a.dev_signs[lane] : (((neg >> lane) & 1u) ? -a.sign_mag : a.sign_mag);
    {
        constexpr int h0 = 0;
#pragma unroll
        for (int hh = 0; hh < 8; ++hh) {
            if (h0 + hh >= g) continue;
            const int head = head0 + h0 + hh;
            float r = acc[hh];
            if (GROUP) {
                a.group_out[((size_t)head * group_stride + gslot) * D + tid] = r;
                continue;
            }
            if (a.rotate) r = wht32(r * sg, lane) * inv_sqrt;
            if (a.num_copies > 0) {
                // (constant indices only: a run-time index would move the argument block to local memory)
#pragma unroll
                for (int c = 0; c < kMaxPeers; ++c)
                    if (c < a.num_copies) a.copy_rec[c][(size_t)head * D + tid] = r;
                continue;
            }
            if (a.lse_out == nullptr) {
                const float L = s_L[h0 + hh];
                r *= L > 0.0f ? 1.0f / L : 0.0f;
            }
            store_out(a.out, a.out_dtype, (size_t)head * D + tid, r);
        }
    }
    if (tid < g) {
        if (GROUP) {
            a.group_max[(size_t)(head0 + tid) * group_stride + gslot] = s_M[tid];
            a.group_sum[(size_t)(head0 + tid) * group_stride + gslot] = s_L[tid];
        } else if (a.num_copies > 0) {
#pragma unroll
            for (int c = 0; c < kMaxPeers; ++c)
                if (c < a.num_copies) {
                    float* lse = a.copy_rec[c] + (size_t)a.num_q_heads * D;
                    lse[(head0 + tid) * 2] = s_M[tid];
                    lse[(head0 + tid) * 2 + 1] = s_L[tid];
                }
        } else if (a.lse_out != nullptr) {
            a.lse_out[(head0 + tid) * 2] = s_M[tid];
            a.lse_out[(head0 + tid) * 2 + 1] = s_L[tid];
        }
    }
}

}  // namespace tqb
