// Fused decode attention over the packed block-32 cache: general kernel.
//
// Algebra (derived from src/cache/cuda/kernels/tq_dequant_kernel.cu:77-97 and
// tq_attention_kernel.cu:161-253).  A stored block decodes to
//     k = |s| * H32(sigma .* c[idx]) / sqrt(32)
// and H32 is symmetric, so  <q_b, k> = |s| * < sigma .* H32(q_b)/sqrt(32), c[idx] >.
// The kernel therefore rotates the query once (q~ = sigma .* H32(q_b)/sqrt(32)), scores
// tokens with a plain code -> centroid lookup, accumulates  sum_t p_t |s_t| c[idx_t]  in the
// rotated domain, and the merge kernel applies one inverse rotation per output block.
// The reference instead runs a 32-point butterfly per key and per value.
//
// One CTA serves one KV head and one partition of the sequence for ALL query heads of the
// GQA group, so packed K/V bytes are fetched from HBM once (the reference launches one CTA
// per query head, tq_attention_kernel.cu:90-93).  Each warp owns whole tokens; there is no
// block-wide barrier inside the token loop.
#include <float.h>

#include <mutex>

#include "tqb_common.cuh"
#include "tqb_merge.cuh"

namespace tqb {

int block_cfg_check(int bits, int head_dim, int norm_mode);
int launch_decode_mma(const tqb_decode_params* p, int num_partitions, float* partial_out, float* partial_max,
                      float* partial_sum, float sign_mag, unsigned* counters, bool counters_clean, cudaStream_t s,
                      const int* gate = nullptr, int gate_want = 0, const float* dev_signs = nullptr, int alias_heads = 0,
                      const PeerPush* peer = nullptr, float* group_area = nullptr);

int launch_chunk_umma(const tqb_decode_params* p, int q_len, cudaStream_t s);

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kHeadTile = 8;  // query heads handled per pass over the partition

struct DecodeArgs {
    const void* q;
    const uint8_t* k_idx;
    const uint16_t* k_sc;
    const uint8_t* v_idx;
    const uint16_t* v_sc;
    float* partial_out;  // [hq, P, D]  rotated domain, un-normalised
    float* partial_max;  // [hq, P]
    float* partial_sum;  // [hq, P]
    const uint8_t* qjl_signs;
    const uint16_t* qjl_norms;
    const float* rq;
    const float* dev_codebook;  // reference entry point: caller's tables on the device
    const float* dev_signs;
    int qjl_enabled;
    int hq, hkv, head_dim, nblk, bits, packed_dim;
    int kv_len, kv_stride, num_partitions, part_size;
    int outlier_mode;  // 0 all normal, 1 all outlier, 2 by sign of the scale
    float softmax_scale;
    float sign_mag;
    const int* gate;     // reference entry point: run only if *gate == 0 (the caller's tables are not the standard ones)
    // causal chunk: grid head x = query position x / alias_heads on cache head x % alias_heads with
    // kv_len0 + x / alias_heads tokens (0: off)
    int alias_heads, kv_len0;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 32-point butterfly with one element per lane.
__device__ __forceinline__ float wht32_lane(float v, int lane) {
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
        float other = __shfl_xor_sync(0xffffffffu, v, h);
        v = (lane & h) ? (other - v) : (v + other);
    }
    return v;
}

template <typename QT, int NB>
__global__ void __launch_bounds__(kThreads)
decode_general_kernel(DecodeArgs a, Codebook normal, Codebook outlier) {
    if (a.gate != nullptr && *a.gate != 0) return;   // a tensor-core kernel of the same call does the work
    extern __shared__ float smem[];
    const int D = a.head_dim;
    const int g = a.hq / a.hkv;
    float* s_q = smem;                                // [kHeadTile][D]
    float* s_rq = s_q + kHeadTile * D;                // [kHeadTile][D]
    float* s_c = s_rq + kHeadTile * D;                // [2][16]
    float* s_sign = s_c + 32;                         // [32]
    float* s_m = s_sign + 32;                         // [kWarps][kHeadTile]
    float* s_l = s_m + kWarps * kHeadTile;            // [kWarps][kHeadTile]
    float* s_o = s_l + kWarps * kHeadTile;            // [kWarps][kHeadTile][D]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kvh = blockIdx.x, part = blockIdx.y;
    const int nwords = a.packed_dim >> 2;
    const int bits = a.bits;
    const uint32_t cmask = (1u << bits) - 1u;

    if (tid < 16) {
        s_c[tid] = normal.c[tid];
        s_c[16 + tid] = a.dev_codebook ? (tid < (1 << bits) ? a.dev_codebook[tid] : 0.0f) : outlier.c[tid];
    }
    if (tid < 32) {
        const uint32_t neg = 0xB1A6D4B2u;  // src/cache/precomputed/rotation.rs:16-20
        s_sign[tid] = a.dev_signs ? a.dev_signs[tid] : (((neg >> tid) & 1u) ? -a.sign_mag : a.sign_mag);
    }
    __syncthreads();

    int kv_len = a.kv_len, cache_head = kvh;
    if (a.alias_heads > 0) {
        const int pos = kvh / a.alias_heads;
        cache_head = kvh - pos * a.alias_heads;
        kv_len = a.kv_len0 + pos;
    }
    const int t0 = part * a.part_size;
    const int t1 = min(t0 + a.part_size, kv_len);
    const float inv_sqrt = 1.0f / sqrtf((float)kBlock);
    const float qjl_c = 1.2533141f * (1.0f / sqrtf((float)D));  // tq_attention_kernel.cu:225

    const size_t row0 = (size_t)cache_head * a.kv_stride;
    const uint32_t* kw = reinterpret_cast<const uint32_t*>(a.k_idx);
    const uint32_t* vw = reinterpret_cast<const uint32_t*>(a.v_idx);

    for (int h0 = 0; h0 < g; h0 += kHeadTile) {
        const int gt = min(kHeadTile, g - h0);
        __syncthreads();
        // rotate the queries of this tile once: (head, block) pairs round-robin over warps
        for (int u = warp; u < gt * a.nblk; u += kWarps) {
            const int hh = u / a.nblk, b = u - hh * a.nblk;
            const int head = kvh * g + h0 + hh;
            float v = to_f32<QT>(reinterpret_cast<const QT*>(a.q)[(size_t)head * D + b * 32 + lane]);
            v = wht32_lane(v, lane);
            s_q[hh * D + b * 32 + lane] = (v * inv_sqrt) * s_sign[lane];
            if (a.qjl_enabled) s_rq[hh * D + b * 32 + lane] = a.rq[(size_t)head * D + b * 32 + lane];
        }
        __syncthreads();

        float m[kHeadTile], l[kHeadTile], o[kHeadTile][NB];
#pragma unroll
        for (int hh = 0; hh < kHeadTile; ++hh) {
            m[hh] = -FLT_MAX;
            l[hh] = 0.0f;
#pragma unroll
            for (int b = 0; b < NB; ++b) o[hh][b] = 0.0f;
        }

        for (int t = t0 + warp; t < t1; t += kWarps) {
            const size_t row = row0 + t;
            const uint32_t kword = lane < nwords ? __ldg(kw + row * nwords + lane) : 0u;
            const uint32_t vword = lane < nwords ? __ldg(vw + row * nwords + lane) : 0u;
            float ksc = 0.0f, vsc = 0.0f;
            if (lane < a.nblk) {
                ksc = f16_bits_to_f32(__ldg(a.k_sc + row * a.nblk + lane));
                vsc = f16_bits_to_f32(__ldg(a.v_sc + row * a.nblk + lane));
            }
            float acc[kHeadTile];
#pragma unroll
            for (int hh = 0; hh < kHeadTile; ++hh) acc[hh] = 0.0f;
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                if (b < a.nblk) {
                    const int bitoff = (b * 32 + lane) * bits;
                    const int wi = bitoff >> 5;
                    const uint32_t w0 = __shfl_sync(0xffffffffu, kword, wi);
                    const uint32_t w1 = __shfl_sync(0xffffffffu, kword, min(wi + 1, 31));
                    uint32_t code = __funnelshift_r(w0, w1, bitoff & 31) & cmask;
                    const float sb = __shfl_sync(0xffffffffu, ksc, b);
                    const int sel = a.outlier_mode == 2 ? (sb < 0.0f ? 1 : 0) : a.outlier_mode;
                    if (sel == 0) code = min(code, (uint32_t)(normal.n - 1));
                    const float kv = s_c[sel * 16 + code] * fabsf(sb);
#pragma unroll
                    for (int hh = 0; hh < kHeadTile; ++hh)
                        if (hh < gt) acc[hh] = fmaf(s_q[hh * D + b * 32 + lane], kv, acc[hh]);
                }
            }
            float corr[kHeadTile];
            float qn = 0.0f;
            if (a.qjl_enabled) {
                // tq_attention_kernel.cu:197-231
                const uint32_t sw = lane < a.nblk
                    ? __ldg(reinterpret_cast<const uint32_t*>(a.qjl_signs) + row * a.nblk + lane) : 0u;
                qn = f16_bits_to_f32(__ldg(a.qjl_norms + row));
#pragma unroll
                for (int hh = 0; hh < kHeadTile; ++hh) corr[hh] = 0.0f;
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    if (b < a.nblk) {
                        const uint32_t w = __shfl_sync(0xffffffffu, sw, b);
                        const float sg = ((w >> lane) & 1u) ? 1.0f : -1.0f;
#pragma unroll
                        for (int hh = 0; hh < kHeadTile; ++hh)
                            if (hh < gt) corr[hh] = fmaf(s_rq[hh * D + b * 32 + lane], sg, corr[hh]);
                    }
                }
            }
            float p[kHeadTile];
#pragma unroll
            for (int hh = 0; hh < kHeadTile; ++hh) {
                if (hh < gt) {
                    float s = warp_sum(acc[hh]) * a.softmax_scale;
                    if (a.qjl_enabled) s += (warp_sum(corr[hh]) * (qn * qjl_c)) * a.softmax_scale;
                    const float mn = fmaxf(m[hh], s);
                    const float resc = expf(m[hh] - mn);
                    p[hh] = expf(s - mn);
                    l[hh] = l[hh] * resc + p[hh];
                    m[hh] = mn;
#pragma unroll
                    for (int b = 0; b < NB; ++b) o[hh][b] *= resc;
                }
            }
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                if (b < a.nblk) {
                    const int bitoff = (b * 32 + lane) * bits;
                    const int wi = bitoff >> 5;
                    const uint32_t w0 = __shfl_sync(0xffffffffu, vword, wi);
                    const uint32_t w1 = __shfl_sync(0xffffffffu, vword, min(wi + 1, 31));
                    uint32_t code = __funnelshift_r(w0, w1, bitoff & 31) & cmask;
                    const float sb = __shfl_sync(0xffffffffu, vsc, b);
                    const int sel = a.outlier_mode == 2 ? (sb < 0.0f ? 1 : 0) : a.outlier_mode;
                    if (sel == 0) code = min(code, (uint32_t)(normal.n - 1));
                    const float vv = s_c[sel * 16 + code] * fabsf(sb);
#pragma unroll
                    for (int hh = 0; hh < kHeadTile; ++hh)
                        if (hh < gt) o[hh][b] = fmaf(p[hh], vv, o[hh][b]);
                }
            }
        }

        // merge the four warps' online-softmax states
#pragma unroll
        for (int hh = 0; hh < kHeadTile; ++hh) {
            if (hh < gt) {
                if (lane == 0) {
                    s_m[warp * kHeadTile + hh] = m[hh];
                    s_l[warp * kHeadTile + hh] = l[hh];
                }
#pragma unroll
                for (int b = 0; b < NB; ++b)
                    if (b < a.nblk) s_o[(warp * kHeadTile + hh) * D + b * 32 + lane] = o[hh][b];
            }
        }
        __syncthreads();
        for (int u = warp; u < gt * a.nblk; u += kWarps) {
            const int hh = u / a.nblk, b = u - hh * a.nblk;
            float M = -FLT_MAX;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w * kHeadTile + hh]);
            float L = 0.0f, O = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float e = expf(s_m[w * kHeadTile + hh] - M);
                L = fmaf(s_l[w * kHeadTile + hh], e, L);
                O = fmaf(s_o[(w * kHeadTile + hh) * D + b * 32 + lane], e, O);
            }
            const int head = kvh * g + h0 + hh;
            const size_t pi = (size_t)head * a.num_partitions + part;
            a.partial_out[pi * D + b * 32 + lane] = O;
            if (b == 0 && lane == 0) {
                a.partial_max[pi] = M;
                a.partial_sum[pi] = L;
            }
        }
    }
}

// Log-sum-exp merge of partitions fused with the single inverse rotation of the output (merge_head in
// tqb_merge.cuh).  Grid: one CTA per query head.
__global__ void __launch_bounds__(kThreads) decode_merge_kernel(MergeArgs a) {
    merge_head(a, blockIdx.x, threadIdx.x & 31, threadIdx.x >> 5, kWarps);
}

// Shard merge: partial_out [S, hq, D] un-normalised and already in the output domain,
// partial_lse [S, hq, 2].
// Shard merge: per shard an un-normalised output [hq, D] already in the output domain and (max, sum) pairs
// [hq, 2]; shard s starts at po + s * po_stride and lse + s * lse_stride (floats).
template <typename OT>
__global__ void lse_combine_kernel(const float* __restrict__ po, const float* __restrict__ lse, size_t po_stride,
                                   size_t lse_stride, int S, int hq, int D, OT* __restrict__ out) {
    const int head = blockIdx.x;
    float M = -FLT_MAX;
    for (int s = 0; s < S; ++s) M = fmaxf(M, lse[s * lse_stride + (size_t)head * 2]);
    float L = 0.0f;
    for (int s = 0; s < S; ++s) L += lse[s * lse_stride + (size_t)head * 2 + 1] * expf(lse[s * lse_stride + (size_t)head * 2] - M);
    const float inv_l = L > 0.0f ? 1.0f / L : 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < S; ++s)
            acc = fmaf(po[s * po_stride + (size_t)head * D + d], expf(lse[s * lse_stride + (size_t)head * 2] - M), acc);
        out[(size_t)head * D + d] = from_f32<OT>(acc * inv_l);
    }
}

// Verdict on the caller's device tables: 1 = the MaxNorm codebook of this width and the standard sign pattern,
// 2 = the L2Norm codebook and the standard sign pattern, 0 = anything else.
__global__ void table_gate_kernel(const float* __restrict__ codebook, const float* __restrict__ signs, int n, Codebook std_max,
                                  Codebook std_l2, int* __restrict__ gate) {
    const int lane = threadIdx.x;
    const uint32_t neg = 0xB1A6D4B2u;   // src/cache/precomputed/rotation.rs:16-20
    // the crate uploads rotation_fwd[0] * sqrt(32) (src/cache/pqo.rs:134-138): +-1 up to one f32 rounding
    const float mag = fabsf(signs[0]);
    const bool sign_ok = fabsf(mag - 1.0f) < 1e-6f && signs[lane] == (((neg >> lane) & 1u) ? -mag : mag);
    const bool is_max = lane >= n || codebook[lane] == std_max.c[lane];
    const bool is_l2 = lane >= n || codebook[lane] == std_l2.c[lane];
    const bool s_ok = __all_sync(0xffffffffu, sign_ok);
    const bool m_ok = __all_sync(0xffffffffu, is_max);
    const bool l_ok = __all_sync(0xffffffffu, is_l2);
    if (lane == 0) *gate = !s_ok ? 0 : (m_ok ? 1 : (l_ok ? 2 : 0));
}

// Gate words: a ring of slots in a static device array, one per call in flight (the ring is far longer than
// any realistic number of concurrent calls).
constexpr int kGateSlots = 4096;
__device__ int g_gate_slots[kGateSlots];
std::mutex g_gate_mutex;
int* g_gate_base[64] = {};
unsigned g_gate_next = 0;

int gate_slot(int** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TQB_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_gate_mutex);
    if (!g_gate_base[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_gate_slots) != cudaSuccess || !ptr) return TQB_ERR_CUDA;
        g_gate_base[dev] = static_cast<int*>(ptr);
    }
    *out = g_gate_base[dev] + (g_gate_next++ % kGateSlots);
    return TQB_OK;
}

size_t general_smem_bytes(int D) {
    return sizeof(float) * ((size_t)2 * kHeadTile * D + 64 + 2 * kWarps * kHeadTile + (size_t)kWarps * kHeadTile * D);
}

template <typename QT, int NB>
int launch_general(const DecodeArgs& a, const Codebook& n, const Codebook& o, cudaStream_t s) {
    const size_t smem = general_smem_bytes(a.head_dim);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(decode_general_kernel<QT, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) { set_cuda_error(e); return TQB_ERR_CUDA; }
    }
    dim3 grid(a.hkv, a.num_partitions);
    decode_general_kernel<QT, NB><<<grid, kThreads, smem, s>>>(a, n, o);
    return check_launch(s);
}

template <typename QT>
int launch_general_nb(const DecodeArgs& a, const Codebook& n, const Codebook& o, cudaStream_t s) {
    if (a.nblk <= 2) return launch_general<QT, 2>(a, n, o, s);
    if (a.nblk <= 4) return launch_general<QT, 4>(a, n, o, s);
    return launch_general<QT, 8>(a, n, o, s);
}

int launch_merge(const MergeArgs& m, int hq, cudaStream_t s) {
    decode_merge_kernel<<<hq, kThreads, 0, s>>>(m);
    return check_launch(s);
}

inline float cpu_sign_magnitude() {
    volatile float inv = 1.0f / sqrtf(32.0f);
    volatile float s = sqrtf(32.0f);
    return inv * s;
}

int run_merge(const DecodeArgs& a, void* out, int out_dtype, float* lse_out, cudaStream_t s);

int run_decode(DecodeArgs& a, const Codebook& cn, const Codebook& co, int q_dtype, void* out, int out_dtype,
               float* lse_out, cudaStream_t s, bool partials_only = false) {
    int st;
    if (q_dtype == TQB_F32) st = launch_general_nb<float>(a, cn, co, s);
    else if (q_dtype == TQB_F16) st = launch_general_nb<__half>(a, cn, co, s);
    else st = launch_general_nb<__nv_bfloat16>(a, cn, co, s);
    if (st != TQB_OK || partials_only) return st;
    return run_merge(a, out, out_dtype, lse_out, s);
}

int run_merge(const DecodeArgs& a, void* out, int out_dtype, float* lse_out, cudaStream_t s) {
    MergeArgs m{};
    m.partial_out = a.partial_out;
    m.partial_max = a.partial_max;
    m.partial_sum = a.partial_sum;
    m.dev_signs = a.dev_signs;
    m.out = out;
    m.lse_out = lse_out;
    m.head_dim = a.head_dim;
    m.nblk = a.nblk;
    m.num_partitions = a.num_partitions;
    m.rotate = 1;
    m.sign_mag = a.sign_mag;
    m.out_dtype = out_dtype;
    return launch_merge(m, a.hq, s);
}

}  // namespace
}  // namespace tqb

using namespace tqb;

extern "C" {

int32_t tqb_decode_num_partitions(int32_t num_kv_heads, int32_t kv_len) {
    if (num_kv_heads <= 0 || kv_len <= 0) return 1;
    // Measured on B200 (tensor-core kernels, 8 to 2048 KV heads, 2K to 128K tokens): the best grids hold
    // between one and two times the 148 x 4 CTAs that are resident at once - 512 heads x 8192 tokens run 4 %
    // faster split in 2 than in 4, and 7 % faster than unsplit (which leaves 14 % of the slots empty); more,
    // shorter partitions pay the per-CTA query prologue and merge again.  So: two residencies' worth of CTAs
    // while a partition keeps at least 768 tokens, else one residency's worth, never below 64 tokens.  One
    // residency's worth is rounded DOWN: 64 heads x 10 partitions are 640 CTAs for 592 slots, and the 48 left over
    // start when the first ones end - the launch takes twice as long as with 9 partitions.
    const long long resident = 148 * 4;
    const int max_p = (kv_len + 63) / 64;
    const long long p1 = resident / num_kv_heads;
    long long p2 = 2 * resident / num_kv_heads;
    if (p2 < 1) p2 = 1;
    // (two residencies only while they merge in one level: 8 heads x 131,072 tokens take 85 us with 148 partitions and
    // 76 us with 74 or 55, whose merge tail is half as long)
    long long p = (kv_len / p2 >= 768 && p2 <= 2 * kMergeGroup) ? p2 : p1;
    if (p > max_p) p = max_p;
    if (p < 1) p = 1;
    return (int32_t)p;
}

// Partition count for launches made with TQB_DECODE_OVERLAP.  Several such launches are resident at once (the next one
// fills the slots the previous one frees), so a launch need not fill the GPU by itself: fewer, longer partitions pay
// the query prologue and the split-K merge less often.  Measured on B200 (PQO4, 8192 tokens, overlapped chain, us per
// launch): 64 heads: P = 2 or 3 -> 15.0, P = 9 -> 18.3; 128 heads: P = 1 or 2 -> 28.2, P = 4 -> 29.8; 256 heads: P = 1 ->
// 55.5, P = 4 -> 61.1; 512 heads: P = 1 -> 110.5, P = 2 -> 112.5.  So: about one CTA per SM and launch, partitions of
// at least 768 tokens.
int32_t tqb_decode_num_partitions_overlapped(int32_t num_kv_heads, int32_t kv_len) {
    if (num_kv_heads <= 0 || kv_len <= 0) return 1;
    long long p = 148 / num_kv_heads;
    const long long cap = kv_len / 768;
    if (p > cap) p = cap;
    if (p < 1) p = 1;
    return (int32_t)p;
}

// Scratch layout: [merge tickets: (1 + G) u32 per query head, rounded up to 256 bytes][partial out [hq, P, D]]
// [partial max [hq, P]][partial sum [hq, P]][group partials: out [hq, G, D], max [hq, G], sum [hq, G]], where
// G = merge_groups(P) is the number of partition groups of the two-level merge (0 up to kMergeGroup partitions).
static size_t ticket_bytes(int32_t num_q_heads, int32_t num_partitions) {
    return (sizeof(unsigned) * (size_t)num_q_heads * (1 + merge_groups(num_partitions)) + 255) / 256 * 256;
}

size_t tqb_decode_scratch_bytes(int32_t num_q_heads, int32_t head_dim, int32_t num_partitions) {
    if (num_q_heads <= 0 || head_dim <= 0 || num_partitions <= 0) return 0;
    return ticket_bytes(num_q_heads, num_partitions) +
           sizeof(float) * (size_t)num_q_heads * (num_partitions + merge_groups(num_partitions)) * ((size_t)head_dim + 2);
}

// alias_heads > 0: p is a causal chunk folded into heads (see tqb_chunk_attention)
static int decode_impl(const tqb_decode_params* p, int alias_heads, tqb_stream_t stream, const PeerPush* peer = nullptr) {
    if (!p) return TQB_ERR_NULL_POINTER;
    int st = block_cfg_check(p->bits, p->head_dim, p->norm_mode);
    if (st != TQB_OK) return st;
    if (p->head_dim > 256) return TQB_ERR_UNSUPPORTED;
    if (p->num_q_heads <= 0 || p->num_kv_heads <= 0 || p->num_q_heads % p->num_kv_heads != 0)
        return TQB_ERR_INVALID_ARGUMENT;
    if (p->kv_len < 0 || p->kv_len > p->kv_stride) return TQB_ERR_RANGE_OUT_OF_BOUNDS;
    if (!p->q || !p->out || !p->scratch) return TQB_ERR_NULL_POINTER;
    if (p->kv_len > 0 && (!p->k_indices || !p->k_scales || !p->v_indices || !p->v_scales)) return TQB_ERR_NULL_POINTER;
    if (p->qjl_enabled && (!p->qjl_signs || !p->qjl_norms || !p->rq)) return TQB_ERR_NULL_POINTER;
    if (p->lse_out && p->out_dtype != TQB_F32) return TQB_ERR_INVALID_ARGUMENT;
    if ((p->append_k == nullptr) != (p->append_v == nullptr)) return TQB_ERR_NULL_POINTER;
    if (p->append_k != nullptr && p->kv_len < 1) return TQB_ERR_RANGE_OUT_OF_BOUNDS;
    if (((uintptr_t)p->k_indices % 4) || ((uintptr_t)p->v_indices % 4) || ((uintptr_t)p->scratch % 16) ||
        ((uintptr_t)p->qjl_signs % 4))
        return TQB_ERR_MISALIGNED;
    int P = p->num_partitions > 0 ? p->num_partitions : tqb_decode_num_partitions(p->num_kv_heads, p->kv_len);
    if (p->scratch_bytes < tqb_decode_scratch_bytes(p->num_q_heads, p->head_dim, P)) return TQB_ERR_INVALID_ARGUMENT;
    Codebook cn, co;
    if (!block_codebook(p->bits - 1, p->norm_mode, cn) || !block_codebook(p->bits, p->norm_mode, co))
        return TQB_ERR_UNSUPPORTED_BITS;
    DecodeArgs a{};
    a.q = p->q;
    a.k_idx = p->k_indices; a.k_sc = p->k_scales; a.v_idx = p->v_indices; a.v_sc = p->v_scales;
    unsigned* tickets = reinterpret_cast<unsigned*>(p->scratch);
    float* sc = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(p->scratch) + ticket_bytes(p->num_q_heads, P));
    a.partial_out = sc;
    a.partial_max = sc + (size_t)p->num_q_heads * P * p->head_dim;
    a.partial_sum = a.partial_max + (size_t)p->num_q_heads * P;
    float* group_area = a.partial_sum + (size_t)p->num_q_heads * P;
    a.qjl_signs = p->qjl_signs; a.qjl_norms = p->qjl_norms; a.rq = p->rq; a.qjl_enabled = p->qjl_enabled ? 1 : 0;
    a.dev_codebook = nullptr; a.dev_signs = nullptr;
    a.hq = p->num_q_heads; a.hkv = p->num_kv_heads; a.head_dim = p->head_dim; a.nblk = p->head_dim / kBlock;
    a.bits = p->bits; a.packed_dim = p->head_dim * p->bits / 8;
    a.kv_len = p->kv_len; a.kv_stride = p->kv_stride; a.num_partitions = P;
    a.alias_heads = alias_heads;
    a.kv_len0 = alias_heads > 0 ? p->kv_len - p->num_kv_heads / alias_heads + 1 : p->kv_len;
    a.part_size = ((p->kv_len + P - 1) / P + kWarps - 1) / kWarps * kWarps;
    if (a.part_size < kWarps) a.part_size = kWarps;
    const int ob = p->outlier_blocks < 0 || p->outlier_blocks >= a.nblk ? a.nblk : p->outlier_blocks;
    a.outlier_mode = ob >= a.nblk ? 1 : (ob == 0 ? 0 : 2);
    a.softmax_scale = p->softmax_scale;
    a.sign_mag = cpu_sign_magnitude();
    const bool partials_only = (p->flags & TQB_DECODE_PARTIALS_ONLY) != 0;
    tqb_decode_params local = *p;
    // The append as a launch of its own (shapes the tensor-core kernels do not cover).
    auto append_separately = [&]() -> int {
        int rc = tqb_block_quantize_pair(p->bits, p->head_dim, p->norm_mode, p->outlier_blocks, p->append_k, p->append_v,
                                         p->q_dtype, p->num_kv_heads, 0, const_cast<uint8_t*>(p->k_indices),
                                         const_cast<uint16_t*>(p->k_scales), const_cast<uint8_t*>(p->v_indices),
                                         const_cast<uint16_t*>(p->v_scales), 1, p->kv_stride, p->kv_len - 1, stream);
        local.append_k = local.append_v = nullptr;
        return rc;
    };
    if (!(p->flags & TQB_DECODE_FORCE_GENERAL)) {
        // tensor-core kernels for the shapes they cover; everything else takes the general kernel
        // (the merge runs inside the kernel, in the CTA that finishes a KV head last)
        st = launch_decode_mma(&local, P, a.partial_out, a.partial_max, a.partial_sum, a.sign_mag,
                               partials_only ? nullptr : tickets, (p->flags & TQB_DECODE_TICKETS_ZERO) != 0, as_stream(stream),
                               nullptr, 0, nullptr, alias_heads, peer, group_area);
        if (peer != nullptr) return st;   // the push exists in the tensor-core kernels only
        if (st == TQB_ERR_UNSUPPORTED && local.append_k != nullptr) {
            st = append_separately();
            if (st != TQB_OK) return st;
            st = launch_decode_mma(&local, P, a.partial_out, a.partial_max, a.partial_sum, a.sign_mag,
                                   partials_only ? nullptr : tickets, (p->flags & TQB_DECODE_TICKETS_ZERO) != 0, as_stream(stream),
                                   nullptr, 0, nullptr, 0, nullptr, group_area);
        }
        if (st != TQB_ERR_UNSUPPORTED) return st;
    }
    if (local.append_k != nullptr) {
        st = append_separately();
        if (st != TQB_OK) return st;
    }
    return run_decode(a, cn, co, p->q_dtype, p->out, p->out_dtype, p->lse_out, as_stream(stream), partials_only);
}

int tqb_decode_attention(const tqb_decode_params* p, tqb_stream_t stream) { return decode_impl(p, 0, stream); }
}  // extern "C"
namespace tqb {
int decode_with_peer_push(const tqb_decode_params* p, const PeerPush& push, tqb_stream_t stream) {
    if (p && (p->append_k || p->flags & (TQB_DECODE_PARTIALS_ONLY | TQB_DECODE_FORCE_GENERAL))) return TQB_ERR_INVALID_ARGUMENT;
    return decode_impl(p, 0, stream, &push);
}
}  // namespace tqb
extern "C" {

// Causal attention of a chunk of q_len consecutive query tokens over the packed cache.  Query position i is
// run as one more "sequence" of a batched decode whose cache rows are those of the one real sequence: grid
// head (i, kv head) reads cache head `kv head` and stops after kv_len - q_len + i + 1 tokens.  The chunk
// re-reads the cache once per query position, mostly from L2.
int tqb_chunk_attention(const tqb_decode_params* p, int32_t q_len, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (!p) return TQB_ERR_NULL_POINTER;
    if (q_len <= 0) return TQB_ERR_INVALID_ARGUMENT;
    if (p->append_k != nullptr || p->append_v != nullptr) return TQB_ERR_INVALID_ARGUMENT;   // the chunk is stored first
    if (p->kv_len < q_len) return TQB_ERR_RANGE_OUT_OF_BOUNDS;
    if (p->num_q_heads <= 0 || p->num_kv_heads <= 0) return TQB_ERR_INVALID_ARGUMENT;
    if ((long long)p->num_q_heads * q_len > (1 << 24)) return TQB_ERR_TOO_LARGE;
    if (!(p->flags & (TQB_DECODE_FORCE_GENERAL | TQB_DECODE_FOLD_CHUNK | TQB_DECODE_PARTIALS_ONLY))) {
        // the dedicated kernel on the tcgen05 tensor cores, for the shapes it covers
        if (!p->q || !p->out) return TQB_ERR_NULL_POINTER;
        if (p->num_q_heads % p->num_kv_heads != 0) return TQB_ERR_INVALID_ARGUMENT;
        if (p->kv_len > p->kv_stride) return TQB_ERR_RANGE_OUT_OF_BOUNDS;
        if (!p->k_indices || !p->k_scales || !p->v_indices || !p->v_scales) return TQB_ERR_NULL_POINTER;
        const int st = launch_chunk_umma(p, q_len, as_stream(stream));
        if (st != TQB_ERR_UNSUPPORTED) return st;
    }
    tqb_decode_params f = *p;
    f.flags &= ~TQB_DECODE_FOLD_CHUNK;
    f.num_q_heads = p->num_q_heads * q_len;
    f.num_kv_heads = p->num_kv_heads * q_len;
    return decode_impl(&f, p->num_kv_heads, stream);
}

static int lse_combine_impl(const float* po, const float* lse, size_t po_stride, size_t lse_stride, int32_t num_shards,
                            int32_t num_q_heads, int32_t head_dim, void* out, int32_t out_dtype, tqb_stream_t stream) {
    if (!po || !lse || !out) return TQB_ERR_NULL_POINTER;
    if (num_shards <= 0 || num_q_heads <= 0 || head_dim <= 0) return TQB_ERR_INVALID_ARGUMENT;
    cudaStream_t s = as_stream(stream);
    if (out_dtype == TQB_F32)
        lse_combine_kernel<float><<<num_q_heads, 128, 0, s>>>(po, lse, po_stride, lse_stride, num_shards, num_q_heads, head_dim, (float*)out);
    else if (out_dtype == TQB_F16)
        lse_combine_kernel<__half><<<num_q_heads, 128, 0, s>>>(po, lse, po_stride, lse_stride, num_shards, num_q_heads, head_dim, (__half*)out);
    else if (out_dtype == TQB_BF16)
        lse_combine_kernel<__nv_bfloat16><<<num_q_heads, 128, 0, s>>>(po, lse, po_stride, lse_stride, num_shards, num_q_heads, head_dim, (__nv_bfloat16*)out);
    else return TQB_ERR_INVALID_ARGUMENT;
    return check_launch(s);
}

int tqb_lse_combine(const float* partial_out, const float* partial_lse, int32_t num_shards, int32_t num_q_heads,
                    int32_t head_dim, void* out, int32_t out_dtype, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    return lse_combine_impl(partial_out, partial_lse, (size_t)num_q_heads * head_dim, (size_t)num_q_heads * 2, num_shards,
                            num_q_heads, head_dim, out, out_dtype, stream);
}

int tqb_lse_combine_packed(const float* gathered, int32_t num_shards, int32_t num_q_heads, int32_t head_dim, void* out,
                           int32_t out_dtype, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (!gathered) return TQB_ERR_NULL_POINTER;
    const size_t rec = (size_t)num_q_heads * ((size_t)head_dim + 2);
    return lse_combine_impl(gathered, gathered + (size_t)num_q_heads * head_dim, rec, rec, num_shards, num_q_heads, head_dim,
                            out, out_dtype, stream);
}

int tqb_fused_attention(const float* q, const uint8_t* k_indices, const uint16_t* k_scales, const uint8_t* v_indices,
                        const uint16_t* v_scales, const float* codebook, const float* sign_pattern, float* output,
                        float* partial_out, float* partial_max, float* partial_sum, const uint8_t* qjl_signs,
                        const uint16_t* qjl_residual_norms, const float* rq, int32_t qjl_enabled,
                        int32_t num_attention_heads, int32_t num_kv_heads, int32_t head_dim, int32_t kv_len,
                        int32_t kv_stride, int32_t packed_dim, int32_t num_qblocks, int32_t bits, float softmax_scale,
                        int32_t num_partitions, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (kv_len == 0 || num_kv_heads == 0) return TQB_OK;  // tq_attention_kernel.cu:366
    if (bits < 2 || bits > 4) return TQB_ERR_UNSUPPORTED_BITS;
    if (head_dim <= 0 || head_dim % kBlock != 0) return TQB_ERR_INVALID_DIMENSION;
    if (head_dim > 256) return TQB_ERR_UNSUPPORTED;  // the reference itself stops at 8 blocks (TQ_NUM_WARPS)
    if (num_qblocks != head_dim / kBlock || packed_dim != head_dim * bits / 8) return TQB_ERR_DIMENSION_MISMATCH;
    if (num_attention_heads <= 0 || num_kv_heads < 0 || num_attention_heads % num_kv_heads != 0 || num_partitions <= 0)
        return TQB_ERR_INVALID_ARGUMENT;
    if (kv_len < 0 || kv_len > kv_stride) return TQB_ERR_RANGE_OUT_OF_BOUNDS;
    if (!q || !k_indices || !k_scales || !v_indices || !v_scales || !codebook || !sign_pattern || !output ||
        !partial_out || !partial_max || !partial_sum)
        return TQB_ERR_NULL_POINTER;
    if (qjl_enabled && (!qjl_signs || !qjl_residual_norms || !rq)) return TQB_ERR_NULL_POINTER;
    if (((uintptr_t)k_indices % 4) || ((uintptr_t)v_indices % 4) || ((uintptr_t)qjl_signs % 4)) return TQB_ERR_MISALIGNED;
    Codebook dummy{};
    dummy.n = 1 << bits;
    DecodeArgs a{};
    a.q = q;
    a.k_idx = k_indices; a.k_sc = k_scales; a.v_idx = v_indices; a.v_sc = v_scales;
    a.partial_out = partial_out; a.partial_max = partial_max; a.partial_sum = partial_sum;
    a.qjl_signs = qjl_signs; a.qjl_norms = qjl_residual_norms; a.rq = rq; a.qjl_enabled = qjl_enabled ? 1 : 0;
    a.dev_codebook = codebook; a.dev_signs = sign_pattern;
    a.hq = num_attention_heads; a.hkv = num_kv_heads; a.head_dim = head_dim; a.nblk = num_qblocks;
    a.bits = bits; a.packed_dim = packed_dim;
    a.kv_len = kv_len; a.kv_stride = kv_stride; a.num_partitions = num_partitions;
    a.part_size = ((kv_len + num_partitions - 1) / num_partitions + kWarps - 1) / kWarps * kWarps;
    a.outlier_mode = 1;  // the caller's codebook decodes every block
    a.softmax_scale = softmax_scale;
    a.sign_mag = 1.0f;
    cudaStream_t s = as_stream(stream);
    // The tables arrive as device pointers, so the host cannot know whether they are the crate's own
    // (src/cache/precomputed/codebooks.rs, rotation.rs) - the only ones the tensor-core kernels decode.  A
    // one-warp kernel compares them on the device and leaves a verdict in a gate word; the tensor-core
    // kernel(s) and the general kernel are all launched and every CTA of those whose verdict it is not
    // returns at once.  No host synchronisation, safe under stream capture.
    const bool fast_shape = head_dim == 128 && !qjl_enabled && (bits == 3 || bits == 4) &&
                            num_attention_heads / num_kv_heads <= 8;
    Codebook std_max{}, std_l2{};
    int* gate = nullptr;
    if (fast_shape && block_codebook(bits, TQB_MAXNORM, std_max) && block_codebook(bits, TQB_L2NORM, std_l2) &&
        gate_slot(&gate) == TQB_OK) {
        table_gate_kernel<<<1, 32, 0, s>>>(codebook, sign_pattern, 1 << bits, std_max, std_l2, gate);
        tqb_decode_params p{};
        p.q = q; p.k_indices = k_indices; p.k_scales = k_scales; p.v_indices = v_indices; p.v_scales = v_scales;
        p.out = output; p.q_dtype = TQB_F32; p.out_dtype = TQB_F32; p.bits = bits; p.head_dim = head_dim;
        p.outlier_blocks = -1; p.num_q_heads = num_attention_heads; p.num_kv_heads = num_kv_heads;
        p.kv_len = kv_len; p.kv_stride = kv_stride; p.num_partitions = num_partitions; p.softmax_scale = softmax_scale;
        bool any_fast = false;
        for (int mode = 0; mode < 2; ++mode) {   // verdict 1: MaxNorm tables, verdict 2: L2Norm tables
            p.norm_mode = mode == 0 ? TQB_MAXNORM : TQB_L2NORM;
            const int st = launch_decode_mma(&p, num_partitions, partial_out, partial_max, partial_sum, 1.0f, nullptr, true, s,
                                             gate, mode + 1, sign_pattern);
            if (st == TQB_OK) any_fast = true;
            else if (st != TQB_ERR_UNSUPPORTED) return st;
        }
        if (any_fast) a.gate = gate;
    }
    return run_decode(a, dummy, dummy, TQB_F32, output, TQB_F32, nullptr, s);
}

void tq_fused_attention(const float* q, const uint8_t* k_indices, const uint16_t* k_scales, const uint8_t* v_indices,
                        const uint16_t* v_scales, const float* codebook, const float* sign_pattern, float* output,
                        float* partial_out, float* partial_max, float* partial_sum, const uint8_t* qjl_signs,
                        const uint16_t* qjl_residual_norms, const float* rq, int32_t qjl_enabled,
                        int32_t num_attention_heads, int32_t num_kv_heads, int32_t head_dim, int32_t kv_len,
                        int32_t kv_stride, int32_t packed_dim, int32_t num_qblocks, int32_t bits, float softmax_scale,
                        int32_t num_partitions, tqb_stream_t stream) {
    (void)tqb_fused_attention(q, k_indices, k_scales, v_indices, v_scales, codebook, sign_pattern, output, partial_out,
                              partial_max, partial_sum, qjl_signs, qjl_residual_norms, rq, qjl_enabled,
                              num_attention_heads, num_kv_heads, head_dim, kv_len, kv_stride, packed_dim, num_qblocks,
                              bits, softmax_scale, num_partitions, stream);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Decode attention with library-resident scratch (no allocation by anybody).
//
// The split-K partials of decode attention normally live in a buffer the caller allocates.  Some
// callers cannot do that: an inference engine that has handed every free byte of device memory to
// its own pool at start-up (a later cudaMalloc fails), or a serving loop that must not take the
// device-wide synchronisation that cudaMalloc / cudaFree imply.  For them the partials go into the
// fixed array below, which every GPU that loads this library holds from load until exit.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;   // 8 MiB: e.g. 2048 query heads x 8 partitions at head_dim 128
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_addr[kMaxDevices] = {};   // device address of g_decode_scratch, per device

// The array's name is only a host-side handle; the address a kernel can use is obtained once per
// device (with that device current) through cudaGetSymbolAddress.
int static_scratch_address(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { tqb::set_cuda_error(e); return TQB_ERR_CUDA; }
    if (dev < 0 || dev >= kMaxDevices) return TQB_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_decode_scratch);
        if (e != cudaSuccess || ptr == nullptr) { tqb::set_cuda_error(e); return TQB_ERR_CUDA; }
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return TQB_OK;
}

}  // namespace

extern "C" {

size_t tqb_decode_static_scratch_capacity(void) { return kStaticScratchBytes; }

int tqb_decode_attention_static(const tqb_decode_params* p, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (!p) return TQB_ERR_NULL_POINTER;
    if (p->num_q_heads <= 0 || p->num_kv_heads <= 0 || p->head_dim <= 0) return TQB_ERR_INVALID_ARGUMENT;
    // the partials would stay in the library's array, whose address the caller cannot obtain
    if (p->flags & TQB_DECODE_PARTIALS_ONLY) return TQB_ERR_INVALID_ARGUMENT;
    const int P = p->num_partitions > 0 ? p->num_partitions : tqb_decode_num_partitions(p->num_kv_heads, p->kv_len);
    const size_t need = tqb_decode_scratch_bytes(p->num_q_heads, p->head_dim, P);
    if (need == 0 || need > kStaticScratchBytes) return TQB_ERR_TOO_LARGE;   // refuse, never spill past the array
    void* scratch = nullptr;
    int st = static_scratch_address(&scratch);
    if (st != TQB_OK) return st;
    tqb_decode_params q = *p;
    q.scratch = scratch;
    q.scratch_bytes = kStaticScratchBytes;
    q.num_partitions = P;
    // Every (head, partition) slot that the merge reads is written by the split-K pass of the same
    // call, and the merge tickets are cleared on the stream before the kernel (their area may hold an
    // earlier call's partials when the head count changes), so stale contents are never read.
    q.flags &= ~TQB_DECODE_TICKETS_ZERO;
    return tqb_decode_attention(&q, stream);
}

}  // extern "C"
