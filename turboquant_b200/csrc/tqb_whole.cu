// Whole-vector ("core crate") kernels: PolarQuant quantize / dequantize, the QJL sign
// sketch, query projections, inner-product scores and weighted values.
//
// Element e of a vector of dimension d = 32*EPL lives in lane e % 32, slot e / 32.  The
// Walsh-Hadamard stages run in the reference's order h = 1, 2, 4, ... (src/rotation.rs:22-40):
// h < 32 through __shfl_xor, h >= 32 between the slots of a lane.  Every stage pairs the
// same two operands as the scalar loop, so the transform is bit-identical to it.
//
// The two order-sensitive reductions of the reference -- the L2 norm (src/quantize.rs:51-53)
// and each Rademacher row product (src/qjl.rs:196-208) -- are sequential f32 sums.  They are
// kept sequential: a warp stages 32 vectors in shared memory and lane r sums vector r, so all
// lanes stay busy while each sum keeps the reference's left-to-right order.
#include <float.h>

#include "tqb_common.cuh"
#include "tqb_pqo_quant.cuh"
#include <type_traits>

namespace tqb {
namespace {

constexpr int kTile = 32;  // vectors per warp tile

// src/rotation.rs:47-70: the multiplier is odd, so the hash's low bit is the parity of seed+i.
__device__ __forceinline__ float sign_of(uint64_t seed, int e) {
    return ((seed + (uint64_t)e) & 1ULL) ? -1.0f : 1.0f;
}

template <int EPL>
__device__ __forceinline__ void wht_lanes(float (&v)[EPL], int lane) {
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
        const bool upper = (lane & h) != 0;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            float other = __shfl_xor_sync(0xffffffffu, v[i], h);
            v[i] = upper ? (other - v[i]) : (v[i] + other);
        }
    }
#pragma unroll
    for (int hs = 1; hs < EPL; hs <<= 1) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            if ((i & hs) == 0) {
                float x = v[i], y = v[i + hs];
                v[i] = x + y;
                v[i + hs] = x - y;
            }
        }
    }
}

// Codes of one vector (bytes in shared memory, dim entries) -> packed bytes, eight codes
// (= `bits` bytes) per lane pass.  src/packed/mod.rs:242-309.
__device__ __forceinline__ void pack_codes(const uint8_t* codes, uint8_t* out, int dim, int bits, int lane) {
    for (int g = lane; g < dim / 8; g += 32) {
        uint32_t acc = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc |= (uint32_t)codes[g * 8 + i] << (bits * i);
        for (int b = 0; b < bits; ++b) out[g * bits + b] = (uint8_t)(acc >> (8 * b));
    }
}

// Code of element e from the packed words of one vector, one word per lane.
__device__ __forceinline__ uint32_t code_at(uint32_t word, int e, int bits) {
    const int bitoff = e * bits;
    const int wi = bitoff >> 5;
    const uint32_t w0 = __shfl_sync(0xffffffffu, word, wi);
    const uint32_t w1 = __shfl_sync(0xffffffffu, word, min(wi + 1, 31));
    return __funnelshift_r(w0, w1, bitoff & 31) & ((1u << bits) - 1u);
}

struct WholeArgs {
    const float* x;
    long long n;
    uint8_t* packed;
    uint16_t* scales;
    uint8_t* signs;       // QJL outputs (may be null)
    uint16_t* rnorms;
    const uint32_t* rbits;  // [dim][dim/32]
    int bits;             // polar bits
    int dim;
    int pb;               // packed bytes per vector
    uint64_t seed;
    float inv_sqrt_d;
};

// Sequential Rademacher row products of one vector held in shared memory.
// Lane handles rows lane, lane+32, ...; s_rb has row stride W+1 words.
template <int EPL>
__device__ __forceinline__ void rademacher_rows(const float* vec, const uint32_t* s_rb, int lane, float inv_sqrt_d,
                                                float (&proj)[EPL]) {
    constexpr int W = EPL;
    float s[EPL];
#pragma unroll
    for (int k = 0; k < EPL; ++k) s[k] = 0.0f;
#pragma unroll 1
    for (int cw = 0; cw < W; ++cw) {
        uint32_t rb[EPL];
#pragma unroll
        for (int k = 0; k < EPL; ++k) rb[k] = s_rb[(lane + 32 * k) * (W + 1) + cw];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            const uint32_t val = __float_as_uint(vec[cw * 32 + c]);
#pragma unroll
            for (int k = 0; k < EPL; ++k)
                s[k] = s[k] + __uint_as_float(val ^ ((rb[k] << (31 - c)) & 0x80000000u));
        }
    }
#pragma unroll
    for (int k = 0; k < EPL; ++k) proj[k] = s[k] * inv_sqrt_d;
}

// quantize_vec (src/quantize.rs:142-192) and, with QJL outputs requested,
// quantize_with_qjl (src/qjl.rs:355-377).  One warp per tile of 32 vectors.
template <int EPL, bool QJL>
__global__ void whole_quantize_kernel(WholeArgs a, Codebook cb) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int D = 32 * EPL;
    constexpr int W = EPL;
    const int warps = blockDim.x >> 5;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // layout: [rbits (D*(W+1) words, QJL only)] [boundaries 16] [centroids 16] then per warp:
    // tile [32][D+1] floats, codes [D] bytes, stage [32*pb] bytes
    uint32_t* s_rb = reinterpret_cast<uint32_t*>(smem_raw);
    float* s_b = reinterpret_cast<float*>(s_rb + (QJL ? D * (W + 1) : 0));
    float* s_c = s_b + 16;
    const size_t per_warp = sizeof(float) * kTile * (D + 1) + D + (size_t)kTile * a.pb;
    unsigned char* wbase = reinterpret_cast<unsigned char*>(s_c + 16) + (size_t)warp * ((per_warp + 15) / 16 * 16);
    float* tile = reinterpret_cast<float*>(wbase);
    uint8_t* codes = reinterpret_cast<uint8_t*>(tile + kTile * (D + 1));
    uint8_t* stage = codes + D;

    if (threadIdx.x < 16) {
        s_b[threadIdx.x] = cb.b[threadIdx.x];
        s_c[threadIdx.x] = cb.c[threadIdx.x];
    }
    if (QJL)
        for (int i = threadIdx.x; i < D * W; i += blockDim.x) s_rb[(i / W) * (W + 1) + (i % W)] = a.rbits[i];
    __syncthreads();

    const long long tiles = (a.n + kTile - 1) / kTile;
    for (long long t = (long long)blockIdx.x * warps + warp; t < tiles; t += (long long)gridDim.x * warps) {
        const long long v0 = t * kTile;
        const int nv = (int)min((long long)kTile, a.n - v0);
        // stage the tile (coalesced 128-byte rows)
        for (int r = 0; r < nv; ++r)
#pragma unroll
            for (int i = 0; i < EPL; ++i) tile[r * (D + 1) + lane + 32 * i] = a.x[(v0 + r) * D + lane + 32 * i];
        __syncwarp();
        // l2_norm: lane r sums vector r left to right
        float norm = 0.0f;
        if (lane < nv) {
            float s = 0.0f;
            const float* row = tile + lane * (D + 1);
#pragma unroll 8
            for (int c = 0; c < D; ++c) s = s + row[c] * row[c];
            norm = __fsqrt_rn(s);
        }
        float rnorm_mine = 0.0f;
        for (int r = 0; r < nv; ++r) {
            const float nr = __shfl_sync(0xffffffffu, norm, r);
            const bool tiny = nr < kMinNorm;
            const float inv = __fdiv_rn(1.0f, nr);
            float x[EPL], v[EPL];
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                x[i] = tile[r * (D + 1) + lane + 32 * i];
                float nx = tiny ? 0.0f : x[i] * inv;                 // normalize_inplace, quantize.rs:60-72
                v[i] = nx * sign_of(a.seed, lane + 32 * i);          // rotation.rs:139-142
            }
            wht_lanes<EPL>(v, lane);
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                v[i] = v[i] * a.inv_sqrt_d;
                codes[lane + 32 * i] = (uint8_t)bucket_index_n(v[i], s_b, cb.n);
            }
            __syncwarp();
            pack_codes(codes, stage + (size_t)r * a.pb, D, a.bits, lane);
            if (QJL) {
                // dequantize (quantize.rs:225-239) with the f16-rounded scale, residual, norm, signs
                const float sc = f16_bits_to_f32(f32_to_f16_bits(tiny ? 0.0f : nr));
                float y[EPL];
#pragma unroll
                for (int i = 0; i < EPL; ++i) y[i] = s_c[codes[lane + 32 * i]];
                wht_lanes<EPL>(y, lane);
#pragma unroll
                for (int i = 0; i < EPL; ++i) {
                    float rec = ((y[i] * a.inv_sqrt_d) * sign_of(a.seed, lane + 32 * i)) * sc;
                    tile[r * (D + 1) + lane + 32 * i] = x[i] - rec;  // compute_residual, qjl.rs:213-219
                }
            }
            __syncwarp();
        }
        if (QJL) {
            if (lane < nv) {
                float s = 0.0f;
                const float* row = tile + lane * (D + 1);
#pragma unroll 8
                for (int c = 0; c < D; ++c) s = s + row[c] * row[c];
                rnorm_mine = __fsqrt_rn(s);
                a.rnorms[v0 + lane] = f32_to_f16_bits(rnorm_mine);
            }
            for (int r = 0; r < nv; ++r) {
                float proj[EPL];
                rademacher_rows<EPL>(tile + r * (D + 1), s_rb, lane, a.inv_sqrt_d, proj);
#pragma unroll
                for (int k = 0; k < EPL; ++k) {
                    const uint32_t word = __ballot_sync(0xffffffffu, proj[k] >= 0.0f);  // qjl.rs:315
                    if (lane == 0) reinterpret_cast<uint32_t*>(a.signs)[(v0 + r) * W + k] = word;
                }
            }
        }
        // write the tile's packed bytes and scales (contiguous in global memory)
        const int nwords = nv * a.pb / 4;
        uint32_t* gout = reinterpret_cast<uint32_t*>(a.packed + v0 * a.pb);
        const uint32_t* sst = reinterpret_cast<const uint32_t*>(stage);
        for (int i = lane; i < nwords; i += 32) gout[i] = sst[i];
        if (lane < nv) a.scales[v0 + lane] = f32_to_f16_bits(norm < kMinNorm ? 0.0f : norm);  // select_scale
        __syncwarp();
    }
}

// quantize_vec for batches (no QJL outputs): EPL lanes share a vector, each owning 32 consecutive elements
// that it loads itself, so the first five butterfly stages run in registers and only log2(EPL) stages
// cross lanes; a warp works on 32 / EPL vectors at a time.  Same arithmetic, in the same order, as
// whole_quantize_kernel: the sum of squares runs left to right (the lanes of a vector take turns), the
// sign flip is folded into the exact multiplication by +-1/norm, and the boundary count comes from a cell
// table: cell = round(255 * sat(t + 0.5)); each cell, widened by kWholeSlop, holds at most one boundary
// (the host checks the table's gaps), so code = boundaries under the cell + (t > the cell's boundary).
constexpr float kWholeSlop = 2e-4f;
constexpr int kWholeCells = 128;
constexpr float kWholeFine = 256.0f * kWholeCells - 1.0f;   // sat(t + 0.5) in [0, 1] -> k in [0, 256 * cells - 1]
constexpr float kWholeMinGap = 256.0f / kWholeFine + 4.0f * kWholeSlop;   // smallest boundary gap the cell table can take
constexpr int kWholeWarps = 8;
constexpr int kWholeRowB = 32 * 4 + 16;   // a lane's 32 staged floats + 16 bytes: rows 9 x 16 bytes apart read without bank conflicts
constexpr size_t kWholeSmem = (size_t)kWholeCells * 32 * sizeof(float2) + (size_t)kWholeWarps * 32 * kWholeRowB;

// Input staging: a warp's 32 / EPL vectors are 4 KB of consecutive floats.  They are copied to shared memory
// in 16-byte pieces, 512 consecutive bytes per warp instruction, and each lane then reads its own 128 bytes
// (one lane per 128-byte line straight from global memory costs 32 L1 wavefronts per load instruction).
// The cell table is stored [cell][lane], so the 32 look-ups of a warp instruction touch 32 different bank pairs.
template <int EPL, int BITS>
__global__ void __launch_bounds__(kWholeWarps * 32, 3)
whole_quantize_lane_kernel(WholeArgs a, Codebook cb) {
    constexpr int D = 32 * EPL, KPW = 32 / EPL, NB = (1 << BITS) - 1;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float2* s_cell = reinterpret_cast<float2*>(smem_raw);   // [kWholeCells][32]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned char* stage = smem_raw + (size_t)kWholeCells * 32 * sizeof(float2) + (size_t)warp * 32 * kWholeRowB;
    // cell of t: k = round(sat(t + 0.5) * kWholeFine) (an integer in the mantissa after the 1.5 * 2^23 add), cell = k >> 8
    for (int c = warp; c < kWholeCells; c += kWholeWarps) {
        const float lo = c == 0 ? -FLT_MAX : (256.0f * c - 0.5f) / kWholeFine - 0.5f - kWholeSlop;
        const float hi = c == kWholeCells - 1 ? FLT_MAX : (256.0f * c + 255.5f) / kWholeFine - 0.5f + kWholeSlop;
        float bnd = FLT_MAX;
        unsigned below = 0;
        for (int k = 0; k < NB; ++k) {
            const float b = cb.b[k];
            if (b < lo) ++below;
            else if (b <= hi) bnd = b;
        }
        s_cell[c * 32 + lane] = make_float2(bnd, __uint_as_float(below));
    }
    __syncthreads();
    const int sub = lane % EPL, kin = lane / EPL;
    const bool seed_odd = (a.seed & 1ULL) != 0;
    const long long wid = (long long)blockIdx.x * kWholeWarps + warp;
    const long long nw = (long long)gridDim.x * kWholeWarps;
    const uint32_t stage_s = (uint32_t)__cvta_generic_to_shared(stage);
    for (long long v0 = wid * KPW; v0 < a.n; v0 += nw * KPW) {
        const long long vi = v0 + kin;
        const bool live = vi < a.n;
        // piece q = 32 * i + lane of the warp's 256 pieces belongs to lane q / 8 (vector q / (8 * EPL))
        const uint32_t dst0 = stage_s + (lane >> 3) * kWholeRowB + (lane & 7) * 16;   // + i * 4 rows
        if (v0 + KPW <= a.n) {
            const float* src0 = a.x + v0 * D + lane * 4;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst0 + i * 4 * kWholeRowB), "l"(src0 + i * 128) : "memory");
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int q = 32 * i + lane;
                long long vec = v0 + q / (8 * EPL);
                if (vec >= a.n) vec = a.n - 1;
                const float* src = a.x + vec * D + (q % (8 * EPL)) * 4;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst0 + i * 4 * kWholeRowB), "l"(src) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
        __syncwarp();
        float v[32];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float4 f = *reinterpret_cast<const float4*>(stage + lane * kWholeRowB + k * 16);
            v[4 * k] = f.x; v[4 * k + 1] = f.y; v[4 * k + 2] = f.z; v[4 * k + 3] = f.w;
        }
        __syncwarp();   // the rows are free for the next pass
        // l2_norm (quantize.rs:51-53): s = s + x*x, left to right over the whole vector
        float s = 0.0f;
#pragma unroll
        for (int p = 0; p < EPL; ++p) {
            if (sub == p) {
#pragma unroll
                for (int j = 0; j < 32; ++j) s = s + v[j] * v[j];
            }
            s = __shfl_sync(0xffffffffu, s, (lane & ~(EPL - 1)) | p);
        }
        const float norm = __fsqrt_rn(s);
        const bool tiny = norm < kMinNorm;
        // normalize_inplace (quantize.rs:60-72) and the sign flip (rotation.rs:139-142): (x * inv) * (+-1)
        const float inv = tiny ? 0.0f : __fdiv_rn(1.0f, norm);
        const float inv_even = seed_odd ? -inv : inv, inv_odd = -inv_even;   // element 32*sub + j has the parity of seed + j
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = v[j] * ((j & 1) ? inv_odd : inv_even);
        butterfly32_regs(v);
#pragma unroll
        for (int hs = 1; hs < EPL; hs <<= 1) {
            const uint32_t flip = (sub & hs) ? 0x80000000u : 0u;   // upper half: other - v, lower half: v + other
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float other = __shfl_xor_sync(0xffffffffu, v[j], hs);
                v[j] = other + __uint_as_float(__float_as_uint(v[j]) ^ flip);
            }
        }
        uint32_t w[BITS];
#pragma unroll
        for (int k = 0; k < BITS; ++k) w[k] = 0u;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float t = v[j] * a.inv_sqrt_d;
            const float y = fmaf(__saturatef(t + 0.5f), kWholeFine, 12582912.0f);
            // byte offset of [cell][lane]: cell * 256 + lane * 8
            const float2 e = *reinterpret_cast<const float2*>(smem_raw + ((__float_as_uint(y) & ((kWholeCells - 1) << 8)) | (lane << 3)));
            const uint32_t c = __float_as_uint(e.y) + (t > e.x ? 1u : 0u);
            const int bit = BITS * j;
            w[bit >> 5] += c << (bit & 31);
            if ((bit & 31) + BITS > 32) w[(bit >> 5) + 1] += c >> (32 - (bit & 31));
        }
        if (live) {
            uint32_t* out = reinterpret_cast<uint32_t*>(a.packed + vi * a.pb) + sub * BITS;
#pragma unroll
            for (int k = 0; k < BITS; ++k) out[k] = w[k];
            if (sub == 0) a.scales[vi] = f32_to_f16_bits(tiny ? 0.0f : norm);   // select_scale
        }
    }
}

// dequantize_vec (src/quantize.rs:225-239) / dequantize_rotated (:306-316); warp per vector.
template <int EPL>
__global__ void whole_dequantize_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scales,
                                        long long n, float* __restrict__ out, Codebook cb, int bits, int pb,
                                        uint64_t seed, float inv_sqrt_d, int rotated_only) {
    constexpr int D = 32 * EPL;
    __shared__ float s_c[16];
    if (threadIdx.x < 16) s_c[threadIdx.x] = cb.c[threadIdx.x];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const int nwords = pb >> 2;
    for (long long i = warp_id; i < n; i += nwarps) {
        const uint32_t word = lane < nwords ? __ldg(reinterpret_cast<const uint32_t*>(packed + i * pb) + lane) : 0u;
        const float sc = f16_bits_to_f32(__ldg(scales + i));
        float v[EPL];
#pragma unroll
        for (int k = 0; k < EPL; ++k) v[k] = s_c[code_at(word, lane + 32 * k, bits)];
        if (!rotated_only) {
            wht_lanes<EPL>(v, lane);
#pragma unroll
            for (int k = 0; k < EPL; ++k) v[k] = (v[k] * inv_sqrt_d) * sign_of(seed, lane + 32 * k);
        }
#pragma unroll
        for (int k = 0; k < EPL; ++k) out[i * D + lane + 32 * k] = v[k] * sc;
    }
}

// The same for batches with the lane layout of whole_quantize_lane_kernel: a lane decodes its 32 codes
// through a [code][lane] centroid table (one bank per lane), runs five butterfly stages in registers and
// log2(EPL) across lanes, and the warp's 32 / EPL output vectors (4 KB of consecutive floats) leave
// through shared memory as 512 consecutive bytes per store instruction.  Values are bit-identical to
// whole_dequantize_kernel (same operations in the same order; the sign flip is an exact negation).
template <int EPL, int BITS>
__global__ void __launch_bounds__(kWholeWarps * 32, 3)
whole_dequantize_lane_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scales, long long n,
                             float* __restrict__ out, Codebook cb, int pb, uint64_t seed, float inv_sqrt_d,
                             int rotated_only) {
    constexpr int D = 32 * EPL, KPW = 32 / EPL;
    __shared__ float s_tab[(1 << BITS) * 32];
    __shared__ __align__(16) unsigned char s_stage[kWholeWarps * 32 * kWholeRowB];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < (1 << BITS) * 32; i += kWholeWarps * 32) s_tab[i] = cb.c[i >> 5];
    __syncthreads();
    const float* tab = s_tab + lane;
    unsigned char* stage = s_stage + warp * 32 * kWholeRowB;
    const int sub = lane % EPL, kin = lane / EPL;
    const bool seed_odd = (seed & 1ULL) != 0;
    const float m_even = seed_odd ? -inv_sqrt_d : inv_sqrt_d, m_odd = -m_even;   // (v * inv_sqrt_d) * (+-1)
    const long long wid = (long long)blockIdx.x * kWholeWarps + warp;
    const long long nw = (long long)gridDim.x * kWholeWarps;
    for (long long v0 = wid * KPW; v0 < n; v0 += nw * KPW) {
        const long long vi = v0 + kin;
        const long long vc = vi < n ? vi : n - 1;
        uint32_t w[BITS];
        {
            const uint32_t* p = reinterpret_cast<const uint32_t*>(packed + vc * pb) + sub * BITS;
#pragma unroll
            for (int k = 0; k < BITS; ++k) w[k] = __ldg(p + k);
        }
        const float sc = f16_bits_to_f32(__ldg(scales + vc));
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int bit = BITS * j, k = bit >> 5, sh = bit & 31;
            const uint32_t code = (sh + BITS <= 32 ? (w[k] >> sh) : __funnelshift_r(w[k], w[k + 1 < BITS ? k + 1 : k], sh)) &
                                  ((1u << BITS) - 1u);
            v[j] = tab[code * 32];
        }
        if (!rotated_only) {
            butterfly32_regs(v);
#pragma unroll
            for (int hs = 1; hs < EPL; hs <<= 1) {
                const uint32_t flip = (sub & hs) ? 0x80000000u : 0u;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float other = __shfl_xor_sync(0xffffffffu, v[j], hs);
                    v[j] = other + __uint_as_float(__float_as_uint(v[j]) ^ flip);
                }
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = v[j] * ((j & 1) ? m_odd : m_even);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k)
            *reinterpret_cast<float4*>(stage + lane * kWholeRowB + k * 16) =
                make_float4(v[4 * k] * sc, v[4 * k + 1] * sc, v[4 * k + 2] * sc, v[4 * k + 3] * sc);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int q = 32 * i + lane;
            const long long vec = v0 + q / (8 * EPL);
            const float4 f = *reinterpret_cast<const float4*>(stage + (q >> 3) * kWholeRowB + (q & 7) * 16);
            if (vec < n) *reinterpret_cast<float4*>(out + vec * D + (q % (8 * EPL)) * 4) = f;
        }
        __syncwarp();
    }
}

// precompute_query_projections (src/qjl.rs:488-492); one warp per query.
template <int EPL>
__global__ void projections_kernel(const float* __restrict__ q, long long nq, const uint32_t* __restrict__ rbits,
                                   float* __restrict__ rq, float inv_sqrt_d) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int D = 32 * EPL, W = EPL;
    uint32_t* s_rb = reinterpret_cast<uint32_t*>(smem_raw);
    float* vecs = reinterpret_cast<float*>(s_rb + D * (W + 1));
    for (int i = threadIdx.x; i < D * W; i += blockDim.x) s_rb[(i / W) * (W + 1) + (i % W)] = rbits[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    float* vec = vecs + warp * D;
    for (long long i = (long long)blockIdx.x * warps + warp; i < nq; i += (long long)gridDim.x * warps) {
#pragma unroll
        for (int k = 0; k < EPL; ++k) vec[lane + 32 * k] = q[i * D + lane + 32 * k];
        __syncwarp();
        float proj[EPL];
        rademacher_rows<EPL>(vec, s_rb, lane, inv_sqrt_d, proj);
#pragma unroll
        for (int k = 0; k < EPL; ++k) rq[i * D + lane + 32 * k] = proj[k];
        __syncwarp();
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// attention_scores (src/attention.rs:319-353, src/qjl.rs:585-606).  The key is never
// rotated back: <q, s * sigma .* H(c)/sqrt(d)> = s * <H(sigma .* q)/sqrt(d), c>.
template <int EPL>
__global__ void scores_kernel(const float* __restrict__ q, const float* __restrict__ rq,
                              const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scales,
                              const uint8_t* __restrict__ signs, const uint16_t* __restrict__ rnorms, long long n,
                              float* __restrict__ scores, Codebook cb, int bits, int pb, uint64_t seed,
                              float inv_sqrt_d, float sqrt_d) {
    constexpr int D = 32 * EPL, W = EPL;
    __shared__ float s_c[16];
    if (threadIdx.x < 16) s_c[threadIdx.x] = cb.c[threadIdx.x];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    float qr[EPL], rqv[EPL];
#pragma unroll
    for (int k = 0; k < EPL; ++k) {
        qr[k] = q[lane + 32 * k] * sign_of(seed, lane + 32 * k);
        rqv[k] = rq[lane + 32 * k];
    }
    wht_lanes<EPL>(qr, lane);
#pragma unroll
    for (int k = 0; k < EPL; ++k) qr[k] = qr[k] * inv_sqrt_d;
    const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const int nwords = pb >> 2;
    // kU keys per warp step: their loads and the two shuffle reductions per key are independent chains, which
    // hides the latency that a one-key-at-a-time loop exposes
    constexpr int kU = 4;
    for (long long i0 = warp_id * kU; i0 < n; i0 += nwarps * kU) {
        uint32_t word[kU], sw[kU];
        float sc[kU], rn[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const long long i = i0 + u < n ? i0 + u : n - 1;
            word[u] = lane < nwords ? __ldg(reinterpret_cast<const uint32_t*>(packed + i * pb) + lane) : 0u;
            sw[u] = lane < W ? __ldg(reinterpret_cast<const uint32_t*>(signs + i * (D / 8)) + lane) : 0u;
            sc[u] = f16_bits_to_f32(__ldg(scales + i));
            rn[u] = f16_bits_to_f32(__ldg(rnorms + i));
        }
        float base[kU], corr[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            base[u] = 0.0f;
            corr[u] = 0.0f;
#pragma unroll
            for (int k = 0; k < EPL; ++k) {
                base[u] = fmaf(qr[k], s_c[code_at(word[u], lane + 32 * k, bits)], base[u]);
                const uint32_t w = __shfl_sync(0xffffffffu, sw[u], k);
                corr[u] = fmaf(rqv[k], ((w >> lane) & 1u) ? 1.0f : -1.0f, corr[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            base[u] = warp_sum(base[u]) * sc[u];
            corr[u] = warp_sum(corr[u]);
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const float cc = (rn[u] * 1.2533141f) / sqrt_d;  // qjl.rs:263-265
            if (lane == 0 && i0 + u < n) scores[i0 + u] = base[u] + cc * corr[u];
        }
    }
}

constexpr int kWvBlocks = 296;  // two CTAs per SM
constexpr long long kListMin = 4096;   // shorter lists stay on the warp-per-key kernels (no table build)

// weighted_values (src/attention.rs:371-408), accumulated in the rotated domain:
// sum_t w_t s_t sigma .* H(c_t)/sqrt(d) = sigma .* H(sum_t w_t s_t c_t)/sqrt(d).
template <int EPL>
__global__ void weighted_values_partial_kernel(const float* __restrict__ w, const uint8_t* __restrict__ packed,
                                               const uint16_t* __restrict__ scales, long long n,
                                               float* __restrict__ partial, Codebook cb, int bits, int pb) {
    constexpr int D = 32 * EPL;
    __shared__ float s_c[16];
    __shared__ float s_acc[8][D];
    if (threadIdx.x < 16) s_c[threadIdx.x] = cb.c[threadIdx.x];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int nwords = pb >> 2;
    float acc[EPL];
#pragma unroll
    for (int k = 0; k < EPL; ++k) acc[k] = 0.0f;
    // four values per warp step (independent loads); each lane still adds its elements in value order, so the
    // result does not depend on the grouping
    constexpr int kU = 4;
    const long long wid = (long long)blockIdx.x * warps + warp, nw = (long long)gridDim.x * warps;
    for (long long i0 = wid * kU; i0 < n; i0 += nw * kU) {
        uint32_t word[kU];
        float ws[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const long long i = i0 + u < n ? i0 + u : n - 1;
            word[u] = lane < nwords ? __ldg(reinterpret_cast<const uint32_t*>(packed + i * pb) + lane) : 0u;
            ws[u] = i0 + u < n ? __ldg(w + i) * f16_bits_to_f32(__ldg(scales + i)) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < kU; ++u)
#pragma unroll
            for (int k = 0; k < EPL; ++k) acc[k] = fmaf(ws[u], s_c[code_at(word[u], lane + 32 * k, bits)], acc[k]);
    }
#pragma unroll
    for (int k = 0; k < EPL; ++k) s_acc[warp][lane + 32 * k] = acc[k];
    __syncthreads();
    for (int e = threadIdx.x; e < D; e += blockDim.x) {
        float s = 0.0f;
        for (int ww = 0; ww < warps; ++ww) s += s_acc[ww][e];
        partial[(size_t)blockIdx.x * D + e] = s;
    }
}

template <int EPL>
__global__ void __launch_bounds__(256)
weighted_values_final_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ out, uint64_t seed,
                             float inv_sqrt_d) {
    constexpr int D = 32 * EPL;
    __shared__ float s_part[8][D];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float v[EPL];
#pragma unroll
    for (int k = 0; k < EPL; ++k) v[k] = 0.0f;
    for (int p = warp; p < nparts; p += 8) {
#pragma unroll
        for (int k = 0; k < EPL; ++k) v[k] += partial[(size_t)p * D + lane + 32 * k];
    }
#pragma unroll
    for (int k = 0; k < EPL; ++k) s_part[warp][lane + 32 * k] = v[k];
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int k = 0; k < EPL; ++k) {
        float s = 0.0f;
#pragma unroll
        for (int ww = 0; ww < 8; ++ww) s += s_part[ww][lane + 32 * k];
        v[k] = s;
    }
    wht_lanes<EPL>(v, lane);
#pragma unroll
    for (int k = 0; k < EPL; ++k) out[lane + 32 * k] = (v[k] * inv_sqrt_d) * sign_of(seed, lane + 32 * k);
}

// ---- long key / value lists: one lane per 32 consecutive elements ---------------------------------------
// The warp-per-key kernels above spend ~170 instructions per key (cross-lane code extraction, two warp
// reductions), which is all that matters once a list holds more than a few thousand entries.  Here a key is
// shared by EPL lanes, each owning 32 consecutive elements = PB packed words + one sign word that it loads
// itself, and a warp works on 32 / EPL keys at a time.
//
// Scores: the query is fixed for the launch, so the dot products are tabulated once per CTA.
//   t_base[j][v][lane] = sum_m q~[32*sub + CH*j + m] * c[code m of chunk value v]   (chunk = two 2-bit codes
//                        or one 3-bit code; sub = lane % EPL)
//   t_sign[j][b][lane] = sum_m Rq[32*sub + 4*j + m] * (bit m of b ? +1 : -1)         (b = four sign bits)
// A key then costs one look-up and one add per chunk and per sign nibble.  The lane index is the innermost
// dimension: every lane reads its own bank, so a look-up of 32 random entries is one shared-memory
// wavefront (tables of 64 or 256 entries without the per-lane copies cost ~3.5 wavefronts per look-up and
// were the bound of the kernel).
template <int I, int N, typename F>
__device__ __forceinline__ void static_loop(F&& f) {   // f(integral_constant<int, I>) for I in [I, N): compile-time indices
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_loop<I + 1, N>(f);
    }
}

template <int PB> struct ChunkGeo;
template <> struct ChunkGeo<2> { static constexpr int kCodes = 2, kBits = 4, kEntries = 16; };
template <> struct ChunkGeo<3> { static constexpr int kCodes = 1, kBits = 3, kEntries = 8; };

template <int PB>
__device__ __forceinline__ void load_words(const uint8_t* packed, long long key, int pb, int sub, uint32_t (&w)[PB]) {
    const uint32_t* p = reinterpret_cast<const uint32_t*>(packed + key * pb) + sub * PB;
#pragma unroll
    for (int k = 0; k < PB; ++k) w[k] = __ldg(p + k);
}
constexpr int kListThreads = 512;

// byte offset of entry (x >> SH) & (ENT - 1) in a [ENT][32 lanes] float table
template <int SH, int ENT>
__device__ __forceinline__ uint32_t entry_offset(uint32_t x) {
    if constexpr (SH >= 7) return (x >> (SH - 7)) & ((ENT - 1) << 7);
    else return (x << (7 - SH)) & ((ENT - 1) << 7);
}

template <int EPL, int PB>
__global__ void __launch_bounds__(kListThreads, 2)
scores_table_kernel(const float* __restrict__ q, const float* __restrict__ rq, const uint8_t* __restrict__ packed,
                    const uint16_t* __restrict__ scales, const uint8_t* __restrict__ signs,
                    const uint16_t* __restrict__ rnorms, long long n, float* __restrict__ scores, Codebook cb, int pb,
                    uint64_t seed, float inv_sqrt_d, float sqrt_d) {
    constexpr int D = 32 * EPL, CH = ChunkGeo<PB>::kCodes, CB = ChunkGeo<PB>::kBits, ENT = ChunkGeo<PB>::kEntries;
    constexpr int NJ = 32 / CH;
    constexpr int KPW = 32 / EPL;   // keys per warp step
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* t_base = reinterpret_cast<float*>(smem_raw);   // [NJ][ENT][32]
    float* t_sign = t_base + NJ * ENT * 32;               // [8][16][32]
    float* s_q = t_sign + 8 * 16 * 32;                    // rotated query
    float* s_rq = s_q + D;
    float* s_c = s_rq + D;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x < 16) s_c[threadIdx.x] = cb.c[threadIdx.x];
    if (warp == 0) {
        float qr[EPL];
#pragma unroll
        for (int k = 0; k < EPL; ++k) qr[k] = q[lane + 32 * k] * sign_of(seed, lane + 32 * k);
        wht_lanes<EPL>(qr, lane);
#pragma unroll
        for (int k = 0; k < EPL; ++k) {
            s_q[lane + 32 * k] = qr[k] * inv_sqrt_d;
            s_rq[lane + 32 * k] = rq[lane + 32 * k];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < NJ * ENT * 32; idx += kListThreads) {
        const int j = idx / (ENT * 32), v = (idx >> 5) % ENT;
        const int e0 = (lane % EPL) * 32 + j * CH;   // idx & 31 == lane: kListThreads is a multiple of 32
        float sum = 0.0f;
#pragma unroll
        for (int m = 0; m < CH; ++m) sum = fmaf(s_q[e0 + m], s_c[(v >> (PB * m)) & ((1 << PB) - 1)], sum);
        t_base[idx] = sum;
    }
    for (int idx = threadIdx.x; idx < 8 * 16 * 32; idx += kListThreads) {
        const int j = idx / (16 * 32), b = (idx >> 5) & 15;
        const int e0 = (lane % EPL) * 32 + j * 4;
        float sum = 0.0f;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const float x = s_rq[e0 + m];
            sum += ((b >> m) & 1) ? x : -x;
        }
        t_sign[idx] = sum;
    }
    __syncthreads();

    const int sub = lane % EPL, kin = lane / EPL;
    const unsigned char* tb = reinterpret_cast<const unsigned char*>(t_base + lane);
    const unsigned char* ts = reinterpret_cast<const unsigned char*>(t_sign + lane);
    const float cfac = 1.2533141f / sqrt_d;
    constexpr int kU = 4;
    const long long wid = (long long)blockIdx.x * (kListThreads / 32) + warp;
    const long long nw = (long long)gridDim.x * (kListThreads / 32);
    for (long long i0 = wid * (kU * KPW); i0 < n; i0 += nw * (kU * KPW)) {
        uint32_t w[kU][PB], sw[kU];
        float sc[kU], rn[kU];
        if (i0 + kU * KPW <= n) {
            // full step: one base address per array, every key of the step at a compile-time offset from it
            constexpr int PBW = D * PB / 32;   // packed words per key (pb == 4 * PBW)
            const long long ib = i0 + kin;
            const uint32_t* pw = reinterpret_cast<const uint32_t*>(packed) + ib * PBW + sub * PB;
            const uint32_t* pg = reinterpret_cast<const uint32_t*>(signs) + ib * EPL + sub;
            const uint16_t* pc = scales + ib;
            const uint16_t* pr = rnorms + ib;
#pragma unroll
            for (int u = 0; u < kU; ++u) {
#pragma unroll
                for (int k = 0; k < PB; ++k) w[u][k] = __ldg(pw + u * KPW * PBW + k);
                sw[u] = __ldg(pg + u * KPW * EPL);
                sc[u] = f16_bits_to_f32(__ldg(pc + u * KPW));
                rn[u] = f16_bits_to_f32(__ldg(pr + u * KPW));
            }
        } else {
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                long long i = i0 + u * KPW + kin;
                if (i >= n) i = n - 1;
                load_words<PB>(packed, i, pb, sub, w[u]);
                sw[u] = __ldg(reinterpret_cast<const uint32_t*>(signs + i * (D / 8)) + sub);
                sc[u] = f16_bits_to_f32(__ldg(scales + i));
                rn[u] = f16_bits_to_f32(__ldg(rnorms + i));
            }
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            float base[2] = {0.0f, 0.0f}, corr = 0.0f;
            static_loop<0, NJ>([&](auto j_) {
                constexpr int j = decltype(j_)::value, pos = CB * j, k = pos >> 5, sh = pos & 31;
                uint32_t off;
                if constexpr (sh + CB <= 32) off = entry_offset<sh, ENT>(w[u][k]);
                else off = entry_offset<0, ENT>(__funnelshift_r(w[u][k], w[u][k + 1 < PB ? k + 1 : k], sh));
                base[j & 1] += *reinterpret_cast<const float*>(tb + j * (ENT * 128) + off);
            });
            static_loop<0, 8>([&](auto j_) {
                constexpr int j = decltype(j_)::value;
                corr += *reinterpret_cast<const float*>(ts + j * (16 * 128) + entry_offset<4 * j, 16>(sw[u]));
            });
            // qjl.rs:263-265: sqrt(pi/2) / sqrt(d) * ||residual||
            float val = fmaf(rn[u] * cfac, corr, (base[0] + base[1]) * sc[u]);
#pragma unroll
            for (int o = 1; o < EPL; o <<= 1) val += __shfl_xor_sync(0xffffffffu, val, o);
            const long long i = i0 + u * KPW + kin;
            if (sub == 0 && i < n) scores[i] = val;
        }
    }
}

// Weighted sum of values: each lane keeps 32 running sums (its elements) over the keys of its lane group;
// a pair of codes indexes a table of centroid pairs.  Lane groups are added at the end.
template <int EPL, int PB>
__global__ void __launch_bounds__(kListThreads, 2)
weighted_values_lane_kernel(const float* __restrict__ w, const uint8_t* __restrict__ packed,
                            const uint16_t* __restrict__ scales, long long n, float* __restrict__ partial, Codebook cb,
                            int pb) {
    constexpr int D = 32 * EPL, KPW = 32 / EPL, NP = 1 << (2 * PB);
    __shared__ float2 s_pair[NP];
    __shared__ float s_acc[kListThreads / 32][D];
    for (int i = threadIdx.x; i < NP; i += kListThreads)
        s_pair[i] = make_float2(cb.c[i & ((1 << PB) - 1)], cb.c[i >> PB]);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % EPL, kin = lane / EPL;
    float acc[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) acc[e] = 0.0f;
    constexpr int kU = 4;
    const long long wid = (long long)blockIdx.x * (kListThreads / 32) + warp;
    const long long nw = (long long)gridDim.x * (kListThreads / 32);
    for (long long i0 = wid * (kU * KPW); i0 < n; i0 += nw * (kU * KPW)) {
        uint32_t cw[kU][PB];
        float ws[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const long long i = i0 + u * KPW + kin;
            const long long ic = i < n ? i : n - 1;
            load_words<PB>(packed, ic, pb, sub, cw[u]);
            ws[u] = i < n ? __ldg(w + ic) * f16_bits_to_f32(__ldg(scales + ic)) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
#pragma unroll
            for (int p = 0; p < 16; ++p) {
                const int pos = 2 * PB * p, k = pos >> 5, sh = pos & 31;
                const uint32_t v = (sh + 2 * PB <= 32 ? (cw[u][k] >> sh)
                                                      : __funnelshift_r(cw[u][k], cw[u][k + 1 < PB ? k + 1 : k], sh)) & (NP - 1);
                const float2 c = s_pair[v];
                acc[2 * p] = fmaf(ws[u], c.x, acc[2 * p]);
                acc[2 * p + 1] = fmaf(ws[u], c.y, acc[2 * p + 1]);
            }
        }
    }
#pragma unroll
    for (int o = EPL; o < 32; o <<= 1) {
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
    }
    if (kin == 0) {
#pragma unroll
        for (int e = 0; e < 32; ++e) s_acc[warp][sub * 32 + e] = acc[e];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < D; e += kListThreads) {
        float sum = 0.0f;
        for (int ww = 0; ww < kListThreads / 32; ++ww) sum += s_acc[ww][e];
        partial[(size_t)blockIdx.x * D + e] = sum;
    }
}

// compute_qjl_signs_and_norms of the block-32 TQ cache (src/cache/tq.rs:380-411): residual =
// original - dequantized, its L2 norm (f16) and the head_dim-wide sign sketch, written at the
// storage rows of CompressedStorage (row i -> (i / rows_per_group) * group_stride + row_offset
// + i % rows_per_group).  One warp per tile of 32 vectors; sums are sequential as in the core crate.
template <int EPL, typename T>
__global__ void residual_sketch_kernel(const T* __restrict__ x, const float* __restrict__ xhat, long long n,
                                       const uint32_t* __restrict__ rbits, uint8_t* __restrict__ signs,
                                       uint16_t* __restrict__ norms, long long rows_per_group, long long group_stride,
                                       long long row_offset, float inv_sqrt_d, int vt) {
    // vt: vectors per warp tile (1..kTile).  A warp sketches the vectors of its tile one after the other (~3 us each),
    // so a small batch - the 512 new keys of a decode step - is spread one vector per warp instead of 32.
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int D = 32 * EPL, W = EPL;
    uint32_t* s_rb = reinterpret_cast<uint32_t*>(smem_raw);
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* tile = reinterpret_cast<float*>(s_rb + D * (W + 1)) + (size_t)warp * vt * (D + 1);
    for (int i = threadIdx.x; i < D * W; i += blockDim.x) s_rb[(i / W) * (W + 1) + (i % W)] = rbits[i];
    __syncthreads();
    const long long tiles = (n + vt - 1) / vt;
    for (long long t = (long long)blockIdx.x * warps + warp; t < tiles; t += (long long)gridDim.x * warps) {
        const long long v0 = t * vt;
        const int nv = (int)min((long long)vt, n - v0);
        for (int r = 0; r < nv; ++r)
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                const long long e = (v0 + r) * D + lane + 32 * i;
                tile[r * (D + 1) + lane + 32 * i] = to_f32<T>(x[e]) - xhat[e];
            }
        __syncwarp();
        long long orow = 0;
        if (lane < nv) {
            float s = 0.0f;
            const float* row = tile + lane * (D + 1);
#pragma unroll 8
            for (int c = 0; c < D; ++c) s = s + row[c] * row[c];
            const long long i = v0 + lane;
            orow = i;
            if (rows_per_group != 0) {
                const long long g = i / rows_per_group;
                orow = g * group_stride + row_offset + (i - g * rows_per_group);
            }
            norms[orow] = f32_to_f16_bits(__fsqrt_rn(s));
        }
        for (int r = 0; r < nv; ++r) {
            float proj[EPL];
            rademacher_rows<EPL>(tile + r * (D + 1), s_rb, lane, inv_sqrt_d, proj);
            const long long dst = __shfl_sync(0xffffffffu, orow, r);
#pragma unroll
            for (int k = 0; k < EPL; ++k) {
                const uint32_t word = __ballot_sync(0xffffffffu, proj[k] >= 0.0f);
                if (lane == 0) reinterpret_cast<uint32_t*>(signs)[dst * W + k] = word;
            }
        }
        __syncwarp();
    }
}

// compute_logit_bias (src/cache/tq.rs:185-253): bias[h, i, t] = (sum_d rq[h, i, d] * (+-1)) * c_t with
// c_t = norm_t * sqrt(pi/2) / sqrt(D).  One thread per token, the group's projected queries in shared memory.
// rq: [hq, q_len, D]; signs: [hkv, stride, D/8]; norms: [hkv, stride]; bias: [hq, q_len, kv_len] of type OT.
template <typename OT>
__global__ void logit_bias_kernel(const float* __restrict__ rq, const uint8_t* __restrict__ signs,
                                  const uint16_t* __restrict__ norms, OT* __restrict__ bias, int hq, int hkv, int q_len,
                                  int D, int kv_len, int kv_stride, float scale_factor) {
    extern __shared__ float s_rq[];   // [g * q_len][D]
    const int kvh = blockIdx.y, g = hq / hkv;
    const int rows = g * q_len;
    for (int i = threadIdx.x; i < rows * D; i += blockDim.x) s_rq[i] = rq[(size_t)kvh * rows * D + i];
    __syncthreads();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= kv_len) return;
    const size_t row = (size_t)kvh * kv_stride + t;
    const uint32_t* sw = reinterpret_cast<const uint32_t*>(signs + row * (D / 8));
    const float c = f16_bits_to_f32(norms[row]) * scale_factor;
    for (int r = 0; r < rows; ++r) {
        float acc = 0.0f;
        for (int w = 0; w < D / 32; ++w) {
            const uint32_t bits = sw[w];
#pragma unroll 8
            for (int b = 0; b < 32; ++b) acc = fmaf(s_rq[r * D + w * 32 + b], ((bits >> b) & 1u) ? 1.0f : -1.0f, acc);
        }
        const int head = kvh * g + r / q_len, qi = r % q_len;
        bias[((size_t)head * q_len + qi) * kv_len + t] = from_f32<OT>(acc * c);
    }
}

size_t quant_smem(int dim, int pb, int warps, bool qjl) {
    const int W = dim / 32;
    size_t per_warp = sizeof(float) * kTile * (dim + 1) + dim + (size_t)kTile * pb;
    per_warp = (per_warp + 15) / 16 * 16;
    return (qjl ? sizeof(uint32_t) * dim * (W + 1) : 0) + 32 * sizeof(float) + per_warp * warps;
}

template <int EPL, bool QJL>
int launch_quant(const WholeArgs& a, const Codebook& cb, cudaStream_t s) {
    const int warps = EPL >= 8 ? 2 : 4;
    const size_t smem = quant_smem(a.dim, a.pb, warps, QJL);
    cudaError_t e = cudaFuncSetAttribute(whole_quantize_kernel<EPL, QJL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return TQB_ERR_CUDA; }
    const long long tiles = (a.n + kTile - 1) / kTile;
    long long grid = (tiles + warps - 1) / warps;
    if (grid > 148 * 8) grid = 148 * 8;
    whole_quantize_kernel<EPL, QJL><<<(int)grid, warps * 32, smem, s>>>(a, cb);
    return check_launch(s);
}

template <int EPL, int BITS>
int launch_quant_lane_bits(const WholeArgs& a, const Codebook& cb, cudaStream_t s) {
    constexpr int kpw = 32 / EPL;
    long long grid = (a.n + kWholeWarps * kpw - 1) / (kWholeWarps * kpw);
    if (grid > 148 * 3) grid = 148 * 3;
    cudaError_t e = cudaFuncSetAttribute(whole_quantize_lane_kernel<EPL, BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kWholeSmem);
    if (e != cudaSuccess) { set_cuda_error(e); return TQB_ERR_CUDA; }
    whole_quantize_lane_kernel<EPL, BITS><<<(int)grid, kWholeWarps * 32, kWholeSmem, s>>>(a, cb);
    return check_launch(s);
}

template <int EPL>
int launch_quant_lane(const WholeArgs& a, const Codebook& cb, cudaStream_t s) {
    switch (a.bits) {
        case 2: return launch_quant_lane_bits<EPL, 2>(a, cb, s);
        case 3: return launch_quant_lane_bits<EPL, 3>(a, cb, s);
        case 4: return launch_quant_lane_bits<EPL, 4>(a, cb, s);
        default: return TQB_ERR_UNSUPPORTED_BITS;
    }
}

// The cell table of whole_quantize_lane_kernel needs every boundary inside (-0.5, 0.5) and gaps wider than a cell.
bool cell_table_fits(const Codebook& cb, int bits) {
    const int nb = (1 << bits) - 1;
    for (int k = 0; k < nb; ++k) {
        if (!(fabsf(cb.b[k]) < 0.49f)) return false;
        if (k > 0 && !(cb.b[k] - cb.b[k - 1] > kWholeMinGap)) return false;
    }
    return true;
}

template <bool QJL>
int dispatch_quant(const WholeArgs& a, const Codebook& cb, cudaStream_t s) {
    if (!QJL && a.bits >= 2 && a.bits <= 4 && ((uintptr_t)a.x % 16) == 0 && cell_table_fits(cb, a.bits)) {
        switch (a.dim) {
            case 32: return launch_quant_lane<1>(a, cb, s);
            case 64: return launch_quant_lane<2>(a, cb, s);
            case 128: return launch_quant_lane<4>(a, cb, s);
            case 256: return launch_quant_lane<8>(a, cb, s);
            default: return TQB_ERR_UNSUPPORTED;
        }
    }
    switch (a.dim) {
        case 32: return launch_quant<1, QJL>(a, cb, s);
        case 64: return launch_quant<2, QJL>(a, cb, s);
        case 128: return launch_quant<4, QJL>(a, cb, s);
        case 256: return launch_quant<8, QJL>(a, cb, s);
        default: return TQB_ERR_UNSUPPORTED;
    }
}

int grid_warps(long long n, int warps_per_block) {
    long long g = (n + warps_per_block - 1) / warps_per_block;
    if (g > 148 * 8) g = 148 * 8;
    if (g < 1) g = 1;
    return (int)g;
}

float host_inv_sqrt(int dim) { return 1.0f / sqrtf((float)dim); }  // rotation.rs:36

}  // namespace
}  // namespace tqb

using namespace tqb;

#define TQB_DISPATCH_EPL(dim, ...)                        \
    switch (dim) {                                         \
        case 32: { constexpr int EPL = 1; __VA_ARGS__; } break;  \
        case 64: { constexpr int EPL = 2; __VA_ARGS__; } break;  \
        case 128: { constexpr int EPL = 4; __VA_ARGS__; } break; \
        case 256: { constexpr int EPL = 8; __VA_ARGS__; } break; \
        default: return TQB_ERR_UNSUPPORTED;               \
    }

extern "C" {

int tqb_quantize_batch(const tqb_config* cfg, const float* x, int64_t n, uint8_t* packed, uint16_t* scales,
                       tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    int st = tqb_config_validate(cfg);
    if (st != TQB_OK) return st;
    if (n < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (n == 0) return TQB_OK;
    if (!x || !packed || !scales) return TQB_ERR_NULL_POINTER;
    if (((uintptr_t)packed % 4) || ((uintptr_t)x % 4)) return TQB_ERR_MISALIGNED;
    Codebook cb;
    if (!whole_codebook(cfg->bits, cfg->dim, cb)) return TQB_ERR_UNSUPPORTED;
    WholeArgs a{};
    a.x = x; a.n = n; a.packed = packed; a.scales = scales;
    a.bits = cfg->bits; a.dim = cfg->dim; a.pb = (int)tqb_packed_bytes(cfg->bits, cfg->dim);
    a.seed = cfg->rotation_seed; a.inv_sqrt_d = host_inv_sqrt(cfg->dim);
    return dispatch_quant<false>(a, cb, as_stream(stream));
}

int tqb_qjl_quantize_batch(const tqb_config* cfg, const uint32_t* rbits, const float* x, int64_t n, uint8_t* packed,
                           uint16_t* scales, uint8_t* signs, uint16_t* rnorms, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (!cfg) return TQB_ERR_NULL_POINTER;
    if (cfg->bits < 3 || cfg->bits > 4) return TQB_ERR_UNSUPPORTED_BITS;  // src/qjl.rs:277-279
    tqb_config polar = *cfg;
    polar.bits = cfg->bits - 1;
    int st = tqb_config_validate(&polar);
    if (st != TQB_OK) return st;
    if (n < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (n == 0) return TQB_OK;
    if (!rbits || !x || !packed || !scales || !signs || !rnorms) return TQB_ERR_NULL_POINTER;
    if (((uintptr_t)packed % 4) || ((uintptr_t)signs % 4) || ((uintptr_t)x % 4)) return TQB_ERR_MISALIGNED;
    Codebook cb;
    if (!whole_codebook(polar.bits, polar.dim, cb)) return TQB_ERR_UNSUPPORTED;
    WholeArgs a{};
    a.x = x; a.n = n; a.packed = packed; a.scales = scales; a.signs = signs; a.rnorms = rnorms; a.rbits = rbits;
    a.bits = polar.bits; a.dim = polar.dim; a.pb = (int)tqb_packed_bytes(polar.bits, polar.dim);
    a.seed = cfg->rotation_seed; a.inv_sqrt_d = host_inv_sqrt(cfg->dim);
    return dispatch_quant<true>(a, cb, as_stream(stream));
}

static int dequant_common(const tqb_config* cfg, const uint8_t* packed, const uint16_t* scales, int64_t n, float* out,
                          int rotated_only, tqb_stream_t stream) {
    int st = tqb_config_validate(cfg);
    if (st != TQB_OK) return st;
    if (n < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (n == 0) return TQB_OK;
    if (!packed || !scales || !out) return TQB_ERR_NULL_POINTER;
    if ((uintptr_t)packed % 4) return TQB_ERR_MISALIGNED;
    Codebook cb;
    if (!whole_codebook(cfg->bits, cfg->dim, cb)) return TQB_ERR_UNSUPPORTED;
    const int pb = (int)tqb_packed_bytes(cfg->bits, cfg->dim);
    cudaStream_t s = as_stream(stream);
    if (((uintptr_t)out % 16) == 0 && cfg->bits >= 2 && cfg->bits <= 4) {
        const long long per_cta = (long long)kWholeWarps * (32 / (cfg->dim / 32));
        long long g = (n + per_cta - 1) / per_cta;
        if (g > 148 * 3) g = 148 * 3;
#define TQB_DEQ_LANE(BITS)                                                                                            \
    TQB_DISPATCH_EPL(cfg->dim, (whole_dequantize_lane_kernel<EPL, BITS><<<(int)g, kWholeWarps * 32, 0, s>>>(            \
        packed, scales, n, out, cb, pb, cfg->rotation_seed, host_inv_sqrt(cfg->dim), rotated_only)))
        if (cfg->bits == 2) { TQB_DEQ_LANE(2); } else if (cfg->bits == 3) { TQB_DEQ_LANE(3); } else { TQB_DEQ_LANE(4); }
#undef TQB_DEQ_LANE
        return check_launch(s);
    }
    const int grid = grid_warps(n, 8);
    TQB_DISPATCH_EPL(cfg->dim, (whole_dequantize_kernel<EPL><<<grid, 256, 0, s>>>(
        packed, scales, n, out, cb, cfg->bits, pb, cfg->rotation_seed, host_inv_sqrt(cfg->dim), rotated_only)));
    return check_launch(s);
}

int tqb_dequantize_batch(const tqb_config* cfg, const uint8_t* packed, const uint16_t* scales, int64_t n, float* out,
                         tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    return dequant_common(cfg, packed, scales, n, out, 0, stream);
}

int tqb_dequantize_rotated_batch(const tqb_config* cfg, const uint8_t* packed, const uint16_t* scales, int64_t n,
                                 float* out, tqb_stream_t stream) {
    return dequant_common(cfg, packed, scales, n, out, 1, stream);
}

int tqb_qjl_query_projections(int32_t dim, const uint32_t* rbits, const float* q, int64_t nq, float* rq,
                              tqb_stream_t stream) {
    if (dim != 32 && dim != 64 && dim != 128 && dim != 256)
        return (dim > 0 && (dim & (dim - 1)) == 0) ? TQB_ERR_UNSUPPORTED : TQB_ERR_INVALID_DIMENSION;
    if (nq < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (nq == 0) return TQB_OK;
    if (!rbits || !q || !rq) return TQB_ERR_NULL_POINTER;
    cudaStream_t s = as_stream(stream);
    const int W = dim / 32, warps = 4;
    const size_t smem = sizeof(uint32_t) * dim * (W + 1) + sizeof(float) * warps * dim;
    const int grid = grid_warps(nq, warps);
    TQB_DISPATCH_EPL(dim, {
        cudaError_t e = cudaFuncSetAttribute(projections_kernel<EPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { set_cuda_error(e); return TQB_ERR_CUDA; }
        projections_kernel<EPL><<<grid, warps * 32, smem, s>>>(q, nq, rbits, rq, host_inv_sqrt(dim));
    });
    return check_launch(s);
}

int tqb_qjl_attention_scores(const tqb_config* cfg, const float* q, const float* rq, const uint8_t* packed,
                             const uint16_t* scales, const uint8_t* signs, const uint16_t* rnorms, int64_t n,
                             float* scores, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (!cfg) return TQB_ERR_NULL_POINTER;
    if (cfg->bits < 3 || cfg->bits > 4) return TQB_ERR_UNSUPPORTED_BITS;
    tqb_config polar = *cfg;
    polar.bits = cfg->bits - 1;
    int st = tqb_config_validate(&polar);
    if (st != TQB_OK) return st;
    if (n < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (n == 0) return TQB_OK;
    if (!q || !rq || !packed || !scales || !signs || !rnorms || !scores) return TQB_ERR_NULL_POINTER;
    if (((uintptr_t)packed % 4) || ((uintptr_t)signs % 4)) return TQB_ERR_MISALIGNED;
    Codebook cb;
    if (!whole_codebook(polar.bits, polar.dim, cb)) return TQB_ERR_UNSUPPORTED;
    const int pb = (int)tqb_packed_bytes(polar.bits, polar.dim);
    cudaStream_t s = as_stream(stream);
    if (n >= kListMin && (polar.bits == 2 || polar.bits == 3) && cfg->dim >= 64) {
        // long lists: tabulated query, one lane per 32 elements
        const int dim = cfg->dim;
        const size_t smem = sizeof(float) * (8192 + 4096 + 2 * dim + 16);   // [chunks][entries][32] + [8][16][32]
        const long long per_cta = (long long)(kListThreads / 32) * 4 * (32 / (dim / 32));
        long long g = (n + per_cta - 1) / per_cta;
        const long long gmax = smem > 100 * 1024 ? 148 : 296;
        if (g > gmax) g = gmax;
#define TQB_SCORES_TABLE(PB)                                                                                          \
    TQB_DISPATCH_EPL(dim, {                                                                                           \
        cudaError_t e = cudaFuncSetAttribute(scores_table_kernel<EPL, PB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) { set_cuda_error(e); return TQB_ERR_CUDA; }                                             \
        scores_table_kernel<EPL, PB><<<(int)g, kListThreads, smem, s>>>(q, rq, packed, scales, signs, rnorms, n, scores, cb, pb, \
                                                                         cfg->rotation_seed, host_inv_sqrt(dim),     \
                                                                         sqrtf((float)dim));                         \
    })
        if (polar.bits == 2) { TQB_SCORES_TABLE(2); } else { TQB_SCORES_TABLE(3); }
#undef TQB_SCORES_TABLE
        return check_launch(s);
    }
    const int grid = grid_warps(n, 8);
    TQB_DISPATCH_EPL(cfg->dim, (scores_kernel<EPL><<<grid, 256, 0, s>>>(
        q, rq, packed, scales, signs, rnorms, n, scores, cb, polar.bits, pb, cfg->rotation_seed,
        host_inv_sqrt(cfg->dim), sqrtf((float)cfg->dim))));
    return check_launch(s);
}

size_t tqb_weighted_values_scratch_bytes(int32_t dim) {
    return dim > 0 ? sizeof(float) * (size_t)kWvBlocks * dim : 0;
}

int tqb_weighted_values(const tqb_config* cfg, const float* w, const uint8_t* packed, const uint16_t* scales, int64_t n,
                        float* out, void* scratch, size_t scratch_bytes, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (!cfg) return TQB_ERR_NULL_POINTER;
    if (cfg->bits < 3 || cfg->bits > 4) return TQB_ERR_UNSUPPORTED_BITS;
    tqb_config polar = *cfg;
    polar.bits = cfg->bits - 1;
    int st = tqb_config_validate(&polar);
    if (st != TQB_OK) return st;
    if (n < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (!out || !scratch) return TQB_ERR_NULL_POINTER;
    if (n > 0 && (!w || !packed || !scales)) return TQB_ERR_NULL_POINTER;
    if (scratch_bytes < tqb_weighted_values_scratch_bytes(cfg->dim)) return TQB_ERR_INVALID_ARGUMENT;
    if ((uintptr_t)packed % 4) return TQB_ERR_MISALIGNED;
    Codebook cb;
    if (!whole_codebook(polar.bits, polar.dim, cb)) return TQB_ERR_UNSUPPORTED;
    const int pb = (int)tqb_packed_bytes(polar.bits, polar.dim);
    cudaStream_t s = as_stream(stream);
    int nparts = (int)((n + 7) / 8);
    if (nparts > kWvBlocks) nparts = kWvBlocks;
    if (nparts < 1) nparts = 1;
    float* partial = reinterpret_cast<float*>(scratch);
    if (n >= kListMin && (polar.bits == 2 || polar.bits == 3) && cfg->dim >= 64) {
        const long long per_cta = (long long)(kListThreads / 32) * 4 * (32 / (cfg->dim / 32));
        long long g = (n + per_cta - 1) / per_cta;
        if (g > kWvBlocks) g = kWvBlocks;
        nparts = (int)g;
#define TQB_WV_LANE(PB)                                                                                               \
    TQB_DISPATCH_EPL(cfg->dim, {                                                                                      \
        weighted_values_lane_kernel<EPL, PB><<<nparts, kListThreads, 0, s>>>(w, packed, scales, n, partial, cb, pb);  \
        weighted_values_final_kernel<EPL><<<1, 256, 0, s>>>(partial, nparts, out, cfg->rotation_seed, host_inv_sqrt(cfg->dim)); \
    })
        if (polar.bits == 2) { TQB_WV_LANE(2); } else { TQB_WV_LANE(3); }
#undef TQB_WV_LANE
        return check_launch(s);
    }
    TQB_DISPATCH_EPL(cfg->dim, {
        weighted_values_partial_kernel<EPL><<<nparts, 256, 0, s>>>(w, packed, scales, n, partial, cb, polar.bits, pb);
        weighted_values_final_kernel<EPL><<<1, 256, 0, s>>>(partial, nparts, out, cfg->rotation_seed, host_inv_sqrt(cfg->dim));
    });
    return check_launch(s);
}

}  // extern "C"

extern "C" {

int tqb_residual_sketch(int32_t dim, const uint32_t* rbits, const void* original, int32_t dtype,
                        const float* dequantized, int64_t n, uint8_t* signs, uint16_t* norms, int64_t rows_per_group,
                        int64_t out_group_stride, int64_t out_row_offset, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (dim != 32 && dim != 64 && dim != 128 && dim != 256)
        return (dim > 0 && dim % 32 == 0) ? TQB_ERR_UNSUPPORTED : TQB_ERR_INVALID_DIMENSION;
    if (n < 0 || rows_per_group < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (n == 0) return TQB_OK;
    if (!rbits || !original || !dequantized || !signs || !norms) return TQB_ERR_NULL_POINTER;
    if ((uintptr_t)signs % 4) return TQB_ERR_MISALIGNED;
    if (dtype != TQB_F32 && dtype != TQB_F16 && dtype != TQB_BF16) return TQB_ERR_INVALID_ARGUMENT;
    cudaStream_t s = as_stream(stream);
    const int W = dim / 32, warps = dim >= 256 ? 2 : 4;
    // vectors per warp tile: enough tiles for ~16 warps on every SM before a warp takes a second vector
    long long vt = (n + 148 * 16 - 1) / (148 * 16);
    if (vt > kTile) vt = kTile;
    if (vt < 1) vt = 1;
    const size_t smem = sizeof(uint32_t) * dim * (W + 1) + sizeof(float) * warps * vt * (dim + 1);
    const long long tiles = (n + vt - 1) / vt;
    long long grid = (tiles + warps - 1) / warps;
    if (grid > 148 * 8) grid = 148 * 8;
    const float inv = host_inv_sqrt(dim);
#define TQB_SKETCH(T)                                                                                            \
    do { TQB_DISPATCH_EPL(dim, {                                                                                 \
        cudaError_t e = cudaFuncSetAttribute(residual_sketch_kernel<EPL, T>,                                      \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
        if (e != cudaSuccess) { set_cuda_error(e); return TQB_ERR_CUDA; }                                        \
        residual_sketch_kernel<EPL, T><<<(int)grid, warps * 32, smem, s>>>(                                       \
            (const T*)original, dequantized, n, rbits, signs, norms, rows_per_group, out_group_stride,           \
            out_row_offset, inv, (int)vt);                                                                       \
    }) } while (0)
    if (dtype == TQB_F32) TQB_SKETCH(float);
    else if (dtype == TQB_F16) TQB_SKETCH(__half);
    else TQB_SKETCH(__nv_bfloat16);
#undef TQB_SKETCH
    return check_launch(s);
}

int tqb_qjl_logit_bias(int32_t head_dim, const float* rq, const uint8_t* signs, const uint16_t* norms, void* bias,
                       int32_t bias_dtype, int32_t num_q_heads, int32_t num_kv_heads, int32_t q_len, int32_t kv_len,
                       int32_t kv_stride, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (head_dim <= 0 || head_dim % 32 != 0) return TQB_ERR_INVALID_DIMENSION;
    if (num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0 || q_len <= 0) return TQB_ERR_INVALID_ARGUMENT;
    if (kv_len < 0 || kv_len > kv_stride) return TQB_ERR_RANGE_OUT_OF_BOUNDS;
    if (kv_len == 0) return TQB_OK;
    if (!rq || !signs || !norms || !bias) return TQB_ERR_NULL_POINTER;
    if ((uintptr_t)signs % 4) return TQB_ERR_MISALIGNED;
    const int g = num_q_heads / num_kv_heads;
    const size_t smem = sizeof(float) * (size_t)g * q_len * head_dim;
    if (smem > 200 * 1024) return TQB_ERR_TOO_LARGE;
    // src/cache/tq.rs:215-216: sqrt(pi/2) as f32 divided by sqrt(head_dim) in f32
    const float scale_factor = (float)sqrt(1.5707963267948966) / sqrtf((float)head_dim);
    cudaStream_t s = as_stream(stream);
    dim3 grid((kv_len + 127) / 128, num_kv_heads);
#define TQB_BIAS(OT)                                                                                                   \
    do {                                                                                                               \
        cudaError_t e = cudaFuncSetAttribute(logit_bias_kernel<OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) { set_cuda_error(e); return TQB_ERR_CUDA; }                                              \
        logit_bias_kernel<OT><<<grid, 128, smem, s>>>(rq, signs, norms, (OT*)bias, num_q_heads, num_kv_heads, q_len,   \
                                                      head_dim, kv_len, kv_stride, scale_factor);                      \
    } while (0)
    if (bias_dtype == TQB_F32) TQB_BIAS(float);
    else if (bias_dtype == TQB_F16) TQB_BIAS(__half);
    else if (bias_dtype == TQB_BF16) TQB_BIAS(__nv_bfloat16);
    else return TQB_ERR_INVALID_ARGUMENT;
#undef TQB_BIAS
    return check_launch(s);
}

}  // extern "C"
