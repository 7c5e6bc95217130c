// Block-32 ("cache module") quantize / dequantize kernels.
//
// Work decomposition: the tensor is a flat array of independent 32-element blocks
// (src/cache/config.rs:9).  Four lanes own one block, eight consecutive elements each, so a
// warp covers eight blocks per pass.  The 32-point Walsh-Hadamard butterfly runs stages
// h = 1, 2, 4 inside a lane and h = 8, 16 through __shfl_xor; every add/sub pairs the same
// two operands as the scalar butterfly of src/cache/wht_tensor.rs:44-59, so the result is
// bit-identical to it.  Eight codes of one lane are 2, 3 or 4 whole bytes of the packed
// stream (src/packed/mod.rs:242-309), which makes packing a lane-local shift/or plus one
// shuffle for the 3-bit width.
#include "tqb_common.cuh"
#include "tqb_pqo_quant.cuh"

namespace tqb {
namespace {

constexpr int kThreads = 256;

struct RowMap {
    // output row of input row i: (i / rows_per_group) * group_stride + row_offset + i % rows_per_group
    long long rows_per_group;  // 0 = identity
    long long group_stride;
    long long row_offset;
    __device__ __forceinline__ long long operator()(long long i) const {
        if (rows_per_group == 0) return i;
        long long g = i / rows_per_group;
        return g * group_stride + row_offset + (i - g * rows_per_group);
    }
};

__device__ __forceinline__ void butterfly8_inlane(float (&v)[8]) {
#pragma unroll
    for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if ((i & h) == 0) {
                float x = v[i], y = v[i + h];
                v[i] = x + y;
                v[i + h] = x - y;
            }
        }
    }
}

// Stages h = 8 and h = 16 across the four lanes of a block (q = lane & 3).
__device__ __forceinline__ void butterfly_cross(float (&v)[8], int q) {
#pragma unroll
    for (int m = 1; m <= 2; m <<= 1) {
        const bool upper = (q & m) != 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float other = __shfl_xor_sync(0xffffffffu, v[i], m);
            v[i] = upper ? (other - v[i]) : (v[i] + other);
        }
    }
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
    float4 a = __ldg(reinterpret_cast<const float4*>(p));
    float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
    uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);            // bf16 -> f32 is exact
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[8]) {
    uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
}
template <>
__device__ __forceinline__ void store8<__half>(__half* p, const float (&v)[8]) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
}

// Writes the 8*BITS bits of one lane (four lanes = one block of 4*BITS bytes).
// `next` is the same quantity of the following lane (fetched by the caller with a
// warp-wide shuffle, outside any divergent branch).
template <int BITS>
__device__ __forceinline__ void store_codes(uint8_t* block_ptr, uint32_t mine, uint32_t next, int q) {
    if (BITS == 4) {
        reinterpret_cast<uint32_t*>(block_ptr)[q] = mine;
    } else if (BITS == 3) {
        // lanes hold 24 bits each; words: w0 = L0 | L1<<24, w1 = L1>>8 | L2<<16, w2 = L2>>16 | L3<<8
        uint32_t w = (mine >> (8 * q)) | (next << (24 - 8 * q));
        if (q < 3) reinterpret_cast<uint32_t*>(block_ptr)[q] = w;
    } else {
        if ((q & 1) == 0) reinterpret_cast<uint32_t*>(block_ptr)[q >> 1] = mine | (next << 16);
    }
}

struct QuantArgs {
    const void* x;
    long long n_rows;
    long long x_row_stride;
    uint8_t* indices;
    uint16_t* scales;
    RowMap map;
    int nblk;            // blocks per row
    int outlier_blocks;  // clamped to [0, nblk]
    int norm_mode;
    int pre_rotated;     // input already rotated (legacy entry point)
    float outer_centroid;
    float scale_sign_outlier;  // multiplies the stored scale of outlier blocks
    float scale_sign_normal;
    const float* dev_boundaries;  // legacy entry point: boundaries on the device (outlier table)
    int dev_num_boundaries;
    // second tensor of a pair launch (grid.y = 2: K and V of one append in one launch), else nullptr
    const void* x2;
    uint8_t* indices2;
    uint16_t* scales2;
};

// src/cache/quantize_tensor.rs:40-176 with the scalar arithmetic of
// src/cache/cuda/kernels/tq_quant_kernel.cu:216-259 (true IEEE division, no fast-math).
template <typename T, int BITS>
__global__ void __launch_bounds__(kThreads)
block_quantize_kernel(QuantArgs a, Codebook normal, Codebook outlier) {
    if (blockIdx.y != 0) { a.x = a.x2; a.indices = a.indices2; a.scales = a.scales2; }
    __shared__ float s_b[2][16];
    __shared__ float s_sign[32];
    if (threadIdx.x < 16) {
        s_b[0][threadIdx.x] = normal.b[threadIdx.x];
        s_b[1][threadIdx.x] = outlier.b[threadIdx.x];
    }
    if (a.dev_boundaries != nullptr && threadIdx.x < 16)
        s_b[1][threadIdx.x] = (int)threadIdx.x < a.dev_num_boundaries ? a.dev_boundaries[threadIdx.x] : INFINITY;
    if (threadIdx.x < 32) {
        // src/cache/precomputed/rotation.rs:16-20, stored as a bit mask
        const uint32_t neg = 0xB1A6D4B2u;  // bit j set <=> sign j is -1
        s_sign[threadIdx.x] = ((neg >> threadIdx.x) & 1u) ? -1.0f : 1.0f;
    }
    __syncthreads();

    const long long total_blocks = a.n_rows * a.nblk;
    const long long lane_stride = (long long)gridDim.x * kThreads;
    const int q = threadIdx.x & 3;
    const int n_out = a.dev_boundaries ? a.dev_num_boundaries + 1 : outlier.n;
    const float inv_sqrt = 1.0f / sqrtf((float)kBlock);

    // all 32 lanes of a warp iterate together (total_blocks*4 is rounded up per warp)
    const long long padded = ((total_blocks * 4 + 31) / 32) * 32;
    for (long long gid = (long long)blockIdx.x * kThreads + threadIdx.x; gid < padded; gid += lane_stride) {
        long long blk = gid >> 2;
        const bool live = blk < total_blocks;
        if (!live) blk = total_blocks - 1;
        const long long row = blk / a.nblk;
        const int bv = (int)(blk - row * a.nblk);
        const long long xrow = a.x_row_stride ? a.x_row_stride : (long long)a.nblk * kBlock;
        const T* xp = reinterpret_cast<const T*>(a.x) + row * xrow + bv * kBlock + q * 8;

        float v[8];
        load8<T>(xp, v);
        const bool outl = bv < a.outlier_blocks;
        float scale;
        if (a.norm_mode == TQB_MAXNORM) {
            if (!a.pre_rotated) {
                butterfly8_inlane(v);
                butterfly_cross(v, q);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = (v[i] * inv_sqrt) * s_sign[q * 8 + i];
            }
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            float raw = __fdiv_rn(amax, a.outer_centroid);
            scale = raw > kMinNorm ? raw : kMinNorm;
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fdiv_rn(v[i], scale);
        } else {
            // src/cache/quantize_tensor.rs:93-102: sequential sum of squares over the block
            float s = 0.0f;
#pragma unroll
            for (int owner = 0; owner < 4; ++owner) {
                if (q == owner) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) s = s + v[i] * v[i];
                }
                s = __shfl_sync(0xffffffffu, s, (threadIdx.x & 28) | owner);
            }
            float norm = __fsqrt_rn(s);
            scale = norm > kMinNorm ? norm : kMinNorm;
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fdiv_rn(v[i], scale);
            butterfly8_inlane(v);
            butterfly_cross(v, q);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = (v[i] * inv_sqrt) * s_sign[q * 8 + i];
        }

        const float* bnd = s_b[outl ? 1 : 0];
        const int n = outl ? n_out : normal.n;
        uint32_t mine = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) mine |= (uint32_t)bucket_index_n(v[i], bnd, n) << (BITS * i);

        const long long orow = a.map(row);
        uint8_t* bp = a.indices + (orow * a.nblk + bv) * (4 * BITS);
        const uint32_t next = (BITS == 4) ? 0u : __shfl_down_sync(0xffffffffu, mine, 1);
        if (live) {
            store_codes<BITS>(bp, mine, next, q);
            if (q == 0) a.scales[orow * a.nblk + bv] = f32_to_f16_bits(scale * (outl ? a.scale_sign_outlier : a.scale_sign_normal));
        }
    }
}

// ---- bulk kernel for the PQO layouts (MaxNorm, every block on the outlier codebook) ---------
// One lane owns one 32-element block: the butterfly is 160 register add/subs with no shuffle,
// the max-abs needs no reduction and the packed codes of a lane are 12 or 16 contiguous bytes.
// Arithmetic is the same as in block_quantize_kernel (so the bytes are identical):
//   rot_i = (W_i * 1/sqrt(32)) * sign_i ;  scale = max(amax / outer, 1e-10) ;  t_i = rot_i / scale.
// * Division: r = RN(1/scale) once per block, then q = v*r, rem = fma(-q, scale, v), t = fma(rem, r, q).
//   With a correctly rounded reciprocal and an exact remainder this is the correctly rounded quotient
//   (checked against IEEE division on 4e8 random operand pairs plus all-ones mantissas: 0 differences).
// * 4-bit uniform grid (codebooks.rs:63-73): the code is round((t + R) / step); it is taken from
//   an approximate u (one FMA from W_i) by the 1.5*2^23 magic add.  Only when u lies within 2e-5 of
//   a half-integer could the approximation disagree with the table comparison; such lanes redo
//   their block with exact division and the f32 boundary table.
// NORMAL: every block is on the narrower "normal" codebook (cb, cb.n levels) stored at BITS width, scale sign +
// (the TQ cache layout, outlier_blocks = 0): the cell table serves any sorted boundary set.
template <typename T, int BITS, bool NORMAL>
__global__ void __launch_bounds__(kThreads)
block_quantize_pqo_kernel(QuantArgs a, Codebook cb) {
    if (blockIdx.y != 0) { a.x = a.x2; a.indices = a.indices2; a.scales = a.scales2; }
    __shared__ float2 s_lut[(BITS == 3 || NORMAL) ? 256 : 1];
    const float2* lut = nullptr;
    if (BITS == 3 || NORMAL) {
        build_cell_table(cb, cb.n - 1, s_lut, threadIdx.x, kThreads);
        __syncthreads();
        lut = s_lut;
    }
    const unsigned total = (unsigned)(a.n_rows * a.nblk);
    const unsigned nblk = (unsigned)a.nblk;
    const long long xrow = a.x_row_stride ? a.x_row_stride : (long long)a.nblk * kBlock;

    for (unsigned blk = blockIdx.x * kThreads + threadIdx.x; blk < total; blk += gridDim.x * kThreads) {
        const unsigned row = blk / nblk, bv = blk - row * nblk;
        uint32_t w[4];
        const float scale = pqo_quantize_block<T, BITS, NORMAL>(reinterpret_cast<const T*>(a.x) + (long long)row * xrow + bv * kBlock, cb,
                                                        a.outer_centroid, w, lut);
        long long orow = row;
        if (a.map.rows_per_group != 0) {   // 32-bit division: row and rows_per_group are below 2^31 here
            const unsigned rpg = (unsigned)a.map.rows_per_group;
            const unsigned gi = row / rpg;
            orow = (long long)gi * a.map.group_stride + a.map.row_offset + (row - gi * rpg);
        }
        uint8_t* bp = a.indices + (orow * a.nblk + bv) * (4 * BITS);
        if (BITS == 4) {
            *reinterpret_cast<uint4*>(bp) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
            uint32_t* wp = reinterpret_cast<uint32_t*>(bp);
            wp[0] = w[0]; wp[1] = w[1]; wp[2] = w[2];
        }
        a.scales[orow * a.nblk + bv] = f32_to_f16_bits(scale * (NORMAL ? a.scale_sign_normal : a.scale_sign_outlier));
    }
}

struct DequantArgs {
    const uint8_t* indices;
    const uint16_t* scales;
    void* out;
    long long n_rows;
    RowMap map;  // maps logical row -> storage row
    int nblk;
    int outlier_blocks;   // clamped to [0, nblk]
    const float* dev_codebook;  // legacy entry point
    const float* dev_signs;     // legacy entry point
    float sign_mag;             // |sign| used by the CPU butterfly of the reference
};

// src/cache/quantize_tensor.rs:179-261 + src/cache/wht_tensor.rs:27-65;
// kernel twin: src/cache/cuda/kernels/tq_dequant_kernel.cu:38-98.
template <typename T, int BITS>
__global__ void __launch_bounds__(kThreads)
block_dequantize_kernel(DequantArgs a, Codebook normal, Codebook outlier) {
    __shared__ float s_c[2][16];
    __shared__ float s_sign[32];
    if (threadIdx.x < 16) {
        s_c[0][threadIdx.x] = normal.c[threadIdx.x];
        s_c[1][threadIdx.x] = a.dev_codebook ? ((int)threadIdx.x < (1 << BITS) ? a.dev_codebook[threadIdx.x] : 0.0f)
                                             : outlier.c[threadIdx.x];
    }
    if (threadIdx.x < 32) {
        const uint32_t neg = 0xB1A6D4B2u;
        s_sign[threadIdx.x] = a.dev_signs ? a.dev_signs[threadIdx.x]
                                          : (((neg >> threadIdx.x) & 1u) ? -a.sign_mag : a.sign_mag);
    }
    __syncthreads();

    const long long total_blocks = a.n_rows * a.nblk;
    const long long lane_stride = (long long)gridDim.x * kThreads;
    const int q = threadIdx.x & 3;
    const float inv_sqrt = 1.0f / sqrtf((float)kBlock);
    const long long padded = ((total_blocks * 4 + 31) / 32) * 32;
    const uint32_t* words = reinterpret_cast<const uint32_t*>(a.indices);

    for (long long gid = (long long)blockIdx.x * kThreads + threadIdx.x; gid < padded; gid += lane_stride) {
        long long blk = gid >> 2;
        const bool live = blk < total_blocks;
        if (!live) blk = total_blocks - 1;
        const long long row = blk / a.nblk;
        const int bv = (int)(blk - row * a.nblk);
        const long long srow = a.map(row);
        const long long sblk = srow * a.nblk + bv;

        // this lane's BITS bytes start at byte BITS*q of the block
        const long long byte0 = sblk * (4 * BITS) + BITS * q;
        uint32_t w0 = __ldg(words + (byte0 >> 2));
        uint32_t code_bits;
        if (BITS == 4) {
            code_bits = w0;
        } else {
            const int sh = (int)(byte0 & 3) * 8;
            uint32_t w1 = (sh + 8 * BITS > 32) ? __ldg(words + (byte0 >> 2) + 1) : 0u;
            code_bits = __funnelshift_r(w0, w1, sh);
        }
        const float sc = f16_bits_to_f32(__ldg(a.scales + sblk));
        bool outl;
        if (a.outlier_blocks >= a.nblk) outl = true;
        else if (a.outlier_blocks == 0) outl = false;
        else outl = sc < 0.0f;
        const float* cb = s_c[outl ? 1 : 0];
        const int nmax = outl ? (1 << BITS) - 1 : normal.n - 1;

        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int id = (int)((code_bits >> (BITS * i)) & ((1u << BITS) - 1u));
            id = id > nmax ? nmax : id;
            v[i] = cb[id] * s_sign[q * 8 + i];
        }
        butterfly8_inlane(v);
        butterfly_cross(v, q);
        const float as = fabsf(sc);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (v[i] * inv_sqrt) * as;
        if (live) store8<T>(reinterpret_cast<T*>(a.out) + (row * a.nblk + bv) * kBlock + q * 8, v);
    }
}

// src/cache/cuda/kernels/tq_quant_kernel.cu:387-414: pack a u8 code tensor; one thread per
// group of eight codes (= BITS output bytes).
template <int BITS>
__global__ void pack_kernel(const uint8_t* __restrict__ idx, uint8_t* __restrict__ out, long long groups) {
    long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= groups) return;
    uint2 r = *reinterpret_cast<const uint2*>(idx + g * 8);
    uint64_t codes = ((uint64_t)r.y << 32) | r.x;
    uint32_t bits = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) bits |= (uint32_t)((codes >> (8 * i)) & ((1u << BITS) - 1u)) << (BITS * i);
#pragma unroll
    for (int b = 0; b < BITS; ++b) out[g * BITS + b] = (uint8_t)(bits >> (8 * b));
}

int grid_for(long long work_items) {
    long long blocks = (work_items + kThreads - 1) / kThreads;
    const long long cap = 148LL * 16;  // 148 SMs x resident CTAs; the kernels grid-stride
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

template <typename T>
int launch_quant(int bits, const QuantArgs& a, const Codebook& n, const Codebook& o, cudaStream_t s) {
    const long long blocks = a.n_rows * a.nblk;
    const bool one_table = a.norm_mode == TQB_MAXNORM && !a.pre_rotated && a.dev_boundaries == nullptr &&
                           (bits == 3 || bits == 4) && blocks < (1LL << 31) && a.map.rows_per_group < (1LL << 31) &&
                           ((uintptr_t)a.indices % 16) == 0 && ((uintptr_t)a.indices2 % 16) == 0;
    if (one_table && a.outlier_blocks >= a.nblk) {   // every block on the outlier codebook
        const dim3 grid(grid_for(blocks), a.x2 ? 2 : 1);
        if (bits == 4) block_quantize_pqo_kernel<T, 4, false><<<grid, kThreads, 0, s>>>(a, o);
        else block_quantize_pqo_kernel<T, 3, false><<<grid, kThreads, 0, s>>>(a, o);
        return check_launch(s);
    }
    if (one_table && a.outlier_blocks == 0) {        // every block on the normal codebook
        const dim3 grid(grid_for(blocks), a.x2 ? 2 : 1);
        if (bits == 4) block_quantize_pqo_kernel<T, 4, true><<<grid, kThreads, 0, s>>>(a, n);
        else block_quantize_pqo_kernel<T, 3, true><<<grid, kThreads, 0, s>>>(a, n);
        return check_launch(s);
    }
    const long long lanes = a.n_rows * a.nblk * 4;
    const dim3 grid(grid_for(lanes), a.x2 ? 2 : 1);
    switch (bits) {
        case 2: block_quantize_kernel<T, 2><<<grid, kThreads, 0, s>>>(a, n, o); break;
        case 3: block_quantize_kernel<T, 3><<<grid, kThreads, 0, s>>>(a, n, o); break;
        default: block_quantize_kernel<T, 4><<<grid, kThreads, 0, s>>>(a, n, o); break;
    }
    return check_launch(s);
}

template <typename T>
int launch_dequant(int bits, const DequantArgs& a, const Codebook& n, const Codebook& o, cudaStream_t s) {
    const long long lanes = a.n_rows * a.nblk * 4;
    const int grid = grid_for(lanes);
    switch (bits) {
        case 2: block_dequantize_kernel<T, 2><<<grid, kThreads, 0, s>>>(a, n, o); break;
        case 3: block_dequantize_kernel<T, 3><<<grid, kThreads, 0, s>>>(a, n, o); break;
        default: block_dequantize_kernel<T, 4><<<grid, kThreads, 0, s>>>(a, n, o); break;
    }
    return check_launch(s);
}

inline float cpu_sign_magnitude() {
    // src/cache/wht_tensor.rs:29-35,43: rotation_fwd[0][j] * sqrt(32), all in f32
    volatile float inv = 1.0f / sqrtf(32.0f);
    volatile float s = sqrtf(32.0f);
    return inv * s;
}

}  // namespace

int block_cfg_check(int bits, int head_dim, int norm_mode) {
    if (bits < 3 || bits > 4) return TQB_ERR_UNSUPPORTED_BITS;          // precomputed/mod.rs:46-51
    if (head_dim <= 0 || head_dim % kBlock != 0) return TQB_ERR_INVALID_DIMENSION;  // pqo.rs:32-39
    if (norm_mode != TQB_MAXNORM && norm_mode != TQB_L2NORM) return TQB_ERR_INVALID_ARGUMENT;
    return TQB_OK;
}

}  // namespace tqb

using namespace tqb;

extern "C" {

static int block_quantize_impl(int32_t bits, int32_t head_dim, int32_t norm_mode, int32_t outlier_blocks, const void* x,
                               const void* x2, int32_t x_dtype, int64_t n, int64_t x_row_stride, uint8_t* indices,
                               uint16_t* scales, uint8_t* indices2, uint16_t* scales2, int64_t rows_per_group,
                               int64_t out_group_stride, int64_t out_row_offset, tqb_stream_t stream) {
    int st = block_cfg_check(bits, head_dim, norm_mode);
    if (st != TQB_OK) return st;
    if (n < 0 || x_row_stride < 0 || rows_per_group < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (n == 0) return TQB_OK;
    if (!x || !indices || !scales) return TQB_ERR_NULL_POINTER;
    if (x2 && (!indices2 || !scales2)) return TQB_ERR_NULL_POINTER;
    if (x_row_stride != 0 && x_row_stride < head_dim) return TQB_ERR_INVALID_ARGUMENT;
    const size_t esz = x_dtype == TQB_F32 ? 4 : 2;
    if (x_dtype != TQB_F32 && x_dtype != TQB_F16 && x_dtype != TQB_BF16) return TQB_ERR_INVALID_ARGUMENT;
    if (((uintptr_t)x % 16) != 0 || ((x_row_stride * esz) % 16) != 0 || ((uintptr_t)indices % 4) != 0 ||
        ((uintptr_t)scales % 2) != 0)
        return TQB_ERR_MISALIGNED;
    if (x2 && (((uintptr_t)x2 % 16) != 0 || ((uintptr_t)indices2 % 4) != 0 || ((uintptr_t)scales2 % 2) != 0))
        return TQB_ERR_MISALIGNED;
    Codebook cn, co;
    if (!block_codebook(bits - 1, norm_mode, cn) || !block_codebook(bits, norm_mode, co)) return TQB_ERR_UNSUPPORTED_BITS;
    QuantArgs a{};
    a.x = x;
    a.n_rows = n;
    a.x_row_stride = x_row_stride;
    a.indices = indices;
    a.scales = scales;
    a.x2 = x2;
    a.indices2 = x2 ? indices2 : nullptr;
    a.scales2 = x2 ? scales2 : nullptr;
    a.map = RowMap{rows_per_group, out_group_stride, out_row_offset};
    a.nblk = head_dim / kBlock;
    a.outlier_blocks = outlier_blocks < 0 || outlier_blocks > a.nblk ? a.nblk : outlier_blocks;
    a.norm_mode = norm_mode;
    a.pre_rotated = 0;
    a.outer_centroid = co.c[co.n - 1];  // precomputed/mod.rs:78
    a.scale_sign_outlier = -1.0f;       // precomputed/mod.rs:103-115
    a.scale_sign_normal = 1.0f;
    a.dev_boundaries = nullptr;
    a.dev_num_boundaries = 0;
    cudaStream_t s = as_stream(stream);
    if (x_dtype == TQB_F32) return launch_quant<float>(bits, a, cn, co, s);
    if (x_dtype == TQB_F16) return launch_quant<__half>(bits, a, cn, co, s);
    return launch_quant<__nv_bfloat16>(bits, a, cn, co, s);
}

int tqb_block_quantize(int32_t bits, int32_t head_dim, int32_t norm_mode, int32_t outlier_blocks, const void* x,
                       int32_t x_dtype, int64_t n, int64_t x_row_stride, uint8_t* indices, uint16_t* scales,
                       int64_t rows_per_group, int64_t out_group_stride, int64_t out_row_offset,
                       tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    return block_quantize_impl(bits, head_dim, norm_mode, outlier_blocks, x, nullptr, x_dtype, n, x_row_stride, indices,
                               scales, nullptr, nullptr, rows_per_group, out_group_stride, out_row_offset, stream);
}

int tqb_block_quantize_pair(int32_t bits, int32_t head_dim, int32_t norm_mode, int32_t outlier_blocks, const void* k,
                            const void* v, int32_t x_dtype, int64_t n, int64_t x_row_stride, uint8_t* k_indices,
                            uint16_t* k_scales, uint8_t* v_indices, uint16_t* v_scales, int64_t rows_per_group,
                            int64_t out_group_stride, int64_t out_row_offset, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (n > 0 && !v) return TQB_ERR_NULL_POINTER;
    return block_quantize_impl(bits, head_dim, norm_mode, outlier_blocks, k, v, x_dtype, n, x_row_stride, k_indices,
                               k_scales, v_indices, v_scales, rows_per_group, out_group_stride, out_row_offset, stream);
}

int tqb_block_dequantize(int32_t bits, int32_t head_dim, int32_t norm_mode, int32_t outlier_blocks,
                         const uint8_t* indices, const uint16_t* scales, int64_t n, int64_t rows_per_group,
                         int64_t in_group_stride, int64_t in_row_offset, void* out, int32_t out_dtype,
                         tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    int st = block_cfg_check(bits, head_dim, norm_mode);
    if (st != TQB_OK) return st;
    if (n < 0 || rows_per_group < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (n == 0) return TQB_OK;
    if (!indices || !scales || !out) return TQB_ERR_NULL_POINTER;
    if (out_dtype != TQB_F32 && out_dtype != TQB_F16 && out_dtype != TQB_BF16) return TQB_ERR_INVALID_ARGUMENT;
    if (((uintptr_t)out % 16) != 0 || ((uintptr_t)indices % 4) != 0 || ((uintptr_t)scales % 2) != 0)
        return TQB_ERR_MISALIGNED;
    Codebook cn, co;
    if (!block_codebook(bits - 1, norm_mode, cn) || !block_codebook(bits, norm_mode, co)) return TQB_ERR_UNSUPPORTED_BITS;
    DequantArgs a{};
    a.indices = indices;
    a.scales = scales;
    a.out = out;
    a.n_rows = n;
    a.map = RowMap{rows_per_group, in_group_stride, in_row_offset};
    a.nblk = head_dim / kBlock;
    a.outlier_blocks = outlier_blocks < 0 || outlier_blocks > a.nblk ? a.nblk : outlier_blocks;
    a.dev_codebook = nullptr;
    a.dev_signs = nullptr;
    a.sign_mag = cpu_sign_magnitude();
    cudaStream_t s = as_stream(stream);
    if (out_dtype == TQB_F32) return launch_dequant<float>(bits, a, cn, co, s);
    if (out_dtype == TQB_F16) return launch_dequant<__half>(bits, a, cn, co, s);
    return launch_dequant<__nv_bfloat16>(bits, a, cn, co, s);
}

// ---- the reference's launchers ------------------------------------------------------------

int tqb_dequant_batch(const uint8_t* packed_indices, const uint16_t* scales, const float* codebook,
                      const float* sign_pattern, float* output, int32_t num_blocks, int32_t block_size, int32_t bits,
                      int32_t bytes_per_block, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (num_blocks == 0) return TQB_OK;  // tq_dequant_kernel.cu:116
    if (num_blocks < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (bits < 2 || bits > 4) return TQB_ERR_UNSUPPORTED_BITS;
    if (block_size != kBlock) return TQB_ERR_UNSUPPORTED;
    if (bytes_per_block != block_size * bits / 8) return TQB_ERR_DIMENSION_MISMATCH;
    if (!packed_indices || !scales || !codebook || !sign_pattern || !output) return TQB_ERR_NULL_POINTER;
    if (((uintptr_t)output % 16) != 0 || ((uintptr_t)packed_indices % 4) != 0) return TQB_ERR_MISALIGNED;
    Codebook dummy{};
    dummy.n = 1 << bits;
    DequantArgs a{};
    a.indices = packed_indices;
    a.scales = scales;
    a.out = output;
    a.n_rows = num_blocks;
    a.map = RowMap{0, 0, 0};
    a.nblk = 1;
    a.outlier_blocks = 1;  // the caller's codebook decodes every block
    a.dev_codebook = codebook;
    a.dev_signs = sign_pattern;
    a.sign_mag = 1.0f;
    return launch_dequant<float>(bits, a, dummy, dummy, as_stream(stream));
}

int tqb_quant_maxnorm_batch(const float* rotated_input, const float* boundaries, uint8_t* packed_out,
                            uint16_t* scales_out, int32_t num_blocks, int32_t block_size, int32_t bits,
                            int32_t num_boundaries, int32_t bytes_per_block, float outer_centroid, float scale_sign,
                            tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (num_blocks == 0) return TQB_OK;  // tq_quant_kernel.cu:430
    if (num_blocks < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (bits < 2 || bits > 4) return TQB_ERR_UNSUPPORTED_BITS;
    if (block_size != kBlock) return TQB_ERR_UNSUPPORTED;
    if (bytes_per_block != block_size * bits / 8) return TQB_ERR_DIMENSION_MISMATCH;
    if (num_boundaries < 1 || num_boundaries > 15) return TQB_ERR_INVALID_ARGUMENT;
    // the bisection needs a power-of-two centroid count
    if (((num_boundaries + 1) & num_boundaries) != 0 || num_boundaries + 1 < 4) return TQB_ERR_UNSUPPORTED;
    if (!rotated_input || !boundaries || !packed_out || !scales_out) return TQB_ERR_NULL_POINTER;
    if (((uintptr_t)rotated_input % 16) != 0 || ((uintptr_t)packed_out % 4) != 0) return TQB_ERR_MISALIGNED;
    Codebook dummy{};
    dummy.n = num_boundaries + 1;
    for (int i = 0; i < 16; ++i) dummy.b[i] = INFINITY;
    QuantArgs a{};
    a.x = rotated_input;
    a.n_rows = num_blocks;
    a.x_row_stride = 0;
    a.indices = packed_out;
    a.scales = scales_out;
    a.map = RowMap{0, 0, 0};
    a.nblk = 1;
    a.outlier_blocks = 1;
    a.norm_mode = TQB_MAXNORM;
    a.pre_rotated = 1;
    a.outer_centroid = outer_centroid;
    a.scale_sign_outlier = scale_sign;
    a.scale_sign_normal = scale_sign;
    a.dev_boundaries = boundaries;
    a.dev_num_boundaries = num_boundaries;
    return launch_quant<float>(bits, a, dummy, dummy, as_stream(stream));
}

int tqb_pack_indices(const uint8_t* indices, uint8_t* packed_out, int32_t num_vectors, int32_t block_size,
                     int32_t bits, int32_t bytes_per_block, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (num_vectors == 0) return TQB_OK;  // tq_quant_kernel.cu:450
    if (num_vectors < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (bits < 2 || bits > 4) return TQB_ERR_UNSUPPORTED_BITS;
    if (block_size <= 0 || block_size % 8 != 0) return TQB_ERR_INVALID_DIMENSION;
    if (bytes_per_block != block_size * bits / 8) return TQB_ERR_DIMENSION_MISMATCH;
    if (!indices || !packed_out) return TQB_ERR_NULL_POINTER;
    if (((uintptr_t)indices % 8) != 0) return TQB_ERR_MISALIGNED;
    const long long groups = (long long)num_vectors * (block_size / 8);
    const int grid = (int)((groups + 255) / 256);
    cudaStream_t s = as_stream(stream);
    switch (bits) {
        case 2: pack_kernel<2><<<grid, 256, 0, s>>>(indices, packed_out, groups); break;
        case 3: pack_kernel<3><<<grid, 256, 0, s>>>(indices, packed_out, groups); break;
        default: pack_kernel<4><<<grid, 256, 0, s>>>(indices, packed_out, groups); break;
    }
    return check_launch(s);
}

void tq_dequant_batch(const uint8_t* packed_indices, const uint16_t* scales, const float* codebook,
                      const float* sign_pattern, float* output, int32_t num_blocks, int32_t block_size, int32_t bits,
                      int32_t bytes_per_block, tqb_stream_t stream) {
    (void)tqb_dequant_batch(packed_indices, scales, codebook, sign_pattern, output, num_blocks, block_size, bits,
                            bytes_per_block, stream);
}

void tq_quant_maxnorm_batch(const float* rotated_input, const float* boundaries, uint8_t* packed_out,
                            uint16_t* scales_out, int32_t num_blocks, int32_t block_size, int32_t bits,
                            int32_t num_boundaries, int32_t bytes_per_block, float outer_centroid, float scale_sign,
                            tqb_stream_t stream) {
    (void)tqb_quant_maxnorm_batch(rotated_input, boundaries, packed_out, scales_out, num_blocks, block_size, bits,
                                  num_boundaries, bytes_per_block, outer_centroid, scale_sign, stream);
}

void tq_pack_indices(const uint8_t* indices, uint8_t* packed_out, int32_t num_vectors, int32_t block_size, int32_t bits,
                     int32_t bytes_per_block, tqb_stream_t stream) {
    (void)tqb_pack_indices(indices, packed_out, num_vectors, block_size, bits, bytes_per_block, stream);
}

}  // extern "C"
