// CPU oracle for the TurboQuant quantize -> pack -> (QJL sketch) -> attend path.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, in plain single-precision C++, the
// arithmetic of the reference crate `turboquant-rs` 0.3.1 so that the CUDA library can
// be checked against it.  Nothing in the shipped library may call into it; only the
// test-suite, the smoke check and the CPU-baseline leg of the benchmark do.
//
// Parity status: the reference's own Rust code cannot be built without a Rust toolchain,
// so this restatement is pinned against (a) the reference's host-compilable header
// `src/cache/cuda/kernels/tq_common.h` (bit packing, sign pattern, Rademacher hash), (b) the
// reference's own block-32 quantize and dequantize CUDA kernels (tq_quant_kernel.cu:204-262,
// tq_dequant_kernel.cu:38-98), compiled from the reference checkout and run on the GPU beside
// this file's block_quantize_one / block_dequantize_one on the same rotated blocks, and (c) the
// known-answer facts asserted by the reference's tests (see tests/).  Two items stay "parity
// unpinned" because their arithmetic lives in the un-vendored `candle-core` dependency: the
// summation order of the block-32 forward rotation (a matmul in the reference, a butterfly
// here) and softmax/SDPA for the non-fused path.
//
// Build: g++ -O3 -march=native -ffp-contract=off -shared -fPIC (see Makefile).
// -ffp-contract=off matters: Rust never fuses a*b+c, so neither may this file.
//
// Every function cites the reference file:line it follows.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

// ---------------------------------------------------------------------------------
// Codebook tables: src/codebook/tables.rs:111-377, transcribed by gen_tables.py.
// ---------------------------------------------------------------------------------
struct Table {
    int bits, dim, n;
    double centroids[16];
    double boundaries[15];
};
#define TQ_UNPAREN(...) __VA_ARGS__
#define TQ_TABLE(bits, dim, n, c, b) {bits, dim, n, {TQ_UNPAREN c}, {TQ_UNPAREN b}},
const Table kTables[] = {
#include "codebook_tables.inc"
};
#undef TQ_TABLE

// src/codebook/tables.rs:89-105 (lookup_static_codebook_ref).  Dimensions outside the
// table would be generated on the fly by the reference (codebook/gen.rs); the oracle
// refuses them.
const Table* find_table(int bits, int dim) {
    for (const Table& t : kTables)
        if (t.bits == bits && t.dim == dim) return &t;
    return nullptr;
}

// IEEE binary16 <-> binary32, round-to-nearest-even, as crate `half` 2.x does
// (src/quantize.rs:125, :236).
inline uint16_t f32_to_f16_bits(float f) {
    _Float16 h = (_Float16)f;
    uint16_t u;
    std::memcpy(&u, &h, 2);
    return u;
}
inline float f16_bits_to_f32(uint16_t u) {
    _Float16 h;
    std::memcpy(&h, &u, 2);
    return (float)h;
}

// src/rotation.rs:22-40 (wht_inplace): stages h = 1, 2, 4, ...; then scale by
// 1.0 / sqrt(n) computed in f32.
void wht_inplace(float* data, int n) {
    for (int h = 1; h < n; h *= 2)
        for (int i = 0; i < n; i += 2 * h)
            for (int j = i; j < i + h; ++j) {
                float x = data[j], y = data[j + h];
                data[j] = x + y;
                data[j + h] = x - y;
            }
    float norm = 1.0f / std::sqrt((float)n);
    for (int i = 0; i < n; ++i) data[i] *= norm;
}

// src/rotation.rs:47-70 (golden_ratio_hash, generate_sign_pattern).
inline float sign_at(uint64_t seed, uint64_t index) {
    uint64_t h = (seed + index) * 0x9E3779B97F4A7C15ULL;
    return (h & 1ULL) == 0 ? 1.0f : -1.0f;
}

// src/quantize.rs:51-53 (l2_norm): sequential f32 sum of squares, then sqrt.
inline float l2_norm(const float* x, int n) {
    float s = 0.0f;
    for (int i = 0; i < n; ++i) s += x[i] * x[i];
    return std::sqrt(s);
}

// src/codebook/mod.rs:66-87 (boundary_binary_search / nearest_centroid): the index is
// the number of interior boundaries strictly below the value, compared in f64.
inline uint8_t nearest_centroid(double v, const double* boundaries, int nb) {
    int lo = 0, hi = nb;
    while (lo < hi) {
        int mid = lo + (hi - lo) / 2;
        if (v > boundaries[mid]) lo = mid + 1; else hi = mid;
    }
    return (uint8_t)lo;
}

// src/packed/mod.rs:242-309 and src/packed/indices.rs:152-281.  All three widths are a
// little-endian LSB-first bit stream: code k occupies bits [k*bits, (k+1)*bits); a
// trailing partial group is zero padded to a whole group (4 codes -> 1 byte for 2-bit,
// 8 codes -> 3 bytes for 3-bit, 2 codes -> 1 byte for 4-bit).
size_t packed_len(int bits, size_t count) {
    switch (bits) {
        case 2: return (count + 3) / 4;
        case 3: return ((count + 7) / 8) * 3;
        default: return (count + 1) / 2;
    }
}
void pack_indices(int bits, const uint8_t* idx, size_t count, uint8_t* out) {
    size_t nbytes = packed_len(bits, count);
    std::memset(out, 0, nbytes);
    const uint8_t mask = (uint8_t)((1u << bits) - 1u);
    for (size_t k = 0; k < count; ++k) {
        uint32_t v = idx[k] & mask;
        size_t bit = k * (size_t)bits;
        out[bit >> 3] |= (uint8_t)(v << (bit & 7));
        if ((bit & 7) + bits > 8) out[(bit >> 3) + 1] |= (uint8_t)(v >> (8 - (bit & 7)));
    }
}
void unpack_indices(int bits, const uint8_t* packed, size_t count, uint8_t* out) {
    const uint32_t mask = (1u << bits) - 1u;
    for (size_t k = 0; k < count; ++k) {
        size_t bit = k * (size_t)bits;
        uint32_t w = packed[bit >> 3];
        if ((bit & 7) + bits > 8) w |= (uint32_t)packed[(bit >> 3) + 1] << 8;
        out[k] = (uint8_t)((w >> (bit & 7)) & mask);
    }
}

// src/qjl.rs:143-171 (mix_seed, rademacher_sign_from_hash).
inline uint64_t mix_seed(uint64_t seed, uint64_t row) {
    uint64_t mixed = seed * 0x517CC1B727220A95ULL + row;
    return mixed ^ (mixed >> 32) ^ 0x6C62272E07BB0142ULL;
}
inline float rademacher_sign(uint64_t row_seed, uint64_t row, uint64_t col) {
    uint64_t z = row_seed + row * 0x9E3779B97F4A7C15ULL + col;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    z = z ^ (z >> 31);
    return (z & 1ULL) == 0 ? 1.0f : -1.0f;
}
// src/qjl.rs:196-208 (rademacher_vector_product): sequential f32 sum of sign*x, then
// one multiply by 1/sqrt(dim).
inline float rademacher_vector_product(const float* x, int dim, uint64_t seed, int row) {
    uint64_t rs = mix_seed(seed, (uint64_t)row);
    float inv = 1.0f / std::sqrt((float)dim);
    float s = 0.0f;
    for (int c = 0; c < dim; ++c) s += rademacher_sign(rs, (uint64_t)row, (uint64_t)c) * x[c];
    return s * inv;
}

struct PolarCtx {
    int bits, dim;
    const Table* tab;
    std::vector<float> signs;
    std::vector<float> centroids_f32;  // src/quantize.rs:97-102: `centroid as f32`
};
bool make_ctx(PolarCtx& c, int bits, int dim, uint64_t seed) {
    if (bits < 2 || bits > 4) return false;
    if (dim <= 0 || (dim & (dim - 1)) != 0) return false;
    c.tab = find_table(bits, dim);
    if (!c.tab) return false;
    c.bits = bits;
    c.dim = dim;
    c.signs.resize(dim);
    for (int i = 0; i < dim; ++i) c.signs[i] = sign_at(seed, (uint64_t)i);
    c.centroids_f32.resize(c.tab->n);
    for (int i = 0; i < c.tab->n; ++i) c.centroids_f32[i] = (float)c.tab->centroids[i];
    return true;
}

// src/quantize.rs:142-192 (quantize_vec / quantize_vec_with_codebook).
void quantize_one(const PolarCtx& c, const float* x, uint8_t* packed, uint16_t* scale_bits,
                  float* work, uint8_t* idx) {
    const int d = c.dim;
    float norm = l2_norm(x, d);
    // src/quantize.rs:60-72 (normalize_inplace)
    if (norm < 1e-10f) {
        for (int i = 0; i < d; ++i) work[i] = 0.0f;
    } else {
        float inv = 1.0f / norm;
        for (int i = 0; i < d; ++i) work[i] = x[i] * inv;
    }
    // src/rotation.rs:137-143 (Forward: sign flip then WHT)
    for (int i = 0; i < d; ++i) work[i] *= c.signs[i];
    wht_inplace(work, d);
    // src/quantize.rs:87-92 (quantize_coordinates)
    for (int i = 0; i < d; ++i)
        idx[i] = nearest_centroid((double)work[i], c.tab->boundaries, c.tab->n - 1);
    // src/quantize.rs:123-126 (select_scale)
    *scale_bits = f32_to_f16_bits(norm < 1e-10f ? 0.0f : norm);
    pack_indices(c.bits, idx, (size_t)d, packed);
}

// src/quantize.rs:225-239 (dequantize_vec_with_codebook).
void dequantize_one(const PolarCtx& c, const uint8_t* packed, uint16_t scale_bits, float* out,
                    uint8_t* idx) {
    const int d = c.dim;
    unpack_indices(c.bits, packed, (size_t)d, idx);
    for (int i = 0; i < d; ++i) out[i] = c.centroids_f32[idx[i]];
    // src/rotation.rs:144-147 (Inverse: WHT then sign flip)
    wht_inplace(out, d);
    for (int i = 0; i < d; ++i) out[i] *= c.signs[i];
    float s = f16_bits_to_f32(scale_bits);
    for (int i = 0; i < d; ++i) out[i] *= s;
}

template <class F>
void parallel_for(int64_t n, int nthreads, F f) {
    if (nthreads <= 1 || n < 2) {
        f(0, n, 0);
        return;
    }
    std::vector<std::thread> th;
    int64_t chunk = (n + nthreads - 1) / nthreads;
    for (int t = 0; t < nthreads; ++t) {
        int64_t lo = t * chunk, hi = std::min<int64_t>(n, lo + chunk);
        if (lo >= hi) break;
        th.emplace_back([=] { f(lo, hi, t); });
    }
    for (auto& x : th) x.join();
}

// ---------------------------------------------------------------------------------
// Block-32 format of the `cache/` module ("PQ", "PQO", "TQ" caches).
// ---------------------------------------------------------------------------------
constexpr int kBlock = 32;  // src/cache/config.rs:9 (QUANT_BLOCK_SIZE)

// src/cache/precomputed/rotation.rs:16-20: fixed sign pattern for block size 32.
const float kBlockSigns[32] = {1, -1, 1, 1, -1, -1, 1, -1, 1, 1, -1, 1, -1, 1, -1, -1,
                               1, -1, -1, 1, 1, -1, 1, -1, -1, 1, 1, 1, -1, -1, 1, -1};

struct BlockCodebook {
    int n;                 // number of centroids
    float centroids[16];
    float boundaries[15];
};

// src/cache/precomputed/codebooks.rs:18-88 (build_codebooks_l2 / build_codebooks_maxnorm).
// `cb_bits` is the width of the codebook itself (bits for outlier blocks, bits-1 for
// normal blocks).  norm_mode: 0 = MaxNorm, 1 = L2Norm.
bool block_codebook(int cb_bits, int norm_mode, BlockCodebook& cb) {
    if (cb_bits < 2 || cb_bits > 4) return false;
    cb.n = 1 << cb_bits;
    if (norm_mode == 1) {
        const Table* t = find_table(cb_bits, kBlock);
        if (!t) return false;
        for (int i = 0; i < t->n; ++i) cb.centroids[i] = (float)t->centroids[i];
        for (int i = 0; i < t->n - 1; ++i) cb.boundaries[i] = (float)t->boundaries[i];
        return true;
    }
    const float R = 2.1573f;
    if (cb_bits == 3) {
        const float c3[8] = {-2.1573f, -1.3336f, -0.7434f, -0.2428f, 0.2428f, 0.7434f, 1.3336f, 2.1573f};
        const float b3[7] = {-1.7455f, -1.0385f, -0.4931f, 0.0f, 0.4931f, 1.0385f, 1.7455f};
        std::copy(c3, c3 + 8, cb.centroids);
        std::copy(b3, b3 + 7, cb.boundaries);
    } else if (cb_bits == 2) {
        const float c2[4] = {-R, -0.7434f, 0.7434f, R};
        const float b2[3] = {-1.0385f, 0.0f, 1.0385f};
        std::copy(c2, c2 + 4, cb.centroids);
        std::copy(b2, b2 + 3, cb.boundaries);
    } else {
        // codebooks.rs:63-73: uniform grid, all arithmetic in f32
        const float full = 2.0f * R;
        const float step = full / 15.0f;
        for (int i = 0; i < 16; ++i) cb.centroids[i] = -R + (float)i * step;
        for (int i = 0; i < 15; ++i) cb.boundaries[i] = -R + ((float)i + 0.5f) * step;
    }
    return true;
}

inline void butterfly32(float* b) {
    for (int h = 1; h < kBlock; h <<= 1)
        for (int i = 0; i < kBlock; i += 2 * h)
            for (int j = i; j < i + h; ++j) {
                float x = b[j], y = b[j + h];
                b[j] = x + y;
                b[j + h] = x - y;
            }
}

// Forward rotation of one block: x @ (H/sqrt(32) * diag(signs))
// (src/cache/precomputed/rotation.rs:26, src/cache/quantize_tensor.rs:100,104).  The
// reference evaluates it as a matmul whose summation order is not specified; the oracle
// fixes it as the butterfly of src/cache/wht_tensor.rs:44-59, then *1/sqrt(32), then the
// sign.
inline void rotate_block_fwd(const float* x, float* out) {
    float b[kBlock];
    std::copy(x, x + kBlock, b);
    butterfly32(b);
    const float inv = 1.0f / std::sqrt((float)kBlock);
    for (int j = 0; j < kBlock; ++j) out[j] = (b[j] * inv) * kBlockSigns[j];
}

inline uint8_t bucketize(float v, const float* boundaries, int nb) {
    // src/cache/quantize_tensor.rs:161-176 (broadcast_gt + sum);
    // src/cache/cuda/kernels/tq_quant_kernel.cu:235-241.
    int c = 0;
    for (int k = 0; k < nb; ++k) c += (v > boundaries[k]) ? 1 : 0;
    return (uint8_t)c;
}

struct BlockCfg {
    int bits, head_dim, norm_mode, outlier_blocks, nblk, packed_dim;
    BlockCodebook normal, outlier;
};
bool make_block_cfg(BlockCfg& c, int bits, int head_dim, int norm_mode, int outlier_blocks) {
    // src/cache/precomputed/mod.rs:45-51 (bits 3 or 4), src/cache/pqo.rs:32-39.
    if (bits < 3 || bits > 4) return false;
    if (head_dim <= 0 || head_dim % kBlock != 0) return false;
    c.bits = bits;
    c.head_dim = head_dim;
    c.norm_mode = norm_mode;
    c.nblk = head_dim / kBlock;
    c.outlier_blocks = std::min(std::max(outlier_blocks, 0), c.nblk);
    c.packed_dim = head_dim * bits / 8;
    return block_codebook(bits - 1, norm_mode, c.normal) && block_codebook(bits, norm_mode, c.outlier);
}

// src/cache/quantize_tensor.rs:40-176 (polar_quantize, normalize_and_rotate,
// bucketize_blocks) with the scalar arithmetic of
// src/cache/cuda/kernels/tq_quant_kernel.cu:216-259 for MaxNorm
// (scale = max(amax / outer_centroid, 1e-10); scaled = rotated / scale).
// The first `outlier_blocks` blocks of each vector use the outlier codebook and store a
// negated scale (src/cache/precomputed/mod.rs:103-115).
// Mixed configurations (0 < outlier_blocks < num_blocks) are ORACLE-DEFINED, not reference-pinned: the
// reference contradicts itself there.  Its scale signs mark the first `outlier_blocks` blocks of EACH vector
// (precomputed/mod.rs:102-114), but bucketize_blocks (quantize_tensor.rs:118-158) gives the outlier codebook
// to the first n * outlier_blocks ROWS of the flattened [n * num_blocks, 32] tensor, i.e. to whole leading
// vectors when n > 1.  This restatement follows the per-vector reading for both, the only one under which
// dequantize (which goes by the sign of the scale) inverts quantize.  The two documented modes, all blocks
// (PQO) and none (PQ / TQ), are unaffected.
void block_quantize_one(const BlockCfg& c, const float* x, uint8_t* packed, uint16_t* scales) {
    std::vector<uint8_t> idx(c.head_dim);
    for (int b = 0; b < c.nblk; ++b) {
        const bool outl = b < c.outlier_blocks;
        const BlockCodebook& cb = outl ? c.outlier : c.normal;
        float rot[kBlock];
        float scale;
        if (c.norm_mode == 0) {
            rotate_block_fwd(x + b * kBlock, rot);
            float amax = 0.0f;
            for (int j = 0; j < kBlock; ++j) amax = std::max(amax, std::fabs(rot[j]));
            // src/cache/precomputed/mod.rs:81: outer centroid always taken from the
            // outlier codebook, also for normal blocks.
            float outer = c.outlier.centroids[c.outlier.n - 1];
            float raw = amax / outer;
            scale = raw > 1e-10f ? raw : 1e-10f;
            for (int j = 0; j < kBlock; ++j) rot[j] = rot[j] / scale;
        } else {
            // src/cache/quantize_tensor.rs:93-102 (L2Norm): norm, clamp, divide, rotate.
            float s = 0.0f;
            for (int j = 0; j < kBlock; ++j) s += x[b * kBlock + j] * x[b * kBlock + j];
            float norm = std::sqrt(s);
            scale = norm > 1e-10f ? norm : 1e-10f;
            float tmp[kBlock];
            for (int j = 0; j < kBlock; ++j) tmp[j] = x[b * kBlock + j] / scale;
            rotate_block_fwd(tmp, rot);
        }
        for (int j = 0; j < kBlock; ++j) idx[b * kBlock + j] = bucketize(rot[j], cb.boundaries, cb.n - 1);
        scales[b] = f32_to_f16_bits(outl ? -scale : scale);
    }
    pack_indices(c.bits, idx.data(), (size_t)c.head_dim, packed);
}

// src/cache/quantize_tensor.rs:179-261 (polar_dequantize, codebook_lookup) with the CPU
// butterfly of src/cache/wht_tensor.rs:27-65: value * (sign/sqrt(32) * sqrt(32)), five
// butterfly stages, * 1/sqrt(32), * |scale|.
void block_dequantize_one(const BlockCfg& c, const uint8_t* packed, const uint16_t* scales, float* out) {
    std::vector<uint8_t> idx(c.head_dim);
    unpack_indices(c.bits, packed, (size_t)c.head_dim, idx.data());
    const float sqrt_n = std::sqrt((float)kBlock);
    const float norm = 1.0f / std::sqrt((float)kBlock);   // precomputed/rotation.rs:52
    const float inv_sqrt_n = 1.0f / sqrt_n;                // wht_tensor.rs:38
    for (int b = 0; b < c.nblk; ++b) {
        float sc = f16_bits_to_f32(scales[b]);
        // quantize_tensor.rs:228-259: all-outlier, all-normal, or by the sign of the scale
        bool outl;
        if (c.outlier_blocks >= c.nblk) outl = true;
        else if (c.outlier_blocks == 0) outl = false;
        else outl = sc < 0.0f;
        const BlockCodebook& cb = outl ? c.outlier : c.normal;
        float blk[kBlock];
        for (int j = 0; j < kBlock; ++j) {
            int id = idx[b * kBlock + j];
            if (!outl && id > cb.n - 1) id = cb.n - 1;  // quantize_tensor.rs:245 clamp
            float sgn = (norm * kBlockSigns[j]) * sqrt_n;  // wht_tensor.rs:29-35,43
            blk[j] = cb.centroids[id] * sgn;
        }
        butterfly32(blk);
        float a = std::fabs(sc);
        for (int j = 0; j < kBlock; ++j) out[b * kBlock + j] = (blk[j] * inv_sqrt_n) * a;
    }
}

}  // namespace

extern "C" {

// ---- scalar helpers -----------------------------------------------------------------
uint16_t tqo_f32_to_f16(float f) { return f32_to_f16_bits(f); }
float tqo_f16_to_f32(uint16_t h) { return f16_bits_to_f32(h); }
float tqo_sign(uint64_t seed, int index) { return sign_at(seed, (uint64_t)index); }
float tqo_rademacher_sign(uint64_t seed, int row, int col) {
    return rademacher_sign(mix_seed(seed, (uint64_t)row), (uint64_t)row, (uint64_t)col);
}
void tqo_wht_inplace(float* data, int n) { wht_inplace(data, n); }
void tqo_sign_pattern(int dim, uint64_t seed, float* out) {
    for (int i = 0; i < dim; ++i) out[i] = sign_at(seed, (uint64_t)i);
}
int tqo_codebook(int bits, int dim, double* centroids, double* boundaries) {
    const Table* t = find_table(bits, dim);
    if (!t) return -1;
    std::copy(t->centroids, t->centroids + t->n, centroids);
    std::copy(t->boundaries, t->boundaries + t->n - 1, boundaries);
    return t->n;
}
int tqo_nearest_centroid(int bits, int dim, double v) {
    const Table* t = find_table(bits, dim);
    if (!t) return -1;
    return nearest_centroid(v, t->boundaries, t->n - 1);
}
size_t tqo_packed_len(int bits, size_t count) { return packed_len(bits, count); }
void tqo_pack_indices(int bits, const uint8_t* idx, size_t count, uint8_t* out) { pack_indices(bits, idx, count, out); }
void tqo_unpack_indices(int bits, const uint8_t* packed, size_t count, uint8_t* out) { unpack_indices(bits, packed, count, out); }

// src/test_utils.rs:4-22 (pseudo_random_vec): 64-bit LCG, top bits -> [-1, 1].
void tqo_pseudo_random_vec(int dim, uint64_t seed, float* out) {
    uint64_t state = seed;
    for (int i = 0; i < dim; ++i) {
        state = state * 6364136223846793005ULL + 1ULL;
        int32_t bits = (int32_t)(state >> 33);
        out[i] = (float)bits / (float)INT32_MAX;
    }
}

// tests/mse_validation.rs:40-79 (Lcg + Box-Muller): fills n*dim normals from one stream,
// restarting the pair for each vector exactly as random_normal_vec does.
void tqo_lcg_normal_vectors(uint64_t seed, int n, int dim, float* out) {
    uint64_t state = seed;
    auto uni = [&]() {
        state = state * 6364136223846793005ULL + 1ULL;
        uint32_t bits = (uint32_t)(state >> 32);
        return ((double)bits + 1.0) / ((double)UINT32_MAX + 2.0);
    };
    const double two_pi = 6.283185307179586476925286766559;
    for (int v = 0; v < n; ++v) {
        int k = 0;
        while (k < dim) {
            double u1 = uni(), u2 = uni();
            double r = std::sqrt(-2.0 * std::log(u1));
            double th = two_pi * u2;
            out[(size_t)v * dim + k++] = (float)(r * std::cos(th));
            if (k < dim) out[(size_t)v * dim + k++] = (float)(r * std::sin(th));
        }
    }
}

// ---- whole-vector format (core crate) -----------------------------------------------
// Returns 0, or the reference's error class: 1 InvalidDimension, 2 UnsupportedBits
// (src/error.rs:4-29, src/packed/mod.rs:124-132).
int tqo_quantize_batch(int bits, int dim, uint64_t seed, const float* x, int64_t n, uint8_t* packed,
                       uint16_t* scales, int nthreads) {
    if (bits < 2 || bits > 4) return 2;
    PolarCtx c;
    if (!make_ctx(c, bits, dim, seed)) return 1;
    const size_t pb = packed_len(bits, dim);
    parallel_for(n, nthreads, [&](int64_t lo, int64_t hi, int) {
        std::vector<float> work(dim);
        std::vector<uint8_t> idx(dim);
        for (int64_t i = lo; i < hi; ++i)
            quantize_one(c, x + i * dim, packed + i * pb, scales + i, work.data(), idx.data());
    });
    return 0;
}

int tqo_dequantize_batch(int bits, int dim, uint64_t seed, const uint8_t* packed, const uint16_t* scales,
                         int64_t n, float* out, int nthreads) {
    if (bits < 2 || bits > 4) return 2;
    PolarCtx c;
    if (!make_ctx(c, bits, dim, seed)) return 1;
    const size_t pb = packed_len(bits, dim);
    parallel_for(n, nthreads, [&](int64_t lo, int64_t hi, int) {
        std::vector<uint8_t> idx(dim);
        for (int64_t i = lo; i < hi; ++i) dequantize_one(c, packed + i * pb, scales[i], out + i * dim, idx.data());
    });
    return 0;
}

// src/quantize.rs:306-316 (dequantize_rotated): no inverse rotation.
int tqo_dequantize_rotated_batch(int bits, int dim, const uint8_t* packed, const uint16_t* scales, int64_t n,
                                 float* out) {
    if (bits < 2 || bits > 4) return 2;
    PolarCtx c;
    if (!make_ctx(c, bits, dim, 0)) return 1;
    const size_t pb = packed_len(bits, dim);
    std::vector<uint8_t> idx(dim);
    for (int64_t i = 0; i < n; ++i) {
        unpack_indices(bits, packed + i * pb, (size_t)dim, idx.data());
        float s = f16_bits_to_f32(scales[i]);
        for (int k = 0; k < dim; ++k) out[i * dim + k] = c.centroids_f32[idx[k]] * s;
    }
    return 0;
}

// src/qjl.rs:305-319 (compute_qjl_signs) + :233-245 (pack_sign_bits).
void tqo_qjl_signs(const float* residual, int dim, uint64_t qjl_seed, uint8_t* signs) {
    std::memset(signs, 0, (size_t)(dim + 7) / 8);
    for (int j = 0; j < dim; ++j) {
        float p = rademacher_vector_product(residual, dim, qjl_seed, j);
        if (p >= 0.0f) signs[j >> 3] |= (uint8_t)(1u << (j & 7));
    }
}

// src/qjl.rs:355-377 / :433-466 (quantize_with_qjl / _resources): polar stage at bits-1,
// residual, residual norm -> f16, sign sketch.  `bits` is the total width (3 or 4).
int tqo_qjl_quantize_batch(int bits, int dim, uint64_t rot_seed, uint64_t qjl_seed, const float* x, int64_t n,
                           uint8_t* packed, uint16_t* scales, uint8_t* signs, uint16_t* rnorms, int nthreads) {
    if (bits < 3 || bits > 4) return 2;  // src/qjl.rs:277-279
    PolarCtx c;
    if (!make_ctx(c, bits - 1, dim, rot_seed)) return 1;
    const size_t pb = packed_len(bits - 1, dim);
    const size_t sb = (size_t)(dim + 7) / 8;
    parallel_for(n, nthreads, [&](int64_t lo, int64_t hi, int) {
        std::vector<float> work(dim), rec(dim), res(dim);
        std::vector<uint8_t> idx(dim);
        for (int64_t i = lo; i < hi; ++i) {
            const float* xi = x + i * dim;
            quantize_one(c, xi, packed + i * pb, scales + i, work.data(), idx.data());
            dequantize_one(c, packed + i * pb, scales[i], rec.data(), idx.data());
            for (int k = 0; k < dim; ++k) res[k] = xi[k] - rec[k];     // qjl.rs:213-219
            rnorms[i] = f32_to_f16_bits(l2_norm(res.data(), dim));     // qjl.rs:369,375
            tqo_qjl_signs(res.data(), dim, qjl_seed, signs + i * sb);
        }
    });
    return 0;
}

// src/qjl.rs:488-492 (precompute_query_projections).
void tqo_query_projections(const float* q, int dim, uint64_t qjl_seed, float* rq) {
    for (int j = 0; j < dim; ++j) rq[j] = rademacher_vector_product(q, dim, qjl_seed, j);
}

// src/attention.rs:319-353 (attention_scores) via src/qjl.rs:585-606
// (estimate_inner_product_with_codebook): full dequantize, sequential f32 dot, plus
// c * sum_j r_q[j] * (2*bit_j - 1) with c = ||res|| * 1.2533141 / sqrt(dim).
int tqo_attention_scores(int bits, int dim, uint64_t rot_seed, uint64_t qjl_seed, const float* q,
                         const uint8_t* packed, const uint16_t* scales, const uint8_t* signs,
                         const uint16_t* rnorms, int64_t n, float* scores, int nthreads) {
    if (bits < 3 || bits > 4) return 2;
    PolarCtx c;
    if (!make_ctx(c, bits - 1, dim, rot_seed)) return 1;
    const size_t pb = packed_len(bits - 1, dim);
    const size_t sb = (size_t)(dim + 7) / 8;
    std::vector<float> rq(dim);
    tqo_query_projections(q, dim, qjl_seed, rq.data());
    parallel_for(n, nthreads, [&](int64_t lo, int64_t hi, int) {
        std::vector<float> rec(dim);
        std::vector<uint8_t> idx(dim);
        for (int64_t i = lo; i < hi; ++i) {
            dequantize_one(c, packed + i * pb, scales[i], rec.data(), idx.data());
            float base = 0.0f;
            for (int k = 0; k < dim; ++k) base += q[k] * rec[k];                    // qjl.rs:224-226
            float rn = f16_bits_to_f32(rnorms[i]);
            float cc = rn * 1.2533141f / std::sqrt((float)dim);                     // qjl.rs:263-265
            float corr = 0.0f;
            const uint8_t* s = signs + i * sb;
            for (int k = 0; k < dim; ++k) {
                float bit = (float)((s[k >> 3] >> (k & 7)) & 1);
                corr += rq[k] * (bit * 2.0f + -1.0f);                               // qjl.rs:227-232,512-518
            }
            scores[i] = base + cc * corr;                                           // qjl.rs:471-473
        }
    });
    return 0;
}

// src/attention.rs:371-408 (weighted_values): polar part of each value block dequantized
// and accumulated as result += v * w, in storage order.
int tqo_weighted_values(int bits, int dim, uint64_t rot_seed, const float* w, const uint8_t* packed,
                        const uint16_t* scales, int64_t n, float* out) {
    if (bits < 3 || bits > 4) return 2;
    PolarCtx c;
    if (!make_ctx(c, bits - 1, dim, rot_seed)) return 1;
    const size_t pb = packed_len(bits - 1, dim);
    std::vector<float> rec(dim);
    std::vector<uint8_t> idx(dim);
    for (int k = 0; k < dim; ++k) out[k] = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        dequantize_one(c, packed + i * pb, scales[i], rec.data(), idx.data());
        for (int k = 0; k < dim; ++k) out[k] += rec[k] * w[i];
    }
    return 0;
}

// ---- block-32 format (cache module) -------------------------------------------------
int tqo_block_codebook(int cb_bits, int norm_mode, float* centroids, float* boundaries) {
    BlockCodebook cb;
    if (!block_codebook(cb_bits, norm_mode, cb)) return -1;
    std::copy(cb.centroids, cb.centroids + cb.n, centroids);
    std::copy(cb.boundaries, cb.boundaries + cb.n - 1, boundaries);
    return cb.n;
}
void tqo_block_signs(float* out) { std::copy(kBlockSigns, kBlockSigns + 32, out); }

// The forward rotation alone (normalize_and_rotate of the MaxNorm branch, src/cache/quantize_tensor.rs:104):
// n_blocks 32-blocks in, their rotated values out.  This is what the reference hands to its
// tq_quant_maxnorm_batch launcher (src/cache/cuda/quantize.rs:111-127).
void tqo_block_rotate(const float* x, int64_t n_blocks, float* out) {
    for (int64_t i = 0; i < n_blocks; ++i) rotate_block_fwd(x + i * kBlock, out + i * kBlock);
}

int tqo_block_quantize(int bits, int head_dim, int norm_mode, int outlier_blocks, const float* x, int64_t n,
                       uint8_t* packed, uint16_t* scales, int nthreads) {
    BlockCfg c;
    if (!make_block_cfg(c, bits, head_dim, norm_mode, outlier_blocks)) return 1;
    parallel_for(n, nthreads, [&](int64_t lo, int64_t hi, int) {
        for (int64_t i = lo; i < hi; ++i)
            block_quantize_one(c, x + i * head_dim, packed + i * c.packed_dim, scales + i * c.nblk);
    });
    return 0;
}

int tqo_block_dequantize(int bits, int head_dim, int norm_mode, int outlier_blocks, const uint8_t* packed,
                         const uint16_t* scales, int64_t n, float* out, int nthreads) {
    BlockCfg c;
    if (!make_block_cfg(c, bits, head_dim, norm_mode, outlier_blocks)) return 1;
    parallel_for(n, nthreads, [&](int64_t lo, int64_t hi, int) {
        for (int64_t i = lo; i < hi; ++i)
            block_dequantize_one(c, packed + i * c.packed_dim, scales + i * c.nblk, out + i * head_dim);
    });
    return 0;
}

// Decode attention over the packed cache with the semantics of
// src/cache/cuda/kernels/tq_attention_kernel.cu:161-253,299-332: every key and value is
// dequantized (|scale|), score = softmax_scale * <q, k> (+ optional QJL correction,
// :197-231), softmax over kv_len, output normalised by the sum (zero when the sum is 0).
// Query head h reads KV head h / (Hq / Hkv) (:92-93).  Layouts: q, out [Hq, D] f32;
// indices [Hkv, kv_stride, packed_dim]; scales [Hkv, kv_stride, D/32];
// qjl_signs [Hkv, kv_stride, D/8]; qjl_norms [Hkv, kv_stride]; rq [Hq, D].
// Dot products and the softmax are accumulated in f64 (the reference pins neither).
int tqo_block_attention(int bits, int head_dim, int norm_mode, int outlier_blocks, const float* q,
                        const uint8_t* k_idx, const uint16_t* k_sc, const uint8_t* v_idx, const uint16_t* v_sc,
                        const uint8_t* qjl_signs, const uint16_t* qjl_norms, const float* rq, int qjl_enabled,
                        int hq, int hkv, int kv_len, int kv_stride, float softmax_scale, float* out,
                        float* scores_out, int nthreads) {
    BlockCfg c;
    if (!make_block_cfg(c, bits, head_dim, norm_mode, outlier_blocks)) return 1;
    if (hkv <= 0 || hq % hkv != 0) return 3;
    const int g = hq / hkv;
    const int D = head_dim;
    parallel_for(hkv, nthreads, [&](int64_t lo, int64_t hi, int) {
        std::vector<float> kd(D), vd(D);
        std::vector<double> sc((size_t)g * kv_len), acc((size_t)g * D);
        for (int64_t kh = lo; kh < hi; ++kh) {
            for (int t = 0; t < kv_len; ++t) {
                size_t row = (size_t)kh * kv_stride + t;
                block_dequantize_one(c, k_idx + row * c.packed_dim, k_sc + row * c.nblk, kd.data());
                for (int gi = 0; gi < g; ++gi) {
                    int h = (int)kh * g + gi;
                    double d = 0.0;
                    for (int k = 0; k < D; ++k) d += (double)q[(size_t)h * D + k] * (double)kd[k];
                    float s = (float)d * softmax_scale;
                    if (qjl_enabled) {
                        double corr = 0.0;
                        const uint8_t* sg = qjl_signs + row * (size_t)(D / 8);
                        for (int k = 0; k < D; ++k)
                            corr += (double)rq[(size_t)h * D + k] * (((sg[k >> 3] >> (k & 7)) & 1) ? 1.0 : -1.0);
                        float nrm = f16_bits_to_f32(qjl_norms[row]);
                        float cterm = (float)corr * (nrm * 1.2533141f * (1.0f / std::sqrt((float)D)));
                        s += cterm * softmax_scale;
                    }
                    sc[(size_t)gi * kv_len + t] = s;
                    if (scores_out) scores_out[(size_t)h * kv_len + t] = s;
                }
            }
            std::fill(acc.begin(), acc.end(), 0.0);
            std::vector<double> mx(g, -INFINITY), sum(g, 0.0);
            for (int gi = 0; gi < g; ++gi)
                for (int t = 0; t < kv_len; ++t) mx[gi] = std::max(mx[gi], sc[(size_t)gi * kv_len + t]);
            for (int t = 0; t < kv_len; ++t) {
                size_t row = (size_t)kh * kv_stride + t;
                block_dequantize_one(c, v_idx + row * c.packed_dim, v_sc + row * c.nblk, vd.data());
                for (int gi = 0; gi < g; ++gi) {
                    double p = std::exp(sc[(size_t)gi * kv_len + t] - mx[gi]);
                    sum[gi] += p;
                    for (int k = 0; k < D; ++k) acc[(size_t)gi * D + k] += p * (double)vd[k];
                }
            }
            for (int gi = 0; gi < g; ++gi) {
                int h = (int)kh * g + gi;
                double inv = sum[gi] > 0.0 ? 1.0 / sum[gi] : 0.0;
                for (int k = 0; k < D; ++k) out[(size_t)h * D + k] = (float)(acc[(size_t)gi * D + k] * inv);
            }
        }
    });
    return 0;
}

// Full float softmax(QK^T * scale) V over already dequantized K, V [Hkv, kv_len, D], the
// step the host engine performs after PqoCache/TqCache return `Dequantized`
// (src/cache/pqo.rs:219-221, src/cache/tq.rs:300-311); `bias` [Hq, kv_len] may be null.
void tqo_sdpa(const float* q, const float* k, const float* v, const float* bias, int hq, int hkv, int kv_len, int D,
              float softmax_scale, float* out) {
    const int g = hq / hkv;
    std::vector<double> s(kv_len);
    for (int h = 0; h < hq; ++h) {
        const float* kk = k + (size_t)(h / g) * kv_len * D;
        const float* vv = v + (size_t)(h / g) * kv_len * D;
        double mx = -INFINITY;
        for (int t = 0; t < kv_len; ++t) {
            double d = 0.0;
            for (int i = 0; i < D; ++i) d += (double)q[(size_t)h * D + i] * (double)kk[(size_t)t * D + i];
            s[t] = d * softmax_scale + (bias ? (double)bias[(size_t)h * kv_len + t] : 0.0);
            mx = std::max(mx, s[t]);
        }
        double sum = 0.0;
        std::vector<double> acc(D, 0.0);
        for (int t = 0; t < kv_len; ++t) {
            double p = std::exp(s[t] - mx);
            sum += p;
            for (int i = 0; i < D; ++i) acc[i] += p * (double)vv[(size_t)t * D + i];
        }
        for (int i = 0; i < D; ++i) out[(size_t)h * D + i] = (float)(sum > 0.0 ? acc[i] / sum : 0.0);
    }
}

int tqo_version() { return 1; }

}  // extern "C"
