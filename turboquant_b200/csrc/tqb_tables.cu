// Host-side constant data: the core crate's Lloyd-Max tables and the cache module's
// MaxNorm / L2Norm codebooks, converted to the single-precision form the kernels use.
#include <cmath>
#include <cstring>

#include "tqb_common.cuh"

namespace tqb {

namespace {
struct Table {
    int bits, dim, n;
    double centroids[16];
    double boundaries[15];
};
#define TQ_UNPAREN(...) __VA_ARGS__
#define TQ_TABLE(bits, dim, n, c, b) {bits, dim, n, {TQ_UNPAREN c}, {TQ_UNPAREN b}},
const Table kTables[] = {
#include "tqb_codebook_tables.inc"
};
#undef TQ_TABLE

const Table* find_table(int bits, int dim) {
    for (const Table& t : kTables)
        if (t.bits == bits && t.dim == dim) return &t;
    return nullptr;
}

// Largest float <= d.
float round_down_f32(double d) {
    float f = (float)d;
    if ((double)f > d) f = std::nextafterf(f, -INFINITY);
    return f;
}

thread_local int g_last_cuda_error = 0;
}  // namespace

// src/cache/precomputed/rotation.rs:16-20
const float kBlockSigns[32] = {1, -1, 1, 1, -1, -1, 1, -1, 1, 1, -1, 1, -1, 1, -1, -1,
                               1, -1, -1, 1, 1, -1, 1, -1, -1, 1, 1, 1, -1, -1, 1, -1};

void set_cuda_error(cudaError_t e) { g_last_cuda_error = (int)e; }

int check_launch(cudaStream_t) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_cuda_error(e);
        return e == cudaErrorMemoryAllocation ? TQB_ERR_OUT_OF_MEMORY : TQB_ERR_CUDA;
    }
    return TQB_OK;
}

bool whole_codebook(int bits, int dim, Codebook& cb) {
    const Table* t = find_table(bits, dim);
    if (!t) return false;
    cb.n = t->n;
    for (int i = 0; i < kMaxCentroids; ++i) {
        cb.c[i] = i < t->n ? (float)t->centroids[i] : 0.0f;
        cb.b[i] = i < t->n - 1 ? round_down_f32(t->boundaries[i]) : INFINITY;
    }
    return true;
}

// src/cache/precomputed/codebooks.rs:18-88
bool block_codebook(int cb_bits, int norm_mode, Codebook& cb) {
    if (cb_bits < 2 || cb_bits > 4) return false;
    const int n = 1 << cb_bits;
    cb.n = n;
    for (int i = 0; i < kMaxCentroids; ++i) { cb.c[i] = 0.0f; cb.b[i] = INFINITY; }
    if (norm_mode == TQB_L2NORM) {
        const Table* t = find_table(cb_bits, kBlock);
        if (!t) return false;
        for (int i = 0; i < n; ++i) cb.c[i] = (float)t->centroids[i];
        for (int i = 0; i < n - 1; ++i) cb.b[i] = (float)t->boundaries[i];  // codebooks.rs:41 `v as f32`
        return true;
    }
    const float R = 2.1573f;
    if (cb_bits == 3) {
        const float c3[8] = {-2.1573f, -1.3336f, -0.7434f, -0.2428f, 0.2428f, 0.7434f, 1.3336f, 2.1573f};
        const float b3[7] = {-1.7455f, -1.0385f, -0.4931f, 0.0f, 0.4931f, 1.0385f, 1.7455f};
        std::memcpy(cb.c, c3, sizeof c3);
        std::memcpy(cb.b, b3, sizeof b3);
    } else if (cb_bits == 2) {
        const float c2[4] = {-R, -0.7434f, 0.7434f, R};
        const float b2[3] = {-1.0385f, 0.0f, 1.0385f};
        std::memcpy(cb.c, c2, sizeof c2);
        std::memcpy(cb.b, b2, sizeof b2);
    } else {
        const float full = 2.0f * R;
        const float step = full / 15.0f;
        for (int i = 0; i < 16; ++i) cb.c[i] = -R + (float)i * step;
        for (int i = 0; i < 15; ++i) cb.b[i] = -R + ((float)i + 0.5f) * step;
    }
    return true;
}

}  // namespace tqb

extern "C" {

const char* tqb_status_string(int s) {
    switch (s) {
        case TQB_OK: return "ok";
        case TQB_ERR_INVALID_DIMENSION: return "invalid dimension";
        case TQB_ERR_UNSUPPORTED_BITS: return "unsupported bit width";
        case TQB_ERR_DIMENSION_MISMATCH: return "dimension mismatch";
        case TQB_ERR_LAYER_OUT_OF_RANGE: return "layer index out of range";
        case TQB_ERR_RANGE_OUT_OF_BOUNDS: return "range out of bounds";
        case TQB_ERR_NULL_POINTER: return "null pointer";
        case TQB_ERR_INVALID_ARGUMENT: return "invalid argument";
        case TQB_ERR_MISALIGNED: return "misaligned pointer";
        case TQB_ERR_UNSUPPORTED: return "unsupported configuration";
        case TQB_ERR_PEER_TIMEOUT: return "a bounded wait for another rank timed out";
        case TQB_ERR_CUDA: return "CUDA error";
        case TQB_ERR_OUT_OF_MEMORY: return "out of device memory";
        case TQB_ERR_TOO_LARGE: return "size exceeds the entry point's fixed capacity";
        default: return "unknown status";
    }
}

int tqb_last_cuda_error(void) { return tqb::g_last_cuda_error; }
int tqb_version(void) { return 1; }

size_t tqb_packed_bytes(int32_t bits, size_t count) {
    switch (bits) {
        case 2: return (count + 3) / 4;
        case 3: return ((count + 7) / 8) * 3;
        case 4: return (count + 1) / 2;
        default: return 0;
    }
}

int tqb_config_validate(const tqb_config* cfg) {
    if (!cfg) return TQB_ERR_NULL_POINTER;
    // src/packed/mod.rs:124-132: bits first, then dim
    if (cfg->bits < 2 || cfg->bits > 4) return TQB_ERR_UNSUPPORTED_BITS;
    if (cfg->dim <= 0 || (cfg->dim & (cfg->dim - 1)) != 0) return TQB_ERR_INVALID_DIMENSION;
    if (!tqb::find_table(cfg->bits, cfg->dim)) return TQB_ERR_UNSUPPORTED;
    return TQB_OK;
}

int tqb_get_codebook(int32_t bits, int32_t dim, double* centroids, double* boundaries) {
    if (!centroids || !boundaries) return TQB_ERR_NULL_POINTER;
    if (bits < 2 || bits > 4) return TQB_ERR_UNSUPPORTED_BITS;
    const tqb::Table* t = tqb::find_table(bits, dim);
    if (!t) return TQB_ERR_UNSUPPORTED;
    std::memcpy(centroids, t->centroids, sizeof(double) * t->n);
    std::memcpy(boundaries, t->boundaries, sizeof(double) * (t->n - 1));
    return TQB_OK;
}

int tqb_generate_sign_pattern(int32_t dim, uint64_t seed, float* out) {
    if (!out) return TQB_ERR_NULL_POINTER;
    if (dim <= 0) return TQB_ERR_INVALID_DIMENSION;
    // src/rotation.rs:47-70
    for (int i = 0; i < dim; ++i) {
        uint64_t h = (seed + (uint64_t)i) * 0x9E3779B97F4A7C15ULL;
        out[i] = (h & 1ULL) == 0 ? 1.0f : -1.0f;
    }
    return TQB_OK;
}

int tqb_block_codebook(int32_t cb_bits, int32_t norm_mode, float* centroids, float* boundaries) {
    tqb::Codebook cb;
    if (!centroids || !boundaries) return -TQB_ERR_NULL_POINTER;
    if (!tqb::block_codebook(cb_bits, norm_mode, cb)) return -TQB_ERR_UNSUPPORTED_BITS;
    std::memcpy(centroids, cb.c, sizeof(float) * cb.n);
    std::memcpy(boundaries, cb.b, sizeof(float) * (cb.n - 1));
    return cb.n;
}

void tqb_block_sign_pattern(float* out32) { std::memcpy(out32, tqb::kBlockSigns, sizeof tqb::kBlockSigns); }

// src/qjl.rs:143-171
int tqb_qjl_rademacher_bits(int32_t dim, uint64_t qjl_seed, uint32_t* host_out) {
    if (!host_out) return TQB_ERR_NULL_POINTER;
    if (dim < 32 || dim % 32 != 0) return TQB_ERR_INVALID_DIMENSION;
    const int words = dim / 32;
    for (int row = 0; row < dim; ++row) {
        uint64_t mixed = qjl_seed * 0x517CC1B727220A95ULL + (uint64_t)row;
        uint64_t row_seed = mixed ^ (mixed >> 32) ^ 0x6C62272E07BB0142ULL;
        for (int w = 0; w < words; ++w) host_out[row * words + w] = 0;
        for (int col = 0; col < dim; ++col) {
            uint64_t z = row_seed + (uint64_t)row * 0x9E3779B97F4A7C15ULL + (uint64_t)col;
            z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
            z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
            z = z ^ (z >> 31);
            if (z & 1ULL) host_out[row * words + col / 32] |= 1u << (col % 32);
        }
    }
    return TQB_OK;
}

}  // extern "C"
