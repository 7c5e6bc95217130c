// Shared device/host helpers of libtqb200.  Compiled with -fmad=false: every a*b+c below is
// two roundings unless written as fmaf(), because the bit-exact paths must round exactly
// like the reference's scalar f32 code.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <nvtx3/nvToolsExt.h>

#include "../../include/tqb200.h"

namespace tqb {

constexpr int kBlock = 32;            // QUANT_BLOCK_SIZE, src/cache/config.rs:9
constexpr int kMaxCentroids = 16;
constexpr float kMinNorm = 1e-10f;    // src/quantize.rs:42, src/cache/quantize_tensor.rs:89

// A codebook in single precision, passed to kernels by value.
//  c[i]  centroid i (the reference's f64 centroid cast to f32, src/quantize.rs:97-102)
//  b[k]  decision boundary k.  For the f64 tables of the core crate the boundary is
//        rounded toward -inf: for f32 v and f64 B,  v > B  <=>  v > round_down_f32(B),
//        so the f32 comparison reproduces the reference's f64 comparison
//        (src/codebook/mod.rs:66-87) exactly.
struct Codebook {
    float c[kMaxCentroids];
    float b[kMaxCentroids];  // b[n-1] = +inf padding
    int n;
};

// Per-thread record of the last CUDA error seen by a launcher.
void set_cuda_error(cudaError_t e);
int check_launch(cudaStream_t s);

bool whole_codebook(int bits, int dim, Codebook& cb);              // core-crate tables
bool block_codebook(int cb_bits, int norm_mode, Codebook& cb);     // cache-module tables
extern const float kBlockSigns[32];

__device__ __forceinline__ float f16_bits_to_f32(uint16_t u) { return __half2float(__ushort_as_half(u)); }
__device__ __forceinline__ uint16_t f32_to_f16_bits(float f) { return __half_as_ushort(__float2half_rn(f)); }

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Number of boundaries strictly below v  (count of `v > b[k]`), by bisection over a
// sorted table of n-1 boundaries held in shared memory or registers.
template <int N>
__device__ __forceinline__ int bucket_index(float v, const float* __restrict__ b) {
    int lo = 0;
#pragma unroll
    for (int step = N / 2; step >= 1; step >>= 1)
        lo += (v > b[lo + step - 1]) ? step : 0;
    return lo;
}
__device__ __forceinline__ int bucket_index_n(float v, const float* __restrict__ b, int n) {
    if (n == 16) return bucket_index<16>(v, b);
    if (n == 8) return bucket_index<8>(v, b);
    return bucket_index<4>(v, b);
}

// Code k of an LSB-first bit stream held as little-endian 32-bit words.
__device__ __forceinline__ uint32_t extract_bits(uint32_t w0, uint32_t w1, int bitoff, int nbits) {
    return __funnelshift_r(w0, w1, bitoff & 31) & ((1u << nbits) - 1u);
}

inline cudaStream_t as_stream(tqb_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// NVTX range around a C-ABI entry point (a few nanoseconds when no tool is attached): profilers show the library's
// calls by name on the host timeline.
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};
#define TQB_NVTX_RANGE() ::tqb::NvtxRange tqb_nvtx_range_(__func__)

// Sequence-parallel decode, fused exchange: where the CTA that finishes a KV head stores the head group's shard-local
// record (un-normalised outputs, then (max, sum) pairs) - once per rank of the group, into that rank's receive buffer
// (peer memory mapped into this process; plain stores, no bulk or multicast copy) - and the flag words it then
// releases.  world == 0: off.
constexpr int kMaxPeers = 8;
constexpr int kPeerFlagHeads = 64;     // flag words per source rank (one per KV head)
struct PeerPush {
    int world;
    unsigned seq;                      // value written to the flags: the exchange's step counter
    float* rec[kMaxPeers];             // this rank's record inside rank p's receive buffer
    unsigned* flag[kMaxPeers];         // this rank's flag row [kPeerFlagHeads] inside rank p's receive buffer
};
// Decode attention (as tqb_decode_attention with lse_out semantics) whose merge CTAs push the result to the peers.
int decode_with_peer_push(const tqb_decode_params* p, const PeerPush& push, tqb_stream_t stream);

}  // namespace tqb
