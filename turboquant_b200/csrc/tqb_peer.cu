// Sequence-parallel decode with the exchange fused into the attention kernel.
//
// One long sequence is split along the tokens over the ranks of one NVLink domain (one process per GPU).  Per layer
// every rank attends over its shard; the CTA that finishes a KV head merges the shard's split-K partials and stores the
// head group's record - un-normalised outputs and (max, sum) pairs - straight into EVERY rank's receive buffer with
// plain global stores over NVLink, then releases one flag word per rank (st.release.sys).  A small combine kernel on
// each rank acquires the flags of all ranks (bounded wait) and merges the records that arrived in its own memory with
// the log-sum-exp algebra of tq_fused_attention_reduce (tq_attention_kernel.cu:299-332).  No NCCL call, no bulk or
// multicast copy, and nothing is ever loaded from peer memory: peers push, consumers read local memory.
//
// The receive buffers are cudaMalloc allocations shared through CUDA IPC handles (the host side exchanges the 64-byte
// handles by whatever channel it has).  Records are multi-buffered by the step counter, so a rank that runs one layer
// ahead writes a different slot than the one its peers are still reading.
//
// Every device-side wait is bounded: when a flag does not arrive within the given number of clock cycles the combine
// kernel counts a time-out, writes zeros and returns; the host reads the counter with tqb_peer_exchange_timeouts().
#include <string.h>

#include <new>

#include "tqb_common.cuh"

using namespace tqb;

namespace {

constexpr int kSlots = 4;
constexpr size_t kHeaderBytes = 4096;   // flags [kMaxPeers][kPeerFlagHeads] u32 (2 KB), then the time-out counter

int cuda_fail(cudaError_t e) {
    set_cuda_error(e);
    return e == cudaErrorMemoryAllocation ? TQB_ERR_OUT_OF_MEMORY : TQB_ERR_CUDA;
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One CTA per query head.  flags: [world][kPeerFlagHeads]; recs: this step's slot, [world][rec_floats].
template <typename OT>
__global__ void __launch_bounds__(128) peer_combine_kernel(const unsigned* flags, const float* recs, int world, int hq, int g,
                                                           size_t rec_floats, unsigned seq, long long wait_cycles,
                                                           unsigned* timeouts, OT* __restrict__ out) {
    const int head = blockIdx.x, kvh = head / g, tid = threadIdx.x;
    constexpr int D = 128;
    __shared__ int s_late;
    if (tid == 0) s_late = 0;
    __syncthreads();
    if (tid < world) {
        const unsigned* f = flags + tid * kPeerFlagHeads + kvh;
        const long long t0 = clock64();
        while ((int)(ld_acquire_sys(f) - seq) < 0) {
            if (clock64() - t0 > wait_cycles) {   // bounded: give up, say so, leave the context usable
                atomicExch(&s_late, 1);
                break;
            }
            __nanosleep(40);
        }
    }
    __syncthreads();
    if (s_late) {
        if (tid == 0) atomicAdd(timeouts, 1u);
        out[(size_t)head * D + tid] = from_f32<OT>(0.0f);
        return;
    }
    const float* lse0 = recs + (size_t)hq * D + (size_t)head * 2;
    float M = -3.402823466e38f;
    for (int r = 0; r < world; ++r) M = fmaxf(M, __ldcg(lse0 + r * rec_floats));
    float L = 0.0f, acc = 0.0f;
    for (int r = 0; r < world; ++r) {
        const float wgt = expf(__ldcg(lse0 + r * rec_floats) - M);
        L += __ldcg(lse0 + r * rec_floats + 1) * wgt;
        acc = fmaf(__ldcg(recs + r * rec_floats + (size_t)head * D + tid), wgt, acc);
    }
    out[(size_t)head * D + tid] = from_f32<OT>(L > 0.0f ? acc * (1.0f / L) : 0.0f);
}

}  // namespace

struct tqb_peer_exchange {
    int world = 0, rank = 0, hq = 0;
    size_t rec_floats = 0, bytes = 0;
    unsigned char* local = nullptr;
    unsigned char* peers[kMaxPeers] = {};
    bool ipc_opened[kMaxPeers] = {};
    bool connected = false;
    unsigned seq = 0;
    cudaIpcMemHandle_t handle{};

    unsigned* flags(int p) const { return reinterpret_cast<unsigned*>(peers[p]); }
    unsigned* timeouts() const { return reinterpret_cast<unsigned*>(local + 2048); }
    float* slot(int p, unsigned s) const {
        return reinterpret_cast<float*>(peers[p] + kHeaderBytes) + (size_t)(s % kSlots) * world * rec_floats;
    }
};

extern "C" {

int tqb_peer_exchange_create(int32_t world, int32_t rank, int32_t num_q_heads, int32_t head_dim, tqb_peer_exchange** out) {
    if (!out) return TQB_ERR_NULL_POINTER;
    *out = nullptr;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || num_q_heads <= 0) return TQB_ERR_INVALID_ARGUMENT;
    if (head_dim != 128) return TQB_ERR_UNSUPPORTED;   // the pushing kernels are the head_dim-128 tensor-core kernels
    tqb_peer_exchange* x = new (std::nothrow) tqb_peer_exchange();
    if (!x) return TQB_ERR_OUT_OF_MEMORY;
    x->world = world; x->rank = rank; x->hq = num_q_heads;
    x->rec_floats = (size_t)num_q_heads * (head_dim + 2);
    x->bytes = kHeaderBytes + sizeof(float) * kSlots * world * x->rec_floats;
    cudaError_t e = cudaMalloc((void**)&x->local, x->bytes);
    if (e == cudaSuccess) e = cudaMemset(x->local, 0, x->bytes);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&x->handle, x->local);
    if (e != cudaSuccess) {
        if (x->local) cudaFree(x->local);
        delete x;
        return cuda_fail(e);
    }
    x->peers[rank] = x->local;
    *out = x;
    return TQB_OK;
}

int tqb_peer_exchange_handle(const tqb_peer_exchange* x, void* handle64) {
    if (!x || !handle64) return TQB_ERR_NULL_POINTER;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    memcpy(handle64, &x->handle, 64);
    return TQB_OK;
}

int tqb_peer_exchange_connect(tqb_peer_exchange* x, const void* handles) {
    if (!x || !handles) return TQB_ERR_NULL_POINTER;
    if (x->connected) return TQB_ERR_INVALID_ARGUMENT;
    const unsigned char* h = static_cast<const unsigned char*>(handles);
    for (int p = 0; p < x->world; ++p) {
        if (p == x->rank) continue;
        cudaIpcMemHandle_t hd;
        memcpy(&hd, h + 64 * p, 64);
        void* ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, hd, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return cuda_fail(e);
        x->peers[p] = static_cast<unsigned char*>(ptr);
        x->ipc_opened[p] = true;
    }
    x->connected = true;
    return TQB_OK;
}

// In-process form (several ranks emulated by one process, e.g. on a single GPU): `all` holds the world's exchange
// objects in rank order; an IPC handle cannot be opened by the process that made it.
int tqb_peer_exchange_connect_local(tqb_peer_exchange* x, tqb_peer_exchange* const* all) {
    if (!x || !all) return TQB_ERR_NULL_POINTER;
    if (x->connected) return TQB_ERR_INVALID_ARGUMENT;
    for (int p = 0; p < x->world; ++p) {
        if (!all[p] || all[p]->world != x->world || all[p]->rank != p || all[p]->rec_floats != x->rec_floats)
            return TQB_ERR_INVALID_ARGUMENT;
        x->peers[p] = all[p]->local;
    }
    x->connected = true;
    return TQB_OK;
}

void tqb_peer_exchange_destroy(tqb_peer_exchange* x) {
    if (!x) return;
    for (int p = 0; p < x->world; ++p)
        if (x->ipc_opened[p]) cudaIpcCloseMemHandle(x->peers[p]);
    if (x->local) cudaFree(x->local);
    delete x;
}

long long tqb_peer_exchange_timeouts(const tqb_peer_exchange* x) {
    if (!x) return -1;
    unsigned v = 0;
    if (cudaMemcpy(&v, x->timeouts(), sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return (long long)v;
}

// TQB_ERR_PEER_TIMEOUT when a bounded wait of a combine kernel has run out since the exchange was created
// (synchronises the device), else TQB_OK.
int tqb_peer_exchange_check(const tqb_peer_exchange* x) {
    const long long n = tqb_peer_exchange_timeouts(x);
    if (n < 0) return TQB_ERR_CUDA;
    return n > 0 ? TQB_ERR_PEER_TIMEOUT : TQB_OK;
}

// Step 2 of a layer (step 1 is tqb_pqo_cache_attend_push): waits (at most wait_cycles clock cycles per flag) for the records of all ranks of the current step and
// merges them: out [num_q_heads, 128] of out_dtype.
int tqb_peer_exchange_combine(tqb_peer_exchange* x, int32_t num_kv_heads, void* out, int32_t out_dtype, int64_t wait_cycles,
                              tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    if (!x || !out) return TQB_ERR_NULL_POINTER;
    if (!x->connected || x->seq == 0) return TQB_ERR_INVALID_ARGUMENT;
    if (num_kv_heads <= 0 || num_kv_heads > kPeerFlagHeads || x->hq % num_kv_heads != 0 || wait_cycles <= 0)
        return TQB_ERR_INVALID_ARGUMENT;
    cudaStream_t s = as_stream(stream);
    const unsigned* fl = x->flags(x->rank);
    const float* recs = x->slot(x->rank, x->seq);
    const int g = x->hq / num_kv_heads;
    if (out_dtype == TQB_F32)
        peer_combine_kernel<float><<<x->hq, 128, 0, s>>>(fl, recs, x->world, x->hq, g, x->rec_floats, x->seq, wait_cycles, x->timeouts(), (float*)out);
    else if (out_dtype == TQB_F16)
        peer_combine_kernel<__half><<<x->hq, 128, 0, s>>>(fl, recs, x->world, x->hq, g, x->rec_floats, x->seq, wait_cycles, x->timeouts(), (__half*)out);
    else if (out_dtype == TQB_BF16)
        peer_combine_kernel<__nv_bfloat16><<<x->hq, 128, 0, s>>>(fl, recs, x->world, x->hq, g, x->rec_floats, x->seq, wait_cycles, x->timeouts(), (__nv_bfloat16*)out);
    else return TQB_ERR_INVALID_ARGUMENT;
    return check_launch(s);
}

}  // extern "C"

// Used by tqb_pqo_cache_attend_push (tqb_host.cu): the push targets of the exchange's next step.
namespace tqb {
int peer_exchange_begin_step(tqb_peer_exchange* x, int num_q_heads, PeerPush& push, float** local_rec) {
    if (!x) return TQB_ERR_NULL_POINTER;
    if (!x->connected || num_q_heads != x->hq) return TQB_ERR_INVALID_ARGUMENT;
    x->seq += 1;
    push = PeerPush{};
    push.world = x->world;
    push.seq = x->seq;
    for (int p = 0; p < x->world; ++p) {
        push.rec[p] = x->slot(p, x->seq) + (size_t)x->rank * x->rec_floats;
        push.flag[p] = x->flags(p) + (size_t)x->rank * kPeerFlagHeads;
    }
    *local_rec = push.rec[x->rank];
    return TQB_OK;
}
}  // namespace tqb
