// Host-side cache objects above the kernels: PqoCache (src/cache/pqo.rs) over
// CompressedStorage (src/cache/storage.rs) and QuantizedKVCache (src/attention.rs).
// They own device memory, keep the reference's growth policy and error behaviour, and
// enqueue the library's own entry points; there is no CPU implementation behind them.
#include <algorithm>
#include <cstring>
#include <new>
#include <vector>

#include "tqb_common.cuh"

namespace {

using namespace tqb;

int cuda_fail(cudaError_t e) {
    set_cuda_error(e);
    return e == cudaErrorMemoryAllocation ? TQB_ERR_OUT_OF_MEMORY : TQB_ERR_CUDA;
}
#define TQB_CUDA(call)                          \
    do {                                        \
        cudaError_t e__ = (call);               \
        if (e__ != cudaSuccess) return cuda_fail(e__); \
    } while (0)
#define TQB_TRY(call)                 \
    do {                              \
        int st__ = (call);            \
        if (st__ != TQB_OK) return st__; \
    } while (0)

size_t dtype_size(int dt) { return dt == TQB_F32 ? 4 : 2; }

// A device buffer that only grows.
struct DevBuf {
    void* p = nullptr;
    size_t bytes = 0;
    int reserve(size_t need) {
        if (need <= bytes) return TQB_OK;
        if (p) TQB_CUDA(cudaFree(p));
        p = nullptr;
        bytes = 0;
        TQB_CUDA(cudaMalloc(&p, need));
        bytes = need;
        return TQB_OK;
    }
    void release() {
        if (p) cudaFree(p);
        p = nullptr;
        bytes = 0;
    }
};

}  // namespace

// ---------------------------------------------------------------------------------------
// PqoCache
// ---------------------------------------------------------------------------------------
// Grows the decode scratch when needed and keeps its ticket area (the first bytes) zero: it is cleared when the
// buffer is new or the (head count, partition count) pair it was laid out for changed - the ticket area's extent
// depends on both; completed decode calls leave it zero.
static int prepare_scratch(DevBuf& scratch, int& ticket_heads, size_t need, int num_q_heads, int head_dim,
                           int num_partitions, cudaStream_t s) {
    if (need > scratch.bytes) {
        TQB_CUDA(cudaStreamSynchronize(s));
        TQB_TRY(scratch.reserve(need + need / 4));
        ticket_heads = -1;
    }
    const int key = num_q_heads * 4096 + num_partitions;
    if (ticket_heads != key) {
        const size_t partials = sizeof(float) * (size_t)num_q_heads * num_partitions * ((size_t)head_dim + 2);
        TQB_CUDA(cudaMemsetAsync(scratch.p, 0, need - partials, s));   // at least the ticket area at the start
        ticket_heads = key;
    }
    return TQB_OK;
}

struct tqb_pqo_cache {
    tqb_cache_config cfg;
    int nblk, packed_dim, heads;  // heads = batch * num_kv_heads
    struct Layer {
        uint8_t *ki = nullptr, *vi = nullptr;
        uint16_t *ks = nullptr, *vs = nullptr;
        int64_t cap = 0, len = 0;
        bool active = false;
    };
    std::vector<Layer> layers;
    DevBuf stage_k, stage_v, stage_q, stage_out, scratch;
    // tqb_pqo_cache_set_overlap: decode launches of different layers may start before their predecessor has finished
    bool overlap = false;
    int last_attend_layer = -1;
    // Host-buffer decode: two staging slots and a copy stream, so that the host->device copies of
    // one call and the device->host copy of the previous call overlap with kernels.
    struct Slot {
        DevBuf k, v, q, out;
        cudaEvent_t in_ready = nullptr, compute_done = nullptr, out_done = nullptr;
    };
    Slot slots[2];
    int next_slot = 0;
    cudaStream_t copy_stream = nullptr;   // host -> device
    cudaStream_t down_stream = nullptr;   // device -> host
    cudaEvent_t last_out = nullptr;   // completion of the most recent device->host output copy
    // Host buffers that are pinned and mapped are read and written by the kernels themselves (no staging copies):
    // the stream of the most recent such call, waited for by tqb_pqo_cache_host_sync
    bool direct_pending = false;
    cudaStream_t direct_stream = nullptr;

    int ensure_pipeline() {
        if (copy_stream) return TQB_OK;
        TQB_CUDA(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking));
        TQB_CUDA(cudaStreamCreateWithFlags(&down_stream, cudaStreamNonBlocking));
        for (auto& sl : slots) {
            TQB_CUDA(cudaEventCreateWithFlags(&sl.in_ready, cudaEventDisableTiming));
            TQB_CUDA(cudaEventCreateWithFlags(&sl.compute_done, cudaEventDisableTiming));
            TQB_CUDA(cudaEventCreateWithFlags(&sl.out_done, cudaEventDisableTiming));
        }
        return TQB_OK;
    }
    void destroy_pipeline() {
        for (auto& sl : slots) {
            sl.k.release(); sl.v.release(); sl.q.release(); sl.out.release();
            if (sl.in_ready) cudaEventDestroy(sl.in_ready);
            if (sl.compute_done) cudaEventDestroy(sl.compute_done);
            if (sl.out_done) cudaEventDestroy(sl.out_done);
        }
        if (copy_stream) cudaStreamDestroy(copy_stream);
        if (down_stream) cudaStreamDestroy(down_stream);
        copy_stream = down_stream = nullptr;
    }

    void free_layer(Layer& l) {
        if (l.ki) cudaFree(l.ki);
        if (l.vi) cudaFree(l.vi);
        if (l.ks) cudaFree(l.ks);
        if (l.vs) cudaFree(l.vs);
        l = Layer{};
    }

    // CompressedStorage::ensure_capacity (src/cache/storage.rs:108-143): grow to
    // needed + max(needed / 4, 128), zero-filled, old rows copied per head.
    int ensure_capacity(int layer, int64_t needed, cudaStream_t s) {
        Layer& l = layers[layer];
        if (l.cap >= needed) return TQB_OK;
        const int64_t grow = std::max<int64_t>(needed / 4, 128);
        const int64_t new_cap = needed + grow;
        Layer nl;
        nl.cap = new_cap;
        nl.len = l.len;
        nl.active = l.active;
        const size_t ib = (size_t)heads * new_cap * packed_dim;
        const size_t sb = (size_t)heads * new_cap * nblk * sizeof(uint16_t);
        cudaError_t e;
        if ((e = cudaMalloc((void**)&nl.ki, ib)) != cudaSuccess || (e = cudaMalloc((void**)&nl.vi, ib)) != cudaSuccess ||
            (e = cudaMalloc((void**)&nl.ks, sb)) != cudaSuccess || (e = cudaMalloc((void**)&nl.vs, sb)) != cudaSuccess) {
            free_layer(nl);
            return cuda_fail(e);
        }
        // on any failure from here on the new buffers are released and the layer is left as it was
        auto fill = [&]() -> cudaError_t {
            cudaError_t r;
            if ((r = cudaMemsetAsync(nl.ki, 0, ib, s)) != cudaSuccess) return r;
            if ((r = cudaMemsetAsync(nl.vi, 0, ib, s)) != cudaSuccess) return r;
            if ((r = cudaMemsetAsync(nl.ks, 0, sb, s)) != cudaSuccess) return r;
            if ((r = cudaMemsetAsync(nl.vs, 0, sb, s)) != cudaSuccess) return r;
            if (l.len > 0) {
                const size_t iw = (size_t)l.len * packed_dim, sw = (size_t)l.len * nblk * 2;
                if ((r = cudaMemcpy2DAsync(nl.ki, (size_t)new_cap * packed_dim, l.ki, (size_t)l.cap * packed_dim, iw, heads,
                                           cudaMemcpyDeviceToDevice, s)) != cudaSuccess) return r;
                if ((r = cudaMemcpy2DAsync(nl.vi, (size_t)new_cap * packed_dim, l.vi, (size_t)l.cap * packed_dim, iw, heads,
                                           cudaMemcpyDeviceToDevice, s)) != cudaSuccess) return r;
                if ((r = cudaMemcpy2DAsync(nl.ks, (size_t)new_cap * nblk * 2, l.ks, (size_t)l.cap * nblk * 2, sw, heads,
                                           cudaMemcpyDeviceToDevice, s)) != cudaSuccess) return r;
                if ((r = cudaMemcpy2DAsync(nl.vs, (size_t)new_cap * nblk * 2, l.vs, (size_t)l.cap * nblk * 2, sw, heads,
                                           cudaMemcpyDeviceToDevice, s)) != cudaSuccess) return r;
            }
            // the old buffers may still be read by queued work, and the copies above must have left them
            return l.ki ? cudaStreamSynchronize(s) : cudaSuccess;
        };
        if ((e = fill()) != cudaSuccess) {
            cudaStreamSynchronize(s);   // nothing queued may still write the buffers that are released next
            free_layer(nl);
            return cuda_fail(e);
        }
        if (l.ki) free_layer(l);
        l = nl;
        return TQB_OK;
    }

    // quantize_and_store (src/cache/pqo.rs:64-104)
    int quantize_and_store(int layer, const void* k_dev, const void* v_dev, int dtype, int new_tokens, cudaStream_t s) {
        Layer& l0 = layers[layer];
        const int64_t old_len = l0.len;
        TQB_TRY(ensure_capacity(layer, old_len + new_tokens, s));
        Layer& l = layers[layer];
        const int64_t rows = (int64_t)heads * new_tokens;
        TQB_TRY(tqb_block_quantize_pair(cfg.bits, cfg.head_dim, cfg.norm_mode, cfg.outlier_blocks, k_dev, v_dev, dtype, rows, 0,
                                        l.ki, l.ks, l.vi, l.vs, new_tokens, l.cap, old_len, s));
        l.len = old_len + new_tokens;
        l.active = true;
        return TQB_OK;
    }

    int dequantize_full(int layer, void* k_out, void* v_out, int dtype, bool host, cudaStream_t s) {
        Layer& l = layers[layer];
        if (l.len == 0) return TQB_OK;
        const int64_t rows = (int64_t)heads * l.len;
        const size_t bytes = (size_t)rows * cfg.head_dim * dtype_size(dtype);
        void* kd = k_out;
        void* vd = v_out;
        if (host) {
            TQB_TRY(stage_k.reserve(bytes));
            TQB_TRY(stage_v.reserve(bytes));
            kd = stage_k.p;
            vd = stage_v.p;
        }
        TQB_TRY(tqb_block_dequantize(cfg.bits, cfg.head_dim, cfg.norm_mode, cfg.outlier_blocks, l.ki, l.ks, rows, l.len,
                                     l.cap, 0, kd, dtype, s));
        TQB_TRY(tqb_block_dequantize(cfg.bits, cfg.head_dim, cfg.norm_mode, cfg.outlier_blocks, l.vi, l.vs, rows, l.len,
                                     l.cap, 0, vd, dtype, s));
        if (host) {
            TQB_CUDA(cudaMemcpyAsync(k_out, kd, bytes, cudaMemcpyDeviceToHost, s));
            TQB_CUDA(cudaMemcpyAsync(v_out, vd, bytes, cudaMemcpyDeviceToHost, s));
        }
        return TQB_OK;
    }

    // One decode step of a layer: append the new token's K / V rows (device, one vector per KV head) and
    // attend, in a single tqb_decode_attention call (the append runs inside the attention kernel where the
    // tensor-core kernels apply).
    int append_and_attend(int layer, const void* k_dev, const void* v_dev, const void* q_dev, int dtype, int num_q_heads,
                          float softmax_scale, void* out_dev, cudaStream_t s) {
        const int64_t old_len = layers[layer].len;
        const bool was_active = layers[layer].active;
        TQB_TRY(ensure_capacity(layer, old_len + 1, s));
        Layer& l = layers[layer];
        l.len = old_len + 1;   // the attention call counts the new token
        l.active = true;
        const int st = attend(layer, q_dev, dtype, num_q_heads, softmax_scale, out_dev, dtype, nullptr, s, k_dev, v_dev);
        if (st != TQB_OK) {    // nothing was launched: the row was never written, so the token is not kept
            l.len = old_len;
            l.active = was_active;
        }
        return st;
    }

    int attend(int layer, const void* q_dev, int dtype, int num_q_heads, float softmax_scale, void* out_dev, int out_dtype,
               float* lse_out, cudaStream_t s, const void* append_k = nullptr, const void* append_v = nullptr) {
        Layer& l = layers[layer];
        tqb_decode_params p{};
        p.q = q_dev;
        p.k_indices = l.ki; p.k_scales = l.ks; p.v_indices = l.vi; p.v_scales = l.vs;
        p.out = out_dev;
        p.lse_out = lse_out;
        p.q_dtype = dtype;
        p.out_dtype = out_dtype;
        p.bits = cfg.bits; p.head_dim = cfg.head_dim; p.norm_mode = cfg.norm_mode; p.outlier_blocks = cfg.outlier_blocks;
        p.num_q_heads = cfg.batch * num_q_heads;
        p.num_kv_heads = heads;
        p.kv_len = (int32_t)l.len;
        p.kv_stride = (int32_t)l.cap;
        // two launches on the same layer in a row stay ordered: the second reads what the first appended
        const bool early = overlap && layer != last_attend_layer;
        last_attend_layer = layer;
        // (with the overlap switched on every launch takes the overlapped partition count, also the ordered ones in
        // between: the scratch layout then stays the same from launch to launch)
        p.num_partitions = overlap ? tqb_decode_num_partitions_overlapped(heads, (int32_t)l.len)
                                   : tqb_decode_num_partitions(heads, (int32_t)l.len);
        p.softmax_scale = softmax_scale;
        const size_t need = tqb_decode_scratch_bytes(p.num_q_heads, cfg.head_dim, p.num_partitions);
        TQB_TRY(prepare_scratch(scratch, ticket_heads, need, p.num_q_heads, cfg.head_dim, p.num_partitions, s));
        p.scratch = scratch.p;
        p.scratch_bytes = scratch.bytes;
        p.flags = TQB_DECODE_TICKETS_ZERO;
        if (early) p.flags |= TQB_DECODE_OVERLAP;
        p.append_k = append_k;
        p.append_v = append_v;
        return tqb_decode_attention(&p, s);
    }
    // Causal attention of the last q_len stored tokens' queries over the layer (q, out: [q_len, batch * Hq, D]).
    int attend_chunk(int layer, const void* q_dev, int dtype, int num_q_heads, int q_len, float softmax_scale, void* out_dev,
                     cudaStream_t s) {
        Layer& l = layers[layer];
        tqb_decode_params p{};
        p.q = q_dev;
        p.k_indices = l.ki; p.k_scales = l.ks; p.v_indices = l.vi; p.v_scales = l.vs;
        p.out = out_dev;
        p.q_dtype = dtype;
        p.out_dtype = dtype;
        p.bits = cfg.bits; p.head_dim = cfg.head_dim; p.norm_mode = cfg.norm_mode; p.outlier_blocks = cfg.outlier_blocks;
        p.num_q_heads = cfg.batch * num_q_heads;
        p.num_kv_heads = heads;
        p.kv_len = (int32_t)l.len;
        p.kv_stride = (int32_t)l.cap;
        p.num_partitions = tqb_decode_num_partitions(heads * q_len, (int32_t)l.len);
        p.softmax_scale = softmax_scale;
        const int folded = p.num_q_heads * q_len;
        const size_t need = tqb_decode_scratch_bytes(folded, cfg.head_dim, p.num_partitions);
        TQB_TRY(prepare_scratch(scratch, ticket_heads, need, folded, cfg.head_dim, p.num_partitions, s));
        p.scratch = scratch.p;
        p.scratch_bytes = scratch.bytes;
        p.flags = TQB_DECODE_TICKETS_ZERO;
        return tqb_chunk_attention(&p, q_len, s);
    }
    // Shard-local attention whose merging CTAs push the record to the ranks of a peer exchange (no append).
    int attend_push(int layer, const void* q_dev, int dtype, int num_q_heads, float softmax_scale, const PeerPush& push,
                    float* local_rec, cudaStream_t s) {
        Layer& l = layers[layer];
        tqb_decode_params p{};
        p.q = q_dev;
        p.k_indices = l.ki; p.k_scales = l.ks; p.v_indices = l.vi; p.v_scales = l.vs;
        p.num_q_heads = cfg.batch * num_q_heads;
        p.out = local_rec;                                        // not written through these two: the kernel stores the
        p.lse_out = local_rec + (size_t)p.num_q_heads * cfg.head_dim;   // record through the push targets
        p.q_dtype = dtype;
        p.out_dtype = TQB_F32;
        p.bits = cfg.bits; p.head_dim = cfg.head_dim; p.norm_mode = cfg.norm_mode; p.outlier_blocks = cfg.outlier_blocks;
        p.num_kv_heads = heads;
        p.kv_len = (int32_t)l.len;
        p.kv_stride = (int32_t)l.cap;
        p.num_partitions = tqb_decode_num_partitions(heads, (int32_t)l.len);
        p.softmax_scale = softmax_scale;
        const size_t need = tqb_decode_scratch_bytes(p.num_q_heads, cfg.head_dim, p.num_partitions);
        TQB_TRY(prepare_scratch(scratch, ticket_heads, need, p.num_q_heads, cfg.head_dim, p.num_partitions, s));
        p.scratch = scratch.p;
        p.scratch_bytes = scratch.bytes;
        p.flags = TQB_DECODE_TICKETS_ZERO;
        return decode_with_peer_push(&p, push, s);
    }
    int ticket_heads = -1;   // head count the zeroed ticket area of `scratch` was sized for
};

namespace tqb {
int peer_exchange_begin_step(tqb_peer_exchange* x, int num_q_heads, PeerPush& push, float** local_rec);
}

extern "C" {

int tqb_pqo_cache_create(const tqb_cache_config* cfg, tqb_pqo_cache** out) {
    if (!cfg || !out) return TQB_ERR_NULL_POINTER;
    *out = nullptr;
    // src/cache/pqo.rs:32-39, src/cache/precomputed/mod.rs:46-51
    if (cfg->head_dim <= 0 || cfg->head_dim % kBlock != 0) return TQB_ERR_INVALID_DIMENSION;
    if (cfg->bits < 3 || cfg->bits > 4) return TQB_ERR_UNSUPPORTED_BITS;
    if (cfg->head_dim > 256) return TQB_ERR_UNSUPPORTED;
    if (cfg->num_kv_heads <= 0 || cfg->num_layers <= 0 || cfg->batch <= 0) return TQB_ERR_INVALID_ARGUMENT;
    if (cfg->norm_mode != TQB_MAXNORM && cfg->norm_mode != TQB_L2NORM) return TQB_ERR_INVALID_ARGUMENT;
    tqb_pqo_cache* c = new (std::nothrow) tqb_pqo_cache();
    if (!c) return TQB_ERR_OUT_OF_MEMORY;
    c->cfg = *cfg;
    c->nblk = cfg->head_dim / kBlock;
    c->packed_dim = cfg->head_dim * cfg->bits / 8;
    c->heads = cfg->batch * cfg->num_kv_heads;
    c->layers.resize(cfg->num_layers);
    *out = c;
    return TQB_OK;
}

void tqb_pqo_cache_destroy(tqb_pqo_cache* c) {
    if (!c) return;
    for (auto& l : c->layers) c->free_layer(l);
    c->stage_k.release(); c->stage_v.release(); c->stage_q.release(); c->stage_out.release(); c->scratch.release();
    c->destroy_pipeline();
    delete c;
}

static int check_layer(const tqb_pqo_cache* c, int32_t layer) {
    if (!c) return TQB_ERR_NULL_POINTER;
    if (layer < 0 || layer >= (int32_t)c->layers.size()) return TQB_ERR_LAYER_OUT_OF_RANGE;
    return TQB_OK;
}

int tqb_pqo_cache_prefill(tqb_pqo_cache* c, int32_t layer, const void* k, const void* v, int32_t dtype,
                          int32_t new_tokens, void* k_out, void* v_out, int32_t host_buffers, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    TQB_TRY(check_layer(c, layer));
    if (new_tokens < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (dtype != TQB_F32 && dtype != TQB_F16 && dtype != TQB_BF16) return TQB_ERR_INVALID_ARGUMENT;
    if (new_tokens == 0) return TQB_OK;
    if (!k || !v) return TQB_ERR_NULL_POINTER;
    cudaStream_t s = as_stream(stream);
    const size_t bytes = (size_t)c->heads * new_tokens * c->cfg.head_dim * dtype_size(dtype);
    const void* kd = k;
    const void* vd = v;
    if (host_buffers) {
        TQB_TRY(c->stage_k.reserve(bytes));
        TQB_TRY(c->stage_v.reserve(bytes));
        TQB_CUDA(cudaMemcpyAsync(c->stage_k.p, k, bytes, cudaMemcpyHostToDevice, s));
        TQB_CUDA(cudaMemcpyAsync(c->stage_v.p, v, bytes, cudaMemcpyHostToDevice, s));
        kd = c->stage_k.p;
        vd = c->stage_v.p;
    }
    const int64_t old_len = c->layers[layer].len;
    TQB_TRY(c->quantize_and_store(layer, kd, vd, dtype, new_tokens, s));
    // pqo.rs:194-199: the first prefill hands back the original tensors
    if (old_len > 0 && k_out && v_out) TQB_TRY(c->dequantize_full(layer, k_out, v_out, dtype, host_buffers != 0, s));
    return TQB_OK;
}

int tqb_pqo_cache_prefill_attend(tqb_pqo_cache* c, int32_t layer, const void* k, const void* v, const void* q, int32_t dtype,
                                 int32_t new_tokens, int32_t num_q_heads, float softmax_scale, void* out,
                                 tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    TQB_TRY(check_layer(c, layer));
    if (new_tokens <= 0) return TQB_ERR_INVALID_ARGUMENT;
    if (dtype != TQB_F32 && dtype != TQB_F16 && dtype != TQB_BF16) return TQB_ERR_INVALID_ARGUMENT;
    if (num_q_heads <= 0 || num_q_heads % c->cfg.num_kv_heads != 0) return TQB_ERR_INVALID_ARGUMENT;
    if (!k || !v || !q || !out) return TQB_ERR_NULL_POINTER;
    cudaStream_t s = as_stream(stream);
    TQB_TRY(c->quantize_and_store(layer, k, v, dtype, new_tokens, s));
    return c->attend_chunk(layer, q, dtype, num_q_heads, new_tokens, softmax_scale, out, s);
}

int tqb_pqo_cache_decode(tqb_pqo_cache* c, int32_t layer, const void* k, const void* v, const void* q, int32_t dtype,
                         int32_t num_q_heads, float softmax_scale, void* out, int32_t host_buffers,
                         tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    TQB_TRY(check_layer(c, layer));
    if (!k || !v || !q || !out) return TQB_ERR_NULL_POINTER;
    if (dtype != TQB_F32 && dtype != TQB_F16 && dtype != TQB_BF16) return TQB_ERR_INVALID_ARGUMENT;
    if (num_q_heads <= 0 || num_q_heads % c->cfg.num_kv_heads != 0) return TQB_ERR_INVALID_ARGUMENT;
    cudaStream_t s = as_stream(stream);
    const size_t esz = dtype_size(dtype);
    const size_t kv_bytes = (size_t)c->heads * c->cfg.head_dim * esz;
    const size_t q_bytes = (size_t)c->cfg.batch * num_q_heads * c->cfg.head_dim * esz;
    if (!host_buffers) return c->append_and_attend(layer, k, v, q, dtype, num_q_heads, softmax_scale, out, s);
    // Pinned, device-mapped host buffers (cudaHostAlloc / cudaHostRegister under unified addressing): the attention
    // kernel reads k, v and q over PCIe itself and the merging CTAs store the result straight into `out`.  No copy
    // engine, no event between two launches - so the launches of successive layers can overlap like device-resident
    // ones - and the bytes cross PCIe once per step all the same.  The caller's buffers are in use until
    // tqb_pqo_cache_host_sync(), exactly as with the staged copies below.
    {
        void* dev[4] = {nullptr, nullptr, nullptr, nullptr};
        const void* host[4] = {k, v, q, out};
        bool mapped = true;
        for (int i = 0; i < 4 && mapped; ++i) {
            cudaPointerAttributes at{};
            if (cudaPointerGetAttributes(&at, host[i]) != cudaSuccess) { cudaGetLastError(); mapped = false; break; }
            mapped = at.type == cudaMemoryTypeHost && at.devicePointer != nullptr;
            dev[i] = at.devicePointer;
        }
        if (mapped) {
            const int st = c->append_and_attend(layer, dev[0], dev[1], dev[2], dtype, num_q_heads, softmax_scale, dev[3], s);
            if (st == TQB_OK) { c->direct_pending = true; c->direct_stream = s; }
            return st;
        }
    }
    // Host buffers: inputs go up on one copy stream into one of two staging slots, the kernels run on
    // the caller's stream once the slot is filled, and the result goes down on a second copy stream
    // once they are done, so the next call's inputs travel while this call's kernels run.  A slot is
    // refilled only after the kernels that read it are done, and its output is overwritten only after
    // the previous result has left it.  tqb_pqo_cache_host_sync() waits for the outstanding results.
    TQB_TRY(c->ensure_pipeline());
    tqb_pqo_cache::Slot& sl = c->slots[c->next_slot];
    c->next_slot ^= 1;
    const bool used = sl.k.p != nullptr;
    TQB_TRY(sl.k.reserve(kv_bytes));
    TQB_TRY(sl.v.reserve(kv_bytes));
    TQB_TRY(sl.q.reserve(q_bytes));
    TQB_TRY(sl.out.reserve(q_bytes));
    if (used) {
        TQB_CUDA(cudaStreamWaitEvent(c->copy_stream, sl.compute_done, 0));
        TQB_CUDA(cudaStreamWaitEvent(s, sl.out_done, 0));
    }
    TQB_CUDA(cudaMemcpyAsync(sl.k.p, k, kv_bytes, cudaMemcpyHostToDevice, c->copy_stream));
    TQB_CUDA(cudaMemcpyAsync(sl.v.p, v, kv_bytes, cudaMemcpyHostToDevice, c->copy_stream));
    TQB_CUDA(cudaMemcpyAsync(sl.q.p, q, q_bytes, cudaMemcpyHostToDevice, c->copy_stream));
    TQB_CUDA(cudaEventRecord(sl.in_ready, c->copy_stream));
    TQB_CUDA(cudaStreamWaitEvent(s, sl.in_ready, 0));
    TQB_TRY(c->append_and_attend(layer, sl.k.p, sl.v.p, sl.q.p, dtype, num_q_heads, softmax_scale, sl.out.p, s));
    TQB_CUDA(cudaEventRecord(sl.compute_done, s));
    TQB_CUDA(cudaStreamWaitEvent(c->down_stream, sl.compute_done, 0));
    TQB_CUDA(cudaMemcpyAsync(out, sl.out.p, q_bytes, cudaMemcpyDeviceToHost, c->down_stream));
    TQB_CUDA(cudaEventRecord(sl.out_done, c->down_stream));
    c->last_out = sl.out_done;
    return TQB_OK;
}

int tqb_pqo_cache_host_sync(tqb_pqo_cache* c) {
    if (!c) return TQB_ERR_NULL_POINTER;
    if (c->last_out) TQB_CUDA(cudaEventSynchronize(c->last_out));
    if (c->direct_pending) {
        c->direct_pending = false;
        TQB_CUDA(cudaStreamSynchronize(c->direct_stream));
    }
    return TQB_OK;
}

int tqb_pqo_cache_attend_partial(tqb_pqo_cache* c, int32_t layer, const void* q, int32_t dtype, int32_t num_q_heads,
                                 float softmax_scale, float* out_unnorm, float* lse_out, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    TQB_TRY(check_layer(c, layer));
    if (!q || !out_unnorm || !lse_out) return TQB_ERR_NULL_POINTER;
    if (num_q_heads <= 0 || num_q_heads % c->cfg.num_kv_heads != 0) return TQB_ERR_INVALID_ARGUMENT;
    return c->attend(layer, q, dtype, num_q_heads, softmax_scale, out_unnorm, TQB_F32, lse_out, as_stream(stream));
}

int tqb_pqo_cache_attend_push(tqb_pqo_cache* c, int32_t layer, const void* q, int32_t dtype, int32_t num_q_heads,
                              float softmax_scale, tqb_peer_exchange* x, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    TQB_TRY(check_layer(c, layer));
    if (!q || !x) return TQB_ERR_NULL_POINTER;
    if (dtype != TQB_F32 && dtype != TQB_F16 && dtype != TQB_BF16) return TQB_ERR_INVALID_ARGUMENT;
    if (num_q_heads <= 0 || num_q_heads % c->cfg.num_kv_heads != 0) return TQB_ERR_INVALID_ARGUMENT;
    if (c->layers[layer].len <= 0) return TQB_ERR_RANGE_OUT_OF_BOUNDS;   // every rank must hold a part of the sequence
    PeerPush push;
    float* local_rec = nullptr;
    TQB_TRY(peer_exchange_begin_step(x, c->cfg.batch * num_q_heads, push, &local_rec));
    return c->attend_push(layer, q, dtype, num_q_heads, softmax_scale, push, local_rec, as_stream(stream));
}

int tqb_pqo_cache_dequantize_full(tqb_pqo_cache* c, int32_t layer, void* k_out, void* v_out, int32_t dtype,
                                  int32_t host_buffers, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    TQB_TRY(check_layer(c, layer));
    if (!k_out || !v_out) return TQB_ERR_NULL_POINTER;
    if (dtype != TQB_F32 && dtype != TQB_F16 && dtype != TQB_BF16) return TQB_ERR_INVALID_ARGUMENT;
    return c->dequantize_full(layer, k_out, v_out, dtype, host_buffers != 0, as_stream(stream));
}

int64_t tqb_pqo_cache_seq_len(const tqb_pqo_cache* c, int32_t layer) {
    return check_layer(c, layer) == TQB_OK ? c->layers[layer].len : -1;
}
int64_t tqb_pqo_cache_capacity(const tqb_pqo_cache* c, int32_t layer) {
    return check_layer(c, layer) == TQB_OK ? c->layers[layer].cap : -1;
}

// No reference counterpart: lets the decode launches of successive layers overlap head to tail (TQB_DECODE_OVERLAP).
int tqb_pqo_cache_set_overlap(tqb_pqo_cache* c, int32_t enabled) {
    if (!c) return TQB_ERR_NULL_POINTER;
    c->overlap = enabled != 0;
    c->last_attend_layer = -1;
    return TQB_OK;
}

// CompressedStorage::reset (src/cache/storage.rs:175-185): drops the buffers.
int tqb_pqo_cache_reset(tqb_pqo_cache* c) {
    if (!c) return TQB_ERR_NULL_POINTER;
    TQB_CUDA(cudaDeviceSynchronize());
    for (auto& l : c->layers) c->free_layer(l);
    return TQB_OK;
}

// CompressedStorage::memory_usage (src/cache/storage.rs:188-202): counts stored tokens.
size_t tqb_pqo_cache_memory_usage(const tqb_pqo_cache* c) {
    if (!c) return 0;
    size_t total = 0;
    for (const auto& l : c->layers) {
        if (l.len == 0) continue;
        total += 2 * (size_t)c->heads * l.len * c->packed_dim;
        total += 2 * (size_t)c->heads * l.len * c->nblk * 2;
    }
    return total;
}

// Dense copy of one layer's stored rows (the capacity padding is dropped): indices [heads, len, packed_dim],
// scales [heads, len, nblk]; `host_buffers` != 0: the destinations are host memory.
int tqb_pqo_cache_export_layer(const tqb_pqo_cache* c, int32_t layer, uint8_t* k_indices, uint16_t* k_scales,
                               uint8_t* v_indices, uint16_t* v_scales, int32_t host_buffers, tqb_stream_t stream) {
    TQB_TRY(check_layer(c, layer));
    if (!k_indices || !k_scales || !v_indices || !v_scales) return TQB_ERR_NULL_POINTER;
    const auto& l = c->layers[layer];
    if (l.len == 0) return TQB_OK;
    cudaStream_t s = as_stream(stream);
    const cudaMemcpyKind kind = host_buffers ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
    const size_t iw = (size_t)l.len * c->packed_dim, sw = (size_t)l.len * c->nblk * 2;
    TQB_CUDA(cudaMemcpy2DAsync(k_indices, iw, l.ki, (size_t)l.cap * c->packed_dim, iw, c->heads, kind, s));
    TQB_CUDA(cudaMemcpy2DAsync(v_indices, iw, l.vi, (size_t)l.cap * c->packed_dim, iw, c->heads, kind, s));
    TQB_CUDA(cudaMemcpy2DAsync(k_scales, sw, l.ks, (size_t)l.cap * c->nblk * 2, sw, c->heads, kind, s));
    TQB_CUDA(cudaMemcpy2DAsync(v_scales, sw, l.vs, (size_t)l.cap * c->nblk * 2, sw, c->heads, kind, s));
    if (host_buffers) TQB_CUDA(cudaStreamSynchronize(s));
    return TQB_OK;
}

int tqb_pqo_cache_layer_ptrs(const tqb_pqo_cache* c, int32_t layer, const uint8_t** k_indices, const uint16_t** k_scales,
                             const uint8_t** v_indices, const uint16_t** v_scales) {
    TQB_TRY(check_layer(c, layer));
    const auto& l = c->layers[layer];
    if (k_indices) *k_indices = l.ki;
    if (k_scales) *k_scales = l.ks;
    if (v_indices) *v_indices = l.vi;
    if (v_scales) *v_scales = l.vs;
    return TQB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// QuantizedKVCache
// ---------------------------------------------------------------------------------------
struct tqb_kv_cache {
    tqb_config cfg;   // total bits
    uint64_t qjl_seed;
    int pb, sb;       // polar bytes and sign bytes per block
    struct Side {
        uint8_t* packed = nullptr;
        uint16_t* scales = nullptr;
        uint8_t* signs = nullptr;
        uint16_t* rnorms = nullptr;
        int64_t cap = 0;
    };
    struct Layer {
        Side k, v;
        int64_t nk = 0, nv = 0;
    };
    std::vector<Layer> layers;
    uint32_t* rbits = nullptr;
    DevBuf stage_a, stage_b, wv_scratch;

    void free_side(Side& s) {
        if (s.packed) cudaFree(s.packed);
        if (s.scales) cudaFree(s.scales);
        if (s.signs) cudaFree(s.signs);
        if (s.rnorms) cudaFree(s.rnorms);
        s = Side{};
    }

    int reserve(Side& s, int64_t used, int64_t needed, cudaStream_t st) {
        if (s.cap >= needed) return TQB_OK;
        int64_t new_cap = std::max<int64_t>(needed, std::max<int64_t>(2 * s.cap, 256));
        Side n;
        n.cap = new_cap;
        cudaError_t e;
        if ((e = cudaMalloc((void**)&n.packed, (size_t)new_cap * pb)) != cudaSuccess ||
            (e = cudaMalloc((void**)&n.scales, (size_t)new_cap * 2)) != cudaSuccess ||
            (e = cudaMalloc((void**)&n.signs, (size_t)new_cap * sb)) != cudaSuccess ||
            (e = cudaMalloc((void**)&n.rnorms, (size_t)new_cap * 2)) != cudaSuccess) {
            free_side(n);
            return cuda_fail(e);
        }
        if (used > 0) {
            TQB_CUDA(cudaMemcpyAsync(n.packed, s.packed, (size_t)used * pb, cudaMemcpyDeviceToDevice, st));
            TQB_CUDA(cudaMemcpyAsync(n.scales, s.scales, (size_t)used * 2, cudaMemcpyDeviceToDevice, st));
            TQB_CUDA(cudaMemcpyAsync(n.signs, s.signs, (size_t)used * sb, cudaMemcpyDeviceToDevice, st));
            TQB_CUDA(cudaMemcpyAsync(n.rnorms, s.rnorms, (size_t)used * 2, cudaMemcpyDeviceToDevice, st));
        }
        TQB_CUDA(cudaStreamSynchronize(st));
        free_side(s);
        s = n;
        return TQB_OK;
    }
};

extern "C" {

int tqb_kv_cache_create(const tqb_config* cfg, int32_t num_layers, uint64_t qjl_seed, tqb_kv_cache** out) {
    if (!cfg || !out) return TQB_ERR_NULL_POINTER;
    *out = nullptr;
    // the QJL stage needs 3 or 4 total bits (src/qjl.rs:277-279); the config itself is
    // validated as TurboQuantConfig::new does (src/packed/mod.rs:124-132)
    int st = tqb_config_validate(cfg);
    if (st != TQB_OK && st != TQB_ERR_UNSUPPORTED) return st;
    if (cfg->bits < 3) return TQB_ERR_UNSUPPORTED_BITS;
    tqb_config polar = *cfg;
    polar.bits = cfg->bits - 1;
    TQB_TRY(tqb_config_validate(&polar));
    if (num_layers < 0) return TQB_ERR_INVALID_ARGUMENT;
    tqb_kv_cache* c = new (std::nothrow) tqb_kv_cache();
    if (!c) return TQB_ERR_OUT_OF_MEMORY;
    c->cfg = *cfg;
    c->qjl_seed = qjl_seed;
    c->pb = (int)tqb_packed_bytes(polar.bits, cfg->dim);
    c->sb = cfg->dim / 8;
    c->layers.resize(num_layers);
    std::vector<uint32_t> rb((size_t)cfg->dim * (cfg->dim / 32));
    st = tqb_qjl_rademacher_bits(cfg->dim, qjl_seed, rb.data());
    if (st == TQB_OK) {
        cudaError_t e = cudaMalloc((void**)&c->rbits, rb.size() * 4);
        if (e == cudaSuccess) e = cudaMemcpy(c->rbits, rb.data(), rb.size() * 4, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) st = cuda_fail(e);
    }
    if (st != TQB_OK) {
        if (c->rbits) cudaFree(c->rbits);
        delete c;
        return st;
    }
    *out = c;
    return TQB_OK;
}

void tqb_kv_cache_destroy(tqb_kv_cache* c) {
    if (!c) return;
    for (auto& l : c->layers) {
        c->free_side(l.k);
        c->free_side(l.v);
    }
    if (c->rbits) cudaFree(c->rbits);
    c->stage_a.release(); c->stage_b.release(); c->wv_scratch.release();
    delete c;
}

static int kv_check_layer(const tqb_kv_cache* c, int32_t layer) {
    if (!c) return TQB_ERR_NULL_POINTER;
    if (layer < 0 || layer >= (int32_t)c->layers.size()) return TQB_ERR_LAYER_OUT_OF_RANGE;  // attention.rs:95-100
    return TQB_OK;
}

int tqb_kv_cache_push_batch(tqb_kv_cache* c, int32_t layer, const float* keys, const float* values, int64_t n,
                            int64_t vec_dim, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    TQB_TRY(kv_check_layer(c, layer));
    if (vec_dim != c->cfg.dim) return TQB_ERR_DIMENSION_MISMATCH;  // attention.rs:241-242, :102-116
    if (n < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (n == 0) return TQB_OK;
    if (!keys || !values) return TQB_ERR_NULL_POINTER;
    cudaStream_t s = as_stream(stream);
    auto& L = c->layers[layer];
    const size_t bytes = (size_t)n * c->cfg.dim * sizeof(float);
    TQB_TRY(c->stage_a.reserve(bytes));
    TQB_TRY(c->stage_b.reserve(bytes));
    TQB_TRY(c->reserve(L.k, L.nk, L.nk + n, s));
    TQB_TRY(c->reserve(L.v, L.nv, L.nv + n, s));
    TQB_CUDA(cudaMemcpyAsync(c->stage_a.p, keys, bytes, cudaMemcpyHostToDevice, s));
    TQB_CUDA(cudaMemcpyAsync(c->stage_b.p, values, bytes, cudaMemcpyHostToDevice, s));
    TQB_TRY(tqb_qjl_quantize_batch(&c->cfg, c->rbits, (const float*)c->stage_a.p, n, L.k.packed + L.nk * c->pb,
                                   L.k.scales + L.nk, L.k.signs + L.nk * c->sb, L.k.rnorms + L.nk, s));
    TQB_TRY(tqb_qjl_quantize_batch(&c->cfg, c->rbits, (const float*)c->stage_b.p, n, L.v.packed + L.nv * c->pb,
                                   L.v.scales + L.nv, L.v.signs + L.nv * c->sb, L.v.rnorms + L.nv, s));
    TQB_CUDA(cudaStreamSynchronize(s));
    L.nk += n;
    L.nv += n;
    return TQB_OK;
}

int tqb_kv_cache_attention_scores(tqb_kv_cache* c, int32_t layer, const float* query, int64_t query_len, float* scores,
                                  tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    TQB_TRY(kv_check_layer(c, layer));
    if (query_len != c->cfg.dim) return TQB_ERR_DIMENSION_MISMATCH;
    auto& L = c->layers[layer];
    if (L.nk == 0) return TQB_OK;  // attention.rs:325-327
    if (!query || !scores) return TQB_ERR_NULL_POINTER;
    cudaStream_t s = as_stream(stream);
    const int d = c->cfg.dim;
    TQB_TRY(c->stage_a.reserve(std::max<size_t>(2 * d * sizeof(float), c->stage_a.bytes)));
    TQB_TRY(c->stage_b.reserve((size_t)L.nk * sizeof(float)));
    float* qd = (float*)c->stage_a.p;
    float* rq = qd + d;
    TQB_CUDA(cudaMemcpyAsync(qd, query, d * sizeof(float), cudaMemcpyHostToDevice, s));
    TQB_TRY(tqb_qjl_query_projections(d, c->rbits, qd, 1, rq, s));
    TQB_TRY(tqb_qjl_attention_scores(&c->cfg, qd, rq, L.k.packed, L.k.scales, L.k.signs, L.k.rnorms, L.nk,
                                     (float*)c->stage_b.p, s));
    TQB_CUDA(cudaMemcpyAsync(scores, c->stage_b.p, (size_t)L.nk * sizeof(float), cudaMemcpyDeviceToHost, s));
    TQB_CUDA(cudaStreamSynchronize(s));
    return TQB_OK;
}

int tqb_kv_cache_weighted_values(tqb_kv_cache* c, int32_t layer, const float* weights, int64_t num_weights, float* out,
                                 tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    TQB_TRY(kv_check_layer(c, layer));
    auto& L = c->layers[layer];
    if (num_weights != L.nk) return TQB_ERR_DIMENSION_MISMATCH;  // attention.rs:373
    if (!out) return TQB_ERR_NULL_POINTER;
    cudaStream_t s = as_stream(stream);
    const int d = c->cfg.dim;
    const int64_t n = std::min(L.nv, num_weights);
    if (n == 0) {
        std::memset(out, 0, sizeof(float) * d);
        return TQB_OK;
    }
    if (!weights) return TQB_ERR_NULL_POINTER;
    TQB_TRY(c->stage_a.reserve((size_t)n * sizeof(float)));
    TQB_TRY(c->stage_b.reserve((size_t)d * sizeof(float)));
    TQB_TRY(c->wv_scratch.reserve(tqb_weighted_values_scratch_bytes(d)));
    TQB_CUDA(cudaMemcpyAsync(c->stage_a.p, weights, (size_t)n * sizeof(float), cudaMemcpyHostToDevice, s));
    TQB_TRY(tqb_weighted_values(&c->cfg, (const float*)c->stage_a.p, L.v.packed, L.v.scales, n, (float*)c->stage_b.p,
                                c->wv_scratch.p, c->wv_scratch.bytes, s));
    TQB_CUDA(cudaMemcpyAsync(out, c->stage_b.p, (size_t)d * sizeof(float), cudaMemcpyDeviceToHost, s));
    TQB_CUDA(cudaStreamSynchronize(s));
    return TQB_OK;
}

int tqb_kv_cache_dequantize_range(tqb_kv_cache* c, int32_t layer, int64_t start, int64_t end, int32_t is_keys, float* out,
                                  tqb_stream_t stream) {
    TQB_TRY(kv_check_layer(c, layer));
    auto& L = c->layers[layer];
    const auto& S = is_keys ? L.k : L.v;
    const int64_t count = is_keys ? L.nk : L.nv;
    if (!(start <= end && end <= count) || start < 0) return TQB_ERR_RANGE_OUT_OF_BOUNDS;  // attention.rs:118-132
    const int64_t n = end - start;
    if (n == 0) return TQB_OK;
    if (!out) return TQB_ERR_NULL_POINTER;
    cudaStream_t s = as_stream(stream);
    const size_t bytes = (size_t)n * c->cfg.dim * sizeof(float);
    TQB_TRY(c->stage_a.reserve(bytes));
    tqb_config polar = c->cfg;
    polar.bits = c->cfg.bits - 1;
    TQB_TRY(tqb_dequantize_batch(&polar, S.packed + start * c->pb, S.scales + start, n, (float*)c->stage_a.p, s));
    TQB_CUDA(cudaMemcpyAsync(out, c->stage_a.p, bytes, cudaMemcpyDeviceToHost, s));
    TQB_CUDA(cudaStreamSynchronize(s));
    return TQB_OK;
}

int tqb_kv_cache_export_packed_range(tqb_kv_cache* c, int32_t layer, int64_t start, int64_t end, int32_t is_keys,
                                     uint8_t* packed_bytes, uint16_t* scales, uint8_t* qjl_signs,
                                     uint16_t* residual_norms, tqb_stream_t stream) {
    TQB_TRY(kv_check_layer(c, layer));
    auto& L = c->layers[layer];
    const auto& S = is_keys ? L.k : L.v;
    const int64_t count = is_keys ? L.nk : L.nv;
    if (!(start <= end && end <= count) || start < 0) return TQB_ERR_RANGE_OUT_OF_BOUNDS;
    const int64_t n = end - start;
    if (n == 0) return TQB_OK;
    if (!packed_bytes || !scales) return TQB_ERR_NULL_POINTER;
    cudaStream_t s = as_stream(stream);
    TQB_CUDA(cudaMemcpyAsync(packed_bytes, S.packed + start * c->pb, (size_t)n * c->pb, cudaMemcpyDeviceToHost, s));
    TQB_CUDA(cudaMemcpyAsync(scales, S.scales + start, (size_t)n * 2, cudaMemcpyDeviceToHost, s));
    if (qjl_signs) TQB_CUDA(cudaMemcpyAsync(qjl_signs, S.signs + start * c->sb, (size_t)n * c->sb, cudaMemcpyDeviceToHost, s));
    if (residual_norms) TQB_CUDA(cudaMemcpyAsync(residual_norms, S.rnorms + start, (size_t)n * 2, cudaMemcpyDeviceToHost, s));
    TQB_CUDA(cudaStreamSynchronize(s));
    return TQB_OK;
}

int tqb_kv_cache_import_packed_range(tqb_kv_cache* c, int32_t layer, int32_t polar_bits, const uint8_t* packed_bytes,
                                     const uint16_t* scales, const uint8_t* qjl_signs_flat,
                                     const uint16_t* residual_norms, int64_t count, int64_t bytes_per_block,
                                     int64_t signs_per_block, int32_t is_keys, tqb_stream_t stream) {
    TQB_TRY(kv_check_layer(c, layer));
    if (count < 0) return TQB_ERR_INVALID_ARGUMENT;
    if (count == 0) return TQB_OK;
    if (polar_bits != c->cfg.bits - 1) return TQB_ERR_UNSUPPORTED;  // one polar width per cache in this build
    if (bytes_per_block != c->pb || signs_per_block != c->sb) return TQB_ERR_DIMENSION_MISMATCH;
    if (!packed_bytes || !scales || !qjl_signs_flat || !residual_norms) return TQB_ERR_NULL_POINTER;
    cudaStream_t s = as_stream(stream);
    auto& L = c->layers[layer];
    auto& S = is_keys ? L.k : L.v;
    int64_t& used = is_keys ? L.nk : L.nv;
    TQB_TRY(c->reserve(S, used, used + count, s));
    TQB_CUDA(cudaMemcpyAsync(S.packed + used * c->pb, packed_bytes, (size_t)count * c->pb, cudaMemcpyHostToDevice, s));
    TQB_CUDA(cudaMemcpyAsync(S.scales + used, scales, (size_t)count * 2, cudaMemcpyHostToDevice, s));
    TQB_CUDA(cudaMemcpyAsync(S.signs + used * c->sb, qjl_signs_flat, (size_t)count * c->sb, cudaMemcpyHostToDevice, s));
    TQB_CUDA(cudaMemcpyAsync(S.rnorms + used, residual_norms, (size_t)count * 2, cudaMemcpyHostToDevice, s));
    TQB_CUDA(cudaStreamSynchronize(s));
    used += count;
    return TQB_OK;
}

int64_t tqb_kv_cache_entry_count(const tqb_kv_cache* c, int32_t layer) {
    return kv_check_layer(c, layer) == TQB_OK ? c->layers[layer].nk : -1;  // attention.rs:443-445
}
int32_t tqb_kv_cache_num_layers(const tqb_kv_cache* c) { return c ? (int32_t)c->layers.size() : 0; }

size_t tqb_kv_cache_memory_usage(const tqb_kv_cache* c) {
    if (!c) return 0;
    // attention.rs:76-78: polar block (2 + packed) + signs + 2 bytes residual norm
    const size_t per = 2 + (size_t)c->pb + c->sb + 2;
    size_t total = 0;
    for (const auto& l : c->layers) total += per * (size_t)(l.nk + l.nv);
    return total;
}

size_t tqb_kv_cache_fp16_equivalent_memory(const tqb_kv_cache* c) {
    if (!c) return 0;
    size_t entries = 0;
    for (const auto& l : c->layers) entries += (size_t)l.nk;
    return entries * c->cfg.dim * 2 * 2;  // attention.rs:437-440
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// TqCache: block-32 polar codes (bits-1 codebook stored at `bits` width when outlier_blocks = 0)
// plus a head_dim-wide QJL sign sketch of the key residual (src/cache/tq.rs:21-412).
// The reference computes the sketch on the CPU after a device->host copy (tq.rs:396-410);
// here it is a kernel and nothing leaves the device.
// ---------------------------------------------------------------------------------------
namespace {

template <typename T>
__global__ void to_f32_kernel(const T* __restrict__ in, float* __restrict__ out, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = tqb::to_f32<T>(in[i]);
}

int convert_to_f32(const void* in, int dtype, float* out, long long n, cudaStream_t s) {
    const int grid = (int)std::min<long long>((n + 255) / 256, 148 * 8);
    if (dtype == TQB_F32) to_f32_kernel<float><<<grid, 256, 0, s>>>((const float*)in, out, n);
    else if (dtype == TQB_F16) to_f32_kernel<__half><<<grid, 256, 0, s>>>((const __half*)in, out, n);
    else to_f32_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)in, out, n);
    return tqb::check_launch(s);
}

}  // namespace

struct tqb_tq_cache {
    tqb_pqo_cache* base = nullptr;
    struct Q {
        uint8_t* signs = nullptr;
        uint16_t* norms = nullptr;
        int64_t cap = 0;
    };
    std::vector<Q> qjl;
    uint32_t* rbits = nullptr;
    DevBuf deq, qf32, rq;

    int sb() const { return base->cfg.head_dim / 8; }

    void free_q(Q& q) {
        if (q.signs) cudaFree(q.signs);
        if (q.norms) cudaFree(q.norms);
        q = Q{};
    }

    // ensure_qjl_capacity (src/cache/tq.rs:64-97)
    int ensure_qjl_capacity(int layer, int64_t needed, int64_t old_len, cudaStream_t s) {
        Q& q = qjl[layer];
        if (q.cap >= needed) return TQB_OK;
        const int64_t new_cap = needed + std::max<int64_t>(needed / 4, 128);
        Q n;
        n.cap = new_cap;
        const int heads = base->heads;
        cudaError_t e;
        if ((e = cudaMalloc((void**)&n.signs, (size_t)heads * new_cap * sb())) != cudaSuccess ||
            (e = cudaMalloc((void**)&n.norms, (size_t)heads * new_cap * 2)) != cudaSuccess) {
            free_q(n);
            return cuda_fail(e);
        }
        auto fill = [&]() -> cudaError_t {
            cudaError_t r;
            if ((r = cudaMemsetAsync(n.signs, 0, (size_t)heads * new_cap * sb(), s)) != cudaSuccess) return r;
            if ((r = cudaMemsetAsync(n.norms, 0, (size_t)heads * new_cap * 2, s)) != cudaSuccess) return r;
            if (old_len > 0 && q.signs) {
                if ((r = cudaMemcpy2DAsync(n.signs, (size_t)new_cap * sb(), q.signs, (size_t)q.cap * sb(), (size_t)old_len * sb(),
                                           heads, cudaMemcpyDeviceToDevice, s)) != cudaSuccess) return r;
                if ((r = cudaMemcpy2DAsync(n.norms, (size_t)new_cap * 2, q.norms, (size_t)q.cap * 2, (size_t)old_len * 2, heads,
                                           cudaMemcpyDeviceToDevice, s)) != cudaSuccess) return r;
            }
            return q.signs ? cudaStreamSynchronize(s) : cudaSuccess;
        };
        if ((e = fill()) != cudaSuccess) {
            cudaStreamSynchronize(s);
            free_q(n);
            return cuda_fail(e);
        }
        if (q.signs) free_q(q);
        q = n;
        return TQB_OK;
    }

    // quantize_and_store + compute_and_store_qjl (src/cache/tq.rs:99-183)
    int store(int layer, const void* k, const void* v, int dtype, int new_tokens, cudaStream_t s) {
        const int64_t old_len = base->layers[layer].len;
        const bool was_active = base->layers[layer].active;
        const auto& cfg = base->cfg;
        const int64_t rows = (int64_t)base->heads * new_tokens;
        // everything that can fail for lack of memory comes before the polar length advances
        TQB_TRY(ensure_qjl_capacity(layer, old_len + new_tokens, old_len, s));
        TQB_TRY(deq.reserve((size_t)rows * cfg.head_dim * sizeof(float)));
        TQB_TRY(base->quantize_and_store(layer, k, v, dtype, new_tokens, s));
        auto& L = base->layers[layer];
        int st = tqb_block_dequantize(cfg.bits, cfg.head_dim, cfg.norm_mode, cfg.outlier_blocks, L.ki, L.ks, rows, new_tokens,
                                      L.cap, old_len, deq.p, TQB_F32, s);
        if (st == TQB_OK)
            st = tqb_residual_sketch(cfg.head_dim, rbits, k, dtype, (const float*)deq.p, rows, qjl[layer].signs,
                                     qjl[layer].norms, new_tokens, qjl[layer].cap, old_len, s);
        if (st != TQB_OK) {   // tokens without a sketch are not kept
            L.len = old_len;
            L.active = was_active;
        }
        return st;
    }

    // compute_logit_bias (src/cache/tq.rs:185-253)
    int project(const void* q, int dtype, int num_q_heads, int q_len, cudaStream_t s) {
        const long long nq = (long long)base->cfg.batch * num_q_heads * q_len;
        const size_t bytes = (size_t)nq * base->cfg.head_dim * sizeof(float);
        TQB_TRY(qf32.reserve(bytes));
        TQB_TRY(rq.reserve(bytes));
        TQB_TRY(convert_to_f32(q, dtype, (float*)qf32.p, nq * base->cfg.head_dim, s));
        return tqb_qjl_query_projections(base->cfg.head_dim, rbits, (const float*)qf32.p, nq, (float*)rq.p, s);
    }

    int logit_bias(int layer, const void* q, int dtype, int num_q_heads, int q_len, void* bias, cudaStream_t s) {
        auto& L = base->layers[layer];
        if (L.len == 0) return TQB_OK;
        TQB_TRY(project(q, dtype, num_q_heads, q_len, s));
        return tqb_qjl_logit_bias(base->cfg.head_dim, (const float*)rq.p, qjl[layer].signs, qjl[layer].norms, bias, dtype,
                                  base->cfg.batch * num_q_heads, base->heads, q_len, (int32_t)L.len, (int32_t)qjl[layer].cap, s);
    }
};

extern "C" {

int tqb_tq_cache_create(const tqb_cache_config* cfg, tqb_tq_cache** out) {
    if (!cfg || !out) return TQB_ERR_NULL_POINTER;
    *out = nullptr;
    // the sign sketch spans the whole head_dim and needs a power of two of at least 32 here
    if (cfg->head_dim != 32 && cfg->head_dim != 64 && cfg->head_dim != 128 && cfg->head_dim != 256)
        return (cfg->head_dim > 0 && cfg->head_dim % kBlock == 0) ? TQB_ERR_UNSUPPORTED : TQB_ERR_INVALID_DIMENSION;
    tqb_pqo_cache* base = nullptr;
    TQB_TRY(tqb_pqo_cache_create(cfg, &base));
    tqb_tq_cache* c = new (std::nothrow) tqb_tq_cache();
    if (!c) { tqb_pqo_cache_destroy(base); return TQB_ERR_OUT_OF_MEMORY; }
    c->base = base;
    c->qjl.resize(cfg->num_layers);
    std::vector<uint32_t> rb((size_t)cfg->head_dim * (cfg->head_dim / 32));
    int st = tqb_qjl_rademacher_bits(cfg->head_dim, cfg->qjl_seed, rb.data());
    if (st == TQB_OK) {
        cudaError_t e = cudaMalloc((void**)&c->rbits, rb.size() * 4);
        if (e == cudaSuccess) e = cudaMemcpy(c->rbits, rb.data(), rb.size() * 4, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) st = cuda_fail(e);
    }
    if (st != TQB_OK) { tqb_tq_cache_destroy(c); return st; }
    *out = c;
    return TQB_OK;
}

void tqb_tq_cache_destroy(tqb_tq_cache* c) {
    if (!c) return;
    for (auto& q : c->qjl) c->free_q(q);
    if (c->rbits) cudaFree(c->rbits);
    c->deq.release(); c->qf32.release(); c->rq.release();
    tqb_pqo_cache_destroy(c->base);
    delete c;
}

static int tq_check(const tqb_tq_cache* c, int32_t layer) {
    if (!c) return TQB_ERR_NULL_POINTER;
    return check_layer(c->base, layer);
}

int tqb_tq_cache_prefill(tqb_tq_cache* c, int32_t layer, const void* k, const void* v, const void* q, int32_t dtype,
                         int32_t new_tokens, int32_t num_q_heads, int32_t q_len, void* k_out, void* v_out,
                         void* logit_bias, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    TQB_TRY(tq_check(c, layer));
    if (new_tokens < 0 || q_len <= 0 || num_q_heads <= 0 || num_q_heads % c->base->cfg.num_kv_heads != 0)
        return TQB_ERR_INVALID_ARGUMENT;
    if (dtype != TQB_F32 && dtype != TQB_F16 && dtype != TQB_BF16) return TQB_ERR_INVALID_ARGUMENT;
    if (!k || !v || !q || !logit_bias) return TQB_ERR_NULL_POINTER;
    cudaStream_t s = as_stream(stream);
    const int64_t old_len = c->base->layers[layer].len;
    if (new_tokens > 0) TQB_TRY(c->store(layer, k, v, dtype, new_tokens, s));
    // tq.rs:272-276: originals on the first call, else the dequantized cache
    if (old_len > 0 && k_out && v_out) TQB_TRY(c->base->dequantize_full(layer, k_out, v_out, dtype, false, s));
    return c->logit_bias(layer, q, dtype, num_q_heads, q_len, logit_bias, s);
}

int tqb_tq_cache_decode(tqb_tq_cache* c, int32_t layer, const void* k, const void* v, const void* q, int32_t dtype,
                        int32_t num_q_heads, void* k_out, void* v_out, void* logit_bias, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    TQB_TRY(tq_check(c, layer));
    if (num_q_heads <= 0 || num_q_heads % c->base->cfg.num_kv_heads != 0) return TQB_ERR_INVALID_ARGUMENT;
    if (dtype != TQB_F32 && dtype != TQB_F16 && dtype != TQB_BF16) return TQB_ERR_INVALID_ARGUMENT;
    if (!k || !v || !q || !k_out || !v_out || !logit_bias) return TQB_ERR_NULL_POINTER;
    cudaStream_t s = as_stream(stream);
    TQB_TRY(c->store(layer, k, v, dtype, 1, s));
    TQB_TRY(c->base->dequantize_full(layer, k_out, v_out, dtype, false, s));   // tq.rs:300-302
    return c->logit_bias(layer, q, dtype, num_q_heads, 1, logit_bias, s);
}

int tqb_tq_cache_decode_fused(tqb_tq_cache* c, int32_t layer, const void* k, const void* v, const void* q, int32_t dtype,
                              int32_t num_q_heads, float softmax_scale, void* out, tqb_stream_t stream) {
    TQB_NVTX_RANGE();
    TQB_TRY(tq_check(c, layer));
    if (num_q_heads <= 0 || num_q_heads % c->base->cfg.num_kv_heads != 0) return TQB_ERR_INVALID_ARGUMENT;
    if (dtype != TQB_F32 && dtype != TQB_F16 && dtype != TQB_BF16) return TQB_ERR_INVALID_ARGUMENT;
    if (!k || !v || !q || !out) return TQB_ERR_NULL_POINTER;
    cudaStream_t s = as_stream(stream);
    TQB_TRY(c->store(layer, k, v, dtype, 1, s));
    TQB_TRY(c->project(q, dtype, num_q_heads, 1, s));
    auto* b = c->base;
    auto& L = b->layers[layer];
    tqb_decode_params p{};
    p.q = q;
    p.k_indices = L.ki; p.k_scales = L.ks; p.v_indices = L.vi; p.v_scales = L.vs;
    p.out = out;
    p.qjl_signs = c->qjl[layer].signs; p.qjl_norms = c->qjl[layer].norms; p.rq = (const float*)c->rq.p;
    p.qjl_enabled = 1;
    p.q_dtype = dtype; p.out_dtype = dtype;
    p.bits = b->cfg.bits; p.head_dim = b->cfg.head_dim; p.norm_mode = b->cfg.norm_mode; p.outlier_blocks = b->cfg.outlier_blocks;
    p.num_q_heads = b->cfg.batch * num_q_heads;
    p.num_kv_heads = b->heads;
    p.kv_len = (int32_t)L.len;
    p.kv_stride = (int32_t)L.cap;
    if (c->qjl[layer].cap != L.cap) return TQB_ERR_UNSUPPORTED;   // both grow by the same rule; the kernel shares one stride
    p.num_partitions = tqb_decode_num_partitions(b->heads, (int32_t)L.len);
    p.softmax_scale = softmax_scale;
    const size_t need = tqb_decode_scratch_bytes(p.num_q_heads, b->cfg.head_dim, p.num_partitions);
    TQB_TRY(prepare_scratch(b->scratch, b->ticket_heads, need, p.num_q_heads, b->cfg.head_dim, p.num_partitions, s));
    p.scratch = b->scratch.p;
    p.scratch_bytes = b->scratch.bytes;
    p.flags = TQB_DECODE_TICKETS_ZERO;
    return tqb_decode_attention(&p, s);
}

int64_t tqb_tq_cache_seq_len(const tqb_tq_cache* c, int32_t layer) { return c ? tqb_pqo_cache_seq_len(c->base, layer) : -1; }

int tqb_tq_cache_reset(tqb_tq_cache* c) {
    if (!c) return TQB_ERR_NULL_POINTER;
    TQB_TRY(tqb_pqo_cache_reset(c->base));
    for (auto& q : c->qjl) c->free_q(q);   // tq.rs:316-324
    return TQB_OK;
}

// tq.rs:322-331: stored tokens of the polar part plus the ALLOCATED sketch tensors
size_t tqb_tq_cache_memory_usage(const tqb_tq_cache* c) {
    if (!c) return 0;
    size_t total = tqb_pqo_cache_memory_usage(c->base);
    for (const auto& q : c->qjl)
        if (q.signs) total += (size_t)c->base->heads * q.cap * (c->sb() + 2);
    return total;
}

int tqb_tq_cache_qjl_ptrs(const tqb_tq_cache* c, int32_t layer, const uint8_t** signs, const uint16_t** norms,
                          int64_t* capacity) {
    TQB_TRY(tq_check(c, layer));
    if (signs) *signs = c->qjl[layer].signs;
    if (norms) *norms = c->qjl[layer].norms;
    if (capacity) *capacity = c->qjl[layer].cap;
    return TQB_OK;
}

}  // extern "C"
