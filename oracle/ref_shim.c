/* Exports the reference's own host-compilable primitives (bit packing, sign pattern,
 * Rademacher hash) from its header src/cache/cuda/kernels/tq_common.h, included from the
 * reference checkout at build time.  Used only to validate the oracle restatement and to
 * generate golden fixtures; test infrastructure, never shipped. */
#include <stdint.h>
#include <string.h>
#include "tq_common.h"

uint8_t ref_unpack(int bits, const uint8_t *packed, int tid) {
    if (bits == 2) return tq_unpack_2bit(packed, tid);
    if (bits == 3) return tq_unpack_3bit(packed, tid);
    return tq_unpack_4bit(packed, tid);
}

/* Packs `count` codes the way the reference kernels do: zeroed output, then one
 * tq_pack_* call per element (tq_quant_kernel.cu:244-252). */
void ref_pack(int bits, const uint8_t *idx, int count, uint8_t *out, int out_bytes) {
    memset(out, 0, (size_t)out_bytes);
    for (int t = 0; t < count; ++t) {
        if (bits == 2) tq_pack_2bit(out, t, idx[t]);
        else if (bits == 3) tq_pack_3bit(out, t, idx[t]);
        else tq_pack_4bit(out, t, idx[t]);
    }
}

float ref_sign(uint64_t seed, int index) { return tq_sign(seed, index); }
uint64_t ref_mix_seed(uint64_t seed, int row) { return tq_mix_seed(seed, row); }
float ref_rademacher_sign(uint64_t seed, int row, int col) { return tq_rademacher_sign(seed, row, col); }
