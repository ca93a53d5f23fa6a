/* CPU restatement of the reference's data indexing (TEST INFRASTRUCTURE ONLY).
 *
 * hash_u64:      utils.h:13-18 (splitmix64 finaliser, 64-bit wrap-around arithmetic).
 * endpoint rule: cuda/dataset.cuh:12-16: endpoint = 8 + hash(seed + step*batch + seq) % (size - 8);
 *                x = data[e-ctx .. e), y = data[e-ctx+1 .. e]  (cuda/dataset.cuh:24-26).
 * The lower bound 8 is the reference's largest context; a longer context would index
 * before the buffer, so the rule is stated with lo = max(8, ctx), which is the same
 * number for every context the reference accepts.  Data-parallel ranks draw global
 * sequence rank*batch + seq of a global batch world*batch, which is the reference rule
 * when world = 1.
 */
#include <stdint.h>

uint64_t oracle_hash_u64(uint64_t x) {
    x += 0x9e3779b97f4a7c15ULL;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
    return x ^ (x >> 31);
}

int64_t oracle_endpoint(uint64_t seed, uint64_t step, int batch, int world, int rank, int sequence,
                        int context, int64_t size) {
    int64_t lo = context > 8 ? context : 8;
    uint64_t global_batch = (uint64_t)batch * (uint64_t)world;
    uint64_t global_sequence = (uint64_t)rank * (uint64_t)batch + (uint64_t)sequence;
    return lo + (int64_t)(oracle_hash_u64(seed + step * global_batch + global_sequence) %
                          (uint64_t)(size - lo));
}

/* Fills x[batch*context], y[batch*context] for one rank's share of one step. */
void oracle_byte_batch(const uint8_t *data, int64_t size, uint64_t seed, uint64_t step, int batch,
                       int world, int rank, int context, uint8_t *x, uint8_t *y) {
    for (int s = 0; s < batch; ++s) {
        int64_t e = oracle_endpoint(seed, step, batch, world, rank, s, context, size);
        for (int p = 0; p < context; ++p) {
            x[(int64_t)s * context + p] = data[e - context + p];
            y[(int64_t)s * context + p] = data[e - context + p + 1];
        }
    }
}
