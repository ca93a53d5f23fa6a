// Fused causal softmax attention on the 5th-generation tensor cores, head size 64, BF16.
// Replaces the reference's per-(query, head) scalar attention loops (cuda/attention.cuh:33-106)
// for the scaled architecture: no T x T matrix ever reaches HBM.
//
// Forward: one CTA per 128 query rows of one (batch, head).  Warp 0 streams K/V in steps of 64
// keys with TMA (four-slot ring); warp 1 issues tcgen05.mma: S = Q K^T into tensor memory, then
// O += P V with P read back from tensor memory as the A operand.  The exponential (16 per clock
// and SM) bounds the kernel, so the softmax work is arranged to keep that unit busy: the steps
// alternate between two chains, each a complete online softmax with its own score buffer,
// reference maximum, row sum and output accumulator in tensor memory and its own four warps (thread
// = query row = TMEM lane, so maxima and sums are thread-local).  While one chain is in its
// exponentials the other waits for its scores or hands its probabilities to the MMA thread; the
// chains never wait for each other and are merged once at the end.  An accumulator is rescaled only
// when its row maximum has grown by more than 2^8.  Two CTAs share an SM (256 TMEM columns and 84 KB
// of shared memory each).
#include "device_utils.cuh"
#include "sm100.cuh"

using namespace sm100;

namespace {
constexpr int BlockM = 128, BlockN = 128, HeadSize = 64;
constexpr int TileBytes = 128 * HeadSize * 2; // 16 KB: a Q, K or V tile
constexpr int KeyStep = 64, KeyBytes = KeyStep * HeadSize * 2; // the forward pass takes 64 keys (8 KB of K, of V) per step
constexpr int ForwardRing = 4;                                 // shared-memory ring of (K, V) steps
constexpr int ForwardThreads = 320;                            // warp 0 TMA, warp 1 MMA, 8 softmax warps
constexpr int ForwardShared = TileBytes + ForwardRing * 2 * KeyBytes + 2048 + 1024 + 256; // Q, ring, merge buffer
constexpr int ForwardTmemColumns = 256; // per chain: 64 score columns, 64 output columns

struct ForwardParams {
    bf16 *out;
    float *lse;
    int batch, context, heads, width, tiles;
    float scale_log2; // log2(e) / sqrt(d_head)
    StepCounters *counters;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(ForwardThreads, 2)
flash_forward_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                     ForwardParams p) {
    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (smem_address(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - smem_address(raw_shared));
    float *exchange = reinterpret_cast<float *>(aligned + TileBytes + ForwardRing * 2 * KeyBytes); // [2 chains][max | sum][128 rows]
    uint64_t *barriers = reinterpret_cast<uint64_t *>(exchange + 4 * BlockM);
    const uint32_t q_full = smem_address(barriers), kv_full0 = q_full + 8, kv_empty0 = kv_full0 + 8 * ForwardRing,
                   s_full0 = kv_empty0 + 8 * ForwardRing, p_full0 = s_full0 + 16, o_full0 = p_full0 + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(barriers + 1 + 2 * ForwardRing + 6);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t smem_q = base, smem_kv = base + TileBytes;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    // Long tiles first: tile index falls as blockIdx grows.
    const int pairs = p.batch * p.heads;
    const int tile = p.tiles - 1 - int(blockIdx.x / pairs);
    const int bh = blockIdx.x % pairs, b = bh / p.heads, h = bh % p.heads;
    const int row0 = b * p.context; // first row of this sequence in the packed qkv matrix
    const int last_key = min(p.context, (tile + 1) * BlockM);
    const int steps = (last_key + KeyStep - 1) / KeyStep; // causal: keys 0 .. last_key - 1, 64 per step

    grid_launch_dependents(); // the next kernel may set itself up while this one runs
    if (threadIdx.x == 0) {
        mbarrier_init(q_full, 1);
        for (int s = 0; s < ForwardRing; ++s) {
            mbarrier_init(kv_full0 + 8 * s, 1);
            mbarrier_init(kv_empty0 + 8 * s, 1);
        }
        for (int c = 0; c < 2; ++c) {
            mbarrier_init(s_full0 + 8 * c, 1);
            mbarrier_init(p_full0 + 8 * c, 4);
            mbarrier_init(o_full0 + 8 * c, 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_map(&map_q);
        prefetch_map(&map_kv);
    }
    if (warp == 1) {
        tmem_alloc(smem_address(tmem_slot), ForwardTmemColumns);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // chain c: scores of its steps at 64 c (the probabilities pack into the first 32 of those columns),
    // its output accumulator at 128 + 64 c
    const uint32_t tmem_s0 = tmem_base, tmem_o0 = tmem_base + 128;

    if (warp == 0) {
        if (elect_one()) {
            mbarrier_expect_tx(q_full, TileBytes);
            tma_load_3d(smem_q, &map_q, h * HeadSize, row0 + tile * BlockM, 0, q_full);
            for (int j = 0; j < steps; ++j) {
                const int ring = j % ForwardRing;
                if (!mbarrier_wait(kv_empty0 + 8 * ring, ((j / ForwardRing) & 1) ^ 1, abort_flag, p.counters, 201))
                    break;
                const uint32_t bar = kv_full0 + 8 * ring, dst = smem_kv + ring * 2 * KeyBytes;
                mbarrier_expect_tx(bar, 2 * KeyBytes);
                tma_load_3d(dst, &map_kv, p.width + h * HeadSize, row0 + j * KeyStep, 0, bar);
                tma_load_3d(dst + KeyBytes, &map_kv, 2 * p.width + h * HeadSize, row0 + j * KeyStep, 0, bar);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc_s = instruction_descriptor(BlockM, KeyStep, 0, 0);
            const uint32_t idesc_o = instruction_descriptor(BlockM, HeadSize, 0, 1);
            const uint64_t q_desc = smem_descriptor(smem_q, 16, 1024), k_desc0 = smem_descriptor(smem_kv, 16, 1024),
                           v_desc0 = smem_descriptor(smem_kv + KeyBytes, 8192, 1024);
            bool ok = mbarrier_wait(q_full, 0, abort_flag, p.counters, 202);
            int issued = 0;
            auto issue_scores = [&]() { // S = Q K_j^T into the buffer of chain j % 2
                const int ring = issued % ForwardRing, chain = issued & 1;
                ok = mbarrier_wait(kv_full0 + 8 * ring, (issued / ForwardRing) & 1, abort_flag, p.counters, 203);
                if (!ok)
                    return;
                tcgen05_fence_after();
                const uint64_t k_desc = descriptor_at(k_desc0, ring * 2 * KeyBytes);
#pragma unroll
                for (int ks = 0; ks < HeadSize / 16; ++ks)
                    tcgen05_mma_bf16(tmem_s0 + 64 * chain, descriptor_at(q_desc, ks * 32), descriptor_at(k_desc, ks * 32),
                                     idesc_s, ks > 0);
                tcgen05_commit(s_full0 + 8 * chain);
                ++issued;
            };
            if (ok)
                issue_scores();
            if (ok && steps > 1)
                issue_scores();
            for (int j = 0; j < steps && ok; ++j) {
                const int chain = j & 1, ring = j % ForwardRing;
                ok = mbarrier_wait(p_full0 + 8 * chain, (j >> 1) & 1, abort_flag, p.counters, 204);
                if (!ok)
                    break;
                tcgen05_fence_after();
                const uint64_t v_desc = descriptor_at(v_desc0, ring * 2 * KeyBytes);
#pragma unroll
                for (int ks = 0; ks < KeyStep / 16; ++ks) // O_chain += P V_j: four 16-key steps
                    tcgen05_mma_bf16_ts(tmem_o0 + 64 * chain, tmem_s0 + 64 * chain + ks * 8,
                                        descriptor_at(v_desc, ks * 2048), idesc_o, (j > 1 || ks > 0) ? 1u : 0u);
                tcgen05_commit(o_full0 + 8 * chain);
                tcgen05_commit(kv_empty0 + 8 * ring); // K_j and V_j are no longer read
                if (issued < steps)
                    issue_scores(); // step j + 2 reuses this chain's buffer: issued after the products that read it
            }
        }
    } else {
        // Eight softmax warps: two per TMEM lane quarter, one for each chain.  A chain takes every
        // other 64-key step and is a complete online softmax of its own (reference maximum, sum and
        // output accumulator), so the two never wait for each other; they are merged at the end.
        const int quarter = warp % 4, chain = (warp - 2) / 4;
        const int row = quarter * 32 + lane;              // query row inside the tile = TMEM lane
        const int position = tile * BlockM + row;          // position inside the sequence
        const int warp_first = tile * BlockM + quarter * 32;
        const uint32_t lanes = uint32_t(quarter * 32) << 16;
        const uint32_t tmem_s = tmem_s0 + 64 * chain + lanes, tmem_o = tmem_o0 + 64 * chain + lanes;
        // Probabilities are taken relative to a reference maximum that is only moved (and the output
        // rescaled) when the true maximum has grown by more than 2^8: values stay inside BF16/FP32 range
        // and the final division by the row sum, accumulated with the same reference, makes the result exact.
        float reference_max = -CUDART_INF_F, running_sum = 0.f;
        bool ok = true;
        int mine = 0; // steps this chain has taken
        for (int j = chain; j < steps; j += 2, ++mine) {
            ok = mbarrier_wait(s_full0 + 8 * chain, mine & 1, abort_flag, p.counters, 206);
            if (!ok)
                break;
            tcgen05_fence_after();
            const int key0 = j * KeyStep;
            const bool diagonal = key0 + KeyStep - 1 > warp_first; // some key of the step lies after some query of the warp
            if (mine > 0 && !diagonal) {
                // One pass: exponentials against the reference maximum this chain already has, the row
                // maximum tracked on the side.  That is exact as long as no row's maximum has grown by
                // more than 2^8; if one has, nothing has been written yet and the step is redone below.
                const float offset = reference_max * p.scale_log2;
                uint32_t packed[32];
                float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, sum0 = 0.f, sum1 = 0.f;
#pragma unroll
                for (int part = 0; part < 4; ++part) { // 16 keys at a time
                    uint32_t s[16];
                    tmem_load_32x16_async(tmem_s + part * 16, s);
                    tmem_wait_load(s);
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        const float x0 = __uint_as_float(s[i]), x1 = __uint_as_float(s[i + 1]);
                        m0 = fmaxf(m0, x0);
                        m1 = fmaxf(m1, x1);
                        const float p0 = fast_exp2(fmaf(x0, p.scale_log2, -offset));
                        const float p1 = fast_exp2(fmaf(x1, p.scale_log2, -offset));
                        sum0 += p0;
                        sum1 += p1;
                        packed[part * 8 + i / 2] = pack_bf16(p0, p1);
                    }
                }
                const bool fits = (fmaxf(m0, m1) - reference_max) * p.scale_log2 <= 8.f; // false for a -inf reference
                if (__all_sync(0xffffffffu, fits)) {
                    tmem_store_32x32(tmem_s, packed);
                    tmem_wait_store();
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0)
                        mbarrier_arrive(p_full0 + 8 * chain);
                    running_sum += sum0 + sum1;
                    continue;
                }
            }
            float block_max = -CUDART_INF_F;
            { // first pass over the scores: the row maximum, 32 keys at a time
                float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t s[32];
                    tmem_load_32x32_async(tmem_s + half * 32, s);
                    tmem_wait_load(s);
                    if (diagonal) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (key0 + half * 32 + i > position)
                                s[i] = 0xff800000u;
                    }
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        m0 = fmaxf(m0, __uint_as_float(s[i]));
                        m1 = fmaxf(m1, __uint_as_float(s[i + 1]));
                    }
                }
                block_max = fmaxf(m0, m1);
            }
            const bool grow = (block_max - reference_max) * p.scale_log2 > 8.f; // true for the first unmasked step
            if (__any_sync(0xffffffffu, grow && reference_max != -CUDART_INF_F)) {
                // the accumulator is rescaled only between this chain's products: wait for the last one
                ok = mbarrier_wait(o_full0 + 8 * chain, (mine - 1) & 1, abort_flag, p.counters, 207);
                if (!ok)
                    break;
                tcgen05_fence_after();
                const float correction =
                    grow && reference_max != -CUDART_INF_F ? fast_exp2((reference_max - block_max) * p.scale_log2) : 1.f;
                running_sum *= correction;
#pragma unroll 1
                for (int half = 0; half < 2; ++half) { // 32 columns at a time keeps the register count down
                    uint32_t a[32];
                    tmem_load_32x32_async(tmem_o + half * 32, a);
                    tmem_wait_load(a);
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        a[i] = __float_as_uint(__uint_as_float(a[i]) * correction);
                    tmem_store_32x32(tmem_o + half * 32, a);
                }
            }
            if (grow)
                reference_max = block_max;
            // a row with nothing unmasked so far (it lies before every key this chain has seen) has
            // reference_max = -inf: every probability below is exp2(-inf) = 0 with offset 0
            const float offset = reference_max == -CUDART_INF_F ? 0.f : reference_max * p.scale_log2;
            float sums[2] = {0.f, 0.f};
#pragma unroll
            for (int half = 0; half < 2; ++half) { // second pass: exponentials, 32 keys at a time
                uint32_t s[32], packed[16];
                tmem_load_32x32_async(tmem_s + half * 32, s);
                tmem_wait_load(s);
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0 = fast_exp2(fmaf(__uint_as_float(s[i]), p.scale_log2, -offset));
                    float p1 = fast_exp2(fmaf(__uint_as_float(s[i + 1]), p.scale_log2, -offset));
                    if (diagonal) {
                        if (key0 + half * 32 + i > position) p0 = 0.f;
                        if (key0 + half * 32 + i + 1 > position) p1 = 0.f;
                    }
                    sums[0] += p0;
                    sums[1] += p1;
                    packed[i / 2] = pack_bf16(p0, p1);
                }
                // the packed half lands on score columns 16 half .. 16 half + 15, which both passes have
                // finished with (half 1 is read from columns 32 .. 63 before this store is issued)
                tmem_store_32x16(tmem_s + half * 16, packed);
            }
            tmem_wait_store();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0)
                mbarrier_arrive(p_full0 + 8 * chain);
            running_sum += sums[0] + sums[1];
        }
        if (ok && mine > 0)
            ok = mbarrier_wait(o_full0 + 8 * chain, (mine - 1) & 1, abort_flag, p.counters, 208);
        // merge the two chains: each publishes its reference maximum and sum, then takes half of the
        // output columns of both accumulators
        exchange[chain * 2 * BlockM + row] = reference_max;
        exchange[chain * 2 * BlockM + BlockM + row] = running_sum;
        tcgen05_fence_before();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        tcgen05_fence_after();
        const int other = chain ^ 1;
        const float other_max = exchange[other * 2 * BlockM + row], other_sum = exchange[other * 2 * BlockM + BlockM + row];
        const float top = fmaxf(reference_max, other_max); // chain 0 has seen key 0: never -inf for a valid row
        const float mine_factor = reference_max == -CUDART_INF_F ? 0.f : fast_exp2((reference_max - top) * p.scale_log2);
        const float other_factor = other_max == -CUDART_INF_F ? 0.f : fast_exp2((other_max - top) * p.scale_log2);
        const float total = running_sum * mine_factor + other_sum * other_factor;
        ok = __all_sync(0xffffffffu, ok && *abort_flag == 0); // the warp stores together or not at all
        if (ok) {
            const float inverse = 1.f / total;
            uint32_t a[32], c[32];
            // this warp's half of the columns (32 chain .. 32 chain + 31) from its own and the other accumulator;
            // an accumulator whose chain took no step was never written and is not read
            const bool other_used = steps > 1 || other == 0;
            tmem_load_32x32_async(tmem_o + chain * 32, a);
            if (other_used)
                tmem_load_32x32_async(tmem_o0 + 64 * other + lanes + chain * 32, c);
            tmem_wait_load(a);
            if (other_used)
                tmem_wait_load(c);
            const bool mine_used = mine > 0;
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                float v[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const float x = mine_used ? __uint_as_float(a[i + u]) * mine_factor : 0.f;
                    const float y = other_used ? __uint_as_float(c[i + u]) * other_factor : 0.f;
                    v[u] = (x + y) * inverse;
                }
                packed[i / 2] = pack_bf16(v[0], v[1]);
            }
            // through the Q tile, which no product reads any more: 2 KB per warp
            const int first = tile * BlockM + (row & ~31);
            store_rows_through_shared(smem_q + (warp - 2) * 2048, packed,
                                      p.out + (int64_t(row0) + first) * p.width + h * HeadSize + chain * 32,
                                      int64_t(p.width) * 2, p.context - first, lane);
            if (chain == 0 && position < p.context) // natural-log sum-exp of the scaled scores
                p.lse[(int64_t(b) * p.heads + h) * p.context + position] =
                    (top * p.scale_log2 + log2f(total)) * 0.6931471805599453f;
        }
    }
    __syncthreads();
    if (*abort_flag)
        __nanosleep(2000000);
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1)
        tmem_dealloc(tmem_base, ForwardTmemColumns);
}

// ------------------------------------------------------------------------------------------
// Backward.  Two kernels, both deterministic (no atomics):
//   dq kernel    : one CTA per 128 query rows, stepping over keys 64 at a time.  S = Q K^T and
//                  dP = dO V^T land in tensor memory; thread = query row computes
//                  dS = P (dP - delta) with P = exp(S / sqrt(d) - lse), packs it to BF16 over S,
//                  and dQ += dS K accumulates in tensor memory; 1 / sqrt(d) is applied once at the end.
//                  It also computes delta = rowsum(dO * O) and leaves it for the second kernel.
//   dk/dv kernel : one CTA per 128 keys, stepping over queries 32 at a time with everything
//                  transposed (S^T = K Q^T, dP^T = V dO^T: thread = key row), so P^T and dS^T are
//                  A operands in tensor memory for dV += P^T dO and dK += dS^T Q.
// Both are software pipelines: score buffers are double-buffered in tensor memory and the MMA thread
// issues the score products ahead of the accumulating products, so the tensor pipe works on the
// neighbouring steps while the compute warps turn one step's scores into dS.  256 TMEM columns and
// under 100 KB of shared memory per CTA: two CTAs share an SM.
// ------------------------------------------------------------------------------------------
constexpr int BackwardThreads = 320, BackwardTmemColumns = 256; // warp 0 TMA, warp 1 MMA, 8 compute warps

struct BackwardParams {
    const bf16 *out; // forward output, for delta = rowsum(dO * O)
    bf16 *dqkv;
    const float *lse;
    // [2][batch * heads][tiles * 128]: every query's lse in base 2, then its delta, in rows padded to whole tiles
    // (zeros in the padding); written by the dq kernel, fetched 64 at a time by the dk/dv kernel that follows it
    float *statistics;
    int batch, context, heads, width, tiles;
    float scale, scale_log2;
    StepCounters *counters;
};

// A warp's 32 accumulator rows x 32 columns from tensor memory, scaled, to BF16 in global memory (whole
// warp; `staging`: 2 KB of shared memory the warp may use; `first_row`: global address of row 0's first column).
__device__ __forceinline__ void store_accumulator(uint32_t address, uint32_t staging, bf16 *first_row, int64_t row_elements,
                                                  int valid_rows, float factor, int lane) {
    uint32_t a[32], packed[16];
    tmem_load_32x32_async(address, a);
    tmem_wait_load(a);
#pragma unroll
    for (int i = 0; i < 16; ++i)
        packed[i] = pack_bf16(__uint_as_float(a[2 * i]) * factor, __uint_as_float(a[2 * i + 1]) * factor);
    store_rows_through_shared(staging, packed, first_row, row_elements * 2, valid_rows, lane);
}

// dq kernel.  64 keys per step.  S = Q K^T is double-buffered in tensor memory and issued two steps
// ahead, so a step's exponentials (the long, SFU-bound part) run while the MMA thread is still
// issuing the previous step's dQ product and this step's dP = dO V^T; dP has one buffer and is only
// needed for the final multiply.  Twelve MMAs per 64 keys (4 S, 4 dP, 4 dQ) keep the issuing thread,
// which pays 40-80 clocks per small MMA, off the critical path.
constexpr int DqStep = 64, DqStepBytes = DqStep * HeadSize * 2, DqRing = 4;
constexpr int DqShared = 2 * TileBytes + DqRing * 2 * DqStepBytes + 1024 + 256; // Q, dO + ring of (K, V)

__global__ void __launch_bounds__(BackwardThreads, 2)
flash_dq_kernel(const __grid_constant__ CUtensorMap map_qkv128, const __grid_constant__ CUtensorMap map_qkv64,
                const __grid_constant__ CUtensorMap map_do128, BackwardParams p) {
    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (smem_address(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - smem_address(raw_shared));
    uint64_t *barriers = reinterpret_cast<uint64_t *>(aligned + 2 * TileBytes + DqRing * 2 * DqStepBytes);
    const uint32_t qdo_full = smem_address(barriers), kv_full0 = qdo_full + 8, kv_empty0 = kv_full0 + 8 * DqRing,
                   s_full0 = kv_empty0 + 8 * DqRing, ds_full0 = s_full0 + 16, dp_full = ds_full0 + 16,
                   dq_done = dp_full + 8; // 1 + 2 DqRing + 2 + 2 + 1 + 1 = 15 barriers
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(barriers + 7 + 2 * DqRing);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t smem_q = base, smem_do = base + TileBytes, smem_kv = base + 2 * TileBytes;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int pairs = p.batch * p.heads;
    const int tile = p.tiles - 1 - int(blockIdx.x / pairs);
    const int bh = blockIdx.x % pairs, b = bh / p.heads, h = bh % p.heads;
    const int row0 = b * p.context;
    const int last_key = min(p.context, (tile + 1) * BlockM); // keys 0..last_key-1 can be attended
    const int blocks = (last_key + DqStep - 1) / DqStep;

    grid_launch_dependents(); // the next kernel may set itself up while this one runs
    if (threadIdx.x == 0) {
        mbarrier_init(qdo_full, 1);
        for (int s = 0; s < DqRing; ++s) {
            mbarrier_init(kv_full0 + 8 * s, 1);
            mbarrier_init(kv_empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbarrier_init(s_full0 + 8 * s, 1);
            mbarrier_init(ds_full0 + 8 * s, 8);
        }
        mbarrier_init(dp_full, 1);
        mbarrier_init(dq_done, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_address(tmem_slot), BackwardTmemColumns);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // S buffers at 0 and 64 (a half's packed dS goes to the first 16 columns of its own 32), dP at 128, dQ at 192
    const uint32_t tmem_dp = tmem_base + 128, tmem_dq = tmem_base + 192;

    if (warp == 0) {
        if (elect_one()) {
            mbarrier_expect_tx(qdo_full, 2 * TileBytes);
            tma_load_3d(smem_q, &map_qkv128, h * HeadSize, row0 + tile * BlockM, 0, qdo_full);
            tma_load_3d(smem_do, &map_do128, h * HeadSize, row0 + tile * BlockM, 0, qdo_full);
            for (int j = 0; j < blocks; ++j) {
                const int ring = j % DqRing;
                if (!mbarrier_wait(kv_empty0 + 8 * ring, ((j / DqRing) & 1) ^ 1, abort_flag, p.counters, 301))
                    break;
                const uint32_t bar = kv_full0 + 8 * ring, dst = smem_kv + ring * 2 * DqStepBytes;
                mbarrier_expect_tx(bar, 2 * DqStepBytes);
                tma_load_3d(dst, &map_qkv64, p.width + h * HeadSize, row0 + j * DqStep, 0, bar);
                tma_load_3d(dst + DqStepBytes, &map_qkv64, 2 * p.width + h * HeadSize, row0 + j * DqStep, 0, bar);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc_s = instruction_descriptor(BlockM, DqStep, 0, 0);
            const uint32_t idesc_dq = instruction_descriptor(BlockM, HeadSize, 0, 1);
            // descriptors are built once; every MMA below only offsets them
            const uint64_t q_desc = smem_descriptor(smem_q, 16, 1024), do_desc = smem_descriptor(smem_do, 16, 1024),
                           kv_desc = smem_descriptor(smem_kv, 16, 1024), k_mn_desc = smem_descriptor(smem_kv, 8192, 1024);
            bool ok = mbarrier_wait(qdo_full, 0, abort_flag, p.counters, 302);
            auto issue_s = [&](int j) { // S = Q K_j^T into buffer j % 2; also the first use of ring slot j
                const int ring = j % DqRing;
                ok = mbarrier_wait(kv_full0 + 8 * ring, (j / DqRing) & 1, abort_flag, p.counters, 303);
                if (!ok)
                    return;
                tcgen05_fence_after();
                const uint64_t k_desc = descriptor_at(kv_desc, ring * 2 * DqStepBytes);
#pragma unroll
                for (int ks = 0; ks < HeadSize / 16; ++ks)
                    tcgen05_mma_bf16(tmem_base + 64 * (j & 1), descriptor_at(q_desc, ks * 32),
                                     descriptor_at(k_desc, ks * 32), idesc_s, ks > 0);
                tcgen05_commit(s_full0 + 8 * (j & 1));
            };
            auto issue_dp = [&](int j) { // dP = dO V_j^T (the slot was awaited by issue_s(j))
                const uint64_t v_desc = descriptor_at(kv_desc, (j % DqRing) * 2 * DqStepBytes + DqStepBytes);
#pragma unroll
                for (int ks = 0; ks < HeadSize / 16; ++ks)
                    tcgen05_mma_bf16(tmem_dp, descriptor_at(do_desc, ks * 32), descriptor_at(v_desc, ks * 32), idesc_s,
                                     ks > 0);
                tcgen05_commit(dp_full);
            };
            if (ok)
                issue_s(0);
            if (ok)
                issue_dp(0);
            if (ok && blocks > 1)
                issue_s(1);
            for (int j = 0; j < blocks && ok; ++j) {
                ok = mbarrier_wait(ds_full0 + 8 * (j & 1), (j >> 1) & 1, abort_flag, p.counters, 304);
                if (!ok)
                    break;
                tcgen05_fence_after();
                const int ring = j % DqRing;
                const uint64_t k_desc = descriptor_at(k_mn_desc, ring * 2 * DqStepBytes);
#pragma unroll
                for (int ks = 0; ks < DqStep / 16; ++ks) // dQ += dS K_j: 16 keys = 8 packed columns at (ks / 2) 32 + (ks % 2) 8
                    tcgen05_mma_bf16_ts(tmem_dq, tmem_base + 64 * (j & 1) + (ks / 2) * 32 + (ks % 2) * 8,
                                        descriptor_at(k_desc, ks * 2048), idesc_dq, (j > 0 || ks > 0) ? 1u : 0u);
                tcgen05_commit(kv_empty0 + 8 * ring);
                if (j + 1 < blocks)
                    issue_dp(j + 1); // every compute warp has finished with dP of step j
                if (j + 2 < blocks)
                    issue_s(j + 2); // into the buffer whose dS the products above have just read
            }
            if (ok)
                tcgen05_commit(dq_done);
        }
    } else {
        // Two warps share each 32-lane quarter; warp `half` takes 32 of the step's 64 keys.
        const int quarter = warp % 4, half = (warp - 2) / 4;
        const int row = quarter * 32 + lane, position = tile * BlockM + row;
        const int warp_first = tile * BlockM + quarter * 32; // earliest query of this warp
        const uint32_t lane_base = tmem_base + (uint32_t(quarter * 32) << 16);
        const bool valid = position < p.context, ragged = warp_first + 31 >= p.context;
        const int64_t padded = int64_t(p.tiles) * BlockM, stat = bh * padded + position;
        const float lse2 = valid ? p.lse[(int64_t(b) * p.heads + h) * p.context + position] * 1.4426950408889634f : 0.f;
        // delta = rowsum(dO * O) for this thread's query: O from global memory, dO from the tile the TMA
        // warp loaded (row r of a 128-byte-swizzled tile keeps its 16-byte chunk c at position c ^ (r % 8)).
        float delta = 0.f;
        bool ok = true;
        {
            uint4 o[8];
            if (valid) {
                const uint4 *source = reinterpret_cast<const uint4 *>(p.out + (int64_t(row0) + position) * p.width + h * HeadSize);
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    o[c] = source[c];
            }
            ok = mbarrier_wait(qdo_full, 0, abort_flag, p.counters, 308);
            if (ok && valid) {
                const uint4 *tile_row = reinterpret_cast<const uint4 *>(aligned + TileBytes + row * 128);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 g = tile_row[c ^ (row & 7)];
                    const unsigned a4[4] = {o[c].x, o[c].y, o[c].z, o[c].w}, b4[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        delta += __uint_as_float(a4[i] << 16) * __uint_as_float(b4[i] << 16) +
                                 __uint_as_float(a4[i] & 0xffff0000u) * __uint_as_float(b4[i] & 0xffff0000u);
                }
            }
            if (ok && half == 0) { // rows past the end of the sequence hold zeros
                p.statistics[stat] = lse2;
                p.statistics[pairs * padded + stat] = delta;
            }
        }
        for (int j = 0; j < blocks && ok; ++j) {
            ok = mbarrier_wait(s_full0 + 8 * (j & 1), (j >> 1) & 1, abort_flag, p.counters, 305);
            if (!ok)
                break;
            tcgen05_fence_after();
            const uint32_t t = lane_base + 64 * (j & 1) + half * 32; // this warp's 32 score columns
            const int key0 = j * DqStep + half * 32;
            const bool none = key0 > warp_first + 31;                  // every key lies after every query of the warp
            const bool masked = key0 + 31 > warp_first || ragged;      // the causal diagonal crosses the warp's block
            uint32_t prob[32]; // scores, then probabilities, as FP32 bits
            if (!none) {
                tmem_load_32x32_async(t, prob);
                tmem_wait_load(prob);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float v = fast_exp2(fmaf(__uint_as_float(prob[i]), p.scale_log2, -lse2));
                    if (masked && (key0 + i > position || !valid))
                        v = 0.f;
                    prob[i] = __float_as_uint(v);
                }
            }
            ok = mbarrier_wait(dp_full, j & 1, abort_flag, p.counters, 309);
            if (!ok)
                break;
            tcgen05_fence_after();
#pragma unroll
            for (int c = 0; c < 2; ++c) { // 16 keys at a time
                uint32_t packed[8];
                if (none) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        packed[i] = 0u;
                } else {
                    uint32_t dp[16];
                    tmem_load_32x16_async(tmem_dp + (uint32_t(quarter * 32) << 16) + half * 32 + c * 16, dp);
                    tmem_wait_load(dp);
#pragma unroll
                    for (int i = 0; i < 16; i += 2)
                        packed[i / 2] = pack_bf16(__uint_as_float(prob[c * 16 + i]) * (__uint_as_float(dp[i]) - delta),
                                                  __uint_as_float(prob[c * 16 + i + 1]) * (__uint_as_float(dp[i + 1]) - delta));
                }
                tmem_store_32x8(t + c * 8, packed); // over this warp's own, already read, score columns
            }
            tmem_wait_store();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0)
                mbarrier_arrive(ds_full0 + 8 * (j & 1));
        }
        if (ok)
            ok = mbarrier_wait(dq_done, 0, abort_flag, p.counters, 306);
        if (__all_sync(0xffffffffu, ok)) { // through the Q tile, which no product reads any more: 2 KB per warp
            tcgen05_fence_after();
            bf16 *out = p.dqkv + (int64_t(row0) + warp_first) * 3 * p.width + h * HeadSize + half * 32;
            store_accumulator(tmem_dq + (uint32_t(quarter * 32) << 16) + half * 32, smem_q + (warp - 2) * 2048, out,
                              3 * int64_t(p.width), p.context - warp_first, p.scale, lane);
        }
    }
    __syncthreads();
    if (*abort_flag)
        __nanosleep(2000000);
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1)
        tmem_dealloc(tmem_base, BackwardTmemColumns);
}

// dk/dv kernel.  64 queries per step, everything transposed (thread = key row).  One buffer each for
// S^T = K Q^T and dP^T = V dO^T: the MMA thread issues, per step, dV += P^T dO (frees the score
// buffer), the next S^T, dK += dS^T Q (frees the dP buffer) and the next dP^T, so the next step's
// exponentials start after eight MMAs and its dP^T is ready when they end.  Sixteen MMAs per 64
// queries instead of 24 with 32-wide steps.
constexpr int DkvStep = 64, DkvStepBytes = DkvStep * HeadSize * 2, DkvRing = 4;
constexpr int DkvShared = 2 * TileBytes + DkvRing * 2 * DkvStepBytes + DkvRing * 128 * 4 + 1024 + 256; // K, V, ring of (Q, dO), statistics

__global__ void __launch_bounds__(BackwardThreads, 2)
flash_dkv_kernel(const __grid_constant__ CUtensorMap map_qkv128, const __grid_constant__ CUtensorMap map_qkv64,
                 const __grid_constant__ CUtensorMap map_do64, BackwardParams p) {
    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (smem_address(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - smem_address(raw_shared));
    // per ring slot: lse (in base 2) of the step's 64 queries, then their delta
    float *statistics = reinterpret_cast<float *>(aligned + 2 * TileBytes + DkvRing * 2 * DkvStepBytes);
    uint64_t *barriers = reinterpret_cast<uint64_t *>(aligned + 2 * TileBytes + DkvRing * 2 * DkvStepBytes + DkvRing * 128 * 4);
    const uint32_t kv_full = smem_address(barriers), qdo_full0 = kv_full + 8, qdo_empty0 = qdo_full0 + 8 * DkvRing,
                   s_full = qdo_empty0 + 8 * DkvRing, dp_full = s_full + 8, p_full = dp_full + 8, ds_full = p_full + 8,
                   acc_done = ds_full + 8; // 6 + 2 DkvRing = 14 barriers
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(barriers + 6 + 2 * DkvRing);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t smem_k = base, smem_v = base + TileBytes, smem_qdo = base + 2 * TileBytes;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int pairs = p.batch * p.heads;
    const int tile = int(blockIdx.x / pairs); // key tile; early tiles have the most query blocks
    const int bh = blockIdx.x % pairs, b = bh / p.heads, h = bh % p.heads;
    const int row0 = b * p.context;
    const int first_block = tile * (BlockN / DkvStep), query_blocks = (p.context + DkvStep - 1) / DkvStep;
    const int blocks = query_blocks - first_block; // query blocks first_block .. query_blocks-1

    grid_launch_dependents(); // the next kernel may set itself up while this one runs
    if (threadIdx.x == 0) {
        mbarrier_init(kv_full, 1);
        for (int s = 0; s < DkvRing; ++s) {
            mbarrier_init(qdo_full0 + 8 * s, 1);
            mbarrier_init(qdo_empty0 + 8 * s, 1);
        }
        mbarrier_init(s_full, 1);
        mbarrier_init(dp_full, 1);
        mbarrier_init(p_full, 8);
        mbarrier_init(ds_full, 8);
        mbarrier_init(acc_done, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_address(tmem_slot), BackwardTmemColumns);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // S^T at 0 (a half's packed P^T goes to the first 16 columns of its own 32), dP^T at 64 (dS^T likewise);
    // dV at 128, dK at 192
    const uint32_t tmem_dp = tmem_base + 64, tmem_dv = tmem_base + 128, tmem_dk = tmem_base + 192;

    if (warp == 0) {
        // One thread issues every load: the tiles by TMA and the step's 64 lse and delta values as two bulk
        // copies from the padded rows, so nothing passes through registers and no load latency sits between steps.
        if (lane == 0) {
            mbarrier_expect_tx(kv_full, 2 * TileBytes);
            tma_load_3d(smem_k, &map_qkv128, p.width + h * HeadSize, row0 + tile * BlockN, 0, kv_full);
            tma_load_3d(smem_v, &map_qkv128, 2 * p.width + h * HeadSize, row0 + tile * BlockN, 0, kv_full);
            const int64_t padded = int64_t(p.tiles) * BlockM;
            const float *lse2 = p.statistics + bh * padded, *delta = lse2 + pairs * padded;
            for (int i = 0; i < blocks; ++i) {
                const int ring = i % DkvRing, q0 = (first_block + i) * DkvStep;
                if (!mbarrier_wait(qdo_empty0 + 8 * ring, ((i / DkvRing) & 1) ^ 1, abort_flag, p.counters, 311))
                    break;
                const uint32_t bar = qdo_full0 + 8 * ring, dst = smem_qdo + ring * 2 * DkvStepBytes,
                               stats = smem_address(statistics + ring * 128);
                mbarrier_expect_tx(bar, 2 * DkvStepBytes + 2 * DkvStep * 4);
                tma_load_3d(dst, &map_qkv64, h * HeadSize, row0 + q0, 0, bar);
                tma_load_3d(dst + DkvStepBytes, &map_do64, h * HeadSize, row0 + q0, 0, bar);
                bulk_load(stats, lse2 + q0, DkvStep * 4, bar);
                bulk_load(stats + DkvStep * 4, delta + q0, DkvStep * 4, bar);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc_s = instruction_descriptor(BlockN, DkvStep, 0, 0);
            const uint32_t idesc_acc = instruction_descriptor(BlockN, HeadSize, 0, 1);
            // descriptors are built once; every MMA below only offsets them
            const uint64_t k_desc = smem_descriptor(smem_k, 16, 1024), v_desc = smem_descriptor(smem_v, 16, 1024),
                           qdo_desc = smem_descriptor(smem_qdo, 16, 1024),
                           qdo_mn_desc = smem_descriptor(smem_qdo, 8192, 1024);
            bool ok = mbarrier_wait(kv_full, 0, abort_flag, p.counters, 312);
            auto issue_s = [&](int i) { // S^T = K Q_i^T; the first use of ring slot i
                const int ring = i % DkvRing;
                ok = mbarrier_wait(qdo_full0 + 8 * ring, (i / DkvRing) & 1, abort_flag, p.counters, 313);
                if (!ok)
                    return;
                tcgen05_fence_after();
                const uint64_t q_desc = descriptor_at(qdo_desc, ring * 2 * DkvStepBytes);
#pragma unroll
                for (int ks = 0; ks < HeadSize / 16; ++ks)
                    tcgen05_mma_bf16(tmem_base, descriptor_at(k_desc, ks * 32), descriptor_at(q_desc, ks * 32), idesc_s,
                                     ks > 0);
                tcgen05_commit(s_full);
            };
            auto issue_dp = [&](int i) { // dP^T = V dO_i^T (the slot was awaited by issue_s(i))
                const uint64_t do_desc = descriptor_at(qdo_desc, (i % DkvRing) * 2 * DkvStepBytes + DkvStepBytes);
#pragma unroll
                for (int ks = 0; ks < HeadSize / 16; ++ks)
                    tcgen05_mma_bf16(tmem_dp, descriptor_at(v_desc, ks * 32), descriptor_at(do_desc, ks * 32), idesc_s,
                                     ks > 0);
                tcgen05_commit(dp_full);
            };
            if (ok)
                issue_s(0);
            if (ok)
                issue_dp(0);
            for (int i = 0; i < blocks && ok; ++i) {
                const int ring = i % DkvRing;
                const uint64_t q_mn = descriptor_at(qdo_mn_desc, ring * 2 * DkvStepBytes),
                               do_mn = descriptor_at(q_mn, DkvStepBytes);
                ok = mbarrier_wait(p_full, i & 1, abort_flag, p.counters, 314);
                if (!ok)
                    break;
                tcgen05_fence_after();
#pragma unroll
                for (int ks = 0; ks < DkvStep / 16; ++ks) // dV += P^T dO_i: 16 queries = 8 packed columns at (ks / 2) 32 + (ks % 2) 8
                    tcgen05_mma_bf16_ts(tmem_dv, tmem_base + (ks / 2) * 32 + (ks % 2) * 8, descriptor_at(do_mn, ks * 2048),
                                        idesc_acc, (i > 0 || ks > 0) ? 1u : 0u);
                if (i + 1 < blocks)
                    issue_s(i + 1); // into the buffer whose P^T the products above have just read
                if (!ok)
                    break;
                ok = mbarrier_wait(ds_full, i & 1, abort_flag, p.counters, 320);
                if (!ok)
                    break;
                tcgen05_fence_after();
#pragma unroll
                for (int ks = 0; ks < DkvStep / 16; ++ks) // dK += dS^T Q_i
                    tcgen05_mma_bf16_ts(tmem_dk, tmem_dp + (ks / 2) * 32 + (ks % 2) * 8, descriptor_at(q_mn, ks * 2048),
                                        idesc_acc, (i > 0 || ks > 0) ? 1u : 0u);
                tcgen05_commit(qdo_empty0 + 8 * ring);
                if (i + 1 < blocks)
                    issue_dp(i + 1); // after the products that read dS^T from the same columns
            }
            if (ok)
                tcgen05_commit(acc_done);
        }
    } else {
        // Two warps share each 32-lane quarter; warp `half` takes 32 of the step's 64 queries.
        const int quarter = warp % 4, half = (warp - 2) / 4;
        const int row = quarter * 32 + lane, key = tile * BlockN + row; // key position inside the sequence
        const int warp_first = tile * BlockN + quarter * 32;            // earliest key of this warp
        const uint32_t lanes = uint32_t(quarter * 32) << 16;
        const uint32_t t_s = tmem_base + lanes + half * 32, t_dp = tmem_dp + lanes + half * 32; // this warp's 32 columns
        bool ok = true;
        for (int i = 0; i < blocks; ++i) {
            const int ring = i % DkvRing;
            ok = mbarrier_wait(qdo_full0 + 8 * ring, (i / DkvRing) & 1, abort_flag, p.counters, 317) && // statistics
                 mbarrier_wait(s_full, i & 1, abort_flag, p.counters, 315);
            if (!ok)
                break;
            tcgen05_fence_after();
            const float *l2 = statistics + ring * 128 + half * 32, *dl = l2 + 64;
            const int qa = (first_block + i) * DkvStep + half * 32;         // first query of this warp's columns
            const bool none = qa + 31 < warp_first;                         // every query lies before every key of the warp
            const bool masked = qa < warp_first + 31 || qa + 32 > p.context; // causal diagonal or ragged end
            uint32_t prob[32]; // scores, then probabilities, as FP32 bits
            {
                uint32_t pp[16];
                if (none) {
#pragma unroll
                    for (int c = 0; c < 16; ++c)
                        pp[c] = 0u;
                } else {
                    tmem_load_32x32_async(t_s, prob);
                    tmem_wait_load(prob);
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        float v = fast_exp2(fmaf(__uint_as_float(prob[c]), p.scale_log2, -l2[c]));
                        if (masked && (qa + c < key || qa + c >= p.context))
                            v = 0.f;
                        prob[c] = __float_as_uint(v);
                    }
#pragma unroll
                    for (int c = 0; c < 32; c += 2)
                        pp[c / 2] = pack_bf16(__uint_as_float(prob[c]), __uint_as_float(prob[c + 1]));
                }
                tmem_store_32x16(t_s, pp); // over this warp's own, already read, score columns
                tmem_wait_store();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbarrier_arrive(p_full);
            }
            ok = mbarrier_wait(dp_full, i & 1, abort_flag, p.counters, 319);
            if (!ok)
                break;
            tcgen05_fence_after();
#pragma unroll
            for (int c = 0; c < 2; ++c) { // 16 queries at a time
                uint32_t pd[8];
                if (none) {
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        pd[e] = 0u;
                } else {
                    uint32_t dp[16];
                    tmem_load_32x16_async(t_dp + c * 16, dp);
                    tmem_wait_load(dp);
#pragma unroll
                    for (int e = 0; e < 16; e += 2)
                        pd[e / 2] = pack_bf16(
                            __uint_as_float(prob[c * 16 + e]) * (__uint_as_float(dp[e]) - dl[c * 16 + e]),
                            __uint_as_float(prob[c * 16 + e + 1]) * (__uint_as_float(dp[e + 1]) - dl[c * 16 + e + 1]));
                }
                tmem_store_32x8(t_dp + c * 8, pd); // over this warp's own, already read, columns
            }
            tmem_wait_store();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0)
                mbarrier_arrive(ds_full);
        }
        if (ok)
            ok = mbarrier_wait(acc_done, 0, abort_flag, p.counters, 316);
        if (__all_sync(0xffffffffu, ok)) { // through the K and V tiles, which no product reads any more: 2 KB per warp
            tcgen05_fence_after();
            const int first = tile * BlockN + quarter * 32; // this warp's first key
            bf16 *out = p.dqkv + (int64_t(row0) + first) * 3 * p.width + h * HeadSize + half * 32;
            const uint32_t staging = smem_k + (warp - 2) * 2048;
            store_accumulator(tmem_dk + lanes + half * 32, staging, out + p.width, 3 * int64_t(p.width), p.context - first,
                              p.scale, lane);
            store_accumulator(tmem_dv + lanes + half * 32, staging, out + 2 * p.width, 3 * int64_t(p.width), p.context - first,
                              1.f, lane);
        }
    }
    __syncthreads();
    if (*abort_flag)
        __nanosleep(2000000);
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1)
        tmem_dealloc(tmem_base, BackwardTmemColumns);
}

} // namespace

bool flash_attention_supported(int width, int heads) {
    return heads > 0 && width == heads * HeadSize;
}

void launch_flash_attention_forward(const void *qkv, void *out, float *lse, int batch, int context, int heads,
                                    StepCounters *counters, cudaStream_t s) {
    static bool configured[64] = {};
    int device = 0;
    CHECK_CUDA(cudaGetDevice(&device));
    if (device < 64 && !configured[device]) {
        CHECK_CUDA(cudaFuncSetAttribute(flash_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        ForwardShared));
        configured[device] = true;
    }
    const int width = heads * HeadSize;
    ForwardParams p{};
    p.out = static_cast<bf16 *>(out), p.lse = lse;
    p.batch = batch, p.context = context, p.heads = heads, p.width = width;
    p.tiles = (context + BlockM - 1) / BlockM;
    p.scale_log2 = 1.4426950408889634f / sqrtf(float(HeadSize));
    p.counters = counters;
    const uint64_t rows = uint64_t(batch) * context;
    CUtensorMap map_q = make_map_bf16(qkv, uint64_t(3) * width, rows, 1, uint64_t(3) * width, 0, HeadSize, BlockM);
    CUtensorMap map_kv = make_map_bf16(qkv, uint64_t(3) * width, rows, 1, uint64_t(3) * width, 0, HeadSize, KeyStep);
    flash_forward_kernel<<<batch * heads * p.tiles, ForwardThreads, ForwardShared, s>>>(map_q, map_kv, p);
    CHECK_CUDA(cudaGetLastError());
}

size_t flash_attention_backward_scratch_bytes(int batch, int context, int heads) {
    return size_t(2) * batch * heads * ((context + BlockM - 1) / BlockM) * BlockM * sizeof(float);
}

void launch_flash_attention_backward(const void *qkv, const void *out, const void *dout, const float *lse,
                                     float *scratch, void *dqkv, int batch, int context, int heads,
                                     StepCounters *counters, cudaStream_t s) {
    static bool configured[64] = {};
    int device = 0;
    CHECK_CUDA(cudaGetDevice(&device));
    if (device < 64 && !configured[device]) {
        CHECK_CUDA(cudaFuncSetAttribute(flash_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DqShared));
        CHECK_CUDA(cudaFuncSetAttribute(flash_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvShared));
        configured[device] = true;
    }
    const int width = heads * HeadSize;
    BackwardParams p{};
    p.out = static_cast<const bf16 *>(out), p.dqkv = static_cast<bf16 *>(dqkv), p.lse = lse, p.statistics = scratch;
    p.batch = batch, p.context = context, p.heads = heads, p.width = width;
    p.tiles = (context + BlockM - 1) / BlockM;
    p.scale = 1.f / sqrtf(float(HeadSize));
    p.scale_log2 = 1.4426950408889634f * p.scale;
    p.counters = counters;
    const uint64_t rows = uint64_t(batch) * context;
    CUtensorMap qkv128 = make_map_bf16(qkv, uint64_t(3) * width, rows, 1, uint64_t(3) * width, 0, HeadSize, 128);

    CUtensorMap do128 = make_map_bf16(dout, width, rows, 1, width, 0, HeadSize, 128);
    CUtensorMap do64 = make_map_bf16(dout, width, rows, 1, width, 0, HeadSize, DkvStep);
    const int grid = batch * heads * p.tiles;
    CUtensorMap qkv64 = make_map_bf16(qkv, uint64_t(3) * width, rows, 1, uint64_t(3) * width, 0, HeadSize, DqStep);
    flash_dq_kernel<<<grid, BackwardThreads, DqShared, s>>>(qkv128, qkv64, do128, p); // also writes delta
    flash_dkv_kernel<<<grid, BackwardThreads, DkvShared, s>>>(qkv128, qkv64, do64, p);
    CHECK_CUDA(cudaGetLastError());
}
