// Fused backward of causal softmax attention, head size 64, BF16: dQ, dK and dV from ONE pass over the
// score blocks, so every probability is exponentiated once (a dq kernel followed by a dk/dv kernel
// evaluates each twice and repeats the S = Q K^T and dP = dO V^T products).  Same role as the
// reference's attention_backward loops (cuda/attention.cuh:69-106), nothing of their structure.
//
// One CTA per 128 keys of one (batch, head), one CTA per SM (all 512 columns of tensor memory).
// It walks the query blocks at or after its keys, 64 queries per step, everything transposed
// (thread = key row):
//   S^T  = K Q_j^T, dP^T = V dO_j^T          -> tensor memory, two buffers each (steps alternate)
//   P^T  = exp(S^T / sqrt(d) - lse)          -> BF16, packed over S^T in tensor memory (A operand)
//   dS^T = P^T (dP^T - delta)                -> BF16, into a swizzled shared-memory tile
//   dV  += P^T dO_j,  dK += dS^T Q_j         -> tensor-memory accumulators for the whole walk
//   dQ   = dS K for two steps (128 queries)  -> its own tensor-memory buffer per pair of steps; the
//          dS^T tile is read once as the K-major A operand of dK and once as the MN-major A operand
//          of dQ: the same bytes serve both.
// Two groups of eight compute warps take alternate steps, so one group's exponentials overlap the
// other's dS arithmetic and the tensor pipe's work on the neighbouring steps; four more warps only
// move finished dQ blocks out of tensor memory.  Registers are redistributed (setmaxnreg): 88 per
// compute thread, 40 for the TMA and MMA warps, the launch count (80) for the drain warps.
//
// dQ of a 128-query block gets a contribution from every key tile at or before it.  The
// contributions are added in global memory in key-tile order: tile t waits (bounded) until a counter
// says tiles 0..t-1 have added theirs, reads the FP32 running sum, adds, writes back and advances the
// counter; the tile on the diagonal is the last one and writes the BF16 result instead.  The order is
// fixed, so the result is the same bits on every run.  A CTA only ever waits for a CTA with a lower
// block index, which the hardware has dispatched before it and which waits only for still lower
// ones, so the wait cannot deadlock; it is bounded all the same.
#include "device_utils.cuh"
#include "sm100.cuh"

using namespace sm100;

namespace {
constexpr int KeyTile = 128, HeadSize = 64, Step = 64, Ring = 4;
constexpr int TileBytes = KeyTile * HeadSize * 2; // 16 KB: K, V, or one step's dS^T tile [128 keys][64 queries]
constexpr int StepBytes = Step * HeadSize * 2;    // 8 KB: Q_j or dO_j
// Warps in groups of four (register budgets are set per group of four warps): 0 TMA + statistics, 1 MMA, 2-3 idle;
// 4-7 move finished dQ blocks out; 8-23 compute.
constexpr int FirstDrainWarp = 4, DrainWarps = 4, FirstComputeWarp = 8, ComputeWarps = 16;
constexpr int Threads = 32 * (FirstComputeWarp + ComputeWarps);
// The kernel starts with LaunchRegisters per thread (65 536 / 768 rounded down to a multiple of 8: what ptxas
// reports; the launcher checks it).  A group of warps can only grow into registers that other groups of the
// same CTA have released, and it waits for them without a limit, so the releases must cover the requests.
constexpr int LaunchRegisters = 80, ControlRegisters = 40, DrainRegisters = 80, ComputeRegisters = 88;
static_assert(32 * (FirstDrainWarp * (LaunchRegisters - ControlRegisters) + DrainWarps * (LaunchRegisters - DrainRegisters)) >=
                  32 * ComputeWarps * (ComputeRegisters - LaunchRegisters),
              "released registers must cover the requested ones");
constexpr int TmemColumns = 512;
// K, V | ring of (Q_j, dO_j) | dS^T tiles: 2 pairs of steps x 2 steps | statistics ring | dQ staging | barriers
constexpr int StagePitch = 68; // floats per staged dQ row (64 + 4): a lane's 16-byte pieces spread over all banks
constexpr int OffsetRing = 2 * TileBytes, OffsetDs = OffsetRing + Ring * 2 * StepBytes, OffsetStats = OffsetDs + 4 * TileBytes,
              OffsetStage = OffsetStats + Ring * 128 * 4, OffsetBarriers = OffsetStage + 128 * StagePitch * 4;
constexpr int SharedBytes = OffsetBarriers + 512 + 1024;

struct FusedParams {
    bf16 *dqkv;
    const float *lse, *delta;
    float *dq_sum;   // [tokens][width] FP32 running sums of dQ between key tiles
    int *dq_count;   // [batch * heads][tiles]: key tiles that have added their share to a 128-query block
    int batch, context, heads, width, tiles;
    float scale, scale_log2;
    StepCounters *counters;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ int load_acquire(const int *p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// 16 bytes global -> shared without passing through registers; completion by copy_async_wait().
__device__ __forceinline__ void copy_async16(uint32_t destination, const void *source) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(destination), "l"(source) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void add_relaxed(int *p, int v) {
    asm volatile("red.relaxed.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Register budget of the calling group of four warps from here on (all four execute it together).
template <int Registers> __device__ __forceinline__ void shrink_registers() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Registers));
}
template <int Registers> __device__ __forceinline__ void grow_registers() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Registers));
}
__device__ __forceinline__ void store_shared16(uint32_t address, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

#ifdef TG_TRACE
__device__ long long g_trace[3 * 8 * 64 * 8];
#define TRACE(role, j, k)                                                                                   \
    do {                                                                                                    \
        const int cta_ = blockIdx.x == 100 ? 0 : blockIdx.x == 900 ? 1 : blockIdx.x == 2500 ? 2 : -1;       \
        if (cta_ >= 0 && (j) < 64)                                                                          \
            g_trace[((cta_ * 8 + (role)) * 64 + (j)) * 8 + (k)] = clock64();                                \
    } while (0)
#else
#define TRACE(role, j, k)
#endif

__global__ void __launch_bounds__(Threads, 1)
flash_backward_kernel(const __grid_constant__ CUtensorMap map_qkv128, const __grid_constant__ CUtensorMap map_qkv64,
                      const __grid_constant__ CUtensorMap map_do64, FusedParams p) {
    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (smem_address(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - smem_address(raw_shared));
    float *statistics = reinterpret_cast<float *>(aligned + OffsetStats); // per ring slot: lse (base 2) of 64 queries, then delta
    uint64_t *barriers = reinterpret_cast<uint64_t *>(aligned + OffsetBarriers);
    const uint32_t kv_full = smem_address(barriers), qdo_full0 = kv_full + 8, qdo_empty0 = qdo_full0 + 8 * Ring,
                   s_full0 = qdo_empty0 + 8 * Ring, dp_full0 = s_full0 + 16, p_full0 = dp_full0 + 16,
                   ds_full0 = p_full0 + 16, ds_free0 = ds_full0 + 16, dq_full0 = ds_free0 + 16, dq_free0 = dq_full0 + 16,
                   acc_done = dq_free0 + 16, stored0 = acc_done + 8; // 1 + 2 Ring + 7 x 2 + 1 + 2 = 26 barriers
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(barriers + 26);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t smem_k = base, smem_v = base + TileBytes, smem_qdo = base + OffsetRing, smem_ds = base + OffsetDs;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int pairs = p.batch * p.heads;
    const int tile = int(blockIdx.x / pairs); // key tile; early tiles walk the most query blocks and are dispatched first
    const int bh = blockIdx.x % pairs, b = bh / p.heads, h = bh % p.heads;
    const int row0 = b * p.context;
    const int first_block = tile * (KeyTile / Step), query_blocks = (p.context + Step - 1) / Step;
    const int blocks = (query_blocks - first_block + 1) & ~1; // an odd count gets one empty step: dQ is formed per pair of steps
    const int supers = blocks / 2;

    grid_launch_dependents(); // the next kernel may set itself up while this one runs
    if (threadIdx.x == 0) {
        mbarrier_init(kv_full, 1);
        for (int s = 0; s < Ring; ++s) {
            mbarrier_init(qdo_full0 + 8 * s, 1);
            mbarrier_init(qdo_empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbarrier_init(s_full0 + 8 * s, 1);
            mbarrier_init(dp_full0 + 8 * s, 1);
            mbarrier_init(p_full0 + 8 * s, ComputeWarps / 2);
            mbarrier_init(ds_full0 + 8 * s, ComputeWarps / 2);
            mbarrier_init(ds_free0 + 8 * s, 1);
            mbarrier_init(dq_full0 + 8 * s, 1);
            mbarrier_init(dq_free0 + 8 * s, DrainWarps);
            mbarrier_init(stored0 + 8 * s, DrainWarps);
        }
        mbarrier_init(acc_done, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_address(tmem_slot), TmemColumns);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // S^T buffers at 0 and 64 (a warp's packed P^T goes to the first 16 columns of its own 32), dP^T at 128 and 192,
    // dV at 256, dK at 320, dQ buffers at 384 and 448
    const uint32_t tmem_st = tmem_base, tmem_dp = tmem_base + 128, tmem_dv = tmem_base + 256, tmem_dk = tmem_base + 320,
                   tmem_dq = tmem_base + 384;

    if (warp < FirstDrainWarp) {
      shrink_registers<ControlRegisters>(); // one instruction for the whole group of four warps
      if (warp == 0) {
        // The whole warp runs the producer loop: lane 0 issues the TMA loads, every lane fetches two
        // queries' statistics into the ring slot before lane 0's arrival releases them.
        if (lane == 0) {
            mbarrier_expect_tx(kv_full, 2 * TileBytes);
            tma_load_3d(smem_k, &map_qkv128, p.width + h * HeadSize, row0 + tile * KeyTile, 0, kv_full);
            tma_load_3d(smem_v, &map_qkv128, 2 * p.width + h * HeadSize, row0 + tile * KeyTile, 0, kv_full);
        }
        const float *lse = p.lse + (int64_t(b) * p.heads + h) * p.context;
        const float *delta = p.delta + (int64_t(b) * p.heads + h) * p.context;
        auto fetch = [&](int j, float (&values)[4]) { // lse (base 2) and delta of queries q0 + lane and q0 + 32 + lane
            const int q0 = (first_block + j) * Step;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const bool inside = j < blocks && q0 + u * 32 + lane < p.context;
                values[u] = inside ? lse[q0 + u * 32 + lane] * 1.4426950408889634f : 0.f;
                values[2 + u] = inside ? delta[q0 + u * 32 + lane] : 0.f;
            }
        };
        bool ok = true;
        auto step = [&](int j, const float (&values)[4]) {
            const int ring = j % Ring, q0 = (first_block + j) * Step;
            if (lane == 0) TRACE(0, j, 0);
            ok = mbarrier_wait(qdo_empty0 + 8 * ring, ((j / Ring) & 1) ^ 1, abort_flag, p.counters, 341);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                return;
            if (lane == 0) TRACE(0, j, 1);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                statistics[ring * 128 + u * 32 + lane] = values[u];
                statistics[ring * 128 + 64 + u * 32 + lane] = values[2 + u];
            }
            __syncwarp();
            if (lane == 0) {
                const uint32_t bar = qdo_full0 + 8 * ring, dst = smem_qdo + ring * 2 * StepBytes;
                mbarrier_expect_tx(bar, 2 * StepBytes);
                // rows past the end of the tensor arrive as zeros; rows of the next sequence are masked by the compute warps
                tma_load_3d(dst, &map_qkv64, h * HeadSize, row0 + q0, 0, bar);
                tma_load_3d(dst + StepBytes, &map_do64, h * HeadSize, row0 + q0, 0, bar);
            }
        };
        // Two register sets, refilled two steps ahead of their use: the loop never waits for a load it has
        // just issued (blocks is even).
        float even[4], odd[4];
        fetch(0, even);
        fetch(1, odd);
        for (int j = 0; j < blocks && ok; j += 2) {
            step(j, even);
            fetch(j + 2, even);
            if (ok)
                step(j + 1, odd);
            fetch(j + 3, odd);
        }
      } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc_s = instruction_descriptor(KeyTile, Step, 0, 0);      // K-major x K-major
            const uint32_t idesc_acc = instruction_descriptor(KeyTile, HeadSize, 0, 1); // (TMEM or K-major A) x MN-major B
            const uint32_t idesc_dq = instruction_descriptor(128, HeadSize, 1, 1);      // MN-major A x MN-major B
            const uint64_t k_desc = smem_descriptor(smem_k, 16, 1024), v_desc = smem_descriptor(smem_v, 16, 1024),
                           k_mn_desc = smem_descriptor(smem_k, TileBytes, 1024),
                           qdo_desc = smem_descriptor(smem_qdo, 16, 1024),
                           qdo_mn_desc = smem_descriptor(smem_qdo, StepBytes, 1024),
                           ds_desc = smem_descriptor(smem_ds, 16, 1024),          // one step's tile as K-major A of dK
                           ds_mn_desc = smem_descriptor(smem_ds, TileBytes, 1024); // two steps' tiles as MN-major A of dQ
            bool ok = mbarrier_wait(kv_full, 0, abort_flag, p.counters, 342);
            auto issue_s = [&](int j) { // S^T = K Q_j^T; the first use of ring slot j
                const int ring = j % Ring;
                ok = mbarrier_wait(qdo_full0 + 8 * ring, (j / Ring) & 1, abort_flag, p.counters, 343);
                if (!ok)
                    return;
                tcgen05_fence_after();
                const uint64_t q_desc = descriptor_at(qdo_desc, ring * 2 * StepBytes);
#pragma unroll
                for (int ks = 0; ks < HeadSize / 16; ++ks)
                    tcgen05_mma_bf16(tmem_st + 64 * (j & 1), descriptor_at(k_desc, ks * 32), descriptor_at(q_desc, ks * 32),
                                     idesc_s, ks > 0);
                tcgen05_commit(s_full0 + 8 * (j & 1));
            };
            auto issue_dp = [&](int j) { // dP^T = V dO_j^T (the slot was awaited by issue_s(j))
                const uint64_t do_desc = descriptor_at(qdo_desc, (j % Ring) * 2 * StepBytes + StepBytes);
#pragma unroll
                for (int ks = 0; ks < HeadSize / 16; ++ks)
                    tcgen05_mma_bf16(tmem_dp + 64 * (j & 1), descriptor_at(v_desc, ks * 32), descriptor_at(do_desc, ks * 32),
                                     idesc_s, ks > 0);
                tcgen05_commit(dp_full0 + 8 * (j & 1));
            };
            for (int j = 0; j < 2 && j < blocks && ok; ++j) {
                issue_s(j);
                if (ok)
                    issue_dp(j);
            }
            for (int j = 0; j < blocks && ok; ++j) {
                const int ring = j % Ring, buffer = j & 1, super = j >> 1;
                const uint64_t q_mn = descriptor_at(qdo_mn_desc, ring * 2 * StepBytes), do_mn = descriptor_at(q_mn, StepBytes);
                TRACE(1, j, 0);
                ok = mbarrier_wait(p_full0 + 8 * buffer, (j >> 1) & 1, abort_flag, p.counters, 344);
                if (!ok)
                    break;
                tcgen05_fence_after();
                TRACE(1, j, 1);
#pragma unroll
                for (int ks = 0; ks < Step / 16; ++ks) // dV += P^T dO_j: 16 queries = 8 packed columns at (ks / 2) 32 + (ks % 2) 8
                    tcgen05_mma_bf16_ts(tmem_dv, tmem_st + 64 * buffer + (ks / 2) * 32 + (ks % 2) * 8,
                                        descriptor_at(do_mn, ks * 2048), idesc_acc, (j > 0 || ks > 0) ? 1u : 0u);
                if (j + 2 < blocks)
                    issue_s(j + 2); // into the buffer whose P^T the products above have just read
                if (!ok)
                    break;
                TRACE(1, j, 2);
                ok = mbarrier_wait(ds_full0 + 8 * buffer, (j >> 1) & 1, abort_flag, p.counters, 345);
                if (!ok)
                    break;
                tcgen05_fence_after();
                TRACE(1, j, 3);
                const uint64_t ds_tile = descriptor_at(ds_desc, ((super & 1) * 2 + buffer) * TileBytes);
#pragma unroll
                for (int ks = 0; ks < Step / 16; ++ks) // dK += dS^T Q_j
                    tcgen05_mma_bf16(tmem_dk, descriptor_at(ds_tile, ks * 32), descriptor_at(q_mn, ks * 2048), idesc_acc,
                                     (j > 0 || ks > 0) ? 1u : 0u);
                tcgen05_commit(qdo_empty0 + 8 * ring); // Q_j and dO_j are no longer read
                if (j + 2 < blocks)
                    issue_dp(j + 2); // the compute warps have read dP^T of step j (they wrote its dS^T)
                TRACE(1, j, 4);
                if (buffer == 1) {
                    // dQ of the pair of steps: (dS^T)^T [128 queries x 128 keys] K [128 keys x 64]
                    if (super >= 2) {
                        ok = mbarrier_wait(dq_free0 + 8 * (super & 1), ((super >> 1) & 1) ^ 1, abort_flag, p.counters, 346);
                        if (!ok)
                            break;
                        tcgen05_fence_after();
                    }
                    const uint64_t ds_pair = descriptor_at(ds_mn_desc, (super & 1) * 2 * TileBytes);
#pragma unroll
                    for (int ks = 0; ks < KeyTile / 16; ++ks)
                        tcgen05_mma_bf16(tmem_dq + 64 * (super & 1), descriptor_at(ds_pair, ks * 2048),
                                         descriptor_at(k_mn_desc, ks * 2048), idesc_dq, ks > 0);
                    tcgen05_commit(dq_full0 + 8 * (super & 1));
                    tcgen05_commit(ds_free0 + 8 * (super & 1)); // both dS^T tiles of the pair may be overwritten
                    TRACE(1, j, 5);
                }
            }
            if (ok)
                tcgen05_commit(acc_done);
        }
      } else if (warp == 2) {
        // Advances the counter of every block the drain warps have added to: their stores are ordered before
        // this warp's device-wide fence by the barrier they arrive on, so the slow fence is off their path.
        // (Warp 3 only completes the group of four.)
        if (lane == 0) {
            for (int super = 0; super < supers; ++super) {
                if (!mbarrier_wait(stored0 + 8 * (super & 1), (super >> 1) & 1, abort_flag, p.counters, 354))
                    break;
                if (super == 0)
                    continue; // the diagonal block is final: nobody waits for it
                __threadfence();
                add_relaxed(p.dq_count + int64_t(bh) * p.tiles + tile + super, DrainWarps);
            }
        }
      }
    } else if (warp < FirstComputeWarp) {
        // Four drain warps, one per 32-lane quarter of tensor memory, add this key tile's dQ of every pair of
        // steps to the running sum in global memory, after the tiles before it; the diagonal tile comes last
        // and writes the BF16 result.  They run beside the compute warps, so the global round trips (counter,
        // running sum, fence) are off the critical path: the running sums are requested before the block is
        // complete in tensor memory, and the counter of a block is advanced after the next block's requests.
        // A block leaves tensor memory with one query row per lane; it is turned through shared memory so that
        // every global access of a warp covers two whole 256-byte rows (lane = row parity x 16-byte piece)
        // instead of 32 different lines: scattered accesses were measured to stall the whole SM's
        // load/store path, shared-memory traffic of the compute warps included.
        const int quarter = warp % 4;
        const uint32_t lanes = uint32_t(quarter * 32) << 16;
        float *stage = reinterpret_cast<float *>(aligned + OffsetStage) + quarter * 32 * StagePitch; // this warp's 32 rows
        const int piece = lane % 16, parity = lane / 16;
        const bool first = tile == 0;
        const int row_pitch = p.width / 2; // float4 elements between rows 2 k + parity and 2 (k + 1) + parity
        bool ok = true;
        // Running sums of block `super`, rows 2 k + parity, as float4 pointers; and their copy into the staging
        // rows, asynchronous (no registers, no wait): issued a whole block ahead of its use.
        auto sums_of = [&](int super) {
            return reinterpret_cast<float4 *>(p.dq_sum + (int64_t(row0) + (tile + super) * 128 + quarter * 32 + parity) * p.width +
                                              h * HeadSize) + piece;
        };
        auto wait_for_tiles_before = [&](int super, int seen) { // `seen`: lane 0's earlier look; bounded; false when it gave up
            seen = __shfl_sync(0xffffffffu, seen, 0);
            if (seen >= DrainWarps * tile)
                return true;
            if (lane == 0) {
                const int *count = p.dq_count + int64_t(bh) * p.tiles + tile + super;
                const unsigned long long start = global_timer();
                while ((seen = load_acquire(count)) < DrainWarps * tile) {
                    if (*abort_flag)
                        break;
                    if (global_timer() - start > WaitLimitNs) {
                        *abort_flag = 1;
                        if (p.counters)
                            atomicCAS(&p.counters->error, 0, 348);
                        break;
                    }
                    __nanosleep(200);
                }
            }
            return __shfl_sync(0xffffffffu, seen, 0) >= DrainWarps * tile;
        };
        auto fetch_sums = [&](int super) {
            const float4 *source = sums_of(super);
            const int position0 = (tile + super) * 128 + quarter * 32;
#pragma unroll
            for (int k = 0; k < 16; ++k)
                if (position0 + 2 * k + parity < p.context)
                    copy_async16(smem_address(stage + (2 * k + parity) * StagePitch + piece * 4), source + k * row_pitch);
            copy_async_commit();
        };
        if (!first) {
            ok = wait_for_tiles_before(0, 0);
            if (ok)
                fetch_sums(0);
        }
        for (int super = 0; super < supers && ok; ++super) {
            const int sb = super & 1;
            const int position0 = (tile + super) * 128 + quarter * 32; // query of this warp's first row
            const bool last = super == 0, more = super + 1 < supers;
            int seen_next = 0; // the next block's counter, read now, looked at when this block is done
            if (!first && more) {
                if (lane == 0)
                    seen_next = load_acquire(p.dq_count + int64_t(bh) * p.tiles + tile + super + 1);
                const float4 *next = sums_of(super + 1);
#pragma unroll
                for (int k = 0; k < 16; ++k) // towards L2, for the copy issued at the end of this block
                    if (position0 + 128 + 2 * k + parity < p.context)
                        prefetch_l2(next + k * row_pitch);
            }
            if (lane == 0 && warp == FirstDrainWarp) TRACE(4, super, 0);
            ok = mbarrier_wait(dq_full0 + 8 * sb, (super >> 1) & 1, abort_flag, p.counters, 347);
            if (!ok)
                break;
            tcgen05_fence_after();
            copy_async_wait();
            __syncwarp(); // the running sums of this block are in the staging rows, whichever lane copied them
            if (lane == 0 && warp == FirstDrainWarp) TRACE(4, super, 1);
#pragma unroll 1
            for (int part = 0; part < 4; ++part) { // 16 columns at a time: tensor memory (+ running sum) -> staging, lane = row
                uint32_t raw[16];
                tmem_load_32x16_async(tmem_dq + 64 * sb + lanes + part * 16, raw);
                tmem_wait_load(raw);
                float4 *cell = reinterpret_cast<float4 *>(stage + lane * StagePitch + part * 16);
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float4 v = make_float4(__uint_as_float(raw[4 * g]), __uint_as_float(raw[4 * g + 1]),
                                           __uint_as_float(raw[4 * g + 2]), __uint_as_float(raw[4 * g + 3]));
                    if (!first) {
                        const float4 o = cell[g];
                        v.x += o.x, v.y += o.y, v.z += o.z, v.w += o.w;
                    }
                    cell[g] = v;
                }
            }
            tcgen05_fence_before();
            __syncwarp(); // the block has left tensor memory and its new sums are complete in the staging rows
            if (lane == 0)
                mbarrier_arrive(dq_free0 + 8 * sb);
            if (lane == 0 && warp == FirstDrainWarp) TRACE(4, super, 2);
            float4 *target = sums_of(super);
#pragma unroll
            for (int k = 0; k < 16; ++k) { // out in whole 256-byte rows: lane = row parity x 16-byte piece
                const int r = 2 * k + parity, position = position0 + r;
                if (position >= p.context)
                    continue;
                const float4 v = *reinterpret_cast<const float4 *>(stage + r * StagePitch + piece * 4);
                if (last) {
                    bf16 *out = p.dqkv + (int64_t(row0) + position) * 3 * p.width + h * HeadSize + piece * 4;
                    *reinterpret_cast<uint2 *>(out) =
                        make_uint2(pack_bf16(v.x * p.scale, v.y * p.scale), pack_bf16(v.z * p.scale, v.w * p.scale));
                } else {
                    __stcg(target + k * row_pitch, v);
                }
            }
            __syncwarp(); // every lane has read the staging rows (and issued its stores) before lane 0 goes on
            if (lane == 0)
                mbarrier_arrive(stored0 + 8 * sb); // warp 2 makes the sums visible and advances the counter
            if (lane == 0 && warp == FirstDrainWarp) TRACE(4, super, 3);
            if (!first && more) {
                ok = wait_for_tiles_before(super + 1, seen_next);
                if (ok)
                    fetch_sums(super + 1);
            }
        }
    } else {
        grow_registers<ComputeRegisters>();
        // Sixteen compute warps in two groups; group g takes the steps j = g, g + 2, ...  Inside a group two
        // warps share each 32-lane quarter of tensor memory; warp `half` takes 32 of the step's 64 queries.
        const int group = (warp - FirstComputeWarp) / 8, quarter = warp % 4, half = ((warp - FirstComputeWarp) / 4) % 2;
        const int row = quarter * 32 + lane, key = tile * KeyTile + row; // key position inside the sequence
        const int warp_first = tile * KeyTile + quarter * 32;            // earliest key of this warp
        const uint32_t lanes = uint32_t(quarter * 32) << 16;
        const uint32_t t_s = tmem_st + 64 * group + lanes + half * 32, t_dp = tmem_dp + 64 * group + lanes + half * 32;
        bool ok = true;

        for (int j = group; j < blocks && ok; j += 2) {
            const int ring = j % Ring, super = j >> 1, use = j >> 1;
            if (lane == 0 && (warp == FirstComputeWarp || warp == FirstComputeWarp + 8)) TRACE(2 + group, j, 0);
            ok = mbarrier_wait(qdo_full0 + 8 * ring, (j / Ring) & 1, abort_flag, p.counters, 349) && // statistics
                 mbarrier_wait(s_full0 + 8 * group, use & 1, abort_flag, p.counters, 350);
            if (!ok)
                break;
            tcgen05_fence_after();
            if (lane == 0 && (warp == FirstComputeWarp || warp == FirstComputeWarp + 8)) TRACE(2 + group, j, 1);
            const float *l2 = statistics + ring * 128 + half * 32, *dl = l2 + 64;
            const int qa = (first_block + j) * Step + half * 32;             // first query of this warp's columns
            const bool none = qa + 31 < warp_first || qa >= p.context;       // every query lies before every key of the warp, or past the end
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
                    mbarrier_arrive(p_full0 + 8 * group);
            }
            if (lane == 0 && (warp == FirstComputeWarp || warp == FirstComputeWarp + 8)) TRACE(2 + group, j, 2);
            ok = mbarrier_wait(dp_full0 + 8 * group, use & 1, abort_flag, p.counters, 351);
            if (ok && super >= 2) // the dS^T tiles of this pair of steps were last read by the products of pair super - 2
                ok = mbarrier_wait(ds_free0 + 8 * (super & 1), ((super >> 1) & 1) ^ 1, abort_flag, p.counters, 352);
            if (!ok)
                break;
            tcgen05_fence_after();
            if (lane == 0 && (warp == FirstComputeWarp || warp == FirstComputeWarp + 8)) TRACE(2 + group, j, 3);
            // dS^T of this warp's 32 queries: four 16-byte chunks of the key's 128-byte row (128-byte swizzle)
            const uint32_t ds_row = smem_ds + ((super & 1) * 2 + group) * TileBytes + row * 128;
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
                const int chunk = half * 4 + c * 2;
                store_shared16(ds_row + (((chunk) ^ (row & 7)) << 4), pd[0], pd[1], pd[2], pd[3]);
                store_shared16(ds_row + (((chunk + 1) ^ (row & 7)) << 4), pd[4], pd[5], pd[6], pd[7]);
            }
            fence_async_proxy(); // the tensor core reads the tile through the asynchronous proxy
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0)
                mbarrier_arrive(ds_full0 + 8 * group);
            if (lane == 0 && (warp == FirstComputeWarp || warp == FirstComputeWarp + 8)) TRACE(2 + group, j, 4);
        }
        if (ok)
            ok = mbarrier_wait(acc_done, 0, abort_flag, p.counters, 353);
        if (ok) {
            tcgen05_fence_after();
            // group 0 stores dK, group 1 dV: thread = key row, 32 columns
            bf16 *out = p.dqkv + (int64_t(row0) + key) * 3 * p.width + h * HeadSize + half * 32;
            uint32_t a[32];
            tmem_load_32x32_async((group == 0 ? tmem_dk : tmem_dv) + lanes + half * 32, a);
            tmem_wait_load(a);
            if (key < p.context) {
                const float factor = group == 0 ? p.scale : 1.f;
                bf16 *target = out + (group == 0 ? p.width : 2 * p.width);
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        v[i] = __uint_as_float(a[g * 8 + i]) * factor;
                    store8(target + g * 8, v);
                }
            }
        }
    }
    __syncthreads();
    if (*abort_flag)
        __nanosleep(2000000);
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1)
        tmem_dealloc(tmem_base, TmemColumns);
}

// delta[b, h, t] = sum_d dO[t, h, d] * O[t, h, d]: eight threads per (token, head), 8 elements each.
__global__ void __launch_bounds__(256) attention_delta_kernel(const bf16 *__restrict__ out, const bf16 *__restrict__ dout,
                                                              float *__restrict__ delta, int64_t vectors, int context,
                                                              int heads) {
    const int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    float sum = 0.f;
    if (i < vectors) {
        float a[8], b[8];
        load8(out + i * 8, a);
        load8(dout + i * 8, b);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            sum += a[j] * b[j];
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    if (i < vectors && (i & 7) == 0) {
        const int64_t pair = i >> 3, token = pair / heads; // (token, head)
        const int head = int(pair % heads);
        delta[(token / context * heads + head) * context + token % context] = sum;
    }
}
} // namespace

#ifdef TG_TRACE
extern "C" int tg_debug_trace(long long *out, int count) {
    return int(cudaMemcpyFromSymbol(out, g_trace, size_t(count) * sizeof(long long)));
}
#endif

size_t flash_backward_scratch_bytes(int batch, int context, int heads) {
    const size_t tiles = size_t(context + KeyTile - 1) / KeyTile;
    return size_t(batch) * context * heads * HeadSize * sizeof(float) + size_t(batch) * heads * tiles * sizeof(int);
}

void launch_flash_attention_backward_fused(const void *qkv, const void *out, const void *dout, const float *lse,
                                           float *delta, void *dqkv, void *scratch, int batch, int context, int heads,
                                           StepCounters *counters, cudaStream_t s) {
    static bool configured[64] = {};
    int device = 0;
    CHECK_CUDA(cudaGetDevice(&device));
    if (device < 64 && !configured[device]) {
        cudaFuncAttributes attributes{};
        CHECK_CUDA(cudaFuncGetAttributes(&attributes, flash_backward_kernel));
        if (attributes.numRegs != LaunchRegisters) // the register hand-over between warp groups is sized for this count
            throw std::runtime_error("attention backward was compiled with " + std::to_string(attributes.numRegs) +
                                     " registers per thread, its register plan needs " + std::to_string(LaunchRegisters));
        CHECK_CUDA(cudaFuncSetAttribute(flash_backward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SharedBytes));
        configured[device] = true;
    }
    const int width = heads * HeadSize;
    FusedParams p{};
    p.dqkv = static_cast<bf16 *>(dqkv), p.lse = lse, p.delta = delta;
    p.batch = batch, p.context = context, p.heads = heads, p.width = width;
    p.tiles = (context + KeyTile - 1) / KeyTile;
    p.dq_sum = static_cast<float *>(scratch);
    p.dq_count = reinterpret_cast<int *>(p.dq_sum + size_t(batch) * context * width);
    p.scale = 1.f / sqrtf(float(HeadSize));
    p.scale_log2 = 1.4426950408889634f * p.scale;
    p.counters = counters;
    const uint64_t rows = uint64_t(batch) * context;
    const int64_t vectors = int64_t(rows) * width / 8;
    attention_delta_kernel<<<unsigned((vectors + 255) / 256), 256, 0, s>>>(
        static_cast<const bf16 *>(out), static_cast<const bf16 *>(dout), delta, vectors, context, heads);
    CHECK_CUDA(cudaMemsetAsync(p.dq_count, 0, size_t(batch) * heads * p.tiles * sizeof(int), s));
    CUtensorMap qkv128 = make_map_bf16(qkv, uint64_t(3) * width, rows, 1, uint64_t(3) * width, 0, HeadSize, 128);
    CUtensorMap qkv64 = make_map_bf16(qkv, uint64_t(3) * width, rows, 1, uint64_t(3) * width, 0, HeadSize, Step);
    CUtensorMap do64 = make_map_bf16(dout, width, rows, 1, width, 0, HeadSize, Step);
    flash_backward_kernel<<<batch * heads * p.tiles, Threads, SharedBytes, s>>>(qkv128, qkv64, do64, p);
    CHECK_CUDA(cudaGetLastError());
}
