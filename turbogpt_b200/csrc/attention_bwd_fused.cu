// Single-pass backward of causal softmax attention, head size 64, BF16: dQ, dK and dV from ONE pass over
// the score blocks, so every probability is exponentiated once (a dq kernel followed by a dk/dv kernel
// evaluates each twice and repeats the S = Q K^T and dP = dO V^T products).  Same role as the
// reference's attention_backward loops (cuda/attention.cuh:69-106), nothing of their structure.
// The engine runs the two-kernel form (attention_tc.cu): measured on B200, this kernel takes 351 us
// against 347 us at 32 x 12 x 1024, 1048 against 928 at 8 x 12 x 4096, 220 against 262 at 64 x 12 x 512
// (both with their statistics kernels).  It is reachable through tg_ex_attention_backward for comparison.
// Where the time goes: tensor memory (512 columns) only leaves room for 64-query steps, whose
// 128 x 64 x 16 products re-read their 4 KB A operand from shared memory every instruction, so a step
// moves about 150 KB through shared memory (1 200 clocks at 128 bytes per clock) for 640 clocks of tensor
// work; a step takes 2 000 clocks; and between two key tiles about 7 000 clocks pass (the last products,
// the dK/dV epilogue, and the first scores and probabilities of the next tile).
//
// One persistent CTA per SM (all 512 columns of tensor memory) takes key tiles of 128 keys of one
// (batch, head) from a fixed list, long tiles first; barriers, tensor memory and the operand ring run on
// from one tile to the next, so a tile's loads and first products overlap the previous tile's last dQ
// blocks leaving.  For a tile it walks the query blocks at or after its keys, 64 queries per step, everything transposed
// (thread = key row):
//   S^T  = K Q_j^T, dP^T = V dO_j^T          -> tensor memory, two buffers each (steps alternate)
//   P^T  = exp(S^T / sqrt(d) - lse)          -> BF16, packed over S^T in tensor memory (A operand)
//   dS^T = P^T (dP^T - delta)                -> BF16, into a swizzled shared-memory tile
//   dV  += P^T dO_j,  dK += dS^T Q_j         -> tensor-memory accumulators for the whole walk
//   dQ   = dS K for two steps (128 queries)  -> its own tensor-memory buffer per pair of steps; the
//          dS^T tile is read once as the K-major A operand of dK and once as the MN-major A operand
//          of dQ: the same bytes serve both.
// One thread issues every load (tiles by TMA, the 64 queries' lse and delta by bulk copies from rows a
// small kernel has prepared), so no load latency sits between two steps.  Two groups of eight compute
// warps take alternate steps, so one group's exponentials overlap the other's dS arithmetic and the
// tensor pipe's work on the neighbouring steps; four more warps only move finished dQ blocks out of
// tensor memory.  Registers are redistributed (setmaxnreg): 88 per compute thread, 48 for the TMA and
// MMA warps, the launch count (80) for the drain warps.
//
// dQ of a 128-query block gets a contribution from every key tile at or before it.  The
// contributions are added in global memory in key-tile order: tile t waits (bounded) until a counter
// says tiles 0..t-1 have added theirs, then hands its block to the copy engine as bulk FP32
// reductions onto the running sum (tile 0 stores), and advances the counter when they have completed;
// the tile on the diagonal is the last one, adds the running sum itself and writes the BF16 result.
// The order is fixed, so the result is the same bits on every run.  A tile only ever waits for a tile
// earlier in the list; every CTA takes its tiles in list order, so the earliest unfinished tile never
// waits for an unfinished one and the waits cannot deadlock while all CTAs are resident; they are bounded
// all the same.
#include "device_utils.cuh"
#include "sm100.cuh"

using namespace sm100;

namespace {
constexpr int KeyTile = 128, HeadSize = 64, Step = 64, Ring = 4;
constexpr int TileBytes = KeyTile * HeadSize * 2; // 16 KB: K, V, or one step's dS^T tile [128 keys][64 queries]
constexpr int StepBytes = Step * HeadSize * 2;    // 8 KB: Q_j or dO_j
// Warps in groups of four (register budgets are set per group of four warps): 0 loads, 1 MMA, 2-3 idle;
// 4-7 move finished dQ blocks out; 8-23 compute.
constexpr int FirstDrainWarp = 4, DrainWarps = 4, FirstComputeWarp = 8, ComputeWarps = 16;
constexpr int Threads = 32 * (FirstComputeWarp + ComputeWarps);
// The kernel starts with LaunchRegisters per thread (65 536 / 768 rounded down to a multiple of 8: what ptxas
// reports; the launcher checks it).  A group of warps can only grow into registers that other groups of the
// same CTA have released, and it waits for them without a limit, so the releases must cover the requests.
constexpr int LaunchRegisters = 80, ControlRegisters = 48, DrainRegisters = 80, ComputeRegisters = 88;
static_assert(32 * (FirstDrainWarp * (LaunchRegisters - ControlRegisters) + DrainWarps * (LaunchRegisters - DrainRegisters)) >=
                  32 * ComputeWarps * (ComputeRegisters - LaunchRegisters),
              "released registers must cover the requested ones");
constexpr int TmemColumns = 512;
// K, V | ring of (Q_j, dO_j) | dS^T tiles: 2 pairs of steps x 2 steps | statistics ring | dQ staging | barriers
constexpr int StagePitch = HeadSize; // floats per staged dQ row; the 16-byte pieces of row r sit at piece ^ (r & 7)
constexpr int OffsetRing = 2 * TileBytes, OffsetDs = OffsetRing + Ring * 2 * StepBytes, OffsetStats = OffsetDs + 4 * TileBytes,
              OffsetStage = OffsetStats + Ring * 128 * 4, OffsetBarriers = OffsetStage + 128 * StagePitch * 4;
constexpr int SharedBytes = OffsetBarriers + 512 + 1024;

struct FusedParams {
    bf16 *dqkv;
    const float *statistics; // [2][batch * heads][tiles * 128]: lse in base 2, then delta (padded rows)
    float *dq_sum;   // [batch * heads][tiles * 128 queries][64] FP32 running sums of dQ between key tiles, rows in staging order
    int *dq_count;   // [batch * heads][tiles]: key tiles that have added their share to a 128-query block
    int batch, context, heads, width, tiles;
    int items;       // work items: tiles x batch x heads
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
// Adds to a counter; everything the calling thread has observed as done is visible to whoever acquires the new value.
__device__ __forceinline__ void add_release(int *p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bulk operations of the copy engine on one contiguous piece of shared memory (16-byte aligned, a multiple of
// 16 bytes): a store to global memory, and an FP32 add onto global memory performed in L2.  bulk_wait() returns
// when all of the calling thread's committed operations are complete.
__device__ __forceinline__ void bulk_store(void *global, uint32_t shared, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(global), "r"(shared), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_add(float *global, uint32_t shared, uint32_t bytes) {
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(global), "r"(shared), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns when at most `Pending` of the calling thread's most recent groups are still incomplete ...
template <int Pending> __device__ __forceinline__ void bulk_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(Pending) : "memory");
}
// ... and when all of them have at least read their shared memory.
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// Register budget of the calling group of four warps from here on (all four execute it together).
template <int Registers> __device__ __forceinline__ void shrink_registers() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Registers));
}
template <int Registers> __device__ __forceinline__ void grow_registers() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Registers));
}



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
                   acc_done = dq_free0 + 16, acc_free = acc_done + 8, kv_free = acc_free + 8; // 1 + 2 Ring + 7 x 2 + 3 barriers
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(barriers + 2 * Ring + 18);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t smem_k = base, smem_v = base + TileBytes, smem_qdo = base + OffsetRing, smem_ds = base + OffsetDs;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int pairs = p.batch * p.heads;
    const int query_blocks = (p.context + Step - 1) / Step;
    // The CTA walks the work items blockIdx.x, blockIdx.x + gridDim.x, ...  Item w is key tile w / pairs of
    // (batch, head) w % pairs: early tiles walk the most query blocks and come first, and every CTA takes its
    // items in ascending order, so the item a dQ block waits for (w - pairs) is never behind the waiting one in
    // any CTA's list.  Barrier phases run on across items: `base` is the number of steps before the item.
    struct Item {
        int tile, bh, h, row0, first_block, blocks, supers;
    };
    auto item_of = [&](int w) {
        Item it;
        it.tile = w / pairs, it.bh = w % pairs, it.h = it.bh % p.heads, it.row0 = it.bh / p.heads * p.context;
        it.first_block = it.tile * (KeyTile / Step);
        it.blocks = (query_blocks - it.first_block + 1) & ~1; // an odd count gets one empty step: dQ is formed per pair of steps
        it.supers = it.blocks / 2;
        return it;
    };

    grid_launch_dependents(); // the next kernel may set itself up while this one runs
    if (threadIdx.x == 32) {
        prefetch_map(&map_qkv128);
        prefetch_map(&map_qkv64);
        prefetch_map(&map_do64);
    }
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
        }
        mbarrier_init(acc_done, 1);
        mbarrier_init(acc_free, ComputeWarps);
        mbarrier_init(kv_free, 1);
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
        // The producer: one thread issues every load, tiles and statistics alike, so nothing passes through
        // its registers and no load latency sits between two steps.
        if (lane == 0) {
            const int64_t padded = int64_t(p.tiles) * KeyTile;
            bool ok = true;
            for (int w = blockIdx.x, n = 0, base = 0; w < p.items && ok; w += gridDim.x, ++n) {
                const Item it = item_of(w);
                if (n > 0) // the products of the item before have finished with K and V
                    ok = mbarrier_wait(kv_free, (n - 1) & 1, abort_flag, p.counters, 340);
                if (!ok)
                    break;
                mbarrier_expect_tx(kv_full, 2 * TileBytes);
                tma_load_3d(smem_k, &map_qkv128, p.width + it.h * HeadSize, it.row0 + it.tile * KeyTile, 0, kv_full);
                tma_load_3d(smem_v, &map_qkv128, 2 * p.width + it.h * HeadSize, it.row0 + it.tile * KeyTile, 0, kv_full);
                const float *lse2 = p.statistics + it.bh * padded, *delta = lse2 + pairs * padded;
                for (int j = 0; j < it.blocks; ++j) {
                    const int g = base + j, ring = g % Ring, q0 = (it.first_block + j) * Step;
                    ok = mbarrier_wait(qdo_empty0 + 8 * ring, ((g / Ring) & 1) ^ 1, abort_flag, p.counters, 341);
                    if (!ok)
                        break;
                    const uint32_t bar = qdo_full0 + 8 * ring, dst = smem_qdo + ring * 2 * StepBytes,
                                   stats = smem_address(statistics + ring * 128);
                    mbarrier_expect_tx(bar, 2 * StepBytes + 2 * Step * 4);
                    // rows past the end of the tensor arrive as zeros; rows of the next sequence are masked by the compute warps
                    tma_load_3d(dst, &map_qkv64, it.h * HeadSize, it.row0 + q0, 0, bar);
                    tma_load_3d(dst + StepBytes, &map_do64, it.h * HeadSize, it.row0 + q0, 0, bar);
                    bulk_load(stats, lse2 + q0, Step * 4, bar);
                    bulk_load(stats + Step * 4, delta + q0, Step * 4, bar);
                }
                base += it.blocks;
            }
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
            bool ok = true;
            int base = 0; // steps before the current item (even)
            auto issue_s = [&](int j) { // S^T = K Q_j^T; the first use of ring slot j
                const int ring = (base + j) % Ring;
                ok = mbarrier_wait(qdo_full0 + 8 * ring, ((base + j) / Ring) & 1, abort_flag, p.counters, 343);
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
                const uint64_t do_desc = descriptor_at(qdo_desc, ((base + j) % Ring) * 2 * StepBytes + StepBytes);
#pragma unroll
                for (int ks = 0; ks < HeadSize / 16; ++ks)
                    tcgen05_mma_bf16(tmem_dp + 64 * (j & 1), descriptor_at(v_desc, ks * 32), descriptor_at(do_desc, ks * 32),
                                     idesc_s, ks > 0);
                tcgen05_commit(dp_full0 + 8 * (j & 1));
            };
          for (int w = blockIdx.x, n = 0; w < p.items && ok; w += gridDim.x, ++n) {
            const Item it = item_of(w);
            const int blocks = it.blocks;
            ok = mbarrier_wait(kv_full, n & 1, abort_flag, p.counters, 342);
            for (int j = 0; j < 2 && j < blocks && ok; ++j) {
                issue_s(j);
                if (ok)
                    issue_dp(j);
            }
            for (int j = 0; j < blocks && ok; ++j) {
                const int ring = (base + j) % Ring, buffer = j & 1, super = (base + j) >> 1; // `super` counts on across items
                const uint64_t q_mn = descriptor_at(qdo_mn_desc, ring * 2 * StepBytes), do_mn = descriptor_at(q_mn, StepBytes);
                ok = mbarrier_wait(p_full0 + 8 * buffer, super & 1, abort_flag, p.counters, 344);
                if (ok && j == 0 && n > 0) // the compute warps have read dK and dV of the item before
                    ok = mbarrier_wait(acc_free, (n - 1) & 1, abort_flag, p.counters, 339);
                if (!ok)
                    break;
                tcgen05_fence_after();
#pragma unroll
                for (int ks = 0; ks < Step / 16; ++ks) // dV += P^T dO_j: 16 queries = 8 packed columns at (ks / 2) 32 + (ks % 2) 8
                    tcgen05_mma_bf16_ts(tmem_dv, tmem_st + 64 * buffer + (ks / 2) * 32 + (ks % 2) * 8,
                                        descriptor_at(do_mn, ks * 2048), idesc_acc, (j > 0 || ks > 0) ? 1u : 0u);
                if (j + 2 < blocks)
                    issue_s(j + 2); // into the buffer whose P^T the products above have just read
                if (!ok)
                    break;
                ok = mbarrier_wait(ds_full0 + 8 * buffer, super & 1, abort_flag, p.counters, 345);
                if (!ok)
                    break;
                tcgen05_fence_after();
                const uint64_t ds_tile = descriptor_at(ds_desc, ((super & 1) * 2 + buffer) * TileBytes);
#pragma unroll
                for (int ks = 0; ks < Step / 16; ++ks) // dK += dS^T Q_j
                    tcgen05_mma_bf16(tmem_dk, descriptor_at(ds_tile, ks * 32), descriptor_at(q_mn, ks * 2048), idesc_acc,
                                     (j > 0 || ks > 0) ? 1u : 0u);
                tcgen05_commit(qdo_empty0 + 8 * ring); // Q_j and dO_j are no longer read
                if (j + 2 < blocks)
                    issue_dp(j + 2); // the compute warps have read dP^T of step j (they wrote its dS^T)
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
                }
            }
            if (ok) {
                tcgen05_commit(acc_done);
                tcgen05_commit(kv_free);
            }
            base += blocks;
          }
        }
      }
    } else if (warp < FirstComputeWarp) {
        // Four drain warps, one per 32-lane quarter of tensor memory, move this key tile's dQ of every pair of
        // steps out, beside the compute warps.  A block leaves tensor memory with one query row per lane and is
        // staged in shared memory, 256 bytes per row.  For every block but the diagonal one, each lane then hands
        // its row to the copy engine as one bulk reduction (FP32 add, performed in L2) onto the running sum in
        // global memory, or a bulk store when this is key tile 0: no load of the running sum, no register
        // traffic, and the round trips (counter, completion, release) overlap the next block's steps, because
        // the counter is read before the block is complete in tensor memory and advanced only when the next
        // block has arrived.  The diagonal block is the last contribution to its queries: the running sum is
        // copied into the staging rows at the start of the CTA, added in place, and written as BF16, every
        // global access of a warp covering two whole 256-byte rows (lane = row parity x 16-byte piece); a
        // lane-per-row pattern there was measured to stall the SM's whole load/store path, the compute
        // warps' shared-memory traffic included.
        const int quarter = warp % 4;
        const uint32_t lanes = uint32_t(quarter * 32) << 16;
        float *stage = reinterpret_cast<float *>(aligned + OffsetStage) + quarter * 32 * StagePitch; // this warp's 32 rows
        const int piece = lane % 16, parity = lane / 16;
        bool ok = true;
        for (int w = blockIdx.x, base_super = 0, n = 0; w < p.items && ok; w += gridDim.x, ++n) {
        const Item it = item_of(w);
        const int tile = it.tile, bh = it.bh, h = it.h, row0 = it.row0, supers = it.supers;
        const bool first = tile == 0;
        // this warp's 32 rows (8 KB) of block tile + s, contiguous, in the staging rows' own order
        auto sums_of = [&](int s) { return p.dq_sum + ((int64_t(bh) * p.tiles + tile + s) * 128 + quarter * 32) * HeadSize; };
        int *count = p.dq_count + int64_t(bh) * p.tiles + tile; // count[s]: drain warps of earlier tiles done with block tile + s
        auto wait_for_tiles_before = [&](int super, int seen) { // `seen`: lane 0's earlier look; bounded; false when it gave up
            seen = __shfl_sync(0xffffffffu, seen, 0);
            if (seen >= DrainWarps * tile)
                return true;
            if (lane == 0) {
                const unsigned long long start = global_timer();
                while ((seen = load_acquire(count + super)) < DrainWarps * tile) {
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
        if (!first) { // the diagonal block's running sum, asynchronously into the staging rows
            ok = wait_for_tiles_before(0, 0);
            if (ok) {
                const float4 *source = reinterpret_cast<const float4 *>(sums_of(0)) + lane;
#pragma unroll
                for (int k = 0; k < 16; ++k) // 8 KB as it lies: 512 bytes per instruction
                    copy_async16(smem_address(stage) + (lane + 32 * k) * 16, source + 32 * k);
                copy_async_commit();
            }
        }
        int released = 0; // blocks 1..released have had their counters advanced (the diagonal block has none)
        for (int super = 0; super < supers && ok; ++super) {
            const int running = base_super + super, sb = running & 1; // tensor-memory buffers alternate across items
            const int position0 = (tile + super) * 128 + quarter * 32; // query of this warp's first row
            const bool last = super == 0;
            int seen = 0; // this block's counter, read now, looked at when the block has been staged
            if (!first && !last && lane == 0)
                seen = load_acquire(count + super);
            if (!first && super + 1 < supers) { // the reduction after this one finds its lines in L2: 32 x 256 bytes
                const char *next = reinterpret_cast<const char *>(sums_of(super + 1)) + lane * 256;
                prefetch_l2(next);
                prefetch_l2(next + 128);
            }
            ok = mbarrier_wait(dq_full0 + 8 * sb, (running >> 1) & 1, abort_flag, p.counters, 347);
            if (!ok)
                break;
            tcgen05_fence_after();
            if (last) {
                copy_async_wait();
                __syncwarp(); // the running sums are in the staging rows, whichever lane copied them
            } else {
                if (lane == 0)
                    bulk_wait_read(); // the copy engine has read the block before from the staging rows
                __syncwarp();
            }
            const bool add = last && !first;
#pragma unroll 1
            for (int part = 0; part < 2; ++part) { // 32 columns at a time: tensor memory -> staging, lane = row
                uint32_t raw[32];
                tmem_load_32x32_async(tmem_dq + 64 * sb + lanes + part * 32, raw);
                tmem_wait_load(raw);
                float4 *row = reinterpret_cast<float4 *>(stage + lane * StagePitch);
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    float4 *cell = row + ((part * 8 + g) ^ (lane & 7)); // eight neighbouring rows use eight different banks
                    float4 v = make_float4(__uint_as_float(raw[4 * g]), __uint_as_float(raw[4 * g + 1]),
                                           __uint_as_float(raw[4 * g + 2]), __uint_as_float(raw[4 * g + 3]));
                    if (add) {
                        const float4 o = *cell;
                        v.x += o.x, v.y += o.y, v.z += o.z, v.w += o.w;
                    }
                    *cell = v;
                }
            }
            tcgen05_fence_before();
            __syncwarp(); // the block has left tensor memory and is complete in the staging rows
            if (lane == 0)
                mbarrier_arrive(dq_free0 + 8 * sb);
            if (last) {
#pragma unroll
                for (int k = 0; k < 16; ++k) { // out in whole rows: lane = row parity x 16-byte piece
                    const int r = 2 * k + parity, position = position0 + r;
                    if (position >= p.context)
                        continue;
                    const float4 v = *reinterpret_cast<const float4 *>(stage + r * StagePitch + (piece ^ (r & 7)) * 4);
                    bf16 *out = p.dqkv + (int64_t(row0) + position) * 3 * p.width + h * HeadSize + piece * 4;
                    *reinterpret_cast<uint2 *>(out) =
                        make_uint2(pack_bf16(v.x * p.scale, v.y * p.scale), pack_bf16(v.z * p.scale, v.w * p.scale));
                }
                __syncwarp(); // every lane has read the staging rows before any lane stages the next block
            } else {
                fence_async_proxy(); // the copy engine reads what this lane has staged
                if (!first)
                    ok = wait_for_tiles_before(super, seen);
                if (!ok)
                    break;
                __syncwarp();
                if (lane == 0) { // one operation for the warp's 32 rows; rows past the end of the sequence are zeros
                    if (first)
                        bulk_store(sums_of(super), smem_address(stage), 32 * HeadSize * 4);
                    else
                        bulk_add(sums_of(super), smem_address(stage), 32 * HeadSize * 4);
                    bulk_commit();
                    bulk_wait<2>(); // two blocks' time for an operation to complete before its counter is advanced
                    while (released < super - 2)
                        add_release(count + ++released, 1);
                }
            }
        }
        if (lane == 0) {
            bulk_wait<0>();
            while (ok && released < supers - 1)
                add_release(count + ++released, 1);
        }
        __syncwarp(); // the staging rows are free for the next item
        base_super += supers;
        }
    } else {
        grow_registers<ComputeRegisters>();
        // Sixteen compute warps in two groups; group g takes the steps j = g, g + 2, ...  Inside a group two
        // warps share each 32-lane quarter of tensor memory; warp `half` takes 32 of the step's 64 queries.
        const int group = (warp - FirstComputeWarp) / 8, quarter = warp % 4, half = ((warp - FirstComputeWarp) / 4) % 2;
        const int row = quarter * 32 + lane;
        const uint32_t lanes = uint32_t(quarter * 32) << 16;
        const uint32_t t_s = tmem_st + 64 * group + lanes + half * 32, t_dp = tmem_dp + 64 * group + lanes + half * 32;
        bool ok = true;

        for (int w = blockIdx.x, n = 0, base = 0; w < p.items && ok; w += gridDim.x, ++n) {
        const Item it = item_of(w);
        const int tile = it.tile, h = it.h, row0 = it.row0, first_block = it.first_block, blocks = it.blocks;
        const int key = tile * KeyTile + row;                 // key position inside the sequence
        const int warp_first = tile * KeyTile + quarter * 32; // earliest key of this warp
        for (int j = group; j < blocks && ok; j += 2) {
            const int ring = (base + j) % Ring, super = (base + j) >> 1, use = super; // counted on across items
            ok = mbarrier_wait(qdo_full0 + 8 * ring, ((base + j) / Ring) & 1, abort_flag, p.counters, 349) && // statistics
                 mbarrier_wait(s_full0 + 8 * group, use & 1, abort_flag, p.counters, 350);
            if (!ok)
                break;
            tcgen05_fence_after();
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
            ok = mbarrier_wait(dp_full0 + 8 * group, use & 1, abort_flag, p.counters, 351);
            if (ok && super >= 2) // the dS^T tiles of this pair of steps were last read by the products of pair super - 2
                ok = mbarrier_wait(ds_free0 + 8 * (super & 1), ((super >> 1) & 1) ^ 1, abort_flag, p.counters, 352);
            if (!ok)
                break;
            tcgen05_fence_after();
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
        }
        if (ok)
            ok = mbarrier_wait(acc_done, n & 1, abort_flag, p.counters, 353);
        if (ok) {
            tcgen05_fence_after();
            // group 0 stores dK, group 1 dV: thread = key row, 32 columns
            uint32_t a[32];
            tmem_load_32x32_async((group == 0 ? tmem_dk : tmem_dv) + lanes + half * 32, a);
            tmem_wait_load(a);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) // the accumulators are in registers: the next item's products may overwrite them
                mbarrier_arrive(acc_free);
            // Out through shared memory, so that a warp's store covers eight 64-byte row pieces instead of 32
            // different lines (thread = row would).  The staging bytes are the ones this same warp writes as dS^T
            // of its group's first tile, which no product reads any more and nobody else ever writes.
            const float factor = group == 0 ? p.scale : 1.f;
            const uint32_t tile_base = smem_ds + group * TileBytes;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                store_shared16(tile_base + row * 128 + (((half * 4 + c) ^ (row & 7)) << 4),
                               pack_bf16(__uint_as_float(a[8 * c]) * factor, __uint_as_float(a[8 * c + 1]) * factor),
                               pack_bf16(__uint_as_float(a[8 * c + 2]) * factor, __uint_as_float(a[8 * c + 3]) * factor),
                               pack_bf16(__uint_as_float(a[8 * c + 4]) * factor, __uint_as_float(a[8 * c + 5]) * factor),
                               pack_bf16(__uint_as_float(a[8 * c + 6]) * factor, __uint_as_float(a[8 * c + 7]) * factor));
            __syncwarp();
            bf16 *target = p.dqkv + (group == 0 ? p.width : 2 * p.width) + h * HeadSize + half * 32 + (lane % 4) * 8;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int r = quarter * 32 + 8 * k + lane / 4, position = tile * KeyTile + r;
                const uint4 v = load_shared16(tile_base + r * 128 + (((half * 4 + lane % 4) ^ (r & 7)) << 4));
                if (position < p.context)
                    *reinterpret_cast<uint4 *>(target + (int64_t(row0) + position) * 3 * p.width) = v;
            }
            __syncwarp(); // every lane has read the staging bytes before the warp writes dS^T there again
        }
        base += blocks;
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

// Per (batch, head, query): lse in base 2 and delta = sum_d dO[t, h, d] * O[t, h, d], into rows padded to whole
// key tiles (the kernel above fetches them 64 at a time).  Eight threads per (token, head), 8 elements each.
__global__ void __launch_bounds__(256) attention_statistics_kernel(const bf16 *__restrict__ out, const bf16 *__restrict__ dout,
                                                                   const float *__restrict__ lse, float *__restrict__ statistics,
                                                                   int64_t vectors, int context, int heads, int64_t padded,
                                                                   int64_t pairs) {
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
        const int64_t bh = token / context * heads + pair % heads, t = token % context;
        statistics[bh * padded + t] = lse[bh * context + t] * 1.4426950408889634f;
        statistics[(pairs + bh) * padded + t] = sum;
    }
}
} // namespace


size_t flash_backward_scratch_bytes(int batch, int context, int heads) {
    const size_t tiles = size_t(context + KeyTile - 1) / KeyTile;
    const size_t pairs = size_t(batch) * heads;
    // running sums of dQ, statistics (lse and delta, padded rows), counters
    return pairs * tiles * KeyTile * HeadSize * sizeof(float) + 2 * pairs * tiles * KeyTile * sizeof(float) + pairs * tiles * sizeof(int);
}

void launch_flash_attention_backward_fused(const void *qkv, const void *out, const void *dout, const float *lse, void *dqkv, void *scratch, int batch, int context, int heads,
                                           StepCounters *counters, cudaStream_t s) {
    static bool configured[64] = {};
    static int sms[64] = {};
    int device = 0;
    CHECK_CUDA(cudaGetDevice(&device));
    if (device >= 64)
        throw std::runtime_error("device index out of range");
    if (!configured[device]) {
        CHECK_CUDA(cudaDeviceGetAttribute(&sms[device], cudaDevAttrMultiProcessorCount, device));
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
    p.dqkv = static_cast<bf16 *>(dqkv);
    p.batch = batch, p.context = context, p.heads = heads, p.width = width;
    p.tiles = (context + KeyTile - 1) / KeyTile;
    const size_t pairs = size_t(batch) * heads, padded = size_t(p.tiles) * KeyTile;
    p.dq_sum = static_cast<float *>(scratch);
    float *statistics = p.dq_sum + pairs * padded * HeadSize;
    p.statistics = statistics;
    p.dq_count = reinterpret_cast<int *>(statistics + 2 * pairs * padded);
    p.scale = 1.f / sqrtf(float(HeadSize));
    p.scale_log2 = 1.4426950408889634f * p.scale;
    p.counters = counters;
    const uint64_t rows = uint64_t(batch) * context;
    const int64_t vectors = int64_t(rows) * width / 8;
    if (padded != size_t(context)) // the padding is read (and masked): keep it finite
        CHECK_CUDA(cudaMemsetAsync(statistics, 0, 2 * pairs * padded * sizeof(float), s));
    attention_statistics_kernel<<<unsigned((vectors + 255) / 256), 256, 0, s>>>(
        static_cast<const bf16 *>(out), static_cast<const bf16 *>(dout), lse, statistics, vectors, context, heads, int64_t(padded),
        int64_t(pairs));
    CHECK_CUDA(cudaMemsetAsync(p.dq_count, 0, pairs * p.tiles * sizeof(int), s));
    CUtensorMap qkv128 = make_map_bf16(qkv, uint64_t(3) * width, rows, 1, uint64_t(3) * width, 0, HeadSize, 128);
    CUtensorMap qkv64 = make_map_bf16(qkv, uint64_t(3) * width, rows, 1, uint64_t(3) * width, 0, HeadSize, Step);
    CUtensorMap do64 = make_map_bf16(dout, width, rows, 1, width, 0, HeadSize, Step);
    p.items = batch * heads * p.tiles;
    flash_backward_kernel<<<std::min(p.items, sms[device]), Threads, SharedBytes, s>>>(qkv128, qkv64, do64, p);
    CHECK_CUDA(cudaGetLastError());
}
