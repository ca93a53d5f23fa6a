// BF16 GEMM on the 5th-generation tensor cores: C[m,n] = sum_k A[m,k] * B[n,k], FP32
// accumulation in tensor memory.  Replaces the reference's warp-level mma.sync products
// (cuda/mma.cuh:69-108, cuda/ops.cuh:30-55,83-117) for every projection, input-gradient and
// weight-gradient GEMM of the step.
//
// One persistent CTA per SM walks output tiles of 128 x BN (BN = 64..256).  Warp 0 streams
// operand slices of 64 K-elements with TMA into a ring of 128-byte-swizzled shared-memory
// stages; warp 1 issues tcgen05.mma (one thread) into one of two TMEM accumulators; warps 2-5
// drain the other accumulator (tcgen05.ld), apply the epilogue and store, so the epilogue of
// tile i overlaps the main loop of tile i+1.  Either operand may be K-major (row = 64
// contiguous K elements) or MN-major (row = 64 contiguous M/N elements for one K index), which
// covers y = x W^T, dx = dy W and dW = dy^T x on row-major tensors without transposes.
//
// Weight-gradient GEMMs have few output tiles and a very long K; they are split along K, each
// split writes an FP32 partial tile to a workspace and the last split to finish a tile (an
// atomic ticket, no spinning) sums the partials in split order, so results are deterministic.
#include "device_utils.cuh"
#include "sm100.cuh"
#include <mutex>
#include <unordered_map>

using namespace sm100;

namespace {
constexpr int BM = 128, BK = 64, MaxBN = 256, Stages = 4;
constexpr int StageABytes = BM * BK * 2, StageBBytes = MaxBN * BK * 2, StageBytes = StageABytes + StageBBytes;
constexpr int Threads = 192; // warp 0: TMA, warp 1: MMA, warps 2-5: epilogue
constexpr int SharedBytes = Stages * StageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int TmemColumns = 512;

struct TcParams {
    int m, n, k, batch;
    int bn;                 // tile width
    int a_mn, b_mn;         // operand majorness
    int splits, k_blocks_per_split;
    int epilogue, out_fp32;
    void *c, *c2;
    const void *r;
    long long ldc, ldr, c_batch, r_batch;
    float alpha, beta;
    float *workspace;       // [splits][batch][m_tiles*BM][n_tiles*bn] FP32 partial tiles
    unsigned *tickets;      // one per output tile, zero between launches
    StepCounters *counters;
};

__device__ __forceinline__ void store_group(const TcParams &p, float (&v)[8], long long row, int col, int z) {
    // Eight consecutive outputs of one row, column multiple of 8.
    const long long ci = z * p.c_batch + row * p.ldc + col, ri = z * p.r_batch + row * p.ldr + col;
    if (p.out_fp32) {
        if (p.epilogue == int(Epilogue::Axpby)) {
            float r[8];
            load8((const float *)p.r + ri, r);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                v[j] = p.alpha * v[j] + p.beta * r[j];
        }
        store8((float *)p.c + ci, v);
        return;
    }
    switch (p.epilogue) {
    case int(Epilogue::Store):
        break;
    case int(Epilogue::Residual): {
        float r[8];
        load8((const bf16 *)p.r + ri, r);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            v[j] = rounded<bf16>(v[j]) + r[j];
        break;
    }
    case int(Epilogue::GeluDual): {
        float act[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] = rounded<bf16>(v[j]);
            act[j] = gelu(v[j]);
        }
        store8((bf16 *)p.c2 + ci, act);
        break;
    }
    case int(Epilogue::GeluGrad): {
        float r[8];
        load8((const bf16 *)p.r + ri, r);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            v[j] = rounded<bf16>(v[j]) * gelu_derivative(r[j]);
        break;
    }
    case int(Epilogue::Axpby): {
        float r[8];
        load8((const bf16 *)p.r + ri, r);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            v[j] = p.alpha * v[j] + p.beta * r[j];
        break;
    }
    }
    store8((bf16 *)p.c + ci, v);
}

// AND of a predicate over the 128 epilogue threads (named barrier 1).
__device__ __forceinline__ bool epilogue_all(bool ok) {
    uint32_t result;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, 1, 128, p;\n\t"
                 "selp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(result)
                 : "r"(uint32_t(ok))
                 : "memory");
    return result != 0;
}

__global__ void __launch_bounds__(Threads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcParams p) {
    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (smem_address(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - smem_address(raw_shared));
    uint64_t *barriers = reinterpret_cast<uint64_t *>(aligned + Stages * StageBytes);
    // barrier slots: full[Stages], empty[Stages], tmem_full[2], tmem_empty[2]
    const uint32_t full0 = smem_address(barriers), empty0 = full0 + 8 * Stages, tfull0 = empty0 + 8 * Stages,
                   tempty0 = tfull0 + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(barriers + 2 * Stages + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    __shared__ int last_split_flag[4];

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) {
        for (int s = 0; s < Stages; ++s) {
            mbarrier_init(full0 + 8 * s, 1);
            mbarrier_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbarrier_init(tfull0 + 8 * b, 1);
            mbarrier_init(tempty0 + 8 * b, 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_map(&map_a);
        prefetch_map(&map_b);
    }
    if (warp == 1) {
        tmem_alloc(smem_address(tmem_slot), TmemColumns);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int m_tiles = (p.m + BM - 1) / BM, n_tiles = (p.n + p.bn - 1) / p.bn;
    const int k_blocks = (p.k + BK - 1) / BK;
    const long long work_items = (long long)m_tiles * n_tiles * p.batch * p.splits;
    const uint32_t stage_tx = StageABytes + p.bn * BK * 2;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            for (long long w = blockIdx.x; w < work_items; w += gridDim.x) {
                const int split = int(w % p.splits);
                long long t = w / p.splits;
                const int nt = int(t % n_tiles), mt = int(t / n_tiles % m_tiles), z = int(t / n_tiles / m_tiles);
                const int kb0 = split * p.k_blocks_per_split;
                const int kb1 = min(k_blocks, kb0 + p.k_blocks_per_split);
                bool ok = true;
                for (int kb = kb0; kb < kb1 && ok; ++kb) {
                    ok = mbarrier_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.counters, 101);
                    if (!ok)
                        break;
                    const uint32_t bar = full0 + 8 * stage, sa = base + stage * StageBytes, sb = sa + StageABytes;
                    mbarrier_expect_tx(bar, stage_tx);
                    if (!p.a_mn) {
                        tma_load_3d(sa, &map_a, kb * BK, mt * BM, z, bar);
                    } else {
                        for (int j = 0; j < BM / 64; ++j)
                            tma_load_3d(sa + j * 64 * BK * 2, &map_a, mt * BM + j * 64, kb * BK, z, bar);
                    }
                    if (!p.b_mn) {
                        tma_load_3d(sb, &map_b, kb * BK, nt * p.bn, z, bar);
                    } else {
                        for (int j = 0; j < p.bn / 64; ++j)
                            tma_load_3d(sb + j * 64 * BK * 2, &map_b, nt * p.bn + j * 64, kb * BK, z, bar);
                    }
                    if (++stage == Stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok)
                    break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (elect_one()) {
            const uint32_t instruction = instruction_descriptor(BM, p.bn, p.a_mn, p.b_mn);
            // Per 16-element K step inside a stage: 32 bytes along a K-major row, or 16 rows of
            // 128 bytes for an MN-major operand.
            const uint32_t a_step = p.a_mn ? 16 * 128 : 32, b_step = p.b_mn ? 16 * 128 : 32;
            const uint32_t a_lbo = p.a_mn ? 64 * BK * 2 : 16, b_lbo = p.b_mn ? 64 * BK * 2 : 16;
            int stage = 0, buffer = 0;
            uint32_t phase = 0, buffer_phase = 0;
            for (long long w = blockIdx.x; w < work_items; w += gridDim.x) {
                const int split = int(w % p.splits);
                const int kb0 = split * p.k_blocks_per_split;
                const int kb1 = min(k_blocks, kb0 + p.k_blocks_per_split);
                if (!mbarrier_wait(tempty0 + 8 * buffer, buffer_phase ^ 1, abort_flag, p.counters, 102))
                    break;
                tcgen05_fence_after();
                const uint32_t accumulator = tmem_base + buffer * MaxBN;
                bool ok = true;
                for (int kb = kb0; kb < kb1; ++kb) {
                    ok = mbarrier_wait(full0 + 8 * stage, phase, abort_flag, p.counters, 103);
                    if (!ok)
                        break;
                    tcgen05_fence_after();
                    const uint32_t sa = base + stage * StageBytes, sb = sa + StageABytes;
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks) {
                        uint64_t da = smem_descriptor(sa + ks * a_step, a_lbo, 1024);
                        uint64_t db = smem_descriptor(sb + ks * b_step, b_lbo, 1024);
                        tcgen05_mma_bf16(accumulator, da, db, instruction, (kb > kb0 || ks > 0) ? 1u : 0u);
                    }
                    tcgen05_commit(empty0 + 8 * stage); // frees the stage once these MMAs have read it
                    if (++stage == Stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok)
                    break;
                tcgen05_commit(tfull0 + 8 * buffer); // accumulator complete
                if (++buffer == 2) {
                    buffer = 0;
                    buffer_phase ^= 1;
                }
            }
        }
    } else {
        // ---------------- epilogue: 4 warps, warp q owns TMEM lanes 32q..32q+31 ----------------
        const int quarter = warp % 4;
        int buffer = 0;
        uint32_t buffer_phase = 0;
        for (long long w = blockIdx.x; w < work_items; w += gridDim.x) {
            const int split = int(w % p.splits);
            long long t = w / p.splits;
            const int nt = int(t % n_tiles), mt = int(t / n_tiles % m_tiles), z = int(t / n_tiles / m_tiles);
            bool ready = mbarrier_wait(tfull0 + 8 * buffer, buffer_phase, abort_flag, p.counters, 104);
            if (p.splits > 1) // the four warps meet at named barriers below: leave together or not at all
                ready = epilogue_all(ready);
            if (!ready)
                break;
            tcgen05_fence_after();
            const long long row = (long long)mt * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buffer * MaxBN;
            if (p.splits == 1) {
                for (int chunk = 0; chunk < p.bn / 32; ++chunk) {
                    float v[32];
                    tmem_load_32x32(taddr + chunk * 32, v);
                    const int col0 = nt * p.bn + chunk * 32;
                    if (row < p.m) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            if (col0 + g * 8 < p.n) {
                                float group[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    group[j] = v[g * 8 + j];
                                store_group(p, group, row, col0 + g * 8, z);
                            }
                        }
                    }
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbarrier_arrive(tempty0 + 8 * buffer);
            } else {
                // Partial tile to the workspace (padded to whole tiles, so no bounds checks).
                const long long padded_m = (long long)m_tiles * BM, padded_n = (long long)n_tiles * p.bn;
                float *partial = p.workspace + ((long long)split * p.batch + z) * padded_m * padded_n;
                for (int chunk = 0; chunk < p.bn / 32; ++chunk) {
                    float v[32];
                    tmem_load_32x32(taddr + chunk * 32, v);
                    float *out = partial + row * padded_n + nt * p.bn + chunk * 32;
#pragma unroll
                    for (int g = 0; g < 8; ++g)
                        *reinterpret_cast<float4 *>(out + g * 4) =
                            make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbarrier_arrive(tempty0 + 8 * buffer);
                // Ticket: the split that arrives last reduces the tile in split order.
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) {
                    unsigned ticket = atomicAdd(&p.tickets[t], 1u);
                    int last = ticket == unsigned(p.splits - 1);
                    if (last)
                        p.tickets[t] = 0; // ready for the next launch
                    last_split_flag[0] = last;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (last_split_flag[0]) {
                    __threadfence();
                    if (row < p.m) {
                        for (int col = 0; col < p.bn; col += 8) {
                            const int c = nt * p.bn + col;
                            if (c >= p.n)
                                break;
                            float sum[8] = {};
                            for (int s = 0; s < p.splits; ++s) {
                                float v[8];
                                // L2 only: the partials were written by other SMs.
                                const float4 *src = reinterpret_cast<const float4 *>(
                                    p.workspace + ((long long)s * p.batch + z) * padded_m * padded_n +
                                    row * padded_n + c);
                                float4 lo = __ldcg(src), hi = __ldcg(src + 1);
                                v[0] = lo.x, v[1] = lo.y, v[2] = lo.z, v[3] = lo.w;
                                v[4] = hi.x, v[5] = hi.y, v[6] = hi.z, v[7] = hi.w;
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    sum[j] += v[j];
                            }
                            store_group(p, sum, row, c, z);
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory"); // last_split_flag is reused next tile
            }
            if (++buffer == 2) {
                buffer = 0;
                buffer_phase ^= 1;
            }
        }
    }

    // Teardown.  After an aborted wait, give copies already in flight time to land before the
    // shared memory and tensor memory are released.
    __syncthreads();
    if (*abort_flag)
        __nanosleep(2000000);
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1)
        tmem_dealloc(tmem_base, TmemColumns);
}

struct Workspace {
    float *partials = nullptr;
    unsigned *tickets = nullptr;
    size_t partial_bytes = 0, ticket_count = 0;
};
std::mutex workspace_mutex;
std::unordered_map<int, Workspace> workspaces; // per device

// Split-K workspace, grown on demand outside stream capture; one per device, shared by the
// engine's single stream.
Workspace &workspace_for(size_t partial_bytes, size_t tickets, cudaStream_t s) {
    int device = 0;
    CHECK_CUDA(cudaGetDevice(&device));
    std::lock_guard<std::mutex> lock(workspace_mutex);
    Workspace &w = workspaces[device];
    if (w.partial_bytes < partial_bytes) {
        CHECK_CUDA(cudaStreamSynchronize(s));
        if (w.partials)
            CHECK_CUDA(cudaFree(w.partials));
        CHECK_CUDA(cudaMalloc(&w.partials, partial_bytes));
        w.partial_bytes = partial_bytes;
    }
    if (w.ticket_count < tickets) {
        CHECK_CUDA(cudaStreamSynchronize(s));
        if (w.tickets)
            CHECK_CUDA(cudaFree(w.tickets));
        CHECK_CUDA(cudaMalloc(&w.tickets, tickets * sizeof(unsigned)));
        CHECK_CUDA(cudaMemset(w.tickets, 0, tickets * sizeof(unsigned)));
        w.ticket_count = tickets;
    }
    return w;
}
} // namespace

int gemm_tc_shared_bytes() { return SharedBytes; }

bool gemm_tc_supported(const GemmArgs &g) {
    if (g.in != Dtype::BF16)
        return false;
    if (g.m < 1 || g.n < 64 || g.k < 64 || g.n % 8)
        return false;
    const bool a_k = g.a_col == 1, a_mn = g.a_row == 1, b_k = g.b_col == 1, b_mn = g.b_row == 1;
    if (!(a_k || a_mn) || !(b_k || b_mn))
        return false;
    const int64_t lda = a_k ? g.a_row : g.a_col, ldb = b_k ? g.b_row : g.b_col;
    if (lda % 8 || ldb % 8 || g.ldc % 8 || (g.r && g.ldr % 8))
        return false;
    if (reinterpret_cast<uintptr_t>(g.a) % 16 || reinterpret_cast<uintptr_t>(g.b) % 16 ||
        reinterpret_cast<uintptr_t>(g.c) % 16 || reinterpret_cast<uintptr_t>(g.r) % 16 ||
        reinterpret_cast<uintptr_t>(g.c2) % 16)
        return false;
    if (g.a_batch % 8 || g.b_batch % 8 || g.c_batch % 8 || g.r_batch % 8)
        return false;
    // An MN-major operand is fetched in 64-wide blocks: its extent must cover whole blocks so a
    // tile never straddles into the next matrix of a batch.
    if (!a_k && a_mn && g.m % 8)
        return false;
    if (g.out == Dtype::FP32 && !(g.epilogue == Epilogue::Store || g.epilogue == Epilogue::Axpby))
        return false;
    return true;
}

void launch_gemm_tc(const GemmArgs &g, int sms, StepCounters *counters, cudaStream_t s) {
    static bool configured[64] = {};
    int device = 0;
    CHECK_CUDA(cudaGetDevice(&device));
    if (device < 64 && !configured[device]) {
        CHECK_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SharedBytes));
        configured[device] = true;
    }
    TcParams p{};
    p.m = g.m, p.n = g.n, p.k = g.k, p.batch = g.batch;
    p.a_mn = g.a_col == 1 ? 0 : 1;
    p.b_mn = g.b_col == 1 ? 0 : 1;
    const int64_t lda = p.a_mn ? g.a_col : g.a_row, ldb = p.b_mn ? g.b_col : g.b_row;
    const int m_tiles = (g.m + BM - 1) / BM, k_blocks = (g.k + BK - 1) / BK;
    // Tile width and K splits by a small cost model, in clocks per 64-deep K block: the MMA
    // takes bn/2, the shared-memory operand reads (128+bn)/4; a tile adds a fixed drain cost and
    // every split one pass over the FP32 partial tile.
    long long best_time = 0;
    p.bn = 0;
    for (int bn : {256, 192, 128, 64}) {
        if (bn > 64 && bn - 64 >= g.n)
            continue; // a narrower tile already covers N
        const long long tiles = (long long)m_tiles * ((g.n + bn - 1) / bn) * g.batch;
        const int block_cost = bn / 2 > (128 + bn) / 4 ? bn / 2 : (128 + bn) / 4;
        for (int splits : {1, 2, 3, 4, 6, 8, 12, 16}) {
            if (splits > 1 && (k_blocks / splits < 8 || tiles * splits > sms))
                continue;
            const int per = (k_blocks + splits - 1) / splits;
            if (splits > 1 && (k_blocks + per - 1) / per != splits)
                continue; // would leave an empty split
            const long long rounds = (tiles * splits + sms - 1) / sms;
            const long long time = rounds * ((long long)per * (block_cost + 16) + bn + (splits > 1 ? splits * bn / 2 : 0));
            if (!p.bn || time < best_time)
                p.bn = bn, p.splits = splits, p.k_blocks_per_split = per, best_time = time;
        }
    }
    const int n_tiles = (g.n + p.bn - 1) / p.bn;
    const long long tiles = (long long)m_tiles * n_tiles * g.batch;
    p.epilogue = int(g.epilogue), p.out_fp32 = g.out == Dtype::FP32;
    p.c = g.c, p.c2 = g.c2, p.r = g.r;
    p.ldc = g.ldc, p.ldr = g.ldr, p.c_batch = g.c_batch, p.r_batch = g.r_batch;
    p.alpha = g.alpha, p.beta = g.beta;
    p.counters = counters;
    if (p.splits > 1) {
        size_t bytes = size_t(p.splits) * g.batch * m_tiles * BM * n_tiles * p.bn * sizeof(float);
        Workspace &w = workspace_for(bytes, size_t(tiles), s);
        p.workspace = w.partials;
        p.tickets = w.tickets;
    }
    CUtensorMap map_a = p.a_mn ? make_map_bf16(g.a, g.m, g.k, g.batch, lda, g.a_batch, 64, BK)
                               : make_map_bf16(g.a, g.k, g.m, g.batch, lda, g.a_batch, BK, BM);
    CUtensorMap map_b = p.b_mn ? make_map_bf16(g.b, g.n, g.k, g.batch, ldb, g.b_batch, 64, BK)
                               : make_map_bf16(g.b, g.k, g.n, g.batch, ldb, g.b_batch, BK, p.bn);
    long long work = tiles * p.splits;
    int grid = int(work < sms ? work : sms);
    gemm_tc_kernel<<<grid, Threads, SharedBytes, s>>>(map_a, map_b, p);
    CHECK_CUDA(cudaGetLastError());
}
