// BF16 GEMM on the 5th-generation tensor cores: C[m,n] = sum_k A[m,k] * B[n,k], FP32
// accumulation in tensor memory.  Replaces the reference's warp-level mma.sync products
// (cuda/mma.cuh:69-108, cuda/ops.cuh:30-55,83-117) for every projection, input-gradient and
// weight-gradient GEMM of the step.
//
// One persistent CTA per SM (or one CTA pair per two SMs, cta_group::2, for 256-row tiles) walks
// output tiles of 128 x BN (BN = 64..256).  Warp 0 streams operand slices of 64 K-elements with
// TMA into a ring of 128-byte-swizzled shared-memory stages; warp 1 issues tcgen05.mma (one
// thread) into one of two 256-column TMEM accumulators; sixteen epilogue warps drain the other
// accumulator, so the epilogue of tile i overlaps the main loop of tile i+1.  Either operand may be
// K-major (row = 64 contiguous K elements) or MN-major (row = 64 contiguous M/N elements for one K
// index), which covers y = x W^T, dx = dy W and dW = dy^T x on row-major tensors without transposes.
//
// Epilogue: four warps share each 32-lane quarter of tensor memory and take every fourth
// 32-column chunk.  A lane owns one output row: it reads its accumulator chunk (tcgen05.ld),
// optionally combines it with the same chunk of a second tensor read straight from global memory
// (residual, saved GELU derivative, or the Newton-Schulz operand) and writes 32-byte pieces with
// 256-bit stores.
//
// Weight-gradient GEMMs have few output tiles and a very long K; they are split along K and each
// split writes an FP32 partial tile to a workspace.  With two or three splits the last one to finish
// a tile (an atomic ticket, no spinning) sums the partials in split order; with four or more a second
// kernel adds them, in the same order, over the whole GPU.  Results are deterministic either way.
// The head GEMM has an epilogue of its own: 256-way softmax cross-entropy on the FP32 accumulators.
#include "device_utils.cuh"
#include "sm100.cuh"
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <mutex>
#include <type_traits>
#include <unordered_map>

using namespace sm100;

namespace {
constexpr int BM = 128, BK = 64, MaxBN = 256, MaxStages = 8;
constexpr int StageABytes = BM * BK * 2;
constexpr int EpilogueWarps = 16;
constexpr int Threads = 64 + 32 * EpilogueWarps; // warp 0: TMA, warp 1: MMA, then the epilogue warps
constexpr int ControlBytes = 512;   // barriers, TMEM slot, flags
constexpr int RowScratchBytes = 2 * 4 * BM * 4; // CrossEntropy: row maxima and row sums of the four column shares
constexpr int MaxShared = 232448 - 1024; // 227 KB less the runtime's own reservation
constexpr int TmemColumns = 512;

struct TcParams {
    int m, n, k, batch;
    int bn;                 // tile width
    int a_mn, b_mn;         // operand majorness
    int splits, k_blocks_per_split;
    int epilogue, out_fp32;
    int stages;             // depth of the operand ring
    int wide;               // C, C2 and R rows are 32-byte aligned: 256-bit epilogue accesses
    int reduce_later;       // K splits only write their partial tiles; splitk_reduce_kernel adds them afterwards
    void *c, *c2;
    const void *r;
    long long ldc, ldr, c_batch, r_batch;
    float alpha, beta;
    float *workspace;       // [splits][batch][m_tiles*BM][n_tiles*bn] FP32 partial tiles
    unsigned *tickets;      // one per output tile, zero between launches
    StepCounters *counters;
};

// Phi(x) = 0.5 (1 + erf(x / sqrt 2)) by Abramowitz & Stegun 7.1.26 (|error| < 3e-7) with every
// constant folded: t = 1 / (1 + p |x| / sqrt 2), e = 2^(-x^2 log2(e) / 2), tail = 0.5 erfc = poly(t) t e.
// Two SFU operations (rcp, ex2) and nine FMA-pipe operations; the exponential also gives the
// Gaussian density of the derivative.
__device__ __forceinline__ void gelu_terms(float x, float &cdf, float &density) {
    float t, e;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.23164189f, fabsf(x), 1.f)));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-0.72134752f * x * x));
    float poly = fmaf(t, 0.5307027145f, -0.7265760135f);
    poly = fmaf(t, poly, 0.7107068705f);
    poly = fmaf(t, poly, -0.142248368f);
    poly = fmaf(t, poly, 0.127414796f);
    const float tail = poly * t * e;
    cdf = x >= 0.f ? 1.f - tail : tail;
    density = 0.3989422804014327f * e; // exp(-x^2/2) / sqrt(2 pi)
}

// Direct global store of eight consecutive outputs (split-K reduction path only).
__device__ __forceinline__ void store_group(const TcParams &p, float (&v)[8], long long row, int col, int z) {
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
    store8((bf16 *)p.c + ci, v);
}

// AND of a predicate over the 512 epilogue threads (named barrier 1).
__device__ __forceinline__ bool epilogue_all(bool ok) {
    uint32_t result;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, 1, 512, p;\n\t"
                 "selp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(result)
                 : "r"(uint32_t(ok))
                 : "memory");
    return result != 0;
}

// 32 bytes to or from global memory: one 256-bit access when `wide` (32-byte aligned), else two
// 128-bit accesses; `second` says whether the upper half is inside the tensor.
__device__ __forceinline__ void load_global32(const void *p, uint32_t (&r)[8], bool wide, bool second) {
    if (wide) {
        asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                     : "l"(p));
    } else {
        uint4 a = *reinterpret_cast<const uint4 *>(p), b = make_uint4(0, 0, 0, 0);
        if (second)
            b = *(reinterpret_cast<const uint4 *>(p) + 1);
        r[0] = a.x, r[1] = a.y, r[2] = a.z, r[3] = a.w, r[4] = b.x, r[5] = b.y, r[6] = b.z, r[7] = b.w;
    }
}
__device__ __forceinline__ void store_global32(void *p, const uint32_t (&r)[8], bool wide, bool second) {
    if (wide) {
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(r[0]), "r"(r[1]),
                     "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                     : "memory");
    } else {
        *reinterpret_cast<uint4 *>(p) = make_uint4(r[0], r[1], r[2], r[3]);
        if (second)
            *(reinterpret_cast<uint4 *>(p) + 1) = make_uint4(r[4], r[5], r[6], r[7]);
    }
}
// Pair = true: the CTA is half of a cluster of two that computes a 256-row tile with
// cta_group::2 MMAs issued by the pair's first CTA.  Each CTA stages its own 128 rows of A and half
// of the B tile (the tensor core reads the other half from the partner's shared memory), so a
// K block costs each SM 16 KB + BN/2 x 128 B instead of 16 KB + BN x 128 B and the ring is deeper.
template <int Kind, bool OutFp32, bool Pair>
__global__ void __launch_bounds__(Threads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcParams p) {
    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (smem_address(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - smem_address(raw_shared));
    constexpr int Unit = Pair ? 2 : 1;
    const uint32_t rank = Pair ? cluster_rank() : 0u;
    const int bn_local = p.bn / Unit; // B rows staged by this CTA
    const int stage_bytes = StageABytes + bn_local * BK * 2;
    uint64_t *barriers = reinterpret_cast<uint64_t *>(aligned + p.stages * stage_bytes);
    // barriers: full[8], empty[8], tmem_full[2], tmem_empty[2]
    const uint32_t full0 = smem_address(barriers), empty0 = full0 + 8 * MaxStages, tfull0 = empty0 + 8 * MaxStages,
                   tempty0 = tfull0 + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(barriers + 2 * MaxStages + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    volatile int *last_split_flag = reinterpret_cast<volatile int *>(tmem_slot + 2);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbarrier_init(full0 + 8 * s, 1);
            mbarrier_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbarrier_init(tfull0 + 8 * b, 1);
            mbarrier_init(tempty0 + 8 * b, EpilogueWarps * Unit);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_map(&map_a);
        prefetch_map(&map_b);
    }
    if (warp == 1) {
        if constexpr (Pair) {
            tmem_alloc_pair(smem_address(tmem_slot), TmemColumns);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_address(tmem_slot), TmemColumns);
            tmem_relinquish();
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if constexpr (Pair)
        cluster_sync_all(); // the partner's barriers exist before anything signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Barriers, tensor memory and descriptors are set up; only now wait for the kernel before this one
    // (its tail overlaps the set-up above when this kernel was launched programmatically).
    grid_launch_dependents();
    grid_dependency_wait();

    // Tiles along M are scheduled per CTA pair; m_tiles counts 128-row tiles including padding.
    const int m_tiles = ((p.m + BM * Unit - 1) / (BM * Unit)) * Unit, n_tiles = (p.n + p.bn - 1) / p.bn;
    const int k_blocks = (p.k + BK - 1) / BK;
    const int m_units = m_tiles / Unit;
    const long long work_items = (long long)m_units * n_tiles * p.batch * p.splits;
    const long long first_item = blockIdx.x / Unit, item_stride = gridDim.x / Unit;
    const uint32_t stage_tx = stage_bytes * Unit; // bytes landing for one stage in both CTAs

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            for (long long w = first_item; w < work_items; w += item_stride) {
                const int split = int(w % p.splits);
                long long t = w / p.splits;
                const int nt = int(t % n_tiles), mt = int(t / n_tiles % m_units) * Unit + int(rank),
                      z = int(t / n_tiles / m_units);
                const int kb0 = split * p.k_blocks_per_split;
                const int kb1 = min(k_blocks, kb0 + p.k_blocks_per_split);
                bool ok = true;
                for (int kb = kb0; kb < kb1 && ok; ++kb) {
                    ok = mbarrier_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.counters, 101);
                    if (!ok)
                        break;
                    const uint32_t sa = base + stage * stage_bytes, sb = sa + StageABytes;
                    // Both CTAs' bytes are counted on the first CTA's barrier, armed by that CTA.
                    const uint32_t bar = Pair ? cluster_address(full0 + 8 * stage, 0) : full0 + 8 * stage;
                    if (rank == 0)
                        mbarrier_expect_tx(full0 + 8 * stage, stage_tx);
                    auto load = [&](uint32_t dst, const CUtensorMap *map, int x, int y) {
                        if constexpr (Pair)
                            tma_load_3d_pair(dst, map, x, y, z, bar);
                        else
                            tma_load_3d(dst, map, x, y, z, bar);
                    };
                    const int n_first = nt * p.bn + int(rank) * bn_local;
                    if (!p.a_mn) {
                        load(sa, &map_a, kb * BK, mt * BM);
                    } else {
                        for (int j = 0; j < BM / 64; ++j)
                            load(sa + j * 64 * BK * 2, &map_a, mt * BM + j * 64, kb * BK);
                    }
                    if (!p.b_mn) {
                        load(sb, &map_b, kb * BK, n_first);
                    } else {
                        for (int j = 0; j < bn_local / 64; ++j)
                            load(sb + j * 64 * BK * 2, &map_b, n_first + j * 64, kb * BK);
                    }
                    if (++stage == p.stages) {
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
        if (rank == 0 && elect_one()) {
            const uint32_t instruction = instruction_descriptor(BM * Unit, p.bn, p.a_mn, p.b_mn);
            // Per 16-element K step inside a stage: 32 bytes along a K-major row, or 16 rows of
            // 128 bytes for an MN-major operand.
            const uint32_t a_step = p.a_mn ? 16 * 128 : 32, b_step = p.b_mn ? 16 * 128 : 32;
            const uint32_t a_lbo = p.a_mn ? 64 * BK * 2 : 16, b_lbo = p.b_mn ? 64 * BK * 2 : 16;
            int stage = 0, buffer = 0;
            uint32_t phase = 0, buffer_phase = 0;
            for (long long w = first_item; w < work_items; w += item_stride) {
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
                    const uint32_t sa = base + stage * stage_bytes, sb = sa + StageABytes;
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks) {
                        uint64_t da = smem_descriptor(sa + ks * a_step, a_lbo, 1024);
                        uint64_t db = smem_descriptor(sb + ks * b_step, b_lbo, 1024);
                        if constexpr (Pair)
                            tcgen05_mma_bf16_pair(accumulator, da, db, instruction, (kb > kb0 || ks > 0) ? 1u : 0u);
                        else
                            tcgen05_mma_bf16(accumulator, da, db, instruction, (kb > kb0 || ks > 0) ? 1u : 0u);
                    }
                    // frees the stage (in both CTAs) once these MMAs have read it
                    if constexpr (Pair) {
                        tcgen05_commit_pair(cluster_address(empty0 + 8 * stage, 0));
                        tcgen05_commit_pair(cluster_address(empty0 + 8 * stage, 1));
                    } else {
                        tcgen05_commit(empty0 + 8 * stage);
                    }
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok)
                    break;
                if constexpr (Pair) { // accumulator complete, in both CTAs' tensor memory
                    tcgen05_commit_pair(cluster_address(tfull0 + 8 * buffer, 0));
                    tcgen05_commit_pair(cluster_address(tfull0 + 8 * buffer, 1));
                } else {
                    tcgen05_commit(tfull0 + 8 * buffer);
                }
                if (++buffer == 2) {
                    buffer = 0;
                    buffer_phase ^= 1;
                }
            }
        }
    } else {
        // ---------------- epilogue: 16 warps; warps q, q+4, q+8, q+12 share TMEM lanes 32q..32q+31 and
        // take every fourth 32-column chunk.  Four warps per scheduler hide one another's TMEM,
        // ALU, SFU and global-load latencies (the epilogue math is a dependent chain per element).
        constexpr int Shares = EpilogueWarps / 4;
        const int quarter = warp % 4, share = (warp - 2) / 4;
        constexpr bool has_r = Kind == int(Epilogue::Residual) || Kind == int(Epilogue::GeluGrad) ||
                               Kind == int(Epilogue::Axpby);
        constexpr bool whole_rows = Kind == int(Epilogue::CrossEntropy); // the sixteen warps meet per tile
        int buffer = 0;
        uint32_t buffer_phase = 0;
        for (long long w = first_item; w < work_items; w += item_stride) {
            const int split = int(w % p.splits);
            long long t = w / p.splits;
            const int nt = int(t % n_tiles), mt = int(t / n_tiles % m_units) * Unit + int(rank),
                      z = int(t / n_tiles / m_units);
            bool ready = mbarrier_wait(tfull0 + 8 * buffer, buffer_phase, abort_flag, p.counters, 104);
            if (p.splits > 1 || whole_rows) // the warps meet at named barriers below: leave together or not at all
                ready = epilogue_all(ready);
            if (!ready)
                break;
            tcgen05_fence_after();
            const long long row = (long long)mt * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buffer * MaxBN;
            const int tile_columns = min(p.bn, p.n - nt * p.bn);
            const int chunks = (tile_columns + 31) / 32;
            if constexpr (whole_rows) {
                // One 256-column tile holds whole rows of logits.  A thread owns row `row` in the 32-column chunks
                // `share` and `share + 4`; the four shares of a row exchange their maxima and sums through shared
                // memory and add them in share order.
                float *row_high = reinterpret_cast<float *>(aligned + p.stages * stage_bytes + ControlBytes);
                float *row_sum = row_high + Shares * BM;
                const int local = quarter * 32 + lane;
                float v[64];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t acc[32];
                    tmem_load_32x32_async(taddr + (share + half * Shares) * 32, acc);
                    tmem_wait_load(acc);
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        v[half * 32 + j] = __uint_as_float(acc[j]);
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) { // the accumulator is in registers: the next tile's products may overwrite it
                    if constexpr (Pair)
                        mbarrier_arrive_cluster(cluster_address(tempty0 + 8 * buffer, 0));
                    else
                        mbarrier_arrive(tempty0 + 8 * buffer);
                }
                const bool row_ok = row < p.m;
                const int target = row_ok ? static_cast<const uint8_t *>(p.r)[row] : 0;
                float high = v[0], picked = 0.f;
#pragma unroll
                for (int j = 0; j < 64; ++j) {
                    high = fmaxf(high, v[j]);
                    const int column = (share + (j / 32) * Shares) * 32 + j % 32;
                    picked = column == target ? v[j] : picked;
                }
                row_high[share * BM + local] = high;
                asm volatile("bar.sync 1, 512;" ::: "memory");
                high = fmaxf(fmaxf(row_high[local], row_high[BM + local]), fmaxf(row_high[2 * BM + local], row_high[3 * BM + local]));
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < 64; ++j) {
                    v[j] = expf(v[j] - high);
                    sum += v[j];
                }
                row_sum[share * BM + local] = sum;
                asm volatile("bar.sync 1, 512;" ::: "memory");
                sum = ((row_sum[local] + row_sum[BM + local]) + row_sum[2 * BM + local]) + row_sum[3 * BM + local];
                if (row_ok) {
                    if (target / 32 % Shares == share)
                        static_cast<float *>(p.c2)[row] = high + logf(sum) - picked;
                    if (p.c) {
                        const float inverse = 1.f / sum;
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            const int column = (share + half * Shares) * 32;
                            char *dst = (char *)p.c + (row * p.ldc + column) * 2;
#pragma unroll
                            for (int g = 0; g < 2; ++g) {
                                uint32_t out[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    const int e = half * 32 + g * 16 + 2 * j;
                                    const float a = (v[e] * inverse - (column + g * 16 + 2 * j == target ? 1.f : 0.f)) * p.alpha;
                                    const float b = (v[e + 1] * inverse - (column + g * 16 + 2 * j + 1 == target ? 1.f : 0.f)) * p.alpha;
                                    out[j] = pack_bf16(a, b);
                                }
                                store_global32(dst + g * 32, out, p.wide, true);
                            }
                        }
                    }
                }
            } else if (p.splits == 1) {
                const bool row_ok = row < p.m;
                const long long c_row = z * p.c_batch + row * p.ldc, r_row = z * p.r_batch + row * p.ldr;
                auto process = [&](uint32_t (&acc)[32], int c) {
                    const int column = nt * p.bn + c * 32;
                    // Second tensor for this chunk: issue the global loads before waiting on TMEM.
                    constexpr int Pieces = OutFp32 ? 4 : 2; // 32-byte pieces per 32-column chunk row
                    constexpr int PieceColumns = 32 / Pieces;
                    uint32_t rv[has_r ? Pieces : 1][8];
                    if (has_r && row_ok) {
                        const char *src = (const char *)p.r + (r_row + column) * (OutFp32 ? 4 : 2);
#pragma unroll
                        for (int g = 0; g < Pieces; ++g)
                            if (column + g * PieceColumns < p.n)
                                load_global32(src + g * 32, rv[g], p.wide && column + (g + 1) * PieceColumns <= p.n,
                                              column + g * PieceColumns + PieceColumns / 2 < p.n);
                    }
                    tmem_wait_load(acc);
                    if (!row_ok)
                        return;
                    char *dst = (char *)p.c + (c_row + column) * (OutFp32 ? 4 : 2);
#pragma unroll
                    for (int g = 0; g < Pieces; ++g) {
                        if (column + g * PieceColumns >= p.n)
                            break;
                        const bool whole = p.wide && column + (g + 1) * PieceColumns <= p.n;
                        uint32_t out[8];
                        if constexpr (OutFp32) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                float v = __uint_as_float(acc[g * 8 + j]);
                                if (has_r) // Axpby on FP32
                                    v = p.alpha * v + p.beta * __uint_as_float(rv[g][j]);
                                out[j] = __float_as_uint(v);
                            }
                        } else {
                            float v[16], r[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                v[j] = __uint_as_float(acc[g * 16 + j]);
                            if (has_r) {
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    r[2 * j] = __uint_as_float(rv[g][j] << 16);
                                    r[2 * j + 1] = __uint_as_float(rv[g][j] & 0xffff0000u);
                                }
                            }
                            if constexpr (Kind == int(Epilogue::Residual)) {
#pragma unroll
                                for (int j = 0; j < 16; ++j)
                                    v[j] = rounded<bf16>(v[j]) + r[j];
                            } else if constexpr (Kind == int(Epilogue::GeluDual)) {
                                uint32_t activated[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) { // v becomes gelu'(pre), `activated` gelu(pre)
                                    float cdf0, cdf1, den0, den1;
                                    const float x0 = rounded<bf16>(v[2 * j]), x1 = rounded<bf16>(v[2 * j + 1]);
                                    gelu_terms(x0, cdf0, den0);
                                    gelu_terms(x1, cdf1, den1);
                                    activated[j] = pack_bf16(x0 * cdf0, x1 * cdf1);
                                    v[2 * j] = fmaf(x0, den0, cdf0);
                                    v[2 * j + 1] = fmaf(x1, den1, cdf1);
                                }
                                store_global32((char *)p.c2 + (c_row + column) * 2 + g * 32, activated, whole,
                                               column + g * 16 + 8 < p.n);
                            } else if constexpr (Kind == int(Epilogue::GeluGrad)) {
#pragma unroll
                                for (int j = 0; j < 16; ++j)
                                    v[j] = rounded<bf16>(v[j]) * r[j];
                            } else if constexpr (Kind == int(Epilogue::Axpby)) {
#pragma unroll
                                for (int j = 0; j < 16; ++j)
                                    v[j] = p.alpha * v[j] + p.beta * r[j];
                            }
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                out[j] = pack_bf16(v[2 * j], v[2 * j + 1]);
                        }
                        store_global32(dst + g * 32, out, whole, column + g * PieceColumns + PieceColumns / 2 < p.n);
                    }
                };
                for (int c = share; c < chunks; c += Shares) {
                    uint32_t acc[32];
                    tmem_load_32x32_async(taddr + c * 32, acc);
                    process(acc, c);
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (Pair)
                        mbarrier_arrive_cluster(cluster_address(tempty0 + 8 * buffer, 0));
                    else
                        mbarrier_arrive(tempty0 + 8 * buffer);
                }
            } else {
                // Partial tile to the workspace (padded to whole tiles, so no bounds checks).  A 32 x 32
                // chunk is stored column by column (lane = row), so every access is one 128-byte line.
                const long long padded_m = (long long)m_tiles * BM, padded_n = (long long)n_tiles * p.bn;
                const long long split_stride = (long long)p.batch * padded_m * padded_n;
                float *partial = p.workspace + ((long long)split * p.batch + z) * padded_m * padded_n;
                const long long chunk_row = ((long long)mt * 4 + quarter) * (padded_n / 32) + nt * (p.bn / 32);
                for (int chunk = share; chunk < p.bn / 32; chunk += Shares) {
                    float v[32];
                    tmem_load_32x32(taddr + chunk * 32, v);
                    float *out = partial + (chunk_row + chunk) * 1024 + lane;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        out[j * 32] = v[j];
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (Pair)
                        mbarrier_arrive_cluster(cluster_address(tempty0 + 8 * buffer, 0));
                    else
                        mbarrier_arrive(tempty0 + 8 * buffer);
                }
                if (p.reduce_later) { // many splits: one SM adding them all would take longer than the products
                    if (++buffer == 2) {
                        buffer = 0;
                        buffer_phase ^= 1;
                    }
                    continue;
                }
                // Ticket: the split that arrives last reduces the tile in split order.
                __threadfence();
                asm volatile("bar.sync 1, 512;" ::: "memory");
                if (threadIdx.x == 64) {
                    unsigned ticket = atomicAdd(&p.tickets[t * Unit + rank], 1u);
                    int last = ticket == unsigned(p.splits - 1);
                    if (last)
                        p.tickets[t * Unit + rank] = 0; // ready for the next launch
                    last_split_flag[0] = last;
                }
                asm volatile("bar.sync 1, 512;" ::: "memory");
                if (last_split_flag[0]) {
                    __threadfence();
                    for (int chunk = share; chunk < p.bn / 32; chunk += Shares) {
                        const int column = nt * p.bn + chunk * 32;
                        if (column >= p.n)
                            break;
                        // L2 only (__ldcg): the partials were written by other SMs.
                        const float *src = p.workspace + ((long long)z * padded_m * padded_n) +
                                           (chunk_row + chunk) * 1024 + lane;
                        float sum[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            sum[j] = 0.f;
                        for (int sp = 0; sp < p.splits; ++sp) {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                sum[j] += __ldcg(src + sp * split_stride + j * 32);
                        }
                        if (row < p.m) {
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                if (column + g * 8 >= p.n)
                                    break;
                                float group[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    group[j] = sum[g * 8 + j];
                                store_group(p, group, row, column + g * 8, z);
                            }
                        }
                    }
                }
                asm volatile("bar.sync 1, 512;" ::: "memory"); // last_split_flag is reused next tile
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
    if constexpr (Pair) {
        cluster_sync_all(); // neither CTA's tensor or shared memory is released while the other may touch it
        if (warp == 1)
            tmem_dealloc_pair(tmem_base, TmemColumns);
    } else {
        if (warp == 1)
            tmem_dealloc(tmem_base, TmemColumns);
    }
}

// C = the K splits' partial tiles added in split order, for schedules with four or more splits: there the last
// arriver of a tile would pull every partial tile through one SM (1 MB per CTA at eight splits: 24 000 clocks
// at the SM's L2 read rate, as long as the products themselves); this kernel spreads the same additions, in the
// same order, over the whole GPU.  One block per 32 x 32 chunk of the padded output (a chunk is stored column
// by column, see the kernel above); rows go out whole through a padded shared-memory tile.
template <bool OutFp32>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(TcParams p, long long padded_m, long long padded_n) {
    __shared__ float tile[32][33];
    const long long chunks_per_row = padded_n / 32, chunks_per_matrix = (padded_m / 32) * chunks_per_row;
    const long long chunk = blockIdx.x % chunks_per_matrix;
    const int z = int(blockIdx.x / chunks_per_matrix);
    const long long split_stride = (long long)p.batch * padded_m * padded_n;
    const float *source = p.workspace + (long long)z * padded_m * padded_n + chunk * 1024;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int e = threadIdx.x + 256 * u; // column e / 32, row e % 32 of the chunk
        float sum = 0.f;
        for (int split = 0; split < p.splits; ++split)
            sum += __ldcg(source + split * split_stride + e);
        tile[e / 32][e % 32] = sum;
    }
    __syncthreads();
    const long long row = chunk / chunks_per_row * 32 + threadIdx.x / 8;
    const int column = int(chunk % chunks_per_row) * 32 + (threadIdx.x % 8) * 4;
    if (row >= p.m || column >= p.n)
        return;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        v[i] = tile[(threadIdx.x % 8) * 4 + i][threadIdx.x / 8];
    const long long index = z * p.c_batch + row * p.ldc + column;
    if (column + 4 <= p.n && p.wide) {
        if constexpr (OutFp32)
            *reinterpret_cast<float4 *>((float *)p.c + index) = make_float4(v[0], v[1], v[2], v[3]);
        else
            *reinterpret_cast<uint2 *>((bf16 *)p.c + index) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
    } else {
        for (int i = 0; i < 4 && column + i < p.n; ++i) {
            if constexpr (OutFp32)
                ((float *)p.c)[index + i] = v[i];
            else
                ((bf16 *)p.c)[index + i] = __float2bfloat16(v[i]);
        }
    }
}

// ---------------------------------------------------------------------------- host side ------
struct Schedule {
    int bn = 0, splits = 1, k_blocks_per_split = 0, pair = 0;
};

// Tile width, K splits and single CTA / CTA pair by a small cost model, in clocks per 64-deep K
// block: the MMA takes bn/2, the shared-memory operand reads (128+bn)/4; a tile adds a fixed drain
// cost and every split one pass over the FP32 partial tile.  CTA pairs (256-row tiles) are tried
// first: they halve the B bytes each SM stages per K block.
Schedule choose_schedule(const GemmArgs &g, int sms) {
    const bool b_mn = g.b_col != 1;
    const bool second_tensor = g.epilogue != Epilogue::Store; // K is split only for plain stores
    const bool whole_rows = g.epilogue == Epilogue::CrossEntropy; // a tile must hold complete rows
    const int m_tiles = (g.m + BM - 1) / BM, k_blocks = (g.k + BK - 1) / BK;
    Schedule best;
    long long best_time = 0;
    for (int unit : {2, 1}) {
        if (unit == 2 && (m_tiles < 2 || sms < 2))
            continue;
        const int slots = sms / unit;
        const long long m_units = (m_tiles + unit - 1) / unit;
        for (int bn : {256, 192, 128, 64}) {
            if (bn > 64 && bn - 64 >= g.n)
                continue; // a narrower tile already covers N
            if (whole_rows && bn != 256)
                continue;
            if (unit == 2 && (bn == 64 || (b_mn && bn == 192)))
                continue; // each CTA stages bn/2 rows of B: whole 64-row blocks when B is MN-major
            const long long tiles = m_units * ((g.n + bn - 1) / bn) * g.batch;
            // Clocks per K block and CTA: the MMA takes bn/2; a single CTA cannot keep its ring full
            // (measured ~65 % of that rate), a pair can.
            const int mma = bn / 2 > (128 + bn) / 4 ? bn / 2 : (128 + bn) / 4;
            const int block_cost = unit == 2 ? mma + 16 : mma * (k_blocks >= 64 ? 9 : 11) / 8 + 16;
            for (int splits : {1, 2, 3, 4, 6, 8, 12, 16}) {
                if (splits > 1 && (k_blocks / splits < 8 || tiles * splits > slots || second_tensor))
                    continue;
                const int per = (k_blocks + splits - 1) / splits;
                if (splits > 1 && (k_blocks + per - 1) / per != splits)
                    continue; // would leave an empty split
                const long long rounds = (tiles * splits + slots - 1) / slots;
                const long long time = rounds * ((long long)per * block_cost + bn + (splits > 1 ? splits * bn / 2 : 0));
                if (!best.bn || time < best_time)
                    best.bn = bn, best.splits = splits, best.k_blocks_per_split = per, best.pair = unit == 2,
                    best_time = time;
            }
        }
    }
    return best;
}

// Scratch a schedule needs: FP32 partial tiles and one ticket per output tile (none without a K split).
struct ScratchNeed {
    size_t partial_bytes = 0, tickets = 0;
};
ScratchNeed scratch_need(const GemmArgs &g, const Schedule &sc) {
    if (sc.splits <= 1)
        return {};
    const int unit = sc.pair ? 2 : 1;
    const int m_tiles = (g.m + BM - 1) / BM, padded_m_tiles = (m_tiles + unit - 1) / unit * unit;
    const int n_tiles = (g.n + sc.bn - 1) / sc.bn;
    return {size_t(sc.splits) * g.batch * padded_m_tiles * BM * n_tiles * sc.bn * sizeof(float),
            size_t(padded_m_tiles) * n_tiles * g.batch};
}

// Stand-alone calls (tg_ex_gemm) share one workspace per device, grown on demand.
std::mutex shared_workspace_mutex;
std::unordered_map<int, GemmWorkspace> shared_workspaces;

void grow(GemmWorkspace &w, const ScratchNeed &need, cudaStream_t s) {
    if (!w.error_word) {
        CHECK_CUDA(cudaMalloc(&w.error_word, sizeof(StepCounters)));
        CHECK_CUDA(cudaMemset(w.error_word, 0, sizeof(StepCounters)));
    }
    if (w.partial_bytes < need.partial_bytes) {
        CHECK_CUDA(cudaStreamSynchronize(s));
        if (w.partials)
            CHECK_CUDA(cudaFree(w.partials));
        w.partials = nullptr, w.partial_bytes = 0;
        CHECK_CUDA(cudaMalloc(&w.partials, need.partial_bytes));
        w.partial_bytes = need.partial_bytes;
        ++w.generation;
    }
    if (w.ticket_count < need.tickets) {
        CHECK_CUDA(cudaStreamSynchronize(s));
        if (w.tickets)
            CHECK_CUDA(cudaFree(w.tickets));
        w.tickets = nullptr, w.ticket_count = 0;
        CHECK_CUDA(cudaMalloc(&w.tickets, need.tickets * sizeof(unsigned)));
        CHECK_CUDA(cudaMemset(w.tickets, 0, need.tickets * sizeof(unsigned)));
        w.ticket_count = need.tickets;
        ++w.generation;
    }
}

// Builds the kernel parameters and tensor maps for `sc` and launches.  `partials` / `tickets` may be
// null when the schedule does not split K.
void launch_schedule(const GemmArgs &g, const Schedule &sc, int sms, float *partials, unsigned *tickets,
                     StepCounters *counters, cudaStream_t s) {
    TcParams p{};
    p.m = g.m, p.n = g.n, p.k = g.k, p.batch = g.batch;
    p.a_mn = g.a_col == 1 ? 0 : 1;
    p.b_mn = g.b_col == 1 ? 0 : 1;
    p.epilogue = int(g.epilogue), p.out_fp32 = g.out == Dtype::FP32;
    p.bn = sc.bn, p.splits = sc.splits, p.k_blocks_per_split = sc.k_blocks_per_split;
    p.reduce_later = sc.splits >= 4; // K is only split for plain stores
    const int64_t lda = p.a_mn ? g.a_col : g.a_row, ldb = p.b_mn ? g.b_col : g.b_row;
    const int unit = sc.pair ? 2 : 1;
    const int m_tiles = (g.m + BM - 1) / BM, padded_m_tiles = (m_tiles + unit - 1) / unit * unit;
    const int n_tiles = (g.n + p.bn - 1) / p.bn;
    const long long tiles = (long long)(padded_m_tiles / unit) * n_tiles * g.batch; // scheduling units
    const int bn_local = p.bn / unit;
    const int stage_bytes = StageABytes + bn_local * BK * 2;
    const int row_scratch = g.epilogue == Epilogue::CrossEntropy ? RowScratchBytes : 0;
    p.stages = (MaxShared - 1024 - ControlBytes - row_scratch) / stage_bytes;
    if (p.stages > MaxStages)
        p.stages = MaxStages;
    const int shared = p.stages * stage_bytes + ControlBytes + row_scratch + 1024;
    p.c = g.c, p.c2 = g.c2, p.r = g.r;
    p.ldc = g.ldc, p.ldr = g.ldr, p.c_batch = g.c_batch, p.r_batch = g.r_batch;
    p.alpha = g.alpha, p.beta = g.beta;
    p.counters = counters;
    p.workspace = partials, p.tickets = tickets;
    {
        const int per32 = p.out_fp32 ? 8 : 16; // elements per 32 bytes
        auto aligned32 = [&](const void *ptr, int64_t ld, int64_t batch_stride) {
            return !ptr || (reinterpret_cast<uintptr_t>(ptr) % 32 == 0 && ld % per32 == 0 && batch_stride % per32 == 0);
        };
        p.wide = g.epilogue == Epilogue::CrossEntropy
                     ? aligned32(g.c, g.ldc, 0)
                     : aligned32(g.c, g.ldc, g.c_batch) && aligned32(g.c2, g.ldc, g.c_batch) && aligned32(g.r, g.ldr, g.r_batch);
    }
    CUtensorMap map_a = p.a_mn ? make_map_bf16(g.a, g.m, g.k, g.batch, lda, g.a_batch, 64, BK)
                               : make_map_bf16(g.a, g.k, g.m, g.batch, lda, g.a_batch, BK, BM);
    CUtensorMap map_b = p.b_mn ? make_map_bf16(g.b, g.n, g.k, g.batch, ldb, g.b_batch, 64, BK)
                               : make_map_bf16(g.b, g.k, g.n, g.batch, ldb, g.b_batch, BK, bn_local);
    const long long work = tiles * p.splits;
    const int slots = sms / unit;
    const int grid = int(work < slots ? work : slots) * unit;
    auto launch = [&](auto kernel) {
        // The opt-in shared-memory size is an attribute of each instantiation on each device.
        static std::mutex guard;
        static std::unordered_map<const void *, unsigned long long> configured; // kernel -> device bit mask
        int device = 0;
        CHECK_CUDA(cudaGetDevice(&device));
        {
            std::lock_guard<std::mutex> lock(guard);
            unsigned long long &mask = configured[reinterpret_cast<const void *>(kernel)];
            if (!(mask >> (device & 63) & 1ull)) {
                CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MaxShared));
                mask |= 1ull << (device & 63);
            }
        }
        cudaLaunchConfig_t config{};
        config.gridDim = dim3(grid), config.blockDim = dim3(Threads);
        config.dynamicSmemBytes = shared, config.stream = s;
        cudaLaunchAttribute attributes[2]{};
        attributes[0].id = cudaLaunchAttributeClusterDimension;
        attributes[0].val.clusterDim.x = unit, attributes[0].val.clusterDim.y = 1, attributes[0].val.clusterDim.z = 1;
        // The kernel's set-up (barriers, tensor memory, descriptors) overlaps the tail of the kernel before it.
        attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[1].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attributes, config.numAttrs = 2;
        CHECK_CUDA(cudaLaunchKernelEx(&config, kernel, map_a, map_b, p));
    };
    auto launch_kind = [&](auto pair_tag) {
        constexpr bool P = decltype(pair_tag)::value;
        if (p.out_fp32) {
            if (g.epilogue == Epilogue::Axpby)
                launch(gemm_tc_kernel<int(Epilogue::Axpby), true, P>);
            else
                launch(gemm_tc_kernel<int(Epilogue::Store), true, P>);
        } else {
            switch (g.epilogue) {
            case Epilogue::Store: launch(gemm_tc_kernel<int(Epilogue::Store), false, P>); break;
            case Epilogue::Residual: launch(gemm_tc_kernel<int(Epilogue::Residual), false, P>); break;
            case Epilogue::GeluDual: launch(gemm_tc_kernel<int(Epilogue::GeluDual), false, P>); break;
            case Epilogue::GeluGrad: launch(gemm_tc_kernel<int(Epilogue::GeluGrad), false, P>); break;
            case Epilogue::Axpby: launch(gemm_tc_kernel<int(Epilogue::Axpby), false, P>); break;
            case Epilogue::CrossEntropy: launch(gemm_tc_kernel<int(Epilogue::CrossEntropy), false, P>); break;
            }
        }
    };
    if (sc.pair)
        launch_kind(std::true_type{});
    else
        launch_kind(std::false_type{});
    CHECK_CUDA(cudaGetLastError());
    if (p.reduce_later) {
        const long long padded_m = (long long)padded_m_tiles * BM, padded_n = (long long)n_tiles * p.bn;
        const unsigned blocks = unsigned(padded_m / 32 * (padded_n / 32) * g.batch);
        if (p.out_fp32)
            splitk_reduce_kernel<true><<<blocks, 256, 0, s>>>(p, padded_m, padded_n);
        else
            splitk_reduce_kernel<false><<<blocks, 256, 0, s>>>(p, padded_m, padded_n);
        CHECK_CUDA(cudaGetLastError());
    }
}
} // namespace

int gemm_tc_shared_bytes() { return MaxShared; }

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
    const bool loss = g.epilogue == Epilogue::CrossEntropy; // R holds one byte per row there
    if (loss && (g.n != 256 || g.batch != 1 || g.out != Dtype::BF16 || !g.r || !g.c2 || g.a_col != 1 || g.b_col != 1))
        return false;
    if (reinterpret_cast<uintptr_t>(g.a) % 16 || reinterpret_cast<uintptr_t>(g.b) % 16 ||
        reinterpret_cast<uintptr_t>(g.c) % 16 || (!loss && reinterpret_cast<uintptr_t>(g.r) % 16) ||
        reinterpret_cast<uintptr_t>(g.c2) % 16)
        return false;
    if (g.a_batch % 8 || g.b_batch % 8 || g.c_batch % 8 || g.r_batch % 8)
        return false;
    if (g.out == Dtype::FP32 && !(g.epilogue == Epilogue::Store || g.epilogue == Epilogue::Axpby))
        return false;
    return true;
}

namespace {
void launch_with(const GemmArgs &g, const Schedule &sc, int sms, StepCounters *counters, cudaStream_t s,
                 GemmWorkspace *workspace);
}

void release_gemm_workspace(GemmWorkspace &w) {
    if (w.partials)
        cudaFree(w.partials);
    if (w.tickets)
        cudaFree(w.tickets);
    if (w.error_word)
        cudaFree(w.error_word);
    w = GemmWorkspace{};
}

// `workspace`: the caller's own split-K scratch (an Engine's: grown here, outside stream capture,
// when a schedule needs more); nullptr: the per-device workspace shared by the stand-alone calls,
// whose device-side give-ups are reported by gemm_tc_take_device_error().
int launch_gemm_tc(const GemmArgs &g, int sms, StepCounters *counters, cudaStream_t s, GemmWorkspace *workspace) {
    const Schedule sc = choose_schedule(g, sms);
    launch_with(g, sc, sms, counters, s, workspace);
    return sc.splits >= 4 ? 2 : 1; // the product kernel, and the kernel that adds many splits' partial tiles
}

namespace {
void launch_with(const GemmArgs &g, const Schedule &sc, int sms, StepCounters *counters, cudaStream_t s,
                 GemmWorkspace *workspace) {
    const ScratchNeed need = scratch_need(g, sc);
    if (workspace) {
        if (need.partial_bytes > workspace->partial_bytes || need.tickets > workspace->ticket_count || !workspace->error_word)
            grow(*workspace, need, s);
        launch_schedule(g, sc, sms, workspace->partials, workspace->tickets, counters, s);
        return;
    }
    int device = 0;
    CHECK_CUDA(cudaGetDevice(&device));
    std::lock_guard<std::mutex> lock(shared_workspace_mutex);
    GemmWorkspace &w = shared_workspaces[device];
    grow(w, need, s);
    launch_schedule(g, sc, sms, w.partials, w.tickets, counters ? counters : w.error_word, s);
}
} // namespace

// ------------------------------------------------------------------------------------------
// Weight gradient without any allocation.  Some hosts may not call cudaMalloc at the moment they
// need a gradient: a serving or training process that has handed the whole device to its own
// memory pool, a caller inside a region where the allocator's implicit device synchronisation is
// not acceptable, or one whose memory budget was fixed when the process started.  For them the
// split-K scratch (FP32 partial tiles, the per-tile tickets and a device error word) lives in the
// array below, which every GPU that loads this library holds until the process exits.
//
// In host code `static_scratch` is only a stand-in for the symbol: its device address comes from
// cudaGetSymbolAddress, fetched once per device with that device current, on the first call for
// that device (so the first call should happen before any stream capture).  All calls share the
// array and it keeps the previous call's contents: the tickets are cleared on the stream before
// every launch, the partial tiles are fully overwritten before they are read.  Two calls that
// overlap on the GPU (different streams, or different threads) race on it.
//
// The schedule (tile width, K splits, CTA pair) and the kernel are exactly those tg_ex_gemm uses
// for the same shape, so the results are bit-identical to it.
// ------------------------------------------------------------------------------------------
namespace {
constexpr size_t StaticPartialBytes = size_t(16) << 20; // 16 MiB of FP32 partial tiles
constexpr int StaticTickets = 1024;                      // output tiles
constexpr size_t StaticErrorOffset = StaticPartialBytes + StaticTickets * sizeof(unsigned);
static __device__ __align__(256) unsigned char static_scratch[StaticErrorOffset + 256];
void *static_scratch_address[64] = {}; // per device, filled on first use
} // namespace

size_t gemm_tc_static_scratch_bytes() { return StaticPartialBytes; }

void launch_weight_gradient_static(const void *dy, const void *x, float *dw, int out, int in, int tokens,
                                   int sms, cudaStream_t s) {
    // dW[out, in] = dy[tokens, out]^T x[tokens, in]: both operands MN-major, K = tokens.
    GemmArgs g;
    g.in = Dtype::BF16, g.out = Dtype::FP32;
    g.a = dy, g.a_row = 1, g.a_col = out, g.b = x, g.b_row = 1, g.b_col = in;
    g.c = dw, g.ldc = in, g.m = out, g.n = in, g.k = tokens;
    if (!gemm_tc_supported(g))
        throw std::runtime_error("weight gradient: sizes must be multiples of 8 (out, in), at least 64, and the "
                                 "pointers 16-byte aligned");
    int device = 0;
    CHECK_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64)
        throw std::runtime_error("weight gradient: device index out of range");
    if (!static_scratch_address[device]) { // set-up, once per device, with that device current
        void *address = nullptr;
        CHECK_CUDA(cudaGetSymbolAddress(&address, static_scratch));
        CHECK_CUDA(cudaMemsetAsync(static_cast<unsigned char *>(address) + StaticErrorOffset, 0, 256, s));
        static_scratch_address[device] = address;
    }
    const Schedule sc = choose_schedule(g, sms);
    const ScratchNeed need = scratch_need(g, sc);
    if (need.partial_bytes > StaticPartialBytes || need.tickets > size_t(StaticTickets))
        throw std::runtime_error("weight gradient: this shape needs " + std::to_string(need.partial_bytes) +
                                 " bytes of scratch in " + std::to_string(need.tickets) +
                                 " tiles; the built-in array holds " + std::to_string(StaticPartialBytes) +
                                 " bytes and " + std::to_string(StaticTickets) + " tiles (use tg_ex_gemm, which allocates)");
    unsigned char *scratch = static_cast<unsigned char *>(static_scratch_address[device]);
    unsigned *tickets = reinterpret_cast<unsigned *>(scratch + StaticPartialBytes);
    CHECK_CUDA(cudaMemsetAsync(tickets, 0, StaticTickets * sizeof(unsigned), s)); // must start at zero
    launch_schedule(g, sc, sms, reinterpret_cast<float *>(scratch), tickets,
                    reinterpret_cast<StepCounters *>(scratch + StaticErrorOffset), s);
}

// First device-side give-up code recorded by the stand-alone GEMM calls (tg_ex_gemm,
// tg_ex_weight_gradient_static) on the current device since the last query; 0 when none.
// Synchronises `s`; allocates nothing.
int gemm_tc_take_device_error(cudaStream_t s) {
    int device = 0;
    CHECK_CUDA(cudaGetDevice(&device));
    CHECK_CUDA(cudaStreamSynchronize(s));
    StepCounters *words[2] = {nullptr, nullptr};
    {
        std::lock_guard<std::mutex> lock(shared_workspace_mutex);
        auto found = shared_workspaces.find(device);
        if (found != shared_workspaces.end())
            words[0] = found->second.error_word;
    }
    if (device >= 0 && device < 64 && static_scratch_address[device])
        words[1] = reinterpret_cast<StepCounters *>(static_cast<unsigned char *>(static_scratch_address[device]) +
                                                    StaticErrorOffset);
    int code = 0;
    for (StepCounters *word : words) {
        if (!word)
            continue;
        StepCounters host{};
        CHECK_CUDA(cudaMemcpy(&host, word, sizeof(host), cudaMemcpyDeviceToHost));
        if (host.error) {
            if (!code)
                code = host.error;
            CHECK_CUDA(cudaMemset(word, 0, sizeof(StepCounters)));
        }
    }
    return code;
}
