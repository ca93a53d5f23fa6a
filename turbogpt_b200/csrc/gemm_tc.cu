// BF16 GEMM on the 5th-generation tensor cores: C[m,n] = sum_k A[m,k] * B[n,k], FP32
// accumulation in tensor memory.  Replaces the reference's warp-level mma.sync products
// (cuda/mma.cuh:69-108, cuda/ops.cuh:30-55,83-117) for every projection, input-gradient and
// weight-gradient GEMM of the step.
//
// One persistent CTA per SM walks output tiles of 128 x BN (BN = 64..256).  Warp 0 streams
// operand slices of 64 K-elements with TMA into a ring of 128-byte-swizzled shared-memory
// stages; warp 1 issues tcgen05.mma (one thread) into one of two TMEM accumulators; warps 2-5
// drain the other accumulator, so the epilogue of tile i overlaps the main loop of tile i+1.
// Either operand may be K-major (row = 64 contiguous K elements) or MN-major (row = 64
// contiguous M/N elements for one K index), which covers y = x W^T, dx = dy W and dW = dy^T x on
// row-major tensors without transposes.
//
// Epilogue: each warp owns 32 rows.  Per 128-byte-wide chunk of its rows it reads the accumulator
// (tcgen05.ld), optionally combines it with a tile of a second tensor fetched by TMA (residual,
// pre-activation, or the Newton-Schulz operand), writes the result into a swizzled staging slot
// and hands the slot to a TMA store: global reads and writes are whole 128-byte lines and the
// tensor's edges are clipped by the TMA unit.
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
constexpr int BM = 128, BK = 64, MaxBN = 256, MaxStages = 8;
constexpr int StageABytes = BM * BK * 2;
constexpr int EpilogueWarps = 16;
constexpr int Threads = 64 + 32 * EpilogueWarps; // warp 0: TMA, warp 1: MMA, then the epilogue warps
constexpr int SlotBytes = 32 * 128; // staging slot: 32 rows x 128 bytes
constexpr int ControlBytes = 512;   // barriers, TMEM slot, flags
constexpr int MaxShared = 232448 - 1024; // 227 KB less the runtime's own reservation
constexpr int TmemColumns = 512;

struct TcParams {
    int m, n, k, batch;
    int bn;                 // tile width
    int a_mn, b_mn;         // operand majorness
    int splits, k_blocks_per_split;
    int epilogue, out_fp32;
    int stages, slots;      // pipeline depth; (slots unused)
    int wide;               // C, C2 and R rows are 32-byte aligned: 256-bit epilogue accesses
    void *c, *c2;
    const void *r;
    long long ldc, ldr, c_batch, r_batch;
    float alpha, beta;
    float *workspace;       // [splits][batch][m_tiles*BM][n_tiles*bn] FP32 partial tiles
    unsigned *tickets;      // one per output tile, zero between launches
    StepCounters *counters;
};

// erf by Abramowitz & Stegun 7.1.26 (|error| < 1.5e-7); the same exponential serves the
// Gaussian term of the derivative.  z = x / sqrt(2).
__device__ __forceinline__ void gelu_terms(float x, float &cdf, float &density) {
    const float z = fabsf(x) * 0.7071067811865475f;
    const float t = __fdividef(1.f, fmaf(0.3275911f, z, 1.f));
    const float e = __expf(-z * z);
    float poly = fmaf(t, 1.061405429f, -1.453152027f);
    poly = fmaf(t, poly, 1.421413741f);
    poly = fmaf(t, poly, -0.284496736f);
    poly = fmaf(t, poly, 0.254829592f);
    const float tail = 0.5f * poly * t * e;       // 0.5 * erfc(|z|)
    cdf = x >= 0.f ? 1.f - tail : tail;           // 0.5 * (1 + erf(z))
    density = 0.3989422804014327f * e;            // exp(-x^2/2) / sqrt(2 pi)
}
__device__ __forceinline__ float fast_gelu(float x) {
    float cdf, density;
    gelu_terms(x, cdf, density);
    return x * cdf;
}
__device__ __forceinline__ float fast_gelu_derivative(float x) {
    float cdf, density;
    gelu_terms(x, cdf, density);
    return fmaf(x, density, cdf);
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

__device__ __forceinline__ uint4 load_shared16(uint32_t address) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address));
    return v;
}
__device__ __forceinline__ void store_shared16(uint32_t address, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
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
__device__ __forceinline__ void unpack8(uint4 u, float (&v)[8]) {
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <int Kind, bool OutFp32>
__global__ void __launch_bounds__(Threads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_c2,
               const __grid_constant__ CUtensorMap map_r, TcParams p) {
    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (smem_address(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - smem_address(raw_shared));
    const int stage_bytes = StageABytes + p.bn * BK * 2;
    uint64_t *barriers = reinterpret_cast<uint64_t *>(aligned + p.stages * stage_bytes + 4 * p.slots * SlotBytes);
    // barrier slots: full[8], empty[8], tmem_full[2], tmem_empty[2], r_full[4 warps][4 slots]
    const uint32_t full0 = smem_address(barriers), empty0 = full0 + 8 * MaxStages, tfull0 = empty0 + 8 * MaxStages,
                   tempty0 = tfull0 + 16, rfull0 = tempty0 + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(barriers + 2 * MaxStages + 4 + 16);
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
            mbarrier_init(tempty0 + 8 * b, EpilogueWarps);
        }
        for (int i = 0; i < 16; ++i)
            mbarrier_init(rfull0 + 8 * i, 1);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_map(&map_a);
        prefetch_map(&map_b);
        prefetch_map(&map_c);
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
    const uint32_t stage_tx = stage_bytes;

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
                    const uint32_t bar = full0 + 8 * stage, sa = base + stage * stage_bytes, sb = sa + StageABytes;
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
                    const uint32_t sa = base + stage * stage_bytes, sb = sa + StageABytes;
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks) {
                        uint64_t da = smem_descriptor(sa + ks * a_step, a_lbo, 1024);
                        uint64_t db = smem_descriptor(sb + ks * b_step, b_lbo, 1024);
                        tcgen05_mma_bf16(accumulator, da, db, instruction, (kb > kb0 || ks > 0) ? 1u : 0u);
                    }
                    tcgen05_commit(empty0 + 8 * stage); // frees the stage once these MMAs have read it
                    if (++stage == p.stages) {
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
        // ---------------- epilogue: 16 warps; warps q, q+4, q+8, q+12 share TMEM lanes 32q..32q+31 and
        // take every fourth 32-column chunk.  Four warps per scheduler hide one another's TMEM,
        // ALU, SFU and global-load latencies (the epilogue math is a dependent chain per element).
        constexpr int Shares = EpilogueWarps / 4;
        const int quarter = warp % 4, share = (warp - 2) / 4;
        constexpr bool has_r = Kind == int(Epilogue::Residual) || Kind == int(Epilogue::GeluGrad) ||
                               Kind == int(Epilogue::Axpby);
        int buffer = 0;
        uint32_t buffer_phase = 0;
        for (long long w = blockIdx.x; w < work_items; w += gridDim.x) {
            const int split = int(w % p.splits);
            long long t = w / p.splits;
            const int nt = int(t % n_tiles), mt = int(t / n_tiles % m_tiles), z = int(t / n_tiles / m_tiles);
            bool ready = mbarrier_wait(tfull0 + 8 * buffer, buffer_phase, abort_flag, p.counters, 104);
            if (p.splits > 1) // the eight warps meet at named barriers below: leave together or not at all
                ready = epilogue_all(ready);
            if (!ready)
                break;
            tcgen05_fence_after();
            const long long row = (long long)mt * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buffer * MaxBN;
            const int tile_columns = min(p.bn, p.n - nt * p.bn);
            const int chunks = (tile_columns + 31) / 32;
            if (p.splits == 1) {
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
                                for (int j = 0; j < 16; ++j)
                                    v[j] = rounded<bf16>(v[j]);
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    activated[j] = pack_bf16(fast_gelu(v[2 * j]), fast_gelu(v[2 * j + 1]));
                                store_global32((char *)p.c2 + (c_row + column) * 2 + g * 32, activated, whole,
                                               column + g * 16 + 8 < p.n);
                            } else if constexpr (Kind == int(Epilogue::GeluGrad)) {
#pragma unroll
                                for (int j = 0; j < 16; ++j)
                                    v[j] = rounded<bf16>(v[j]) * fast_gelu_derivative(r[j]);
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
                if (lane == 0)
                    mbarrier_arrive(tempty0 + 8 * buffer);
            } else {
                // Partial tile to the workspace (padded to whole tiles, so no bounds checks).
                const long long padded_m = (long long)m_tiles * BM, padded_n = (long long)n_tiles * p.bn;
                float *partial = p.workspace + ((long long)split * p.batch + z) * padded_m * padded_n;
                for (int chunk = share; chunk < p.bn / 32; chunk += Shares) {
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
                asm volatile("bar.sync 1, 512;" ::: "memory");
                if (threadIdx.x == 64) {
                    unsigned ticket = atomicAdd(&p.tickets[t], 1u);
                    int last = ticket == unsigned(p.splits - 1);
                    if (last)
                        p.tickets[t] = 0; // ready for the next launch
                    last_split_flag[0] = last;
                }
                asm volatile("bar.sync 1, 512;" ::: "memory");
                if (last_split_flag[0]) {
                    __threadfence();
                    if (row < p.m) {
                        for (int col = share * 32; col < p.bn; col += 32 * Shares) {
                            for (int sub = 0; sub < 32; sub += 8) {
                                const int c = nt * p.bn + col + sub;
                                if (c >= p.n)
                                    break;
                                float sum[8] = {};
                                for (int s = 0; s < p.splits; ++s) {
                                    // L2 only: the partials were written by other SMs.
                                    const float4 *src = reinterpret_cast<const float4 *>(
                                        p.workspace + ((long long)s * p.batch + z) * padded_m * padded_n +
                                        row * padded_n + c);
                                    float4 lo = __ldcg(src), hi = __ldcg(src + 1);
                                    sum[0] += lo.x, sum[1] += lo.y, sum[2] += lo.z, sum[3] += lo.w;
                                    sum[4] += hi.x, sum[5] += hi.y, sum[6] += hi.z, sum[7] += hi.w;
                                }
                                store_group(p, sum, row, c, z);
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
    if (reinterpret_cast<uintptr_t>(g.a) % 16 || reinterpret_cast<uintptr_t>(g.b) % 16 ||
        reinterpret_cast<uintptr_t>(g.c) % 16 || reinterpret_cast<uintptr_t>(g.r) % 16 ||
        reinterpret_cast<uintptr_t>(g.c2) % 16)
        return false;
    if (g.a_batch % 8 || g.b_batch % 8 || g.c_batch % 8 || g.r_batch % 8)
        return false;
    if (g.out == Dtype::FP32 && !(g.epilogue == Epilogue::Store || g.epilogue == Epilogue::Axpby))
        return false;
    return true;
}

void launch_gemm_tc(const GemmArgs &g, int sms, StepCounters *counters, cudaStream_t s) {
    TcParams p{};
    p.m = g.m, p.n = g.n, p.k = g.k, p.batch = g.batch;
    p.a_mn = g.a_col == 1 ? 0 : 1;
    p.b_mn = g.b_col == 1 ? 0 : 1;
    p.epilogue = int(g.epilogue), p.out_fp32 = g.out == Dtype::FP32;
    const bool second_tensor = g.epilogue != Epilogue::Store;
    p.slots = 0;
    const int64_t lda = p.a_mn ? g.a_col : g.a_row, ldb = p.b_mn ? g.b_col : g.b_row;
    const int m_tiles = (g.m + BM - 1) / BM, k_blocks = (g.k + BK - 1) / BK;
    // Tile width and K splits by a small cost model, in clocks per 64-deep K block: the MMA
    // takes bn/2, the shared-memory operand reads (128+bn)/4; a tile adds a fixed drain cost and
    // every split one pass over the FP32 partial tile.  Four staging slots leave room for 192 columns.
    long long best_time = 0;
    p.bn = 0;
    for (int bn : {256, 192, 128, 64}) {
        if (bn > 64 && bn - 64 >= g.n)
            continue; // a narrower tile already covers N
        const long long tiles = (long long)m_tiles * ((g.n + bn - 1) / bn) * g.batch;
        const int block_cost = bn / 2 > (128 + bn) / 4 ? bn / 2 : (128 + bn) / 4;
        for (int splits : {1, 2, 3, 4, 6, 8, 12, 16}) {
            if (splits > 1 && (k_blocks / splits < 8 || tiles * splits > sms || second_tensor))
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
    const int stage_bytes = StageABytes + p.bn * BK * 2;
    const int staging = 4 * p.slots * SlotBytes;
    p.stages = (MaxShared - 1024 - ControlBytes - staging) / stage_bytes;
    if (p.stages > MaxStages)
        p.stages = MaxStages;
    const int shared = p.stages * stage_bytes + staging + ControlBytes + 1024;
    p.c = g.c, p.c2 = g.c2, p.r = g.r;
    p.ldc = g.ldc, p.ldr = g.ldr, p.c_batch = g.c_batch, p.r_batch = g.r_batch;
    p.alpha = g.alpha, p.beta = g.beta;
    p.counters = counters;
    {
        const int per32 = p.out_fp32 ? 8 : 16; // elements per 32 bytes
        auto aligned32 = [&](const void *ptr, int64_t ld, int64_t batch_stride) {
            return !ptr || (reinterpret_cast<uintptr_t>(ptr) % 32 == 0 && ld % per32 == 0 && batch_stride % per32 == 0);
        };
        p.wide = aligned32(g.c, g.ldc, g.c_batch) && aligned32(g.c2, g.ldc, g.c_batch) &&
                 aligned32(g.r, g.ldr, g.r_batch);
    }
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
    const int element = p.out_fp32 ? 4 : 2;
    CUtensorMap map_c = make_map(g.c, element, g.n, g.m, g.batch, g.ldc, g.c_batch, 128 / element, 32);
    CUtensorMap map_c2 = g.c2 ? make_map(g.c2, element, g.n, g.m, g.batch, g.ldc, g.c_batch, 128 / element, 32) : map_c;
    CUtensorMap map_r = g.r ? make_map(g.r, element, g.n, g.m, g.batch, g.ldr, g.r_batch, 128 / element, 32) : map_c;
    long long work = tiles * p.splits;
    int grid = int(work < sms ? work : sms);
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
        kernel<<<grid, Threads, shared, s>>>(map_a, map_b, map_c, map_c2, map_r, p);
    };
    if (p.out_fp32) {
        if (g.epilogue == Epilogue::Axpby)
            launch(gemm_tc_kernel<int(Epilogue::Axpby), true>);
        else
            launch(gemm_tc_kernel<int(Epilogue::Store), true>);
    } else {
        switch (g.epilogue) {
        case Epilogue::Store: launch(gemm_tc_kernel<int(Epilogue::Store), false>); break;
        case Epilogue::Residual: launch(gemm_tc_kernel<int(Epilogue::Residual), false>); break;
        case Epilogue::GeluDual: launch(gemm_tc_kernel<int(Epilogue::GeluDual), false>); break;
        case Epilogue::GeluGrad: launch(gemm_tc_kernel<int(Epilogue::GeluGrad), false>); break;
        case Epilogue::Axpby: launch(gemm_tc_kernel<int(Epilogue::Axpby), false>); break;
        }
    }
    CHECK_CUDA(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------
// Weight gradient without any allocation.  Some hosts may not call cudaMalloc at the moment they
// need a gradient: a serving or training process that has handed the whole device to its own
// memory pool, a caller inside a region where the allocator's implicit device synchronisation is
// not acceptable, or one whose memory budget was fixed when the process started.  For them the
// split-K scratch (FP32 partial tiles and the per-tile tickets) lives in the array below, which
// every GPU that loads this library holds until the process exits.
//
// In host code `static_scratch` is only a stand-in for the symbol: its device address comes from
// cudaGetSymbolAddress, fetched once per device with that device current, on the first call for
// that device (so the first call should happen before any stream capture).  All calls share the
// array and it keeps the previous call's contents: the tickets are cleared on the stream before
// every launch, the partial tiles are fully overwritten before they are read.  Two calls that
// overlap on the GPU (different streams, or different threads) race on it.
// ------------------------------------------------------------------------------------------
namespace {
constexpr size_t StaticPartialBytes = size_t(16) << 20; // 16 MiB of FP32 partial tiles
constexpr int StaticTickets = 1024;                      // output tiles
static __device__ __align__(256) unsigned char static_scratch[StaticPartialBytes + StaticTickets * sizeof(unsigned)];
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
    auto kernel = gemm_tc_kernel<int(Epilogue::Store), true>;
    if (!static_scratch_address[device]) { // set-up, once per device, with that device current
        void *address = nullptr;
        CHECK_CUDA(cudaGetSymbolAddress(&address, static_scratch));
        CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MaxShared));
        static_scratch_address[device] = address;
    }
    TcParams p{};
    p.m = g.m, p.n = g.n, p.k = g.k, p.batch = 1;
    p.a_mn = 1, p.b_mn = 1, p.epilogue = int(Epilogue::Store), p.out_fp32 = 1;
    const int m_tiles = (g.m + BM - 1) / BM, k_blocks = (g.k + BK - 1) / BK;
    long long best_time = 0;
    for (int bn : {256, 192, 128, 64}) { // same cost model as launch_gemm_tc
        if (bn > 64 && bn - 64 >= g.n)
            continue;
        const long long tiles = (long long)m_tiles * ((g.n + bn - 1) / bn);
        const int block_cost = bn / 2 > (128 + bn) / 4 ? bn / 2 : (128 + bn) / 4;
        for (int splits : {1, 2, 3, 4, 6, 8, 12, 16}) {
            if (splits > 1 && (k_blocks / splits < 8 || tiles * splits > sms))
                continue;
            const int per = (k_blocks + splits - 1) / splits;
            if (splits > 1 && (k_blocks + per - 1) / per != splits)
                continue;
            const long long rounds = (tiles * splits + sms - 1) / sms;
            const long long time = rounds * ((long long)per * (block_cost + 16) + bn + (splits > 1 ? splits * bn / 2 : 0));
            if (!p.bn || time < best_time)
                p.bn = bn, p.splits = splits, p.k_blocks_per_split = per, best_time = time;
        }
    }
    const int n_tiles = (g.n + p.bn - 1) / p.bn;
    const long long tiles = (long long)m_tiles * n_tiles;
    const size_t needed = p.splits > 1 ? size_t(p.splits) * m_tiles * BM * n_tiles * p.bn * sizeof(float) : 0;
    if (needed > StaticPartialBytes || (p.splits > 1 && tiles > StaticTickets))
        throw std::runtime_error("weight gradient: this shape needs " + std::to_string(needed) + " bytes of scratch in " +
                                 std::to_string(tiles) + " tiles; the built-in array holds " +
                                 std::to_string(StaticPartialBytes) + " bytes and " + std::to_string(StaticTickets) +
                                 " tiles (use tg_ex_gemm, which allocates)");
    const int stage_bytes = StageABytes + p.bn * BK * 2;
    p.stages = (MaxShared - 1024 - ControlBytes) / stage_bytes;
    if (p.stages > MaxStages)
        p.stages = MaxStages;
    const int shared = p.stages * stage_bytes + ControlBytes + 1024;
    p.c = g.c, p.ldc = g.ldc, p.alpha = 1.f, p.beta = 0.f;
    p.wide = reinterpret_cast<uintptr_t>(g.c) % 32 == 0 && g.ldc % 8 == 0;
    unsigned char *scratch = static_cast<unsigned char *>(static_scratch_address[device]);
    p.workspace = reinterpret_cast<float *>(scratch);
    p.tickets = reinterpret_cast<unsigned *>(scratch + StaticPartialBytes);
    CHECK_CUDA(cudaMemsetAsync(p.tickets, 0, StaticTickets * sizeof(unsigned), s)); // must start at zero
    CUtensorMap map_a = make_map_bf16(g.a, g.m, g.k, 1, g.a_col, 0, 64, BK);
    CUtensorMap map_b = make_map_bf16(g.b, g.n, g.k, 1, g.b_col, 0, 64, BK);
    CUtensorMap map_c = make_map(g.c, 4, g.n, g.m, 1, g.ldc, 0, 32, 32);
    const long long work = tiles * p.splits;
    kernel<<<int(work < sms ? work : sms), Threads, shared, s>>>(map_a, map_b, map_c, map_c, map_c, p);
    CHECK_CUDA(cudaGetLastError());
}
