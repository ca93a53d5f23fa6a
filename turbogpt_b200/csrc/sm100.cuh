// sm_100a primitives in inline PTX: mbarrier, TMA tile loads, tcgen05 (TMEM allocation, MMA,
// commit, TMEM loads), shared-memory and instruction descriptors, and host-side tensor maps.
// Every wait is bounded: a wait that gives up records a code in StepCounters::error and makes
// the kernel drain and return instead of hanging the GPU.
#pragma once
#include "common.h"
#include "kernels.cuh"
#include <cstdlib>
#include <cuda.h>

namespace sm100 {

// ------------------------------------------------------------------ host: tensor maps -------
// cuTensorMapEncodeTiled is fetched through the runtime so the library has no link-time
// dependency on libcuda.
using TensorMapEncoder = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                      const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                      CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                      CUtensorMapFloatOOBfill);
inline TensorMapEncoder tensor_map_encoder() {
    static TensorMapEncoder fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult status;
        CHECK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &status));
        if (!p || status != cudaDriverEntryPointSuccess)
            throw std::runtime_error("cuTensorMapEncodeTiled is not available in this driver");
        return reinterpret_cast<TensorMapEncoder>(p);
    }();
    return fn;
}
// BF16 tensor [batch][outer][inner] with `inner` contiguous, `ld` elements between outer rows and
// `batch_stride` elements between batches; box [1][box_outer][box_inner]; 128-byte swizzle.
// Out-of-range box parts are filled with zeros.
// `element` is 2 (BF16) or 4 (FP32) bytes; the box is always 128 bytes wide.
inline CUtensorMap make_map(const void *base, int element, uint64_t inner, uint64_t outer, uint64_t batch,
                            uint64_t ld, uint64_t batch_stride, uint32_t box_inner, uint32_t box_outer) {
    if (reinterpret_cast<uintptr_t>(base) % 16 || (ld * element) % 16 || (batch_stride * element) % 16 ||
        box_inner * element != 128 || box_outer > 256)
        throw std::runtime_error("tensor map: operand is not 16-byte aligned or the box is out of range");
    CUtensorMap map;
    cuuint64_t dims[3] = {inner, outer, batch};
    cuuint64_t strides[2] = {ld * element, (batch > 1 ? batch_stride : ld * outer) * element};
    cuuint32_t box[3] = {box_inner, box_outer, 1};
    cuuint32_t element_strides[3] = {1, 1, 1};
    CUresult r = tensor_map_encoder()(
        &map, element == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
        const_cast<void *>(base), dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
    return map;
}
inline CUtensorMap make_map_bf16(const void *base, uint64_t inner, uint64_t outer, uint64_t batch, uint64_t ld,
                                 uint64_t batch_stride, uint32_t box_inner, uint32_t box_outer) {
    return make_map(base, 2, inner, outer, batch, ld, batch_stride, box_inner, box_outer);
}

#ifdef __CUDACC__
// ------------------------------------------------------------------ device ------------------
__device__ __forceinline__ uint32_t smem_address(const void *p) {
    return uint32_t(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ bool elect_one() {
    uint32_t is_elected;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(is_elected));
    return is_elected != 0;
}
__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may
// start (and run its prologue) once every CTA of the kernel before it in the stream has called
// grid_launch_dependents() or exited; grid_dependency_wait() then blocks until that kernel has
// completed and its writes are visible.  Both are no-ops for kernels launched the ordinary way.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void mbarrier_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_async_proxy() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbarrier_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarrier_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbarrier_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    // The third operand lets the hardware park the thread for up to that many nanoseconds while the
    // phase is incomplete (it is woken when the phase completes): fewer polls from idle warps.
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(bar), "r"(parity), "r"(100000u)
                 : "memory");
    return done != 0;
}
// Waits for the phase with the given parity.  Gives up after ~2 s of wall time or as soon as
// another role of this CTA has raised `*abort_flag`; then raises the flag, records `code` and
// returns false.  Callers leave their loops on false.
constexpr unsigned long long WaitLimitNs = 2000000000ull;
__device__ __forceinline__ bool mbarrier_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                              StepCounters *counters, int code,
                                              unsigned long long limit_ns = WaitLimitNs) {
    if (mbarrier_try_wait(bar, parity))
        return true;
    const unsigned long long start = global_timer();
    // the clock is read every 256 polls (a poll may park the thread for up to 0.1 ms); short limits read it every poll
    const unsigned stride_mask = limit_ns < 100000000ull ? 0u : 0xffu;
    for (unsigned spins = 1;; ++spins) {
        if (mbarrier_try_wait(bar, parity))
            return true;
        if ((spins & stride_mask) == 0) {
            if (*abort_flag)
                return false;
            if (global_timer() - start > limit_ns) {
                *abort_flag = 1;
                if (counters)
                    atomicCAS(&counters->error, 0, code);
                return false;
            }
        }
    }
}

// 3-D tile load (inner, outer, batch coordinates) completing on an mbarrier.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z,
                                            uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ uint4 load_shared16(uint32_t address) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address) : "memory");
    return v;
}
__device__ __forceinline__ void store_shared16(uint32_t address, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// A warp's 32 rows x 32 BF16 columns (lane = row, `packed` = the lane's 64 bytes) to global memory through 2 KB of
// shared memory owned by the warp, so that one store instruction covers eight 64-byte row pieces.  Storing with
// lane = row makes every instruction touch 32 different lines, which was measured to hold up the SM's whole
// load/store path (the shared-memory traffic of the other warps included).  Rows at or after `valid_rows` are
// not written.  The 16-byte pieces of a row sit at piece ^ (row / 2 % 4): no bank conflicts either way.
__device__ __forceinline__ void store_rows_through_shared(uint32_t staging, const uint32_t (&packed)[16], void *first_row,
                                                          int64_t row_bytes, int valid_rows, int lane) {
#pragma unroll
    for (int c = 0; c < 4; ++c)
        store_shared16(staging + lane * 64 + ((c ^ ((lane >> 1) & 3)) << 4), packed[4 * c], packed[4 * c + 1], packed[4 * c + 2],
                       packed[4 * c + 3]);
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int r = 8 * k + lane / 4, c = lane % 4;
        const uint4 v = load_shared16(staging + r * 64 + ((c ^ ((r >> 1) & 3)) << 4));
        if (r < valid_rows)
            *reinterpret_cast<uint4 *>(static_cast<char *>(first_row) + r * row_bytes + c * 16) = v;
    }
    __syncwarp();
}
// Contiguous global memory -> shared memory by the copy engine (both 16-byte aligned, a multiple of 16 bytes);
// the bytes count towards the barrier's phase like those of a tile load.
__device__ __forceinline__ void bulk_load(uint32_t shared, const void *global, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(shared),
                 "l"(global), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory ----
__device__ __forceinline__ void tmem_alloc(uint32_t result_slot, uint32_t columns) { // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_slot),
                 "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) { // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives on the mbarrier once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; BF16 operands, FP32 accumulator.
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t instruction, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(instruction), "r"(accumulate)
                 : "memory");
}
// 32 lanes x 32 consecutive FP32 columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_load_32x32(uint32_t address, float (&v)[32]) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
                   "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
                   "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
                   "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(address)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i)
        v[i] = __uint_as_float(r[i]);
}

// Same load without the wait: issue several, then tmem_wait_load() on each register group
// before reading it (the wait takes the registers as operands so no use can move above it).
__device__ __forceinline__ void tmem_load_32x32_async(uint32_t address, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
                   "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
                   "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
                   "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(address)
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_load(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                   "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                   "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}
// 16-column forms of the asynchronous load and its wait.
__device__ __forceinline__ void tmem_load_32x16_async(uint32_t address, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
                   "=r"(r[15])
                 : "r"(address)
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_load(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15])
                 :
                 : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns from registers: thread i writes row (lane base + i).
__device__ __forceinline__ void tmem_store_32x32(uint32_t address, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(address),
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
                 "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
                 "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
                 "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_store_32x16(uint32_t address, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(address),
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
                 "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
// 32 lanes x 8 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_store_32x8(uint32_t address, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(address),
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_store() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: A is M x K BF16 held in tensor memory, row i in lane i, two
// K-elements per 32-bit column (even index in the low half).
__device__ __forceinline__ void tcgen05_mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                                    uint32_t instruction, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "r"(a_tmem), "l"(b_desc), "r"(instruction), "r"(accumulate)
                 : "memory");
}

// ---- CTA pairs (cluster of two CTAs driving one M = 256 MMA, cta_group::2) ----
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t cluster_address(uint32_t local_address, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_address), "r"(rank));
    return a;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on an mbarrier of another CTA of the cluster.
__device__ __forceinline__ void mbarrier_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// Tile load into this CTA's shared memory whose completion is counted on an mbarrier that may live
// in the pair's other CTA (`cluster_bar` is a shared::cluster address).
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, int z,
                                                 uint32_t cluster_bar) {
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t result_slot, uint32_t columns) { // one warp in each CTA
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_slot),
                 "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
// Issued by the pair's leader: D (128 rows in each CTA's tensor memory) (+)= A (128 rows from each
// CTA's shared memory) * B (N/2 columns from each CTA's shared memory).
__device__ __forceinline__ void tcgen05_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                      uint32_t instruction, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(instruction), "r"(accumulate)
                 : "memory");
}
// Arrives on one mbarrier (a shared::cluster address, in either CTA) when the pair's MMAs issued so
// far have completed.
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
                 : "memory");
}

// ---- descriptors ----
// Shared-memory matrix descriptor for 128-byte-swizzled BF16 tiles (version 1 = Blackwell).
//   K-major  (rows of 64 K-elements = 128 B, 8-row atoms of 1024 B): SBO = 1024 B between atoms.
//   MN-major (rows of 64 MN-elements = 128 B per K index, 8-K atoms of 1024 B): SBO = 1024 B
//   between 8-K atoms, LBO = bytes between consecutive 64-element MN blocks.
__device__ __forceinline__ uint64_t smem_descriptor(uint32_t address, uint32_t leading_bytes, uint32_t stride_bytes) {
    uint64_t d = 0;
    d |= uint64_t((address & 0x3ffff) >> 4);
    d |= uint64_t((leading_bytes >> 4) & 0x3fff) << 16;
    d |= uint64_t((stride_bytes >> 4) & 0x3fff) << 32;
    d |= uint64_t(1) << 46; // descriptor version
    d |= uint64_t(2) << 61; // 128-byte swizzle
    return d;
}
// The same descriptor `bytes` further into shared memory (the address field holds address / 16 in
// the low 14 bits; tiles never wrap it).  One 32-bit add instead of rebuilding the descriptor:
// the MMA-issuing thread is a serial bottleneck when the MMAs are small.
__device__ __forceinline__ uint64_t descriptor_at(uint64_t descriptor, uint32_t bytes) {
    uint32_t lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(descriptor));
    lo += bytes >> 4;
    uint64_t moved;
    asm("mov.b64 %0, {%1, %2};" : "=l"(moved) : "r"(lo), "r"(hi));
    return moved;
}
// Instruction descriptor: BF16 x BF16 -> FP32, M x N tile, operand majorness (0 = K, 1 = MN).
__host__ __device__ inline uint32_t instruction_descriptor(int m, int n, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(a_mn_major) << 15) | (uint32_t(b_mn_major) << 16) |
           (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}
#endif // __CUDACC__

} // namespace sm100
