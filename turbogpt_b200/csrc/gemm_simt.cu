// GEMM on CUDA cores: C[m,n] = sum_k A[m,k] * B[n,k] with arbitrary element strides, BF16 or
// FP32 operands, FP32 accumulation.  It serves the shapes the tensor-core kernel does not take
// (the reference architecture's 16/48-wide matrices), the FP32 check mode, and is the on-device
// cross-check of the tcgen05 kernel.  64x64 output tile, 16-deep shared-memory slices, 4x4
// outputs per thread.
#include "device_utils.cuh"
#include "kernels.cuh"

constexpr int TileM = 64, TileN = 64, TileK = 16;

template <class Out> struct EpilogueOps {
    // `value` is the FP32 accumulator; returns what is stored to C (already in storage rounding).
    __device__ static void apply(const GemmArgs &g, float value, int64_t c_index, int64_t r_index, int z) {
        Out *c = (Out *)g.c + z * g.c_batch;
        switch (g.epilogue) {
        case Epilogue::Store:
            c[c_index] = from_float<Out>(value);
            break;
        case Epilogue::Residual: {
            const Out *r = (const Out *)g.r + z * g.r_batch;
            c[c_index] = from_float<Out>(rounded<Out>(value) + to_float(r[r_index]));
            break;
        }
        case Epilogue::GeluDual: {
            float pre = rounded<Out>(value);
            c[c_index] = from_float<Out>(gelu_derivative(pre));
            ((Out *)g.c2 + z * g.c_batch)[c_index] = from_float<Out>(gelu(pre));
            break;
        }
        case Epilogue::GeluGrad: {
            const Out *r = (const Out *)g.r + z * g.r_batch;
            c[c_index] = from_float<Out>(rounded<Out>(value) * to_float(r[r_index]));
            break;
        }
        case Epilogue::Axpby: {
            const Out *r = (const Out *)g.r + z * g.r_batch;
            c[c_index] = from_float<Out>(g.alpha * value + g.beta * to_float(r[r_index]));
            break;
        }
        }
    }
};

// `partials` == nullptr: blockIdx.z is the batch index and the block walks all of K.  Otherwise (batch 1)
// blockIdx.z is a slice of K, `slice_k` elements long, and the block writes its FP32 partial tile to
// partials[slice][m][n]; gemm_simt_reduce_kernel adds the slices in order.
template <class In, class Out>
__global__ void __launch_bounds__(256) gemm_simt_kernel(GemmArgs g, float *partials, int slice_k) {
    __shared__ float as[TileK][TileM + 4], bs[TileK][TileN + 4];
    const int z = partials ? 0 : blockIdx.z;
    const In *a = (const In *)g.a + z * g.a_batch, *b = (const In *)g.b + z * g.b_batch;
    const int m0 = blockIdx.y * TileM, n0 = blockIdx.x * TileN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int k_begin = partials ? blockIdx.z * slice_k : 0;
    const int k_end = partials ? min(g.k, k_begin + slice_k) : g.k;
    float acc[4][4] = {};
    for (int k0 = k_begin; k0 < k_end; k0 += TileK) {
        // 64x16 elements per operand, 4 per thread.  Thread order follows the unit stride.
        for (int i = threadIdx.x; i < TileM * TileK; i += 256) {
            int mm, kk;
            if (g.a_col == 1) {
                kk = i % TileK, mm = i / TileK;
            } else {
                mm = i % TileM, kk = i / TileM;
            }
            int m = m0 + mm, k = k0 + kk;
            as[kk][mm] = (m < g.m && k < k_end) ? to_float(a[m * g.a_row + k * g.a_col]) : 0.f;
        }
        for (int i = threadIdx.x; i < TileN * TileK; i += 256) {
            int nn, kk;
            if (g.b_col == 1) {
                kk = i % TileK, nn = i / TileK;
            } else {
                nn = i % TileN, kk = i / TileN;
            }
            int n = n0 + nn, k = k0 + kk;
            bs[kk][nn] = (n < g.n && k < k_end) ? to_float(b[n * g.b_row + k * g.b_col]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TileK; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                av[i] = as[kk][ty * 4 + i];
                bv[i] = bs[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    acc[i][j] += av[i] * bv[j];
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < g.m && n < g.n) {
                if (partials)
                    partials[(int64_t(blockIdx.z) * g.m + m) * g.n + n] = acc[i][j];
                else
                    EpilogueOps<Out>::apply(g, acc[i][j], int64_t(m) * g.ldc + n, int64_t(m) * g.ldr + n, z);
            }
        }
}

// C = the K slices' partial tiles added in slice order (the same bits on every run).
template <class Out> __global__ void gemm_simt_reduce_kernel(GemmArgs g, const float *partials, int slices) {
    const int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x, count = int64_t(g.m) * g.n;
    if (i >= count)
        return;
    float sum = 0.f;
    for (int slice = 0; slice < slices; ++slice)
        sum += partials[slice * count + i];
    const int64_t m = i / g.n, n = i % g.n;
    EpilogueOps<Out>::apply(g, sum, m * g.ldc + n, m * g.ldr + n, 0);
}

// A weight gradient of the reference architecture is a 16..96-wide output over tens of thousands of
// tokens: one or two tiles that would each walk all of K alone.  Such shapes are cut along K.
int gemm_simt_slices(const GemmArgs &g) {
    const int64_t tiles = int64_t((g.n + TileN - 1) / TileN) * ((g.m + TileM - 1) / TileM);
    if (g.batch != 1 || tiles > 32 || g.k < 2048)
        return 1;
    const int64_t wanted = (296 + tiles - 1) / tiles, longest = g.k / 64; // at least four 16-deep steps per slice
    return int(wanted < longest ? wanted : longest);
}
size_t gemm_simt_scratch_bytes(const GemmArgs &g) {
    const int slices = gemm_simt_slices(g);
    return slices > 1 ? size_t(slices) * g.m * g.n * sizeof(float) : 0;
}

void launch_gemm_simt(const GemmArgs &g, cudaStream_t s, float *scratch) {
    const int slices = scratch ? gemm_simt_slices(g) : 1;
    float *partials = slices > 1 ? scratch : nullptr;
    const int slice_k = slices > 1 ? ((g.k + slices - 1) / slices + TileK - 1) / TileK * TileK : 0;
    const int used = slices > 1 ? (g.k + slice_k - 1) / slice_k : 1;
    dim3 grid((g.n + TileN - 1) / TileN, (g.m + TileM - 1) / TileM, slices > 1 ? used : g.batch);
    const unsigned reduce_blocks = unsigned((int64_t(g.m) * g.n + 255) / 256);
    if (g.in == Dtype::BF16 && g.out == Dtype::BF16) {
        gemm_simt_kernel<bf16, bf16><<<grid, 256, 0, s>>>(g, partials, slice_k);
        if (partials)
            gemm_simt_reduce_kernel<bf16><<<reduce_blocks, 256, 0, s>>>(g, partials, used);
    } else if (g.in == Dtype::BF16 && g.out == Dtype::FP32) {
        gemm_simt_kernel<bf16, float><<<grid, 256, 0, s>>>(g, partials, slice_k);
        if (partials)
            gemm_simt_reduce_kernel<float><<<reduce_blocks, 256, 0, s>>>(g, partials, used);
    } else if (g.in == Dtype::FP32 && g.out == Dtype::FP32) {
        gemm_simt_kernel<float, float><<<grid, 256, 0, s>>>(g, partials, slice_k);
        if (partials)
            gemm_simt_reduce_kernel<float><<<reduce_blocks, 256, 0, s>>>(g, partials, used);
    } else {
        throw std::runtime_error("GEMM: FP32 operands with BF16 output are not used");
    }
}
