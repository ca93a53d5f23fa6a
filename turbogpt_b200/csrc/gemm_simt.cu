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

template <class In, class Out> __global__ void __launch_bounds__(256) gemm_simt_kernel(GemmArgs g) {
    __shared__ float as[TileK][TileM + 4], bs[TileK][TileN + 4];
    const int z = blockIdx.z;
    const In *a = (const In *)g.a + z * g.a_batch, *b = (const In *)g.b + z * g.b_batch;
    const int m0 = blockIdx.y * TileM, n0 = blockIdx.x * TileN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < g.k; k0 += TileK) {
        // 64x16 elements per operand, 4 per thread.  Thread order follows the unit stride.
        for (int i = threadIdx.x; i < TileM * TileK; i += 256) {
            int mm, kk;
            if (g.a_col == 1) {
                kk = i % TileK, mm = i / TileK;
            } else {
                mm = i % TileM, kk = i / TileM;
            }
            int m = m0 + mm, k = k0 + kk;
            as[kk][mm] = (m < g.m && k < g.k) ? to_float(a[m * g.a_row + k * g.a_col]) : 0.f;
        }
        for (int i = threadIdx.x; i < TileN * TileK; i += 256) {
            int nn, kk;
            if (g.b_col == 1) {
                kk = i % TileK, nn = i / TileK;
            } else {
                nn = i % TileN, kk = i / TileN;
            }
            int n = n0 + nn, k = k0 + kk;
            bs[kk][nn] = (n < g.n && k < g.k) ? to_float(b[n * g.b_row + k * g.b_col]) : 0.f;
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
            if (m < g.m && n < g.n)
                EpilogueOps<Out>::apply(g, acc[i][j], int64_t(m) * g.ldc + n, int64_t(m) * g.ldr + n, z);
        }
}

void launch_gemm_simt(const GemmArgs &g, cudaStream_t s) {
    dim3 grid((g.n + TileN - 1) / TileN, (g.m + TileM - 1) / TileM, g.batch);
    if (g.in == Dtype::BF16 && g.out == Dtype::BF16)
        gemm_simt_kernel<bf16, bf16><<<grid, 256, 0, s>>>(g);
    else if (g.in == Dtype::BF16 && g.out == Dtype::FP32)
        gemm_simt_kernel<bf16, float><<<grid, 256, 0, s>>>(g);
    else if (g.in == Dtype::FP32 && g.out == Dtype::FP32)
        gemm_simt_kernel<float, float><<<grid, 256, 0, s>>>(g);
    else
        throw std::runtime_error("GEMM: FP32 operands with BF16 output are not used");
}
