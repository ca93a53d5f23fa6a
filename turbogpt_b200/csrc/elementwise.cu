// HBM-bound kernels of the step: byte sampling, embedding gather/scatter, norms, rotation,
// MLP activations, softmax cross-entropy, loss history.  Each is one pass over its operands
// with 128-bit accesses; rows are handled by one warp so the row statistics are shuffle
// reductions.
#include "device_utils.cuh"
#include <atomic>
#include "kernels.cuh"
#include "sm100.cuh"

#define DISPATCH(t, ...)                                                                                    \
    do {                                                                                                    \
        if ((t) == Dtype::BF16) {                                                                           \
            using T = bf16;                                                                                 \
            __VA_ARGS__;                                                                                    \
        } else {                                                                                            \
            using T = float;                                                                                \
            __VA_ARGS__;                                                                                    \
        }                                                                                                   \
    } while (0)

static inline int blocks_for(int64_t items, int per_block, int64_t cap = 1 << 30) {
    int64_t b = (items + per_block - 1) / per_block;
    return int(b < 1 ? 1 : (b > cap ? cap : b));
}

// ------------------------------------------------------------------------------------------
// Byte sampling: one block per sequence.  endpoint = lo + hash(seed + step*B_global + s_global)
// % (size - lo), lo = max(8, context); x = data[e-ctx .. e), y = data[e-ctx+1 .. e].
// ------------------------------------------------------------------------------------------
__global__ void sample_kernel(SampleArgs a) {
    __shared__ long long endpoint;
    const int sequence = blockIdx.x;
    if (threadIdx.x == 0) {
        const uint64_t step = a.fixed_step >= 0 ? uint64_t(a.fixed_step) : uint64_t(a.counters->step);
        const int64_t lo = a.context > 8 ? a.context : 8;
        const uint64_t global_batch = uint64_t(a.batch) * uint64_t(a.world);
        const uint64_t global_sequence = uint64_t(a.rank) * uint64_t(a.batch) + uint64_t(sequence);
        endpoint = lo + (long long)(hash_u64(a.seed + step * global_batch + global_sequence) %
                                    uint64_t(a.size - lo));
    }
    __syncthreads();
    const uint8_t *source = a.data + endpoint - a.context;
    for (int p = threadIdx.x; p < a.context; p += blockDim.x) {
        a.x[int64_t(sequence) * a.context + p] = source[p];
        a.y[int64_t(sequence) * a.context + p] = source[p + 1];
    }
}
void launch_sample(const SampleArgs &a, cudaStream_t s) {
    sample_kernel<<<a.batch, 128, 0, s>>>(a);
}

template <class T>
__global__ void embedding_kernel(const T *__restrict__ table, const uint8_t *__restrict__ x, T *__restrict__ hidden,
                                 int64_t vectors, int width8) {
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < vectors;
         i += int64_t(gridDim.x) * blockDim.x) {
        int64_t token = i / width8;
        int c = int(i % width8) * 8;
        float v[8];
        load8(table + int64_t(x[token]) * width8 * 8 + c, v);
        store8(hidden + token * width8 * 8 + c, v);
    }
}
void launch_embedding(Dtype t, const void *table, const uint8_t *x, void *hidden, int tokens, int width,
                      cudaStream_t s) {
    int64_t vectors = int64_t(tokens) * (width / 8);
    DISPATCH(t, (embedding_kernel<T><<<blocks_for(vectors, 256, 148 * 16), 256, 0, s>>>(
                    (const T *)table, x, (T *)hidden, vectors, width / 8)));
}

// One block per byte value; each warp owns a slice of columns and scans all tokens in order,
// so the FP32 sums have a fixed order (the reference uses atomicAdd, cuda/model.cuh:96-97).
template <class T>
__global__ void embedding_backward_kernel(const T *__restrict__ dhidden, const uint8_t *__restrict__ x,
                                          float *__restrict__ grad, int tokens, int width, bool accumulate) {
    const int value = blockIdx.x, lane = threadIdx.x % 32, warp = threadIdx.x / 32, warps = blockDim.x / 32;
    for (int c0 = warp * 32; c0 < width; c0 += warps * 32) {
        const int c = c0 + lane;
        float sum = 0;
        for (int t0 = 0; t0 < tokens; t0 += 32) {
            int t = t0 + lane;
            unsigned hits = __ballot_sync(0xffffffffu, t < tokens && x[t] == value);
            while (hits) {
                int bit = __ffs(hits) - 1;
                hits &= hits - 1;
                if (c < width)
                    sum += to_float(dhidden[int64_t(t0 + bit) * width + c]);
            }
        }
        if (c < width) {
            float *out = grad + int64_t(value) * width + c;
            *out = accumulate ? *out + sum : sum;
        }
    }
}
// Sliced variant for wide models: block (value, slice) sums the rows of its token slice whose byte
// equals `value` (warp w scans the w-th eighth of the slice in order, lanes hold 8 columns per 256),
// warps are added in order through shared memory, slices in order by the second kernel.
template <class T>
__global__ void __launch_bounds__(256) embedding_backward_slices_kernel(const T *__restrict__ dhidden,
                                                                        const uint8_t *__restrict__ x,
                                                                        float *__restrict__ partial, int tokens,
                                                                        int width) {
    extern __shared__ float sums[]; // [8 warps][width]
    const int value = blockIdx.x, slice = blockIdx.y, lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int per_slice = (tokens + gridDim.y - 1) / gridDim.y;
    const int per_warp = ((per_slice + 7) / 8 + 31) / 32 * 32;
    const int begin = slice * per_slice + warp * per_warp;
    const int end = min(min(begin + per_warp, (slice + 1) * per_slice), tokens);
    float acc[4][8] = {};
    for (int t0 = begin; t0 < end; t0 += 32) {
        const int t = t0 + lane;
        unsigned hits = __ballot_sync(0xffffffffu, t < end && x[t] == value);
        while (hits) {
            const int bit = __ffs(hits) - 1;
            hits &= hits - 1;
            const T *row = dhidden + int64_t(t0 + bit) * width;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const int c = (v * 32 + lane) * 8;
                if (c < width) {
                    float r[8];
                    load8(row + c, r);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        acc[v][j] += r[j];
                }
            }
        }
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        const int c = (v * 32 + lane) * 8;
        if (c < width)
#pragma unroll
            for (int j = 0; j < 8; ++j)
                sums[warp * width + c + j] = acc[v][j];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float total = 0;
        for (int w = 0; w < 8; ++w)
            total += sums[w * width + c];
        partial[(int64_t(slice) * Vocabulary + value) * width + c] = total;
    }
}
__global__ void embedding_backward_sum_kernel(const float *partial, float *grad, int width, int slices,
                                              bool accumulate) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= Vocabulary * width)
        return;
    float total = accumulate ? grad[i] : 0.f;
    for (int s = 0; s < slices; ++s)
        total += partial[int64_t(s) * Vocabulary * width + i];
    grad[i] = total;
}
void launch_embedding_backward(Dtype t, const void *dhidden, const uint8_t *x, float *grad, int tokens,
                               int width, bool accumulate, float *scratch, cudaStream_t s) {
    if (scratch && width <= 1024 && tokens >= 4096) {
        DISPATCH(t, (embedding_backward_slices_kernel<T><<<dim3(Vocabulary, EmbeddingSlices), 256,
                                                          8 * width * sizeof(float), s>>>(
                        (const T *)dhidden, x, scratch, tokens, width)));
        embedding_backward_sum_kernel<<<(Vocabulary * width + 255) / 256, 256, 0, s>>>(scratch, grad, width,
                                                                                     EmbeddingSlices, accumulate);
        return;
    }
    int threads = width >= 256 ? 256 : (width + 31) / 32 * 32;
    DISPATCH(t, (embedding_backward_kernel<T><<<Vocabulary, threads, 0, s>>>((const T *)dhidden, x, grad, tokens,
                                                                           width, accumulate)));
}

// ------------------------------------------------------------------------------------------
// Norms.  RMSNorm: y = x * rsqrt(mean(x^2) + 1e-6) * w.  LayerNorm: y = (x - mean) *
// rsqrt(var + 1e-5) * w + b.  FP32 math on FP32 master scales, one rounding to the activation
// type at the end.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void load_scale8(const bf16 *high, const uint16_t *low, int c, float (&w)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
        w[j] = join_weight(high[c + j], low[c + j]);
}
template <class T>
__device__ __forceinline__ void row_statistics(int kind, const T *row, int width, int lane, float &mean,
                                               float &inv) {
    float sum = 0, squares = 0;
    for (int c = lane * 8; c < width; c += 256) {
        float v[8];
        load8(row + c, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            sum += v[j];
            squares += v[j] * v[j];
        }
    }
    if (kind == TG_NORM_RMS) {
        mean = 0;
        inv = rsqrtf(warp_sum(squares) / width + 1e-6f);
        return;
    }
    mean = warp_sum(sum) / width;
    float centred = 0;
    for (int c = lane * 8; c < width; c += 256) {
        float v[8];
        load8(row + c, v);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            centred += (v[j] - mean) * (v[j] - mean);
    }
    inv = rsqrtf(warp_sum(centred) / width + 1e-5f);
}
template <class T> __global__ void __launch_bounds__(256) norm_kernel(NormArgs a) {
    const int lane = threadIdx.x % 32;
    const int row = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (row >= a.rows)
        return;
    const T *x = (const T *)a.x + int64_t(row) * a.width;
    T *y = (T *)a.y + int64_t(row) * a.width;
    float mean, inv;
    row_statistics(a.kind, x, a.width, lane, mean, inv);
    for (int c = lane * 8; c < a.width; c += 256) {
        float v[8], w[8], out[8];
        load8(x + c, v);
        load_scale8(a.scale_high, a.scale_low, c, w);
        if (a.kind == TG_NORM_RMS) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                out[j] = v[j] * inv * w[j];
        } else {
            float b[8];
            load_scale8(a.bias_high, a.bias_low, c, b);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                out[j] = (v[j] - mean) * inv * w[j] + b[j];
        }
        store8(y + c, out);
    }
}
// Eight elements as they arrive from memory, converted when used: the row fetched ahead of its turn
// costs half the registers of its FP32 form.
template <class T> struct Packet;
template <> struct Packet<bf16> { uint4 u; };
template <> struct Packet<float> { float4 a, b; };
__device__ __forceinline__ void fetch8(const bf16 *p, Packet<bf16> &r) { r.u = *reinterpret_cast<const uint4 *>(p); }
__device__ __forceinline__ void fetch8(const float *p, Packet<float> &r) {
    r.a = *reinterpret_cast<const float4 *>(p), r.b = *reinterpret_cast<const float4 *>(p + 4);
}
__device__ __forceinline__ void unpack8(const Packet<bf16> &r, float (&v)[8]) {
    const unsigned w[4] = {r.u.x, r.u.y, r.u.z, r.u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void unpack8(const Packet<float> &r, float (&v)[8]) {
    v[0] = r.a.x, v[1] = r.a.y, v[2] = r.a.z, v[3] = r.a.w, v[4] = r.b.x, v[5] = r.b.y, v[6] = r.b.z, v[7] = r.b.w;
}

// Widths of 256..1024 in steps of 256: the row lives in registers (one 128-bit load per 256
// columns and lane), so x is read once; scale and bias are read once per block into shared memory.
//
// Per-lane vectors of 8 floats in shared memory are stored as two float4 planes,
// [v][half][lane][4]: consecutive lanes then touch consecutive 16-byte words and a warp-wide access
// has no bank conflicts (the natural [column] order puts lanes 32 bytes apart: two-way conflicts).
__device__ __forceinline__ int plane_index(int v, int half, int lane) { return ((v * 2 + half) * 32 + lane) * 4; }
__device__ __forceinline__ int plane_of_column(int c) { // column -> index in the plane layout
    const int v = c / 256, lane = c % 256 / 8, half = c % 8 / 4, j = c % 4;
    return plane_index(v, half, lane) + j;
}
__device__ __forceinline__ void load_planes(const float *base, int v, int lane, float (&w)[8]) {
    const float4 a = *reinterpret_cast<const float4 *>(base + plane_index(v, 0, lane));
    const float4 b = *reinterpret_cast<const float4 *>(base + plane_index(v, 1, lane));
    w[0] = a.x, w[1] = a.y, w[2] = a.z, w[3] = a.w, w[4] = b.x, w[5] = b.y, w[6] = b.z, w[7] = b.w;
}
__device__ __forceinline__ void store_planes(float *base, int v, int lane, const float (&w)[8]) {
    *reinterpret_cast<float4 *>(base + plane_index(v, 0, lane)) = make_float4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<float4 *>(base + plane_index(v, 1, lane)) = make_float4(w[4], w[5], w[6], w[7]);
}
// Two sums over the warp at once: the shuffles of the two values interleave, so the pair costs the
// latency of one reduction.
__device__ __forceinline__ void warp_sum2(float &a, float &b) {
#pragma unroll
    for (int k = 16; k; k >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, a, k), ob = __shfl_xor_sync(0xffffffffu, b, k);
        a += oa, b += ob;
    }
}
// Mean and 1/sqrt(variance + eps) of a register-resident row.  FP32 rows (the check mode) take two
// passes like the FP32 model they are compared with; BF16 rows take one pass over values shifted by
// the row's first element (exact for the shift, immune to a large common offset), whose two sums
// share one warp reduction: the row's dependent chain is one shuffle plus one reduction.
template <class T, int V> __device__ __forceinline__ void row_moments(int kind, const float (&x)[V][8], int width,
                                                                       float &mean, float &inv) {
    float sums[4] = {0, 0, 0, 0}, squares[4] = {0, 0, 0, 0};
    if (kind == TG_NORM_RMS) {
#pragma unroll
        for (int v = 0; v < V; ++v)
#pragma unroll
            for (int j = 0; j < 8; ++j)
                squares[j % 4] += x[v][j] * x[v][j];
        mean = 0;
        inv = rsqrtf(warp_sum((squares[0] + squares[1]) + (squares[2] + squares[3])) / width + 1e-6f);
        return;
    }
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int v = 0; v < V; ++v)
#pragma unroll
            for (int j = 0; j < 8; ++j)
                sums[j % 4] += x[v][j];
        mean = warp_sum((sums[0] + sums[1]) + (sums[2] + sums[3])) / width;
#pragma unroll
        for (int v = 0; v < V; ++v)
#pragma unroll
            for (int j = 0; j < 8; ++j)
                squares[j % 4] += (x[v][j] - mean) * (x[v][j] - mean);
        inv = rsqrtf(warp_sum((squares[0] + squares[1]) + (squares[2] + squares[3])) / width + 1e-5f);
    } else {
        const float shift = __shfl_sync(0xffffffffu, x[0][0], 0);
#pragma unroll
        for (int v = 0; v < V; ++v)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float d = x[v][j] - shift;
                sums[j % 4] += d;
                squares[j % 4] += d * d;
            }
        float s1 = (sums[0] + sums[1]) + (sums[2] + sums[3]), s2 = (squares[0] + squares[1]) + (squares[2] + squares[3]);
        warp_sum2(s1, s2);
        const float offset = s1 / width;
        mean = shift + offset;
        inv = rsqrtf(fmaxf(s2 / width - offset * offset, 0.f) + 1e-5f);
    }
}
template <class T, int V> __global__ void __launch_bounds__(256, 4) norm_rows_kernel(NormArgs a) {
    sm100::grid_launch_dependents(); // the next kernel may set itself up while this one runs
    __shared__ __align__(16) float sw[V * 256], sb[V * 256]; // FP32 scale and bias in the plane layout
    const int lane = threadIdx.x % 32, warps = blockDim.x / 32;
    for (int c = threadIdx.x; c < V * 256; c += blockDim.x) {
        sw[plane_of_column(c)] = join_weight(a.scale_high[c], a.scale_low[c]);
        sb[plane_of_column(c)] = a.kind == TG_NORM_LAYER ? join_weight(a.bias_high[c], a.bias_low[c]) : 0.f;
    }
    __syncthreads();
    const int stride = gridDim.x * warps;
    int row = blockIdx.x * warps + threadIdx.x / 32;
    Packet<T> next[V]; // the warp's next row, fetched while the current one is normalised
    if (row < a.rows)
#pragma unroll
        for (int k = 0; k < V; ++k)
            fetch8((const T *)a.x + int64_t(row) * a.width + (k * 32 + lane) * 8, next[k]);
    for (; row < a.rows; row += stride) {
        T *y = (T *)a.y + int64_t(row) * a.width;
        float v[V][8];
#pragma unroll
        for (int k = 0; k < V; ++k)
            unpack8(next[k], v[k]);
        if (row + stride < a.rows)
#pragma unroll
            for (int k = 0; k < V; ++k)
                fetch8((const T *)a.x + int64_t(row + stride) * a.width + (k * 32 + lane) * 8, next[k]);
        float mean, inv;
        row_moments<T, V>(a.kind, v, a.width, mean, inv);
        if (a.stats && lane == 0)
            reinterpret_cast<float2 *>(a.stats)[row] = make_float2(mean, inv); // kept for the backward pass
#pragma unroll
        for (int k = 0; k < V; ++k) {
            float out[8], w[8], b[8];
            load_planes(sw, k, lane, w);
            load_planes(sb, k, lane, b);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                out[j] = a.kind == TG_NORM_RMS ? v[k][j] * inv * w[j] : (v[k][j] - mean) * inv * w[j] + b[j];
            store8(y + (k * 32 + lane) * 8, out);
        }
    }
}
template <class T> static void launch_norm_rows(const NormArgs &a, cudaStream_t s) {
    const int blocks = blocks_for(a.rows, 8, 148 * 4);
    switch (a.width / 256) {
    case 1: norm_rows_kernel<T, 1><<<blocks, 256, 0, s>>>(a); break;
    case 2: norm_rows_kernel<T, 2><<<blocks, 256, 0, s>>>(a); break;
    case 3: norm_rows_kernel<T, 3><<<blocks, 256, 0, s>>>(a); break;
    default: norm_rows_kernel<T, 4><<<blocks, 256, 0, s>>>(a); break;
    }
}
void launch_norm(Dtype t, const NormArgs &a, cudaStream_t s) {
    if (a.width % 256 == 0 && a.width <= 1024) {
        DISPATCH(t, launch_norm_rows<T>(a, s));
        return;
    }
    DISPATCH(t, (norm_kernel<T><<<blocks_for(a.rows, 8), 256, 0, s>>>(a)));
}

// dx = (dz - [mean(dz)] - z * mean(dz * z)) * inv with dz = dy * w, z the normalised input;
// rounded to the activation type, then added to the running residual gradient with a second
// rounding (reference cuda/ops.cuh:67-80).  Scale/bias gradients: each warp sums its rows in its own
// slice of shared memory (a lane owns its columns there, so no atomics), the warps are added in
// order, then a fixed-order sum over blocks: the same bits on every run.
template <class T> __global__ void __launch_bounds__(256) norm_backward_kernel(NormBackwardArgs a) {
    extern __shared__ float sums[]; // [warps][2][width]
    const int lane = threadIdx.x % 32, warps = blockDim.x / 32;
    float *mine = sums + (threadIdx.x / 32) * 2 * a.width;
    for (int c = threadIdx.x; c < warps * 2 * a.width; c += blockDim.x)
        sums[c] = 0;
    __syncthreads();
    for (int row = blockIdx.x * warps + threadIdx.x / 32; row < a.rows; row += gridDim.x * warps) {
        const T *x = (const T *)a.x + int64_t(row) * a.width;
        const T *dy = (const T *)a.dy + int64_t(row) * a.width;
        float mean, inv;
        row_statistics(a.kind, x, a.width, lane, mean, inv);
        float sum_dz = 0, sum_dzz = 0;
        for (int c = lane * 8; c < a.width; c += 256) {
            float v[8], g[8], w[8];
            load8(x + c, v);
            load8(dy + c, g);
            load_scale8(a.scale_high, a.scale_low, c, w);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float z = (v[j] - mean) * inv, dz = g[j] * w[j];
                sum_dz += dz;
                sum_dzz += dz * z;
                mine[c + j] += g[j] * z;
                if (a.kind == TG_NORM_LAYER)
                    mine[a.width + c + j] += g[j];
            }
        }
        sum_dzz = warp_sum(sum_dzz) / a.width;
        sum_dz = a.kind == TG_NORM_LAYER ? warp_sum(sum_dz) / a.width : 0.f;
        for (int c = lane * 8; c < a.width; c += 256) {
            float v[8], g[8], w[8], out[8];
            load8(x + c, v);
            load8(dy + c, g);
            load_scale8(a.scale_high, a.scale_low, c, w);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float z = (v[j] - mean) * inv, dz = g[j] * w[j];
                out[j] = (dz - sum_dz - z * sum_dzz) * inv;
            }
            if (a.residual_in) {
                float r[8];
                load8((const T *)a.residual_in + int64_t(row) * a.width + c, r);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    out[j] = r[j] + rounded<T>(out[j]);
            }
            store8((T *)a.dx + int64_t(row) * a.width + c, out);
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < 2 * a.width; c += blockDim.x) {
        float total = 0;
        for (int w = 0; w < warps; ++w)
            total += sums[w * 2 * a.width + c];
        a.partial[int64_t(blockIdx.x) * 2 * a.width + c] = total;
    }
}
// 8 columns per block, 32 threads per column: thread g sums blocks g, g+32, ...; the 32 sums are
// added in order.  Same result on every run.
__global__ void __launch_bounds__(256) norm_backward_reduce_kernel(const float *partial, float *dscale,
                                                                   float *dbias, int width, int blocks) {
    __shared__ float sums[32][9];
    const int column = threadIdx.x % 8, group = threadIdx.x / 8;
    const int c = blockIdx.x * 8 + column;
    float sum = 0;
    if (c < 2 * width)
        for (int b = group; b < blocks; b += 32)
            sum += partial[int64_t(b) * 2 * width + c];
    sums[group][column] = sum;
    __syncthreads();
    if (group == 0 && c < 2 * width) {
        float total = 0;
        for (int g = 0; g < 32; ++g)
            total += sums[g][column];
        if (c < width)
            dscale[c] = total;
        else if (dbias)
            dbias[c - width] = total;
    }
}
// Register-resident variant for widths 256..1024: x, dy and the residual gradient are read once, and
// a warp fetches its next row while it works on the current one.  The row's mean and 1/sigma come
// from the forward pass when it saved them (`stats`), so the only reduction a row waits for is the
// pair sum(dz), sum(dz z).  Each warp keeps the scale/bias gradient sums of its rows in its own slice
// of shared memory (plane layout: a lane owns its words, no conflicts, no atomics); warps are summed
// in order at the end, blocks in order by the reduce kernel: deterministic.
template <class T, int V> __global__ void __launch_bounds__(256, 2) norm_backward_rows_kernel(NormBackwardArgs a) {
    sm100::grid_launch_dependents(); // the next kernel may set itself up while this one runs
    extern __shared__ float sums[]; // [V * 256] scale, then [warps][2][V * 256] gradient sums, all in the plane layout
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32, warps = blockDim.x / 32;
    float *scale = sums, *mine = sums + V * 256 + warp * 2 * V * 256;
    for (int c = threadIdx.x; c < V * 256; c += blockDim.x)
        scale[plane_of_column(c)] = join_weight(a.scale_high[c], a.scale_low[c]);
    for (int c = lane; c < 2 * V * 256; c += 32)
        mine[c] = 0.f;
    __syncthreads();
    const bool residual = a.residual_in != nullptr, saved = a.stats != nullptr;
    const int stride = gridDim.x * warps;
    Packet<T> nx[V], ng[V], nr[V];
    float2 nstat = make_float2(0.f, 1.f);
    auto fetch = [&](int row) {
        const int64_t offset = int64_t(row) * a.width;
        if (saved)
            nstat = reinterpret_cast<const float2 *>(a.stats)[row];
#pragma unroll
        for (int v = 0; v < V; ++v) {
            fetch8((const T *)a.x + offset + (v * 32 + lane) * 8, nx[v]);
            fetch8((const T *)a.dy + offset + (v * 32 + lane) * 8, ng[v]);
            if (residual)
                fetch8((const T *)a.residual_in + offset + (v * 32 + lane) * 8, nr[v]);
        }
    };
    int row = blockIdx.x * warps + warp;
    if (row < a.rows)
        fetch(row);
    for (; row < a.rows; row += stride) {
        const int64_t offset = int64_t(row) * a.width;
        float x[V][8], g[V][8];
        Packet<T> r[V];
#pragma unroll
        for (int v = 0; v < V; ++v) {
            unpack8(nx[v], x[v]);
            unpack8(ng[v], g[v]);
            r[v] = nr[v];
        }
        float mean = nstat.x, inv = nstat.y;
        if (row + stride < a.rows)
            fetch(row + stride); // in flight during this row's arithmetic
        if (!saved)
            row_moments<T, V>(a.kind, x, a.width, mean, inv);
        float part_dz[4] = {0, 0, 0, 0}, part_dzz[4] = {0, 0, 0, 0};
#pragma unroll
        for (int v = 0; v < V; ++v) {
            float w[8], dw[8], db[8];
            load_planes(scale, v, lane, w);
            load_planes(mine, v, lane, dw);
            load_planes(mine + V * 256, v, lane, db);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float z = (x[v][j] - mean) * inv, dz = g[v][j] * w[j];
                x[v][j] = z; // keep the normalised value
                part_dz[j % 4] += dz;
                part_dzz[j % 4] += dz * z;
                dw[j] += g[v][j] * z;
                db[j] += g[v][j];
                g[v][j] = dz; // keep dy * scale
            }
            store_planes(mine, v, lane, dw);
            store_planes(mine + V * 256, v, lane, db);
        }
        float sum_dzz = (part_dzz[0] + part_dzz[1]) + (part_dzz[2] + part_dzz[3]);
        float sum_dz = (part_dz[0] + part_dz[1]) + (part_dz[2] + part_dz[3]);
        warp_sum2(sum_dzz, sum_dz);
        sum_dzz /= a.width;
        sum_dz = a.kind == TG_NORM_LAYER ? sum_dz / a.width : 0.f;
#pragma unroll
        for (int v = 0; v < V; ++v) {
            float out[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                out[j] = (g[v][j] - sum_dz - x[v][j] * sum_dzz) * inv;
            if (residual) {
                float res[8];
                unpack8(r[v], res);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    out[j] = res[j] + rounded<T>(out[j]);
            }
            store8((T *)a.dx + offset + (v * 32 + lane) * 8, out);
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < 2 * a.width; c += blockDim.x) {
        const int which = c / a.width, index = plane_of_column(c % a.width) + which * V * 256;
        float total = 0;
        for (int k = 0; k < warps; ++k)
            total += sums[V * 256 + k * 2 * V * 256 + index];
        a.partial[int64_t(blockIdx.x) * 2 * a.width + c] = total;
    }
}
template <class T, int V> static void launch_norm_backward_rows(const NormBackwardArgs &a, cudaStream_t s) {
    const size_t shared = size_t(V * 256 + 8 * 2 * a.width) * sizeof(float);
    static std::atomic<unsigned long long> configured{0}; // one bit per device; engines on other devices run on other threads
    int device = 0;
    CHECK_CUDA(cudaGetDevice(&device));
    if (shared > 48 * 1024 && (device >= 64 || !(configured.load() >> device & 1))) {
        CHECK_CUDA(cudaFuncSetAttribute(norm_backward_rows_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        int(shared)));
        if (device < 64)
            configured.fetch_or(1ull << device);
    }
    norm_backward_rows_kernel<T, V><<<a.blocks, 256, shared, s>>>(a);
}
int norm_backward_blocks(int rows, int sms) {
    return blocks_for(rows, 8, int64_t(sms) * 2);
}
void launch_norm_backward(Dtype t, const NormBackwardArgs &a, cudaStream_t s) {
    size_t shared = size_t(2) * a.width * sizeof(float);
    const int reduce_blocks = blocks_for(2 * a.width, 8);
    if (a.width % 256 == 0 && a.width <= 1024) {
        DISPATCH(t, {
            switch (a.width / 256) {
            case 1: launch_norm_backward_rows<T, 1>(a, s); break;
            case 2: launch_norm_backward_rows<T, 2>(a, s); break;
            case 3: launch_norm_backward_rows<T, 3>(a, s); break;
            default: launch_norm_backward_rows<T, 4>(a, s); break;
            }
        });
        norm_backward_reduce_kernel<<<reduce_blocks, 256, 0, s>>>(a.partial, a.dscale, a.dbias, a.width, a.blocks);
        return;
    }
    // as many warps per block (up to 8) as 200 KB of per-warp sums allow
    int warps = 8;
    while (warps > 1 && shared * warps > 200 * 1024)
        warps /= 2;
    shared *= warps;
    DISPATCH(t, {
        if (shared > 48 * 1024)
            CHECK_CUDA(cudaFuncSetAttribute(norm_backward_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            int(shared)));
        norm_backward_kernel<T><<<a.blocks, warps * 32, shared, s>>>(a);
    });
    norm_backward_reduce_kernel<<<reduce_blocks, 256, 0, s>>>(a.partial, a.dscale, a.dbias, a.width, a.blocks);
}

// ------------------------------------------------------------------------------------------
// Partial rotary embedding: dims (0, 1) of every query and key head turn `position` radians.
// Products are kept unfused so the rounding matches the PyTorch model.
// ------------------------------------------------------------------------------------------
template <class T>
__global__ void rope_kernel(T *qkv, int64_t pairs, int context, int width, int heads, bool inverse) {
    int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    if (i >= pairs)
        return;
    const int d_head = width / heads;
    int64_t token = i / (2 * heads);
    int slot = int(i % (2 * heads)); // query heads, then key heads
    int position = int(token % context);
    T *pair = qkv + token * 3 * width + (slot / heads) * width + (slot % heads) * d_head;
    float x = to_float(pair[0]), y = to_float(pair[1]);
    float c = float(cos(double(position))), sn = float(sin(double(position)));
    if (inverse)
        sn = -sn;
    pair[0] = from_float<T>(__fsub_rn(__fmul_rn(x, c), __fmul_rn(y, sn)));
    pair[1] = from_float<T>(__fadd_rn(__fmul_rn(x, sn), __fmul_rn(y, c)));
}
void launch_rope(Dtype t, void *qkv, int tokens, int context, int width, int heads, bool inverse,
                 cudaStream_t s) {
    int64_t pairs = int64_t(tokens) * 2 * heads;
    DISPATCH(t, (rope_kernel<T><<<blocks_for(pairs, 256), 256, 0, s>>>((T *)qkv, pairs, context, width, heads,
                                                                      inverse)));
}

// ------------------------------------------------------------------------------------------
// MLP activations with the forward's roundings: act = round(g * sigmoid(g)); out = round(act * u).
// ------------------------------------------------------------------------------------------
template <class T>
__global__ void swiglu_kernel(const T *__restrict__ wide, T *__restrict__ out, int64_t vectors, int hidden8) {
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < vectors;
         i += int64_t(gridDim.x) * blockDim.x) {
        int64_t token = i / hidden8;
        int c = int(i % hidden8) * 8;
        float g[8], u[8], r[8];
        load8(wide + token * hidden8 * 16 + c, g);
        load8(wide + token * hidden8 * 16 + hidden8 * 8 + c, u);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            r[j] = rounded<T>(g[j] * sigmoid(g[j])) * u[j];
        store8(out + token * hidden8 * 8 + c, r);
    }
}
void launch_swiglu(Dtype t, const void *wide, void *out, int tokens, int hidden, cudaStream_t s) {
    int64_t vectors = int64_t(tokens) * (hidden / 8);
    DISPATCH(t, (swiglu_kernel<T><<<blocks_for(vectors, 256, 148 * 16), 256, 0, s>>>((const T *)wide, (T *)out,
                                                                                 vectors, hidden / 8)));
}
template <class T>
__global__ void swiglu_backward_kernel(const T *__restrict__ wide, const T *__restrict__ dout,
                                       T *__restrict__ dwide, int64_t vectors, int hidden8) {
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < vectors;
         i += int64_t(gridDim.x) * blockDim.x) {
        int64_t token = i / hidden8;
        int c = int(i % hidden8) * 8;
        float g[8], u[8], dy[8], dg[8], du[8];
        load8(wide + token * hidden8 * 16 + c, g);
        load8(wide + token * hidden8 * 16 + hidden8 * 8 + c, u);
        load8(dout + token * hidden8 * 8 + c, dy);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float sig = sigmoid(g[j]);
            float activated = rounded<T>(g[j] * sig);
            float da = rounded<T>(dy[j] * u[j]);
            dg[j] = da * sig * (1.f + g[j] * (1.f - sig));
            du[j] = dy[j] * activated;
        }
        store8(dwide + token * hidden8 * 16 + c, dg);
        store8(dwide + token * hidden8 * 16 + hidden8 * 8 + c, du);
    }
}
void launch_swiglu_backward(Dtype t, const void *wide, const void *dout, void *dwide, int tokens, int hidden,
                            cudaStream_t s) {
    int64_t vectors = int64_t(tokens) * (hidden / 8);
    DISPATCH(t, (swiglu_backward_kernel<T><<<blocks_for(vectors, 256, 148 * 16), 256, 0, s>>>(
                    (const T *)wide, (const T *)dout, (T *)dwide, vectors, hidden / 8)));
}

// ------------------------------------------------------------------------------------------
// 256-way softmax cross-entropy, one warp per row, 8 logits per lane (one 128-bit load):
// loss = max + log(sum exp) - logit[y]; dlogit = round((softmax - onehot) / divisor).
// ------------------------------------------------------------------------------------------
template <class T> __global__ void __launch_bounds__(256) cross_entropy_kernel(CrossEntropyArgs a) {
    const int lane = threadIdx.x % 32;
    const int row = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (row >= a.rows)
        return;
    float v[8];
    load8((const T *)a.logits + int64_t(row) * Vocabulary + lane * 8, v);
    float high = v[0];
#pragma unroll
    for (int j = 1; j < 8; ++j)
        high = fmaxf(high, v[j]);
    high = warp_max(high);
    float e[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        e[j] = expf(v[j] - high);
        sum += e[j];
    }
    sum = warp_sum(sum);
    const int target = a.targets[row];
    float picked;
    { // select the target's logit without dynamic register indexing
        float chosen = v[0];
#pragma unroll
        for (int j = 1; j < 8; ++j)
            chosen = (target % 8 == j) ? v[j] : chosen;
        picked = __shfl_sync(0xffffffffu, chosen, target / 8);
    }
    if (lane == 0)
        a.losses[row] = high + logf(sum) - picked;
    if (a.logits_fp32)
        store8(a.logits_fp32 + int64_t(row) * Vocabulary + lane * 8, v);
    if (a.dlogits) {
        float g[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            g[j] = (e[j] / sum - (lane * 8 + j == target ? 1.f : 0.f)) / a.divisor;
        store8((T *)a.dlogits + int64_t(row) * Vocabulary + lane * 8, g);
    }
}
void launch_cross_entropy(Dtype t, const CrossEntropyArgs &a, cudaStream_t s) {
    DISPATCH(t, (cross_entropy_kernel<T><<<blocks_for(a.rows, 8), 256, 0, s>>>(a)));
}

// Mean over the batch for every position, summed in double like the reference
// (cuda/trainer.cuh:94-98); row `iteration` of the history.
__global__ void loss_history_kernel(const float *token_losses, float *history, const StepCounters *counters,
                                    int batch, int context) {
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= context)
        return;
    double total = 0;
    for (int b = 0; b < batch; ++b)
        total += token_losses[int64_t(b) * context + p];
    history[int64_t(counters->iteration) * context + p] = float(total / batch);
}
void launch_loss_history(const float *token_losses, float *history, const StepCounters *counters, int batch,
                         int context, cudaStream_t s) {
    loss_history_kernel<<<blocks_for(context, 64), 64, 0, s>>>(token_losses, history, counters, batch, context);
}

// ------------------------------------------------------------------------------------------
// Conversions.
// ------------------------------------------------------------------------------------------
__global__ void split_weights_kernel(const float *w, bf16 *high, uint16_t *low, int64_t count) {
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < count;
         i += int64_t(gridDim.x) * blockDim.x) {
        unsigned bits = __float_as_uint(w[i]);
        high[i] = __ushort_as_bfloat16((unsigned short)(bits >> 16));
        low[i] = uint16_t(bits);
    }
}
void launch_split_weights(const float *w, bf16 *high, uint16_t *low, int64_t count, cudaStream_t s) {
    split_weights_kernel<<<blocks_for(count, 256, 148 * 8), 256, 0, s>>>(w, high, low, count);
}
__global__ void join_weights_kernel(const bf16 *high, const uint16_t *low, float *w, int64_t count) {
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < count;
         i += int64_t(gridDim.x) * blockDim.x)
        w[i] = join_weight(high[i], low[i]);
}
void launch_join_weights(const bf16 *high, const uint16_t *low, float *w, int64_t count, cudaStream_t s) {
    join_weights_kernel<<<blocks_for(count, 256, 148 * 8), 256, 0, s>>>(high, low, w, count);
}
template <class A, class B> __global__ void cast_kernel(const A *in, B *out, int64_t count) {
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < count;
         i += int64_t(gridDim.x) * blockDim.x)
        out[i] = from_float<B>(to_float(in[i]));
}
void launch_cast(Dtype from, const void *in, Dtype to, void *out, int64_t count, cudaStream_t s) {
    int blocks = blocks_for(count, 256, 148 * 8);
    if (from == Dtype::FP32 && to == Dtype::BF16)
        cast_kernel<<<blocks, 256, 0, s>>>((const float *)in, (bf16 *)out, count);
    else if (from == Dtype::BF16 && to == Dtype::FP32)
        cast_kernel<<<blocks, 256, 0, s>>>((const bf16 *)in, (float *)out, count);
    else
        CHECK_CUDA(cudaMemcpyAsync(out, in, count * dtype_size(from), cudaMemcpyDeviceToDevice, s));
}
