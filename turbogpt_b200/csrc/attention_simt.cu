// Attention on CUDA cores.
//  * Arg-max attention of the reference architecture (cuda/attention.cuh:33-106): per (query,
//    head) the single causal key with the largest q.k wins (first index on ties); the output is
//    v[key] * GELU(score).  Scalar FP32, exact restatement with sizes as parameters.
//  * Causal softmax attention for any head size up to 256 in BF16 or FP32: the check-mode and
//    small-shape path beside the tcgen05 kernel.  One warp per query (or key) row, online
//    softmax, deterministic (no atomics).
#include "device_utils.cuh"
#include "kernels.cuh"

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

// ---------------------------------------------------------------- arg-max attention ----------
template <class T> __global__ void argmax_attention_kernel(ArgmaxAttentionArgs a) {
    const int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    const int64_t tokens = int64_t(a.batch) * a.context;
    if (i >= tokens * a.heads)
        return;
    const int d = a.width / a.heads, head = int(i % a.heads);
    const int64_t row = i / a.heads, start = row / a.context * a.context;
    const T *qkv = (const T *)a.qkv;
    const T *q = qkv + row * 3 * a.width + head * d;
    float top = -CUDART_INF_F;
    int64_t best = start;
    for (int64_t key = start; key <= row; ++key) {
        const T *k = qkv + key * 3 * a.width + a.width + head * d;
        float score = 0;
        for (int c = 0; c < d; ++c)
            score += to_float(q[c]) * to_float(k[c]);
        if (score > top) { // first index wins ties
            top = score;
            best = key;
        }
    }
    float e = 1.f + erff(top * 0.7071067811865475f);
    float g = 0.5f * top * e;
    a.selected[i] = int(best - start);
    a.gates[i] = g;
    a.derivatives[i] = 0.5f * e + top * 0.3989422804014327f * expf(-0.5f * top * top);
    const T *v = qkv + best * 3 * a.width + 2 * a.width + head * d;
    T *out = (T *)a.out + row * a.width + head * d;
    for (int c = 0; c < d; ++c)
        out[c] = from_float<T>(to_float(v[c]) * g);
}
void launch_argmax_attention(Dtype t, const ArgmaxAttentionArgs &a, cudaStream_t s) {
    int64_t items = int64_t(a.batch) * a.context * a.heads;
    DISPATCH(t, (argmax_attention_kernel<T><<<int((items + 127) / 128), 128, 0, s>>>(a)));
}

// Pass 1: dt[query, head] = (dy . v[key]) * GELU'(top).
template <class T> __global__ void argmax_attention_dt_kernel(ArgmaxAttentionBackwardArgs a) {
    const int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    const int64_t tokens = int64_t(a.batch) * a.context;
    if (i >= tokens * a.heads)
        return;
    const int d = a.width / a.heads, head = int(i % a.heads);
    const int64_t row = i / a.heads, key = row / a.context * a.context + a.selected[i];
    const T *dy = (const T *)a.dout + row * a.width + head * d;
    const T *v = (const T *)a.qkv + key * 3 * a.width + 2 * a.width + head * d;
    float dt = 0;
    for (int c = 0; c < d; ++c)
        dt += to_float(dy[c]) * to_float(v[c]);
    a.dt[i] = dt * a.derivatives[i];
}
// Pass 2: one thread per element of dqkv; keys gather from the queries that selected them.
template <class T> __global__ void argmax_attention_backward_kernel(ArgmaxAttentionBackwardArgs a) {
    const int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    const int64_t tokens = int64_t(a.batch) * a.context;
    if (i >= tokens * 3 * a.width)
        return;
    const int d = a.width / a.heads;
    const int64_t row = i / (3 * a.width);
    const int kind = int(i % (3 * a.width)) / a.width, col = int(i % a.width), head = col / d;
    const int64_t start = row / a.context * a.context;
    const T *qkv = (const T *)a.qkv;
    float value = 0;
    if (kind == 0) {
        int64_t key = start + a.selected[row * a.heads + head];
        value = a.dt[row * a.heads + head] * to_float(qkv[key * 3 * a.width + a.width + col]);
    } else {
        for (int64_t query = row; query < start + a.context; ++query) {
            if (start + a.selected[query * a.heads + head] != row)
                continue;
            if (kind == 1)
                value += a.dt[query * a.heads + head] * to_float(qkv[query * 3 * a.width + col]);
            else
                value += to_float(((const T *)a.dout)[query * a.width + col]) * a.gates[query * a.heads + head];
        }
    }
    ((T *)a.dqkv)[i] = from_float<T>(value);
}
void launch_argmax_attention_backward(Dtype t, const ArgmaxAttentionBackwardArgs &a, cudaStream_t s) {
    int64_t tokens = int64_t(a.batch) * a.context;
    DISPATCH(t, {
        argmax_attention_dt_kernel<T><<<int((tokens * a.heads + 127) / 128), 128, 0, s>>>(a);
        argmax_attention_backward_kernel<T><<<int((tokens * 3 * a.width + 255) / 256), 256, 0, s>>>(a);
    });
}

// ---------------------------------------------------------------- softmax attention ----------
constexpr int MaxHeadChunks = 8; // head size up to 256 = 8 chunks of 32 lanes
constexpr int AttentionWarps = 4;

// Dot product of a row held in shared memory (FP32) with a row in global memory.
template <class T> __device__ __forceinline__ float dot_row(const float *shared_row, const T *row, int d) {
    float sum = 0;
    for (int c = 0; c < d; c += 8) {
        float v[8];
        load8(row + c, v);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            sum += shared_row[c + j] * v[j];
    }
    return sum;
}

// One warp per query row.  Lanes take 32 keys at a time; the probabilities are then broadcast
// lane by lane while every lane accumulates its own output columns.
template <class T> __global__ void __launch_bounds__(AttentionWarps * 32) softmax_attention_kernel(SoftmaxAttentionArgs a) {
    extern __shared__ float shared[]; // [warps][d]
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int d = a.width / a.heads;
    const int64_t item = blockIdx.x * int64_t(AttentionWarps) + warp; // (batch, head, query)
    if (item >= int64_t(a.batch) * a.heads * a.context)
        return;
    const int query = int(item % a.context), head = int(item / a.context % a.heads);
    const int64_t b = item / a.context / a.heads, base = b * a.context;
    const T *qkv = (const T *)a.qkv;
    const int64_t ld = 3 * a.width;
    float *q = shared + warp * d;
    for (int c = lane; c < d; c += 32)
        q[c] = to_float(qkv[(base + query) * ld + head * d + c]);
    __syncwarp();
    const float scale = rsqrtf(float(d));
    float running_max = -CUDART_INF_F, running_sum = 0, acc[MaxHeadChunks] = {};
    for (int k0 = 0; k0 <= query; k0 += 32) {
        const int key = k0 + lane;
        float score = -CUDART_INF_F;
        if (key <= query)
            score = dot_row(q, qkv + (base + key) * ld + a.width + head * d, d) * scale;
        float new_max = fmaxf(running_max, warp_max(score));
        float correction = expf(running_max - new_max);
        float p = key <= query ? expf(score - new_max) : 0.f;
        running_sum = running_sum * correction + warp_sum(p);
        running_max = new_max;
#pragma unroll
        for (int j = 0; j < MaxHeadChunks; ++j)
            acc[j] *= correction;
        const int limit = min(32, query - k0 + 1);
        for (int i = 0; i < limit; ++i) {
            float pi = __shfl_sync(0xffffffffu, p, i);
            const T *v = qkv + (base + k0 + i) * ld + 2 * a.width + head * d;
#pragma unroll
            for (int j = 0; j < MaxHeadChunks; ++j)
                if (j * 32 + lane < d)
                    acc[j] += pi * to_float(v[j * 32 + lane]);
        }
    }
    T *out = (T *)a.out + (base + query) * a.width + head * d;
#pragma unroll
    for (int j = 0; j < MaxHeadChunks; ++j)
        if (j * 32 + lane < d)
            out[j * 32 + lane] = from_float<T>(acc[j] / running_sum);
    if (lane == 0)
        a.lse[(b * a.heads + head) * a.context + query] = running_max + logf(running_sum);
}
void launch_softmax_attention(Dtype t, const SoftmaxAttentionArgs &a, cudaStream_t s) {
    int64_t items = int64_t(a.batch) * a.heads * a.context;
    int d = a.width / a.heads;
    DISPATCH(t, (softmax_attention_kernel<T><<<int((items + AttentionWarps - 1) / AttentionWarps),
                                              AttentionWarps * 32, AttentionWarps * d * sizeof(float), s>>>(a)));
}

// delta[b, h, t] = sum_c dout * out.
template <class T> __global__ void attention_delta_kernel(SoftmaxAttentionBackwardArgs a) {
    const int lane = threadIdx.x % 32;
    const int d = a.width / a.heads;
    const int64_t item = blockIdx.x * int64_t(blockDim.x / 32) + threadIdx.x / 32;
    if (item >= int64_t(a.batch) * a.heads * a.context)
        return;
    const int t = int(item % a.context), head = int(item / a.context % a.heads);
    const int64_t b = item / a.context / a.heads, row = b * a.context + t;
    float sum = 0;
    for (int c = lane; c < d; c += 32)
        sum += to_float(((const T *)a.dout)[row * a.width + head * d + c]) *
               to_float(((const T *)a.out)[row * a.width + head * d + c]);
    sum = warp_sum(sum);
    if (lane == 0)
        a.delta[(b * a.heads + head) * a.context + t] = sum;
}
// dq: one warp per query row, lanes over keys.
template <class T> __global__ void __launch_bounds__(AttentionWarps * 32) attention_dq_kernel(SoftmaxAttentionBackwardArgs a) {
    extern __shared__ float shared[]; // [warps][2][d]: q row, dout row
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int d = a.width / a.heads;
    const int64_t item = blockIdx.x * int64_t(AttentionWarps) + warp;
    if (item >= int64_t(a.batch) * a.heads * a.context)
        return;
    const int query = int(item % a.context), head = int(item / a.context % a.heads);
    const int64_t b = item / a.context / a.heads, base = b * a.context;
    const T *qkv = (const T *)a.qkv;
    const int64_t ld = 3 * a.width;
    float *q = shared + warp * 2 * d, *dy = q + d;
    for (int c = lane; c < d; c += 32) {
        q[c] = to_float(qkv[(base + query) * ld + head * d + c]);
        dy[c] = to_float(((const T *)a.dout)[(base + query) * a.width + head * d + c]);
    }
    __syncwarp();
    const float scale = rsqrtf(float(d));
    const float lse = a.lse[(b * a.heads + head) * a.context + query];
    const float delta = a.delta[(b * a.heads + head) * a.context + query];
    float acc[MaxHeadChunks] = {};
    for (int k0 = 0; k0 <= query; k0 += 32) {
        const int key = k0 + lane;
        float ds = 0;
        if (key <= query) {
            float score = dot_row(q, qkv + (base + key) * ld + a.width + head * d, d) * scale;
            float dp = dot_row(dy, qkv + (base + key) * ld + 2 * a.width + head * d, d);
            ds = expf(score - lse) * (dp - delta) * scale;
        }
        const int limit = min(32, query - k0 + 1);
        for (int i = 0; i < limit; ++i) {
            float dsi = __shfl_sync(0xffffffffu, ds, i);
            const T *k = qkv + (base + k0 + i) * ld + a.width + head * d;
#pragma unroll
            for (int j = 0; j < MaxHeadChunks; ++j)
                if (j * 32 + lane < d)
                    acc[j] += dsi * to_float(k[j * 32 + lane]);
        }
    }
    T *dq = (T *)a.dqkv + (base + query) * ld + head * d;
#pragma unroll
    for (int j = 0; j < MaxHeadChunks; ++j)
        if (j * 32 + lane < d)
            dq[j * 32 + lane] = from_float<T>(acc[j]);
}
// dk, dv: one warp per key row, lanes over the queries at or after it.
template <class T> __global__ void __launch_bounds__(AttentionWarps * 32) attention_dkv_kernel(SoftmaxAttentionBackwardArgs a) {
    extern __shared__ float shared[]; // [warps][2][d]: k row, v row
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int d = a.width / a.heads;
    const int64_t item = blockIdx.x * int64_t(AttentionWarps) + warp;
    if (item >= int64_t(a.batch) * a.heads * a.context)
        return;
    const int key = int(item % a.context), head = int(item / a.context % a.heads);
    const int64_t b = item / a.context / a.heads, base = b * a.context;
    const T *qkv = (const T *)a.qkv;
    const T *dout = (const T *)a.dout;
    const int64_t ld = 3 * a.width;
    float *k = shared + warp * 2 * d, *v = k + d;
    for (int c = lane; c < d; c += 32) {
        k[c] = to_float(qkv[(base + key) * ld + a.width + head * d + c]);
        v[c] = to_float(qkv[(base + key) * ld + 2 * a.width + head * d + c]);
    }
    __syncwarp();
    const float scale = rsqrtf(float(d));
    const float *lse = a.lse + (b * a.heads + head) * a.context;
    const float *delta = a.delta + (b * a.heads + head) * a.context;
    float dk[MaxHeadChunks] = {}, dv[MaxHeadChunks] = {};
    for (int q0 = key; q0 < a.context; q0 += 32) {
        const int query = q0 + lane;
        float p = 0, ds = 0;
        if (query < a.context) {
            float score = dot_row(k, qkv + (base + query) * ld + head * d, d) * scale;
            float dp = dot_row(v, dout + (base + query) * a.width + head * d, d);
            p = expf(score - lse[query]);
            ds = p * (dp - delta[query]) * scale;
        }
        const int limit = min(32, a.context - q0);
        for (int i = 0; i < limit; ++i) {
            float pi = __shfl_sync(0xffffffffu, p, i), dsi = __shfl_sync(0xffffffffu, ds, i);
            const T *q = qkv + (base + q0 + i) * ld + head * d;
            const T *dy = dout + (base + q0 + i) * a.width + head * d;
#pragma unroll
            for (int j = 0; j < MaxHeadChunks; ++j)
                if (j * 32 + lane < d) {
                    dv[j] += pi * to_float(dy[j * 32 + lane]);
                    dk[j] += dsi * to_float(q[j * 32 + lane]);
                }
        }
    }
    T *out = (T *)a.dqkv + (base + key) * ld + head * d;
#pragma unroll
    for (int j = 0; j < MaxHeadChunks; ++j)
        if (j * 32 + lane < d) {
            out[a.width + j * 32 + lane] = from_float<T>(dk[j]);
            out[2 * a.width + j * 32 + lane] = from_float<T>(dv[j]);
        }
}
void launch_softmax_attention_backward(Dtype t, const SoftmaxAttentionBackwardArgs &a, cudaStream_t s) {
    int64_t items = int64_t(a.batch) * a.heads * a.context;
    int d = a.width / a.heads;
    int blocks = int((items + AttentionWarps - 1) / AttentionWarps);
    size_t shared = AttentionWarps * 2 * d * sizeof(float);
    DISPATCH(t, {
        attention_delta_kernel<T><<<blocks, AttentionWarps * 32, 0, s>>>(a);
        attention_dq_kernel<T><<<blocks, AttentionWarps * 32, shared, s>>>(a);
        attention_dkv_kernel<T><<<blocks, AttentionWarps * 32, shared, s>>>(a);
    });
}
