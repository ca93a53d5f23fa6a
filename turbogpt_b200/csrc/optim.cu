// Optimizer kernels (reference cuda/optim.cuh).  One fused pass over the flat parameter arena
// applies "mantissa" AdamW: FP32 masters are kept as a BF16 high half (the compute weight) and
// the 16 low mantissa bits, so updates below one BF16 ulp are retained.  Muon's elementwise
// stages sit either side of Newton-Schulz GEMMs issued by the host.
#include "device_utils.cuh"
#include "kernels.cuh"

// Fixed-order partial sums of squares: block b covers a contiguous slice.
__global__ void __launch_bounds__(256) sum_squares_kernel(const float *gradient, int64_t count, float *partial) {
    __shared__ float scratch[32];
    int64_t per = (count + gridDim.x - 1) / gridDim.x;
    per = (per + 3) / 4 * 4;
    int64_t begin = blockIdx.x * per, end = begin + per < count ? begin + per : count;
    float sum = 0;
    int64_t i = begin + threadIdx.x * 4;
    for (; i + 3 * 1024 + 4 <= end; i += 4 * 1024) { // four independent 128-bit loads in flight per thread
        float4 g[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            g[u] = *reinterpret_cast<const float4 *>(gradient + i + u * 1024);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            sum += g[u].x * g[u].x + g[u].y * g[u].y + g[u].z * g[u].z + g[u].w * g[u].w;
    }
    for (; i < end; i += 256 * 4) {
        if (i + 4 <= end) {
            float4 g = *reinterpret_cast<const float4 *>(gradient + i);
            sum += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
        } else {
            for (int64_t j = i; j < end; ++j)
                sum += gradient[j] * gradient[j];
        }
    }
    sum = block_sum(sum, scratch);
    if (threadIdx.x == 0)
        partial[blockIdx.x] = sum;
}
void launch_sum_squares(const float *gradient, int64_t count, float *partial, int blocks, cudaStream_t s) {
    sum_squares_kernel<<<blocks, 256, 0, s>>>(gradient, count, partial);
}

// clip = min(1, clip / (|g| + 1e-6)) from the per-block sums, same order in every block.
__device__ __forceinline__ float clip_factor(const float *norm_partial, int norm_blocks, float clip,
                                             float *scratch) {
    if (!(clip > 0))
        return 1.f;
    float local = 0;
    for (int b = threadIdx.x; b < norm_blocks; b += blockDim.x)
        local += norm_partial[b];
    float norm = block_sum(local, scratch);
    return fminf(1.f, clip / (sqrtf(norm) + 1e-6f));
}

__global__ void __launch_bounds__(256) adamw_kernel(AdamArgs a) {
    __shared__ float scratch[32];
    const float clip = clip_factor(a.norm_partial, a.norm_blocks, a.clip, scratch);
    const unsigned long long step = a.counters->step;
    float multiplier = 1, beta1 = a.beta1;
    if (a.schedule) { // every update reads its own schedule point (reference cuda/optim.cuh:82-89)
        TgStepRates rates = a.schedule[step];
        multiplier = rates.multiplier;
        beta1 = rates.momentum;
    }
    const float lr = a.learning_rate * multiplier;
    // Bias correction with the current, possibly cycled, beta1 as torch.optim.AdamW does.
    const float bc1 = 1 - powf(beta1, float(step + 1)), bc2 = 1 - powf(a.beta2, float(step + 1));
    const float step_size = lr / bc1, inv_sqrt_bc2 = 1.f / sqrtf(bc2);
    const int64_t groups = a.count / 8;
    for (int64_t group = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; group < groups;
         group += int64_t(gridDim.x) * blockDim.x) {
        const int mode = a.mode[group];
        if (mode == 0)
            continue;
        const int64_t i = group * 8;
        const float decay = 1 - lr * (mode == 2 ? a.weight_decay : 0.f);
        float g[8], m[8], v[8], w[8];
        load8(a.gradient + i, g);
        load8(a.momentum + i, m);
        load8(a.variance + i, v);
        uint4 high = *reinterpret_cast<const uint4 *>(a.weight_high + i);
        uint4 low = *reinterpret_cast<const uint4 *>(a.weight_low + i);
        const unsigned hw[4] = {high.x, high.y, high.z, high.w}, lw[4] = {low.x, low.y, low.z, low.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            w[2 * j] = __uint_as_float((hw[j] << 16) | (lw[j] & 0xffffu));
            w[2 * j + 1] = __uint_as_float((hw[j] & 0xffff0000u) | (lw[j] >> 16));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float gj = g[j] * clip;
            m[j] = m[j] + (1 - beta1) * (gj - m[j]);
            v[j] = a.beta2 * v[j] + (1 - a.beta2) * gj * gj;
            w[j] = w[j] * decay - step_size * m[j] / (sqrtf(v[j]) * inv_sqrt_bc2 + a.epsilon);
        }
        store8(a.momentum + i, m);
        store8(a.variance + i, v);
        unsigned ho[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            unsigned b0 = __float_as_uint(w[2 * j]), b1 = __float_as_uint(w[2 * j + 1]);
            ho[j] = (b0 >> 16) | (b1 & 0xffff0000u);
            lo[j] = (b0 & 0xffffu) | (b1 << 16);
        }
        *reinterpret_cast<uint4 *>(a.weight_high + i) = make_uint4(ho[0], ho[1], ho[2], ho[3]);
        *reinterpret_cast<uint4 *>(a.weight_low + i) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        if (a.weight_fp32)
            store8(a.weight_fp32 + i, w);
    }
}
void launch_adamw(const AdamArgs &a, int sms, cudaStream_t s) {
    int64_t groups = a.count / 8;
    int64_t blocks = (groups + 255) / 256;
    if (blocks > int64_t(sms) * 8)
        blocks = int64_t(sms) * 8;
    adamw_kernel<<<int(blocks < 1 ? 1 : blocks), 256, 0, s>>>(a);
}

// ---- Muon (reference cuda/optim.cuh:16-65) ----

__global__ void __launch_bounds__(256) muon_prepare_kernel(MuonPrepareArgs a) {
    __shared__ float scratch[32];
    const float clip = clip_factor(a.norm_partial, a.norm_blocks, a.clip, scratch);
    float mu = a.momentum_rate;
    if (a.schedule)
        mu = a.schedule[a.counters->step].momentum;
    const int matrix = blockIdx.y;
    const int64_t size = int64_t(a.rows) * a.cols, base = matrix * a.stride;
    const bool transpose = a.rows > a.cols;
    float squares = 0;
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < size;
         i += int64_t(gridDim.x) * blockDim.x) {
        float g = a.gradient[base + i] * clip;
        float m = a.momentum[base + i] + (1 - mu) * (g - a.momentum[base + i]);
        a.momentum[base + i] = m;
        bf16 u = __float2bfloat16_rn(g + mu * (m - g));
        int64_t index = transpose ? (i % a.cols) * a.rows + i / a.cols : i;
        a.x[matrix * size + index] = u;
        squares += __bfloat162float(u) * __bfloat162float(u);
    }
    squares = block_sum(squares, scratch);
    if (threadIdx.x == 0)
        a.sumsq[matrix * MuonBlocks + blockIdx.x] = squares;
}
void launch_muon_prepare(const MuonPrepareArgs &a, cudaStream_t s) {
    muon_prepare_kernel<<<dim3(MuonBlocks, a.batch), 256, 0, s>>>(a);
}
// x /= max(bf16(|x|_F), bf16(1e-7)), rounded to BF16.
__global__ void __launch_bounds__(256) muon_normalize_kernel(bf16 *x, const float *sumsq, int64_t per_matrix) {
    const int matrix = blockIdx.y;
    float total = 0;
    for (int b = 0; b < MuonBlocks; ++b)
        total += sumsq[matrix * MuonBlocks + b];
    const float norm = fmaxf(__bfloat162float(__float2bfloat16_rn(sqrtf(total))),
                             __bfloat162float(__float2bfloat16_rn(1e-7f)));
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < per_matrix;
         i += int64_t(gridDim.x) * blockDim.x)
        x[matrix * per_matrix + i] = __float2bfloat16_rn(__bfloat162float(x[matrix * per_matrix + i]) / norm);
}
void launch_muon_normalize(bf16 *x, const float *sumsq, int64_t per_matrix, int batch, cudaStream_t s) {
    muon_normalize_kernel<<<dim3(MuonBlocks, batch), 256, 0, s>>>(x, sumsq, per_matrix);
}
// w = w * (1 - lr * wd) - lr * sqrt(max(1, rows/cols)) * x, x transposed back when rows > cols.
__global__ void __launch_bounds__(256) muon_apply_kernel(MuonApplyArgs a) {
    float multiplier = 1;
    if (a.schedule)
        multiplier = a.schedule[a.counters->step].multiplier;
    const float lr = a.muon_lr * multiplier;
    const float adjusted = lr * sqrtf(fmaxf(1.f, float(a.rows) / a.cols));
    const int matrix = blockIdx.y;
    const int64_t size = int64_t(a.rows) * a.cols, base = matrix * a.stride;
    const bool transpose = a.rows > a.cols;
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < size;
         i += int64_t(gridDim.x) * blockDim.x) {
        int64_t index = transpose ? (i % a.cols) * a.rows + i / a.cols : i;
        float w = join_weight(a.weight_high[base + i], a.weight_low[base + i]) * (1 - lr * a.weight_decay);
        w -= adjusted * __bfloat162float(a.x[matrix * size + index]);
        unsigned bits = __float_as_uint(w);
        a.weight_high[base + i] = __ushort_as_bfloat16((unsigned short)(bits >> 16));
        a.weight_low[base + i] = uint16_t(bits);
        if (a.weight_fp32)
            a.weight_fp32[base + i] = w;
    }
}
void launch_muon_apply(const MuonApplyArgs &a, cudaStream_t s) {
    muon_apply_kernel<<<dim3(MuonBlocks, a.batch), 256, 0, s>>>(a);
}

__global__ void advance_kernel(StepCounters *counters) {
    counters->step += 1;
    counters->iteration += 1;
}
void launch_advance(StepCounters *counters, cudaStream_t s) {
    advance_kernel<<<1, 1, 0, s>>>(counters);
}
