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
// The same stage, 128-bit: eight consecutive elements per thread (matrices stored in the orientation the
// iterations use, rows <= cols).
__global__ void __launch_bounds__(256) muon_prepare_vector_kernel(MuonPrepareArgs a) {
    __shared__ float scratch[32];
    const float clip = clip_factor(a.norm_partial, a.norm_blocks, a.clip, scratch);
    float mu = a.momentum_rate;
    if (a.schedule)
        mu = a.schedule[a.counters->step].momentum;
    const int matrix = blockIdx.y;
    const int64_t size = int64_t(a.rows) * a.cols, base = matrix * a.stride;
    float squares = 0;
    for (int64_t i = (blockIdx.x * int64_t(blockDim.x) + threadIdx.x) * 8; i < size;
         i += int64_t(gridDim.x) * blockDim.x * 8) {
        float g[8], m[8], u[8];
        load8(a.gradient + base + i, g);
        load8(a.momentum + base + i, m);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            g[j] *= clip;
            m[j] += (1 - mu) * (g[j] - m[j]);
            u[j] = rounded<bf16>(g[j] + mu * (m[j] - g[j]));
            squares += u[j] * u[j];
        }
        store8(a.momentum + base + i, m);
        store8(a.x + matrix * size + i, u);
    }
    squares = block_sum(squares, scratch);
    if (threadIdx.x == 0)
        a.sumsq[matrix * MuonBlocks + blockIdx.x] = squares;
}
// Tall matrices (rows > cols) are orthogonalised transposed.  64 x 64 tiles go through shared memory so
// that gradient and momentum are read, and the transposed BF16 matrix written, in whole 128-byte lines.
constexpr int MuonTile = 64, MuonTilePitch = 66; // BF16 elements per tile row in shared memory (33 words: spreads the banks)
__global__ void __launch_bounds__(256) muon_prepare_transpose_kernel(MuonPrepareArgs a) {
    __shared__ float scratch[32];
    __shared__ __align__(16) bf16 tile[MuonTile * MuonTilePitch]; // [column][row]
    const float clip = clip_factor(a.norm_partial, a.norm_blocks, a.clip, scratch);
    float mu = a.momentum_rate;
    if (a.schedule)
        mu = a.schedule[a.counters->step].momentum;
    const int matrix = blockIdx.y;
    const int64_t size = int64_t(a.rows) * a.cols, base = matrix * a.stride;
    const int tiles_across = a.cols / MuonTile, tiles = (a.rows / MuonTile) * tiles_across;
    float squares = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int r0 = t / tiles_across * MuonTile, c0 = t % tiles_across * MuonTile;
        for (int item = threadIdx.x; item < MuonTile * 8; item += blockDim.x) { // (row, group of 8 columns)
            const int rr = item / 8, chunk = item % 8;
            const int64_t at = base + int64_t(r0 + rr) * a.cols + c0 + chunk * 8;
            float g[8], m[8];
            load8(a.gradient + at, g);
            load8(a.momentum + at, m);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                g[j] *= clip;
                m[j] += (1 - mu) * (g[j] - m[j]);
                const bf16 u = __float2bfloat16_rn(g[j] + mu * (m[j] - g[j]));
                tile[(chunk * 8 + j) * MuonTilePitch + rr] = u;
                squares += __bfloat162float(u) * __bfloat162float(u);
            }
            store8(a.momentum + at, m);
        }
        __syncthreads();
        for (int item = threadIdx.x; item < MuonTile * 8; item += blockDim.x) { // (column, group of 8 rows)
            const int cc = item / 8, chunk = item % 8;
            const uint32_t *source = reinterpret_cast<const uint32_t *>(tile + cc * MuonTilePitch + chunk * 8);
            *reinterpret_cast<uint4 *>(a.x + matrix * size + int64_t(c0 + cc) * a.rows + r0 + chunk * 8) =
                make_uint4(source[0], source[1], source[2], source[3]);
        }
        __syncthreads();
    }
    squares = block_sum(squares, scratch);
    if (threadIdx.x == 0)
        a.sumsq[matrix * MuonBlocks + blockIdx.x] = squares;
}
void launch_muon_prepare(const MuonPrepareArgs &a, cudaStream_t s) {
    const dim3 grid(MuonBlocks, a.batch);
    const bool aligned = a.stride % 8 == 0 && reinterpret_cast<uintptr_t>(a.gradient) % 32 == 0 &&
                         reinterpret_cast<uintptr_t>(a.momentum) % 32 == 0;
    if (aligned && a.rows > a.cols && a.rows % MuonTile == 0 && a.cols % MuonTile == 0)
        muon_prepare_transpose_kernel<<<grid, 256, 0, s>>>(a);
    else if (aligned && a.rows <= a.cols && (int64_t(a.rows) * a.cols) % 8 == 0)
        muon_prepare_vector_kernel<<<grid, 256, 0, s>>>(a);
    else
        muon_prepare_kernel<<<grid, 256, 0, s>>>(a);
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
__global__ void __launch_bounds__(256) muon_normalize_vector_kernel(bf16 *x, const float *sumsq, int64_t per_matrix) {
    const int matrix = blockIdx.y;
    float total = 0;
    for (int b = 0; b < MuonBlocks; ++b)
        total += sumsq[matrix * MuonBlocks + b];
    const float norm = fmaxf(__bfloat162float(__float2bfloat16_rn(sqrtf(total))),
                             __bfloat162float(__float2bfloat16_rn(1e-7f)));
    for (int64_t i = (blockIdx.x * int64_t(blockDim.x) + threadIdx.x) * 8; i < per_matrix;
         i += int64_t(gridDim.x) * blockDim.x * 8) {
        float v[8];
        load8(x + matrix * per_matrix + i, v);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            v[j] /= norm;
        store8(x + matrix * per_matrix + i, v);
    }
}
void launch_muon_normalize(bf16 *x, const float *sumsq, int64_t per_matrix, int batch, cudaStream_t s) {
    if (per_matrix % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0)
        muon_normalize_vector_kernel<<<dim3(MuonBlocks, batch), 256, 0, s>>>(x, sumsq, per_matrix);
    else
        muon_normalize_kernel<<<dim3(MuonBlocks, batch), 256, 0, s>>>(x, sumsq, per_matrix);
}
// All Newton-Schulz iterations of one small matrix (the reference architecture's 16 x 16 .. 16 x 48) in one
// block's shared memory, with the roundings of the three-GEMM form: BF16 operands, FP32 sums over ascending k,
// A = X X^T, B = 2.0315 A A - 4.775 A and X' = B X + 3.4445 X each rounded to BF16 (reference
// cuda/optim.cuh:60-106).  One launch instead of three per iteration.
__global__ void __launch_bounds__(256) muon_newton_schulz_small_kernel(bf16 *x_all, int r, int n, int steps) {
    extern __shared__ float shared[];
    float *x = shared, *a = x + r * n, *b = a + r * r, *next = b + r * r;
    bf16 *matrix = x_all + int64_t(blockIdx.x) * r * n;
    for (int i = threadIdx.x; i < r * n; i += blockDim.x)
        x[i] = __bfloat162float(matrix[i]);
    __syncthreads();
    for (int step = 0; step < steps; ++step) {
        for (int i = threadIdx.x; i < r * r; i += blockDim.x) {
            const float *p = x + (i / r) * n, *q = x + (i % r) * n;
            float sum = 0.f;
            for (int k = 0; k < n; ++k)
                sum = fmaf(p[k], q[k], sum);
            a[i] = rounded<bf16>(sum);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < r * r; i += blockDim.x) {
            const float *p = a + (i / r) * r;
            const int column = i % r;
            float sum = 0.f;
            for (int k = 0; k < r; ++k)
                sum = fmaf(p[k], a[k * r + column], sum);
            b[i] = rounded<bf16>(2.0315f * sum + -4.775f * a[i]);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < r * n; i += blockDim.x) {
            const float *p = b + (i / n) * r;
            const int column = i % n;
            float sum = 0.f;
            for (int k = 0; k < r; ++k)
                sum = fmaf(p[k], x[k * n + column], sum);
            next[i] = rounded<bf16>(1.f * sum + 3.4445f * x[i]);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < r * n; i += blockDim.x)
            x[i] = next[i];
        __syncthreads();
    }
    for (int i = threadIdx.x; i < r * n; i += blockDim.x)
        matrix[i] = __float2bfloat16(x[i]);
}
bool muon_newton_schulz_small_supported(int r, int n) { return r <= 32 && n <= 128; }
void launch_muon_newton_schulz_small(bf16 *x, int r, int n, int steps, int matrices, cudaStream_t s) {
    const size_t bytes = size_t(2 * r * n + 2 * r * r) * sizeof(float); // at most 40 KB
    muon_newton_schulz_small_kernel<<<matrices, 256, bytes, s>>>(x, r, n, steps);
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
// Eight consecutive weights per thread: both 16-bit halves of the FP32 masters as 128-bit accesses.
__device__ __forceinline__ void muon_update8(const MuonApplyArgs &a, int64_t at, const float (&x)[8], float keep,
                                             float adjusted) {
    const uint4 high = *reinterpret_cast<const uint4 *>(a.weight_high + at);
    const uint4 low = *reinterpret_cast<const uint4 *>(a.weight_low + at);
    const unsigned h[4] = {high.x, high.y, high.z, high.w}, l[4] = {low.x, low.y, low.z, low.w};
    unsigned ho[4], lo[4];
    float w[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        w[2 * j] = __uint_as_float((h[j] << 16) | (l[j] & 0xffffu));
        w[2 * j + 1] = __uint_as_float((h[j] & 0xffff0000u) | (l[j] >> 16));
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        w[j] *= keep;
        w[j] -= adjusted * x[j];
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const unsigned b0 = __float_as_uint(w[2 * j]), b1 = __float_as_uint(w[2 * j + 1]);
        ho[j] = (b0 >> 16) | (b1 & 0xffff0000u);
        lo[j] = (b0 & 0xffffu) | (b1 << 16);
    }
    *reinterpret_cast<uint4 *>(a.weight_high + at) = make_uint4(ho[0], ho[1], ho[2], ho[3]);
    *reinterpret_cast<uint4 *>(a.weight_low + at) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    if (a.weight_fp32)
        store8(a.weight_fp32 + at, w);
}
__global__ void __launch_bounds__(256) muon_apply_vector_kernel(MuonApplyArgs a) {
    float multiplier = 1;
    if (a.schedule)
        multiplier = a.schedule[a.counters->step].multiplier;
    const float lr = a.muon_lr * multiplier;
    const float adjusted = lr * sqrtf(fmaxf(1.f, float(a.rows) / a.cols)), keep = 1 - lr * a.weight_decay;
    const int matrix = blockIdx.y;
    const int64_t size = int64_t(a.rows) * a.cols, base = matrix * a.stride;
    for (int64_t i = (blockIdx.x * int64_t(blockDim.x) + threadIdx.x) * 8; i < size;
         i += int64_t(gridDim.x) * blockDim.x * 8) {
        float x[8];
        load8(a.x + matrix * size + i, x);
        muon_update8(a, base + i, x, keep, adjusted);
    }
}
__global__ void __launch_bounds__(256) muon_apply_transpose_kernel(MuonApplyArgs a) {
    __shared__ __align__(16) bf16 tile[MuonTile * MuonTilePitch]; // [column][row], as stored
    float multiplier = 1;
    if (a.schedule)
        multiplier = a.schedule[a.counters->step].multiplier;
    const float lr = a.muon_lr * multiplier;
    const float adjusted = lr * sqrtf(fmaxf(1.f, float(a.rows) / a.cols)), keep = 1 - lr * a.weight_decay;
    const int matrix = blockIdx.y;
    const int64_t size = int64_t(a.rows) * a.cols, base = matrix * a.stride;
    const int tiles_across = a.cols / MuonTile, tiles = (a.rows / MuonTile) * tiles_across;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int r0 = t / tiles_across * MuonTile, c0 = t % tiles_across * MuonTile;
        for (int item = threadIdx.x; item < MuonTile * 8; item += blockDim.x) { // (column, group of 8 rows)
            const int cc = item / 8, chunk = item % 8;
            const uint4 v = *reinterpret_cast<const uint4 *>(a.x + matrix * size + int64_t(c0 + cc) * a.rows + r0 + chunk * 8);
            uint32_t *target = reinterpret_cast<uint32_t *>(tile + cc * MuonTilePitch + chunk * 8);
            target[0] = v.x, target[1] = v.y, target[2] = v.z, target[3] = v.w;
        }
        __syncthreads();
        for (int item = threadIdx.x; item < MuonTile * 8; item += blockDim.x) { // (row, group of 8 columns)
            const int rr = item / 8, chunk = item % 8;
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                x[j] = __bfloat162float(tile[(chunk * 8 + j) * MuonTilePitch + rr]);
            muon_update8(a, base + int64_t(r0 + rr) * a.cols + c0 + chunk * 8, x, keep, adjusted);
        }
        __syncthreads();
    }
}
void launch_muon_apply(const MuonApplyArgs &a, cudaStream_t s) {
    const dim3 grid(MuonBlocks, a.batch);
    const bool aligned = a.stride % 8 == 0 && reinterpret_cast<uintptr_t>(a.weight_high) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(a.weight_low) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(a.weight_fp32) % 32 == 0 && reinterpret_cast<uintptr_t>(a.x) % 16 == 0;
    if (aligned && a.rows > a.cols && a.rows % MuonTile == 0 && a.cols % MuonTile == 0)
        muon_apply_transpose_kernel<<<grid, 256, 0, s>>>(a);
    else if (aligned && a.rows <= a.cols && (int64_t(a.rows) * a.cols) % 8 == 0)
        muon_apply_vector_kernel<<<grid, 256, 0, s>>>(a);
    else
        muon_apply_kernel<<<grid, 256, 0, s>>>(a);
}

__global__ void advance_kernel(StepCounters *counters) {
    counters->step += 1;
    counters->iteration += 1;
}
void launch_advance(StepCounters *counters, cudaStream_t s) {
    advance_kernel<<<1, 1, 0, s>>>(counters);
}
