// Launchers of every device kernel of the training step.  All take the stream to enqueue on;
// all element counts are in elements, all leading dimensions in elements.
#pragma once
#include "common.h"

// Element type of activations and compute weights: BF16 (training) or FP32 (check mode).
enum class Dtype { BF16 = 0, FP32 = 1 };
inline size_t dtype_size(Dtype t) { return t == Dtype::BF16 ? 2 : 4; }

// Device-resident step counters, advanced by a kernel so that a captured step replays
// without host involvement (the reference keeps them in the persistent kernel's loop,
// cuda/trainer.cuh:108-124).
struct StepCounters {
    unsigned long long step; // absolute optimizer step: data sampling, schedule, bias correction
    int iteration;           // index inside the current tg_train launch: row of loss_history
    int error;               // first device-side error code (bounded waits that gave up), 0 = none
};

// ---- data + embedding (reference cuda/dataset.cuh:7-34) ----
struct SampleArgs {
    const uint8_t *data;
    int64_t size;
    uint64_t seed;
    const StepCounters *counters; // step read on device unless fixed_step >= 0
    long long fixed_step;
    int batch, context, world, rank;
    uint8_t *x, *y; // [batch*context]
};
void launch_sample(const SampleArgs &a, cudaStream_t s);
void launch_embedding(Dtype t, const void *table, const uint8_t *x, void *hidden, int tokens, int width,
                      cudaStream_t s);
// grad[x[t]*width + c] += dhidden[t, c] in FP32 (reference cuda/model.cuh:96-97), deterministic:
// one CTA per byte value scans the tokens in order.
// `scratch`: EmbeddingSlices x 256 x width floats (nullptr: single-pass kernel for small shapes).
constexpr int EmbeddingSlices = 8;
void launch_embedding_backward(Dtype t, const void *dhidden, const uint8_t *x, float *grad, int tokens,
                               int width, bool accumulate, float *scratch, cudaStream_t s);

// ---- norms (reference cuda/ops.cuh:56-80) ----
struct NormArgs {
    int kind; // TG_NORM_RMS / TG_NORM_LAYER
    const void *x;
    const bf16 *scale_high, *bias_high; // FP32 master values as their two 16-bit halves;
    const uint16_t *scale_low, *bias_low; // bias pointers are nullptr for RMSNorm
    void *y;
    int rows, width;
    float *stats = nullptr; // optional [rows][2]: mean and 1/sqrt(variance + eps) of every row, for the backward pass
};
void launch_norm(Dtype t, const NormArgs &a, cudaStream_t s);
struct NormBackwardArgs {
    int kind;
    const void *x, *dy;
    const bf16 *scale_high;
    const uint16_t *scale_low;
    const void *residual_in; // running residual-stream gradient to add (nullptr: none)
    void *dx;
    float *partial;          // [blocks][2][width] scratch for scale/bias gradients
    float *dscale, *dbias;   // outputs (overwritten); dbias nullptr for RMSNorm
    int rows, width, blocks;
    const float *stats = nullptr; // [rows][2] from the forward pass (nullptr: recomputed from x)
};
void launch_norm_backward(Dtype t, const NormBackwardArgs &a, cudaStream_t s);
int norm_backward_blocks(int rows, int sms);

// ---- positional rotation (reference cuda/attention.cuh:19-30) ----
void launch_rope(Dtype t, void *qkv, int tokens, int context, int width, int heads, bool inverse,
                 cudaStream_t s);

// ---- arg-max attention (reference cuda/attention.cuh:33-106) ----
struct ArgmaxAttentionArgs {
    const void *qkv; // [tokens, 3*width]
    void *out;       // [tokens, width]
    int *selected;   // [tokens, heads]
    float *gates, *derivatives;
    int batch, context, width, heads;
};
void launch_argmax_attention(Dtype t, const ArgmaxAttentionArgs &a, cudaStream_t s);
struct ArgmaxAttentionBackwardArgs {
    const void *qkv, *dout;
    const int *selected;
    const float *gates, *derivatives;
    float *dt;  // [tokens, heads] scratch
    void *dqkv; // [tokens, 3*width]
    int batch, context, width, heads;
};
void launch_argmax_attention_backward(Dtype t, const ArgmaxAttentionBackwardArgs &a, cudaStream_t s);

// ---- causal softmax attention on CUDA cores (any head size up to 256, BF16 or FP32) ----
struct SoftmaxAttentionArgs {
    const void *qkv; // [batch*context, 3*width], q | k | v
    void *out;       // [batch*context, width]
    float *lse;      // [batch, heads, context]
    int batch, context, width, heads;
};
void launch_softmax_attention(Dtype t, const SoftmaxAttentionArgs &a, cudaStream_t s);
struct SoftmaxAttentionBackwardArgs {
    const void *qkv, *out, *dout;
    const float *lse;
    float *delta; // [batch, heads, context] scratch: rowsum(dout * out)
    void *dqkv;
    int batch, context, width, heads;
};
void launch_softmax_attention_backward(Dtype t, const SoftmaxAttentionBackwardArgs &a, cudaStream_t s);

// ---- causal softmax attention on tcgen05 (BF16, head size 64) ----
bool flash_attention_supported(int width, int heads);
void launch_flash_attention_forward(const void *qkv, void *out, float *lse, int batch, int context, int heads,
                                    StepCounters *counters, cudaStream_t s);

// `scratch`: flash_attention_backward_scratch_bytes() bytes; the dq kernel fills it with every query's lse
// (base 2) and rowsum(dout * out) for the dk/dv kernel.
size_t flash_attention_backward_scratch_bytes(int batch, int context, int heads);
void launch_flash_attention_backward(const void *qkv, const void *out, const void *dout, const float *lse,
                                     float *scratch, void *dqkv, int batch, int context, int heads,
                                     StepCounters *counters, cudaStream_t s);

// One fused kernel for dQ, dK and dV (attention_bwd_fused.cu): every probability is exponentiated once.
// `scratch` (flash_backward_scratch_bytes) holds the FP32 running sums of dQ between key tiles and their
// counters; `delta` as above.
size_t flash_backward_scratch_bytes(int batch, int context, int heads);
void launch_flash_attention_backward_fused(const void *qkv, const void *out, const void *dout, const float *lse, void *dqkv, void *scratch, int batch, int context, int heads,
                                           StepCounters *counters, cudaStream_t s);

// ---- MLP activations (reference cuda/ops.cuh:118-144) ----
// wide: [tokens, 2*hidden] = gate | up.  out: [tokens, hidden].
void launch_swiglu(Dtype t, const void *wide, void *out, int tokens, int hidden, cudaStream_t s);
// dwide = d(gate | up) from dout, recomputing the activation with the forward's roundings.
void launch_swiglu_backward(Dtype t, const void *wide, const void *dout, void *dwide, int tokens, int hidden,
                            cudaStream_t s);

// ---- 256-way softmax cross-entropy (reference cuda/model.cuh:33-57) ----
struct CrossEntropyArgs {
    const void *logits;  // [rows, 256]
    const uint8_t *targets;
    float *losses;       // [rows]
    void *dlogits;       // [rows, 256], may alias logits; nullptr: forward only
    float *logits_fp32;  // optional FP32 copy of the logits (diagnostic calls)
    float divisor;       // global batch * context
    int rows;
};
void launch_cross_entropy(Dtype t, const CrossEntropyArgs &a, cudaStream_t s);

// ---- per-position loss history (reference cuda/trainer.cuh:79-100) ----
void launch_loss_history(const float *token_losses, float *history, const StepCounters *counters, int batch,
                         int context, cudaStream_t s);

// ---- GEMM dispatcher: C[m,n] = sum_k A[m,k] * B[n,k] (reference cuda/mma.cuh:77-108,
//      cuda/ops.cuh:30-55,83-117) ----
enum class Epilogue {
    Store = 0,     // C = acc
    Residual = 1,  // C = round(acc) + R            (reference cuda/mma.cuh:96-99)
    GeluDual = 2,  // pre = round(acc); C = gelu'(pre) (kept for backward); C2 = gelu(pre)
    GeluGrad = 3,  // C = round(acc) * R, R = the saved gelu'(pre)
    Axpby = 4,     // C = alpha * acc + beta * R    (Newton-Schulz updates)
    // 256-way softmax cross-entropy on the FP32 accumulators (reference cuda/model.cuh:31-58 fuses the head
    // and the loss the same way; the logits never reach memory): n = 256; R = uint8 targets [m];
    // C2 = FP32 losses [m]; C = BF16 (softmax - onehot) * alpha, or nullptr for the loss alone.
    CrossEntropy = 5,
};
struct GemmArgs {
    Dtype in = Dtype::BF16, out = Dtype::BF16;
    const void *a = nullptr;
    int64_t a_row = 0, a_col = 1;
    const void *b = nullptr;
    int64_t b_row = 0, b_col = 1;
    void *c = nullptr;
    int64_t ldc = 0;
    int m = 0, n = 0, k = 0;
    Epilogue epilogue = Epilogue::Store;
    const void *r = nullptr; // residual / pre-activation / axpby operand, [m, n] with ldr, type `out` (GeluGrad: `in`)
    int64_t ldr = 0;
    void *c2 = nullptr;      // second output of GeluDual, ldc
    float alpha = 1.f, beta = 0.f;
    int batch = 1;           // batched over z with element strides below
    int64_t a_batch = 0, b_batch = 0, c_batch = 0, r_batch = 0;
};
// `scratch`: gemm_simt_scratch_bytes(g) bytes for shapes that are cut along K (small outputs over a long K,
// partial tiles added in a fixed order); nullptr: never cut.
size_t gemm_simt_scratch_bytes(const GemmArgs &g);
void launch_gemm_simt(const GemmArgs &g, cudaStream_t s, float *scratch = nullptr);
// tcgen05 path; returns false when the shape/layout is outside what it supports.
bool gemm_tc_supported(const GemmArgs &g);
// Split-K scratch of the tcgen05 GEMM: FP32 partial tiles, one ticket per output tile (zero between
// launches) and a device error word.  An Engine owns one, so engines never share scratch; it is grown
// by launch_gemm_tc when a schedule needs more (never during stream capture: the engine runs one eager
// step first) and `generation` changes whenever a pointer does.
struct GemmWorkspace {
    float *partials = nullptr;
    unsigned *tickets = nullptr;
    StepCounters *error_word = nullptr;
    size_t partial_bytes = 0, ticket_count = 0;
    uint64_t generation = 1;
};
void release_gemm_workspace(GemmWorkspace &w);
// Returns the number of kernels it launched.
int launch_gemm_tc(const GemmArgs &g, int sms, StepCounters *counters, cudaStream_t s,
                    GemmWorkspace *workspace = nullptr);
int gemm_tc_shared_bytes();
int gemm_tc_take_device_error(cudaStream_t s);
// Weight gradient dW[out, in] = dy^T x whose split-K scratch is a fixed array inside the library:
// allocates nothing (see gemm_tc.cu).  Throws when the shape needs more scratch than the array holds.
void launch_weight_gradient_static(const void *dy, const void *x, float *dw, int out, int in, int tokens, int sms,
                                   cudaStream_t s);
size_t gemm_tc_static_scratch_bytes();

// ---- optimizer (reference cuda/optim.cuh) ----
void launch_sum_squares(const float *gradient, int64_t count, float *partial, int blocks, cudaStream_t s);
struct AdamArgs {
    const float *gradient;
    float *momentum, *variance;
    bf16 *weight_high;
    uint16_t *weight_low;
    float *weight_fp32;        // optional FP32 compute copy (check mode)
    const uint8_t *mode;       // per 8 parameters: 0 skip (Muon), 1 AdamW, 2 AdamW + decay
    const float *norm_partial; // per-block sums of squares
    int norm_blocks;
    const TgStepRates *schedule; // nullptr: constant rates
    const StepCounters *counters;
    float learning_rate, beta1, beta2, weight_decay, epsilon, clip;
    int64_t count;
};
void launch_adamw(const AdamArgs &a, int sms, cudaStream_t s);
constexpr int MuonBlocks = 32; // blocks per matrix in the Muon prepare stage = partial sums per matrix
struct MuonPrepareArgs { // momentum, Nesterov direction, BF16 cast (+ transpose when rows > cols), sum of squares
    const float *gradient;
    float *momentum;
    bf16 *x;             // [batch][min(rows,cols)][max(rows,cols)]
    float *sumsq;        // [batch][MuonBlocks] partial sums of squares, summed in order by the normalise stage
    const float *norm_partial;
    int norm_blocks;
    const TgStepRates *schedule;
    const StepCounters *counters;
    float momentum_rate, clip;
    int rows, cols, batch;
    int64_t stride;      // elements between consecutive matrices of the batch in the flat arrays
};
void launch_muon_prepare(const MuonPrepareArgs &a, cudaStream_t s);
void launch_muon_normalize(bf16 *x, const float *sumsq, int64_t per_matrix, int batch, cudaStream_t s);
// `matrices` consecutive [r, n] BF16 matrices (r <= n), orthogonalised in place by `steps` Newton-Schulz iterations.
bool muon_newton_schulz_small_supported(int r, int n);
void launch_muon_newton_schulz_small(bf16 *x, int r, int n, int steps, int matrices, cudaStream_t s);
struct MuonApplyArgs {
    const bf16 *x;
    bf16 *weight_high;
    uint16_t *weight_low;
    float *weight_fp32;
    const TgStepRates *schedule;
    const StepCounters *counters;
    float muon_lr, weight_decay;
    int rows, cols, batch;
    int64_t stride;
};
void launch_muon_apply(const MuonApplyArgs &a, cudaStream_t s);
void launch_advance(StepCounters *counters, cudaStream_t s);

// ---- self-test: a wait on a barrier nothing arms, with a short limit (selftest.cu) ----
int launch_starved_wait(StepCounters *counters, double limit_ms, int code, cudaStream_t s);

// ---- conversions ----
void launch_split_weights(const float *w, bf16 *high, uint16_t *low, int64_t count, cudaStream_t s);
void launch_join_weights(const bf16 *high, const uint16_t *low, float *w, int64_t count, cudaStream_t s);
void launch_cast(Dtype from, const void *in, Dtype to, void *out, int64_t count, cudaStream_t s);
