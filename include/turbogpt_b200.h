/* turbogpt_b200 — C ABI of the B200-native training engine.
 *
 * Part 1 is the reference's engine interface: the same 22 exported names, argument
 * order, struct layouts and error convention as the reference's runtime.h:12-37, so its
 * host program (train.cpp, trainer.cpp, checkpoint.cpp, dataset.cpp, sampling.cpp,
 * report.cpp, training_log.cpp) and its ctypes bridge (tests/bridge.py:29-49) link
 * against this library unchanged.  Part 2 adds what the reference's fixed 16-wide model
 * cannot express: model dimensions, the scaled architecture, data parallelism, and the
 * kernel microbenchmarks.
 *
 * Error convention (runtime.h:39-42): int results are < 0 on failure and pointer
 * results are NULL; tg_error() returns the calling thread's last message.  No C++
 * exception crosses this boundary.  An Engine is not thread-safe; it owns one CUDA
 * stream, every call selects the engine's device first, and all its scratch memory (the GEMM's split-K
 * workspace included) is its own, so several engines may run on one GPU at once.  The stand-alone
 * kernel calls of part 2 (tg_ex_gemm, ...) share one per-device workspace: calls that overlap on the
 * GPU (different streams or threads) race on it.
 */
#ifndef TURBOGPT_B200_H
#define TURBOGPT_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- structs crossing the boundary (layouts pinned by tests/bridge.py:7-26) ---- */

/* config.h:5-13 — 72 bytes. */
typedef struct TgConfig {
    int32_t depth, context, batch, device;
    int32_t blocks, ns_steps;
    float learning_rate, muon_lr;
    float beta1, beta2, momentum;
    float weight_decay, epsilon, clip;
    uint64_t seed;
    int32_t inflight; /* 1 only; >1 is the reference's optional stale-gradient pipeline */
    int32_t reserved_;
} TgConfig;

/* optim.h:6-13 — 48 bytes. */
typedef struct TgOneCycle {
    int32_t total_steps;
    int32_t pad_;
    double warmup_fraction, initial_lr_fraction, final_lr_fraction, low_momentum, high_momentum;
} TgOneCycle;

/* optim.h:14-16. */
typedef struct TgStepRates {
    float multiplier, momentum;
} TgStepRates;

typedef struct Engine Engine;

/* ---- Part 1: the reference's interface ---- */

const char *tg_error(void);                                  /* runtime.h:13, cuda/runtime.cu:30 */
Engine *tg_create(const TgConfig *config);                   /* runtime.h:14, cuda/runtime.cu:62 — reference architecture (width 16, 4 heads, SwiGLU 48) */
void tg_destroy(Engine *engine);                             /* runtime.h:15, cuda/runtime.cu:156 */
int tg_parameter_count(Engine *engine);                      /* runtime.h:16, cuda/runtime.cu:159 */
int tg_blocks(Engine *engine);                               /* runtime.h:17, cuda/runtime.cu:162 — informational: SM count used to size grids */
int tg_shared_bytes(Engine *engine);                         /* runtime.h:18, cuda/runtime.cu:165 — informational: largest dynamic shared memory of a kernel */
int tg_set_weights(Engine *engine, const float *weights);    /* runtime.h:19, cuda/engine_state.cu:7 — also zeroes optimizer state and the step */
int tg_get_weights(Engine *engine, float *weights);          /* runtime.h:20, cuda/engine_state.cu:36 */
int tg_get_optimizer_state(Engine *engine, float *momentum, float *variance, uint64_t *step); /* runtime.h:21, cuda/engine_state.cu:57 */
int tg_set_optimizer_state(Engine *engine, const float *momentum, const float *variance,
                           uint64_t step);                   /* runtime.h:22, cuda/engine_state.cu:94 */
int tg_memory(Engine *engine, double *used_gb);              /* runtime.h:24, cuda/runtime.cu:178 */
int tg_set_data(Engine *engine, const uint8_t *bytes, int64_t size); /* runtime.h:25, cuda/runtime.cu:190 */
int tg_train(Engine *engine, int steps);                     /* runtime.h:26, cuda/runtime.cu:213 — asynchronous, 1..4096 steps */
int tg_get_training_losses(Engine *engine, float *per_position, int count); /* runtime.h:27, cuda/engine_state.cu:76 — synchronises */
int tg_training_versions(Engine *engine, int *versions, int count);         /* runtime.h:28, cuda/runtime.cu:243 */
int tg_pipeline_stats(Engine *engine, double *mean_staleness, int *max_staleness); /* runtime.h:29, cuda/runtime.cu:263 */
int tg_onecycle_point(const TgOneCycle *schedule, int step, TgStepRates *rates);   /* runtime.h:30, cuda/runtime.cu:33 */
int tg_set_onecycle(Engine *engine, const TgOneCycle *schedule);                   /* runtime.h:31, cuda/runtime.cu:42 */
int tg_batch(Engine *engine, const uint8_t *x, const uint8_t *y, float *logits, float *gradients,
             float *per_position);                           /* runtime.h:33, cuda/runtime.cu:291 */
int tg_predict(Engine *engine, const uint8_t *context, float *logits); /* runtime.h:35, cuda/runtime.cu:322 */
int tg_optimizer_test(Engine *engine, const float *gradients, int steps); /* runtime.h:36, cuda/runtime.cu:352 */
int tg_synchronize(Engine *engine);                          /* runtime.h:37, cuda/runtime.cu:168 */

/* ---- Part 2: extensions ---- */

enum { TG_NORM_RMS = 0, TG_NORM_LAYER = 1 };
enum { TG_ATTENTION_ARGMAX = 0, TG_ATTENTION_SOFTMAX = 1 };
enum { TG_MLP_SWIGLU = 0, TG_MLP_GELU = 1 };
enum { TG_ROPE_NONE = 0, TG_ROPE_PARTIAL = 1 };
enum { TG_HIDDEN_MUON = 0, TG_HIDDEN_ADAMW = 1 };
enum { TG_PRECISION_BF16 = 0, TG_PRECISION_FP32 = 1 };
enum { TG_FLAG_NO_TENSOR_CORES = 1, /* route every GEMM and attention through the plain CUDA-core kernels */
       TG_FLAG_PROFILE = 2,         /* time every kernel family with CUDA events (serialises nothing, disables graph replay) */
       TG_FLAG_BF16_GRADIENT_EXCHANGE = 4, /* all-reduce gradients as BF16 instead of FP32 */
       TG_FLAG_NO_GRAPH = 8,        /* launch every kernel of tg_train directly instead of replaying a CUDA graph of the step */
       TG_FLAG_NO_COMMUNICATOR = 16 /* world > 1 without NCCL: world/rank only shard the sampling (tg_ex_sample) and scale the
                                       loss by the global batch (tg_batch gradients are this rank's share of the global mean);
                                       the caller sums gradients itself, tg_train and tg_ex_train_batch are refused */ };

/* Replaces the compile-time "Width=16, heads=4" of config.h:4 and the hard-wired sizes of
 * model.h:20-34.  `base` keeps the reference's meaning.  struct_size must be
 * sizeof(TgConfigEx).  world/rank select data parallelism: global batch = world*base.batch,
 * this engine draws global sequences rank*batch .. rank*batch+batch-1 (cuda/dataset.cuh:14
 * applied to the global batch) and sums gradients over ranks with NCCL. */
typedef struct TgConfigEx {
    TgConfig base;
    int32_t struct_size;
    int32_t width, heads, hidden;
    int32_t norm, attention, mlp, tied, rope;
    int32_t hidden_optimizer, precision;
    int32_t world, rank;
    int32_t flags;
    uint8_t nccl_id[128]; /* from tg_ex_nccl_unique_id on rank 0, identical on all ranks; ignored when world == 1 */
} TgConfigEx;

/* Fills *config with the reference architecture around `base` (model.h:12-37). */
void tg_ex_reference_config(const TgConfig *base, TgConfigEx *config);
/* Fills *config with the scaled architecture: LayerNorm, softmax attention, GELU MLP, tied head. */
void tg_ex_gpt_config(const TgConfig *base, int width, int heads, int hidden, TgConfigEx *config);
/* tg_create for any architecture (cuda/runtime.cu:62-155 generalised). */
Engine *tg_create_ex(const TgConfigEx *config);
/* parameter_layout(depth).count of model.h:12-37 for any architecture; < 0 on bad dimensions. */
int64_t tg_ex_parameter_count(const TgConfigEx *config);
/* Flat offsets of every tensor, in layout order; returns the number of tensors, writes at most
 * `capacity` entries: offsets[i], rows[i], cols[i] (cols = 0 for vectors). */
int tg_ex_parameter_layout(const TgConfigEx *config, int64_t *offsets, int32_t *rows, int32_t *cols,
                           int capacity);
/* initialize_weights of model.cpp:7-31 for any architecture (same seeds per tensor role). */
int tg_ex_initialize_weights(const TgConfigEx *config, float *weights);
/* Training state as the reference's checkpoint.h:7-14 holds it, with caller-owned arrays. */
typedef struct TgCheckpoint {
    float *weights, *momentum, *variance; /* [tg_ex_parameter_count(config)] each */
    double *final_loss_sums;              /* [config->base.context] */
    uint64_t step, final_loss_batches;
    double train_seconds;
    TgOneCycle scheduler;
} TgCheckpoint;
/* save_training_state / load_training_state of checkpoint.cpp:506-579 for any architecture: the same
 * torch.load-able archive with the same fifteen records the reference host reads by name, plus one
 * record holding width, heads, hidden and the architecture selectors (checkpoint.cpp:164-166 stores
 * depth and context only).  Files of the reference architecture load in the reference host; files
 * the reference host wrote load here as the reference architecture.  Host-only: no device is touched.
 * Loading fills the caller's arrays and fails with "Checkpoint architecture mismatch" when the file
 * was written for other dimensions. */
int tg_ex_save_checkpoint(const char *path, const TgConfigEx *config, const TgCheckpoint *state);
int tg_ex_load_checkpoint(const char *path, const TgConfigEx *config, TgCheckpoint *state);
/* A digest of everything the ranks of one data-parallel job must agree on (every field of *config
 * except rank and base.device; nccl_id included).  Ranks exchange it over their own channel and
 * refuse to call tg_create_ex when the values differ: a communicator created from mismatched
 * configurations would hang or train garbage.  0 (and tg_error) when *config is invalid. */
uint64_t tg_ex_config_digest(const TgConfigEx *config);
/* 128-byte NCCL unique id for TgConfigEx.nccl_id. */
int tg_ex_nccl_unique_id(uint8_t *id128);
/* The engine's CUDA stream (cudaStream_t), for callers that time with their own events. */
void *tg_ex_stream(Engine *engine);
/* Bytes sampled for the next training step of this rank (cuda/dataset.cuh:9-29), without training. */
int tg_ex_sample(Engine *engine, uint64_t step, uint8_t *x, uint8_t *y);
/* Device-resident variant of tg_train + tg_get_training_losses for benchmarks: runs `steps`
 * steps and returns the mean loss of the last one. */
int tg_ex_train_mean_loss(Engine *engine, int steps, float *mean_loss);
/* One optimizer step on caller-supplied host bytes x, y [batch*context] (instead of sampling the
 * resident corpus); writes the per-position mean loss [context] when per_position != NULL, which
 * synchronises.  The host-buffer counterpart of tg_train for callers that stream their own batches. */
int tg_ex_train_batch(Engine *engine, const uint8_t *x, const uint8_t *y, float *per_position);
/* Per-kernel-family device time accumulated since the last reset (TG_FLAG_PROFILE engines).
 * names: up to `capacity` pointers to static strings; returns the number of families. */
int tg_ex_profile(Engine *engine, const char **names, double *milliseconds, int64_t *launches,
                  int capacity, int reset);
/* Number of kernels this library launched on the engine's stream since creation. */
int64_t tg_ex_launch_count(Engine *engine);
/* Diagnostic: copies an activation saved by the last forward pass (tg_batch / tg_train keep them for
 * backward; the reference keeps the same set in its Activation struct, cuda/types.cuh:40-44) to
 * host FP32.  layer >= 0: "x", "normed1", "qkv", "attended", "middle", "normed2", "activated";
 * layer < 0: "final_x", "final_normed".  Returns the element count (tokens x features), also when
 * out == NULL; < 0 on an unknown name or a short buffer. */
int64_t tg_ex_read_activation(Engine *engine, int layer, const char *name, float *out, int64_t capacity);

/* Self-test of the bounded device waits (the reference's waits are unbounded, cuda/pipeline.cuh:24-25):
 * one CTA waits, for at most `limit_ms` (0 < limit_ms <= 100), on a barrier that nothing arms, with no
 * copy or tensor-core operation in flight.  Returns 1 when the wait gave up as designed and left code
 * 901 in the engine's device error word (0 if it reported completion, < 0 on a host error).  The
 * engine's next synchronising call (tg_batch, tg_get_training_losses, tg_predict, tg_optimizer_test)
 * then fails with "a device-side wait gave up (code 901)"; tg_set_weights clears the error word. */
int tg_ex_selftest_bounded_wait(Engine *engine, double limit_ms);

/* Kernel microbenchmarks on device pointers (BF16 unless noted), enqueued on `stream`.
 * C[M,N] = A . B^T with element strides: A[m,k] at m*a_row + k*a_col, B[n,k] at n*b_row + k*b_col;
 * exactly one stride of each operand is 1.  Replaces project/matmul/weight_gradient of
 * cuda/mma.cuh:77-108 and cuda/ops.cuh:30-55,83-109.  out_fp32: C is float, else BF16. */
int tg_ex_gemm(const void *a, int64_t a_row, int64_t a_col, const void *b, int64_t b_row, int64_t b_col,
               void *c, int64_t ldc, int m, int n, int k, int out_fp32, int tensor_cores, void *stream);
/* No counterpart in the reference (its engine allocates everything in tg_create).  Weight gradient
 * dw[out, in] (FP32) = dy[tokens, out]^T x[tokens, in] (BF16, row-major, device pointers) for callers
 * that must not allocate device memory when they need it — a process whose memory pool already owns
 * the whole GPU, or a loop that cannot afford the allocator's device-wide synchronisation.  The
 * split-K scratch is a 16 MiB array built into the library (every GPU that loads the library holds it
 * until exit): shapes needing more, or more than 1024 output tiles, are refused with a message; no
 * cudaMalloc/cudaFree or allocating library call is made.  The first call on a device looks up the
 * array's device address (cudaGetSymbolAddress) and should come before any stream capture.  All calls
 * share the array, which keeps the previous call's contents (the part that must start at zero is
 * cleared on `stream` first): calls that overlap on the GPU race.  Results equal tg_ex_gemm's. */
int tg_ex_weight_gradient_static(const void *dy, const void *x, float *dw, int out, int in, int tokens,
                                 void *stream);
/* tg_ex_gemm and tg_ex_weight_gradient_static return once their kernel is enqueued.  Every wait inside
 * the kernel is bounded (about two seconds); one that gives up leaves a code in a device error word
 * and the output partly unwritten.  This call synchronises `stream` and returns the first such code
 * recorded on the current device since the last query (0: none; < 0: host error), clearing it.
 * Allocates nothing. */
int tg_ex_last_device_error(void *stream);
/* Causal softmax attention over packed qkv [batch*context, 3*heads*d_head] (q | k | v);
 * out [batch*context, heads*d_head]; lse [batch, heads, context] floats. */
int tg_ex_attention_forward(const void *qkv, void *out, float *lse, int batch, int context, int heads,
                            int d_head, int tensor_cores, void *stream);
/* tensor_cores: 0 = SIMT kernels; 1 = the engine's tensor-core kernels (dQ by query tile, then dK and dV by key
 * tile); TG_ATTENTION_BACKWARD_SINGLE_PASS = one tensor-core kernel that forms dQ, dK and dV from a single
 * pass over the score blocks (same results up to rounding; slower at the measured shapes, kept for comparison).
 * The tensor-core forms keep one grow-only scratch allocation per device; calls on a device must not overlap. */
#define TG_ATTENTION_BACKWARD_SINGLE_PASS 2
int tg_ex_attention_backward(const void *qkv, const void *out, const void *dout, const float *lse,
                             void *dqkv, int batch, int context, int heads, int d_head, int tensor_cores,
                             void *stream);
/* RMSNorm (kind TG_NORM_RMS, eps 1e-6) or LayerNorm (TG_NORM_LAYER, eps 1e-5) over BF16 rows
 * [rows, width] (cuda/ops.cuh:56-66).  Scale and bias are FP32 values passed as the engine stores
 * them: the high 16 bits as BF16 (`*_high`) and the low 16 bits (`*_low`, uint16) in separate arrays;
 * bias pointers are ignored for RMSNorm.  `stats` (optional, [rows][2] floats) receives every row's
 * mean and 1/sqrt(variance + eps) for the backward pass; it is written for widths 256, 512, 768 and
 * 1024 (the register-resident kernels) and left untouched otherwise. */
int tg_ex_norm_forward(int kind, const void *x, const void *scale_high, const void *scale_low, const void *bias_high,
                       const void *bias_low, void *y, float *stats, int rows, int width, void *stream);
/* Its backward (cuda/ops.cuh:67-80): dx = norm'(dy) rounded to BF16, plus residual_in when not NULL
 * (the running residual-stream gradient); dscale / dbias [width] FP32 are overwritten, summed over
 * rows in a fixed order.  `stats`: what tg_ex_norm_forward wrote for the same x (NULL: recomputed). */
int tg_ex_norm_backward(int kind, const void *x, const void *dy, const void *scale_high, const void *scale_low,
                        const void *residual_in, const float *stats, void *dx, float *dscale, float *dbias, int rows,
                        int width, void *stream);
/* 256-way softmax cross-entropy (cuda/model.cuh:33-57): losses[rows] floats, dlogits BF16
 * = (softmax - onehot) * scale, written in place over logits when dlogits == logits. */
int tg_ex_cross_entropy(const void *logits, const uint8_t *targets, float *losses, void *dlogits, int rows,
                        float scale, void *stream);
/* The language-model head and its loss in one tensor-core kernel, as a training step runs them
 * (cuda/model.cuh:31-58): logits = x[rows, width] head[256, width]^T stay in FP32 inside the kernel;
 * losses[rows] floats; dlogits BF16 [rows, 256] = (softmax - onehot) * scale, or NULL for the loss alone. */
int tg_ex_head_cross_entropy(const void *x, const void *head, const uint8_t *targets, float *losses, void *dlogits,
                             int rows, int width, float scale, void *stream);

#ifdef __cplusplus
}
#endif
#endif
