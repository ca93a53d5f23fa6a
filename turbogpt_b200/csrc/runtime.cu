// The C ABI: the reference's 22 engine functions (runtime.h:12-37, implemented there by
// cuda/runtime.cu and cuda/engine_state.cu) plus the extensions declared in
// include/turbogpt_b200.h.  Every function converts exceptions to the error convention:
// negative int / NULL and a thread-local message.
#include "engine.h"
#include <mutex>
#include <cstring>

static thread_local std::string last_error;

template <class F> static int guarded(F &&body) {
    try {
        body();
        return 0;
    } catch (const std::exception &error) {
        last_error = error.what();
        return -1;
    }
}

extern "C" {

const char *tg_error(void) { return last_error.c_str(); }

void tg_ex_reference_config(const TgConfig *base, TgConfigEx *c) {
    memset(c, 0, sizeof(*c));
    c->base = *base;
    c->struct_size = sizeof(TgConfigEx);
    c->width = 16, c->heads = 4, c->hidden = 48;
    c->norm = TG_NORM_RMS, c->attention = TG_ATTENTION_ARGMAX, c->mlp = TG_MLP_SWIGLU, c->tied = 0;
    c->rope = TG_ROPE_PARTIAL, c->hidden_optimizer = TG_HIDDEN_MUON, c->precision = TG_PRECISION_BF16;
    c->world = 1, c->rank = 0;
}
void tg_ex_gpt_config(const TgConfig *base, int width, int heads, int hidden, TgConfigEx *c) {
    tg_ex_reference_config(base, c);
    c->width = width, c->heads = heads, c->hidden = hidden;
    c->norm = TG_NORM_LAYER, c->attention = TG_ATTENTION_SOFTMAX, c->mlp = TG_MLP_GELU, c->tied = 1;
    c->rope = TG_ROPE_NONE, c->hidden_optimizer = TG_HIDDEN_ADAMW;
}

Engine *tg_create_ex(const TgConfigEx *config) {
    try {
        if (!config)
            throw std::runtime_error("Missing configuration");
        return new Engine(*config);
    } catch (const std::exception &error) {
        last_error = error.what();
        return nullptr;
    }
}
Engine *tg_create(const TgConfig *config) {
    try {
        if (!config)
            throw std::runtime_error("Missing configuration");
        // The reference's own limits (cuda/runtime.cu:65-68), minus the tile-balance rule of its
        // persistent kernel: any depth up to 64 and any context are accepted here.
        if (config->batch < 4 || int64_t(config->batch) * config->context % 16)
            throw std::runtime_error("Supported: batch at least 4 with batch*context divisible by 16");
        TgConfigEx ex;
        tg_ex_reference_config(config, &ex);
        return new Engine(ex);
    } catch (const std::exception &error) {
        last_error = error.what();
        return nullptr;
    }
}
void tg_destroy(Engine *engine) { delete engine; }
int tg_parameter_count(Engine *e) { return int(e->layout.count); }
int tg_blocks(Engine *e) { return e->sms; }
int tg_shared_bytes(Engine *e) { return e->tensor_cores ? gemm_tc_shared_bytes() : 0; }

int tg_set_weights(Engine *e, const float *w) {
    return guarded([&] {
        if (!w)
            throw std::runtime_error("Missing weights");
        e->set_weights(w);
    });
}
int tg_get_weights(Engine *e, float *w) {
    return guarded([&] {
        if (!w)
            throw std::runtime_error("Missing weights output");
        e->get_weights(w);
    });
}
int tg_get_optimizer_state(Engine *e, float *m, float *v, uint64_t *step) {
    return guarded([&] { e->get_optimizer_state(m, v, step); });
}
int tg_set_optimizer_state(Engine *e, const float *m, const float *v, uint64_t step) {
    return guarded([&] { e->set_optimizer_state(m, v, step); });
}
int tg_memory(Engine *e, double *used_gb) {
    return guarded([&] {
        if (!used_gb)
            throw std::runtime_error("Missing memory output");
        *used_gb = double(e->allocated_bytes) / (1024.0 * 1024.0 * 1024.0);
    });
}
int tg_set_data(Engine *e, const uint8_t *bytes, int64_t size) {
    return guarded([&] {
        if (!bytes)
            throw std::runtime_error("Missing dataset");
        e->set_data(bytes, size);
    });
}
int tg_train(Engine *e, int steps) {
    return guarded([&] { e->train(steps); });
}
int tg_get_training_losses(Engine *e, float *per_position, int count) {
    return guarded([&] { e->training_losses(per_position, count); });
}
int tg_training_versions(Engine *e, int *versions, int count) {
    return guarded([&] { // synchronous training: every step sees the weights of the step before it
        if (count < 0 || count > e->last_train_steps)
            throw std::runtime_error("Version trace exceeds last training launch");
        for (int i = 0; i < count; ++i)
            versions[i] = int(e->step) - e->last_train_steps + i;
    });
}
int tg_pipeline_stats(Engine *, double *mean_staleness, int *max_staleness) {
    return guarded([&] {
        *mean_staleness = 0;
        *max_staleness = 0;
    });
}
int tg_onecycle_point(const TgOneCycle *schedule, int step, TgStepRates *rates) {
    return guarded([&] { *rates = onecycle_point(*schedule, step); });
}
int tg_set_onecycle(Engine *e, const TgOneCycle *schedule) {
    return guarded([&] { e->set_onecycle(*schedule); });
}
int tg_batch(Engine *e, const uint8_t *x, const uint8_t *y, float *logits, float *gradients, float *per_position) {
    return guarded([&] {
        if (!x || !y)
            throw std::runtime_error("Missing batch input");
        e->batch(x, y, logits, gradients, per_position);
    });
}
int tg_predict(Engine *e, const uint8_t *context, float *logits) {
    return guarded([&] { e->predict(context, logits); });
}
int tg_optimizer_test(Engine *e, const float *gradients, int steps) {
    return guarded([&] {
        if (!gradients)
            throw std::runtime_error("Missing gradients");
        e->optimizer_test(gradients, steps);
    });
}
int tg_synchronize(Engine *e) {
    return guarded([&] {
        e->set_device();
        CHECK_CUDA(cudaStreamSynchronize(e->stream));
    });
}

// ---------------------------------------------------------------------------- extensions -----
int64_t tg_ex_parameter_count(const TgConfigEx *config) {
    try {
        validate_config(*config);
        return make_layout(*config).count;
    } catch (const std::exception &error) {
        last_error = error.what();
        return -1;
    }
}
int tg_ex_parameter_layout(const TgConfigEx *config, int64_t *offsets, int32_t *rows, int32_t *cols, int capacity) {
    try {
        validate_config(*config);
        Layout p = make_layout(*config);
        int n = int(p.tensors.size());
        for (int i = 0; i < n && i < capacity; ++i) {
            offsets[i] = p.tensors[i].offset;
            rows[i] = p.tensors[i].rows;
            cols[i] = p.tensors[i].cols;
        }
        return n;
    } catch (const std::exception &error) {
        last_error = error.what();
        return -1;
    }
}
int tg_ex_initialize_weights(const TgConfigEx *config, float *weights) {
    return guarded([&] {
        validate_config(*config);
        initialize_weights(*config, weights);
    });
}
int tg_ex_save_checkpoint(const char *path, const TgConfigEx *config, const TgCheckpoint *state) {
    return guarded([&] {
        if (!path || !config || !state)
            throw std::runtime_error("Missing checkpoint argument");
        save_checkpoint(path, *config, *state);
    });
}
int tg_ex_load_checkpoint(const char *path, const TgConfigEx *config, TgCheckpoint *state) {
    return guarded([&] {
        if (!path || !config || !state)
            throw std::runtime_error("Missing checkpoint argument");
        load_checkpoint(path, *config, *state);
    });
}
uint64_t tg_ex_config_digest(const TgConfigEx *config) {
    try {
        validate_config(*config);
    } catch (const std::exception &error) {
        last_error = error.what();
        return 0;
    }
    // Everything every rank of one job must agree on: all fields except the rank and the device.
    TgConfigEx c = *config;
    c.rank = 0, c.base.device = 0, c.base.reserved_ = 0;
    uint64_t digest = 0x243f6a8885a308d3ull;
    const unsigned char *bytes = reinterpret_cast<const unsigned char *>(&c);
    for (size_t i = 0; i < sizeof(c); i += 8) {
        uint64_t word = 0;
        memcpy(&word, bytes + i, sizeof(c) - i < 8 ? sizeof(c) - i : 8);
        digest = hash_u64(digest ^ word);
    }
    return digest ? digest : 1;
}
int tg_ex_nccl_unique_id(uint8_t *id128) {
    return guarded([&] {
        const Nccl &nccl = Nccl::get();
        Nccl::UniqueId id;
        nccl.check(nccl.GetUniqueId(&id), "ncclGetUniqueId");
        memcpy(id128, id.internal, 128);
    });
}
void *tg_ex_stream(Engine *e) { return e->stream; }
int tg_ex_sample(Engine *e, uint64_t step, uint8_t *x, uint8_t *y) {
    return guarded([&] { e->sample(step, x, y); });
}
int tg_ex_train_mean_loss(Engine *e, int steps, float *mean_loss) {
    return guarded([&] { *mean_loss = e->train_mean_loss(steps); });
}
int tg_ex_train_batch(Engine *e, const uint8_t *x, const uint8_t *y, float *per_position) {
    return guarded([&] { e->train_batch(x, y, per_position); });
}
int tg_ex_profile(Engine *e, const char **names, double *milliseconds, int64_t *launches, int capacity, int reset) {
    try {
        e->set_device();
        e->flush_profile();
        for (int i = 0; i < FamilyCount && i < capacity; ++i) {
            names[i] = family_names[i];
            milliseconds[i] = e->family_ms[i];
            launches[i] = e->family_launches[i];
        }
        if (reset)
            for (int i = 0; i < FamilyCount; ++i)
                e->family_ms[i] = 0, e->family_launches[i] = 0;
        return FamilyCount;
    } catch (const std::exception &error) {
        last_error = error.what();
        return -1;
    }
}
int64_t tg_ex_launch_count(Engine *e) { return e->launches; }
int64_t tg_ex_read_activation(Engine *e, int layer, const char *name, float *out, int64_t capacity) {
    try {
        return e->read_activation(layer, name, out, capacity);
    } catch (const std::exception &error) {
        last_error = error.what();
        return -1;
    }
}

int tg_ex_selftest_bounded_wait(Engine *e, double limit_ms) {
    try {
        e->set_device();
        return launch_starved_wait(e->counters, limit_ms, 901, e->stream);
    } catch (const std::exception &error) {
        last_error = error.what();
        return -1;
    }
}

static int device_sms() {
    int device = 0, sms = 0;
    CHECK_CUDA(cudaGetDevice(&device));
    CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    return sms;
}
static void require_sm100() {
    int device = 0, major = 0;
    CHECK_CUDA(cudaGetDevice(&device));
    CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10)
        throw std::runtime_error("This library is built for sm_100a (B200)");
}

int tg_ex_gemm(const void *a, int64_t a_row, int64_t a_col, const void *b, int64_t b_row, int64_t b_col, void *c,
               int64_t ldc, int m, int n, int k, int out_fp32, int tensor_cores, void *stream) {
    return guarded([&] {
        require_sm100();
        GemmArgs g;
        g.a = a, g.a_row = a_row, g.a_col = a_col, g.b = b, g.b_row = b_row, g.b_col = b_col;
        g.c = c, g.ldc = ldc, g.m = m, g.n = n, g.k = k;
        g.in = Dtype::BF16, g.out = out_fp32 ? Dtype::FP32 : Dtype::BF16;
        if (tensor_cores) {
            if (!gemm_tc_supported(g))
                throw std::runtime_error("GEMM shape or layout is outside the tensor-core kernel's range");
            launch_gemm_tc(g, device_sms(), nullptr, static_cast<cudaStream_t>(stream));
        } else {
            launch_gemm_simt(g, static_cast<cudaStream_t>(stream));
        }
        CHECK_CUDA(cudaGetLastError());
    });
}
int tg_ex_head_cross_entropy(const void *x, const void *head, const uint8_t *targets, float *losses, void *dlogits,
                             int rows, int width, float scale, void *stream) {
    return guarded([&] {
        require_sm100();
        if (!x || !head || !targets || !losses)
            throw std::runtime_error("Missing head or loss operand");
        GemmArgs g;
        g.a = x, g.a_row = width, g.b = head, g.b_row = width, g.c = dlogits, g.ldc = Vocabulary;
        g.m = rows, g.n = Vocabulary, g.k = width;
        g.in = Dtype::BF16, g.out = Dtype::BF16;
        g.epilogue = Epilogue::CrossEntropy, g.r = targets, g.c2 = losses, g.alpha = scale;
        if (!gemm_tc_supported(g))
            throw std::runtime_error("head + loss: width must be a multiple of 8 and at least 64, operands 16-byte aligned");
        launch_gemm_tc(g, device_sms(), nullptr, static_cast<cudaStream_t>(stream));
        CHECK_CUDA(cudaGetLastError());
    });
}
int tg_ex_weight_gradient_static(const void *dy, const void *x, float *dw, int out, int in, int tokens,
                                 void *stream) {
    return guarded([&] {
        require_sm100();
        if (!dy || !x || !dw)
            throw std::runtime_error("Missing weight-gradient operand");
        launch_weight_gradient_static(dy, x, dw, out, in, tokens, device_sms(), static_cast<cudaStream_t>(stream));
    });
}
int tg_ex_last_device_error(void *stream) {
    try {
        require_sm100();
        return gemm_tc_take_device_error(static_cast<cudaStream_t>(stream));
    } catch (const std::exception &error) {
        last_error = error.what();
        return -1;
    }
}
int tg_ex_attention_forward(const void *qkv, void *out, float *lse, int batch, int context, int heads, int d_head,
                            int tensor_cores, void *stream) {
    return guarded([&] {
        require_sm100();
        if (tensor_cores) {
            if (!flash_attention_supported(heads * d_head, heads))
                throw std::runtime_error("tensor-core attention needs a head size of 64");
            launch_flash_attention_forward(qkv, out, lse, batch, context, heads, nullptr,
                                           static_cast<cudaStream_t>(stream));
        } else {
            SoftmaxAttentionArgs a{qkv, out, lse, batch, context, heads * d_head, heads};
            launch_softmax_attention(Dtype::BF16, a, static_cast<cudaStream_t>(stream));
        }
        CHECK_CUDA(cudaGetLastError());
    });
}
namespace {
// Scratch of the stand-alone attention backward call: one grow-only allocation per device, kept until the
// process ends, so that repeated calls cost no allocator traffic.  Calls on the same device must not overlap.
void *attention_scratch(size_t bytes) {
    static std::mutex guard;
    static void *memory[64] = {};
    static size_t capacity[64] = {};
    int device = 0;
    CHECK_CUDA(cudaGetDevice(&device));
    if (device >= 64)
        throw std::runtime_error("device index out of range");
    std::lock_guard<std::mutex> lock(guard);
    if (capacity[device] < bytes) {
        CHECK_CUDA(cudaDeviceSynchronize());
        if (memory[device])
            CHECK_CUDA(cudaFree(memory[device]));
        memory[device] = nullptr, capacity[device] = 0;
        CHECK_CUDA(cudaMalloc(&memory[device], bytes));
        capacity[device] = bytes;
    }
    return memory[device];
}
} // namespace
int tg_ex_attention_backward(const void *qkv, const void *out, const void *dout, const float *lse, void *dqkv,
                             int batch, int context, int heads, int d_head, int tensor_cores, void *stream) {
    return guarded([&] {
        require_sm100();
        if (tensor_cores && !flash_attention_supported(heads * d_head, heads))
            throw std::runtime_error("tensor-core attention needs a head size of 64");
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        if (tensor_cores == TG_ATTENTION_BACKWARD_SINGLE_PASS) {
            launch_flash_attention_backward_fused(qkv, out, dout, lse, dqkv,
                                                  attention_scratch(flash_backward_scratch_bytes(batch, context, heads)), batch,
                                                  context, heads, nullptr, s);
        } else if (tensor_cores) { // what the engine runs: dQ by query tile, then dK and dV by key tile
            float *scratch = static_cast<float *>(attention_scratch(flash_attention_backward_scratch_bytes(batch, context, heads)));
            launch_flash_attention_backward(qkv, out, dout, lse, scratch, dqkv, batch, context, heads, nullptr, s);
        } else {
            float *delta = static_cast<float *>(attention_scratch(size_t(batch) * heads * context * sizeof(float)));
            SoftmaxAttentionBackwardArgs a{qkv, out, dout, lse, delta, dqkv, batch, context, heads * d_head, heads};
            launch_softmax_attention_backward(Dtype::BF16, a, s);
        }
        CHECK_CUDA(cudaGetLastError());
    });
}
int tg_ex_norm_forward(int kind, const void *x, const void *scale_high, const void *scale_low, const void *bias_high,
                       const void *bias_low, void *y, float *stats, int rows, int width, void *stream) {
    return guarded([&] {
        require_sm100();
        if (!x || !y || !scale_high || !scale_low || (kind == TG_NORM_LAYER && (!bias_high || !bias_low)))
            throw std::runtime_error("Missing norm operand");
        if (width < 8 || width % 8 || rows < 1)
            throw std::runtime_error("norm: width must be a positive multiple of 8");
        NormArgs a{kind, x, static_cast<const bf16 *>(scale_high),
                   kind == TG_NORM_LAYER ? static_cast<const bf16 *>(bias_high) : nullptr,
                   static_cast<const uint16_t *>(scale_low),
                   kind == TG_NORM_LAYER ? static_cast<const uint16_t *>(bias_low) : nullptr, y, rows, width,
                   width % 256 == 0 && width <= 1024 ? stats : nullptr};
        launch_norm(Dtype::BF16, a, static_cast<cudaStream_t>(stream));
        CHECK_CUDA(cudaGetLastError());
    });
}
int tg_ex_norm_backward(int kind, const void *x, const void *dy, const void *scale_high, const void *scale_low,
                        const void *residual_in, const float *stats, void *dx, float *dscale, float *dbias, int rows,
                        int width, void *stream) {
    return guarded([&] {
        require_sm100();
        if (!x || !dy || !dx || !scale_high || !scale_low || !dscale || (kind == TG_NORM_LAYER && !dbias))
            throw std::runtime_error("Missing norm operand");
        if (width < 8 || width % 8 || rows < 1)
            throw std::runtime_error("norm: width must be a positive multiple of 8");
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        const int blocks = norm_backward_blocks(rows, device_sms());
        float *partial = nullptr;
        CHECK_CUDA(cudaMallocAsync(&partial, size_t(blocks) * 2 * width * sizeof(float), s));
        NormBackwardArgs a{kind, x, dy, static_cast<const bf16 *>(scale_high), static_cast<const uint16_t *>(scale_low),
                           residual_in, dx, partial, dscale, kind == TG_NORM_LAYER ? dbias : nullptr, rows, width, blocks,
                           width % 256 == 0 && width <= 1024 ? stats : nullptr};
        launch_norm_backward(Dtype::BF16, a, s);
        CHECK_CUDA(cudaFreeAsync(partial, s));
        CHECK_CUDA(cudaGetLastError());
    });
}
int tg_ex_cross_entropy(const void *logits, const uint8_t *targets, float *losses, void *dlogits, int rows,
                        float scale, void *stream) {
    return guarded([&] {
        require_sm100();
        CrossEntropyArgs a{logits, targets, losses, dlogits, nullptr, 1.f / scale, rows};
        launch_cross_entropy(Dtype::BF16, a, static_cast<cudaStream_t>(stream));
        CHECK_CUDA(cudaGetLastError());
    });
}

} // extern "C"
