// Engine: allocation and the kernel sequence of the dense training step.  The reference runs the
// whole step inside one persistent cooperative kernel sized for a 16-wide model
// (cuda/trainer.cuh:103-125); here a step is a stream of large kernels — tcgen05 GEMMs, fused
// attention, 128-bit elementwise passes, one optimizer pass — with all per-step control
// (sampling seed, schedule point, loss-history row) read from device-resident counters.
#include "engine.h"
#include <algorithm>
#include <cstring>
#include <dlfcn.h>

constexpr size_t SimtScratchBytes = size_t(6) << 20; // bounds gemm_simt_scratch_bytes for every shape it cuts

const char *const family_names[FamilyCount] = {
    "sample", "embedding", "norm", "gemm_forward", "gemm_input_grad", "gemm_weight_grad", "attention_forward",
    "attention_backward", "activation", "cross_entropy", "norm_backward", "embedding_backward", "optimizer",
    "muon", "gradient_exchange", "misc"};

// ------------------------------------------------------------------------------- NCCL --------
const Nccl &Nccl::get() {
    static Nccl api;
    static bool loaded = false;
    static std::string failure;
    if (!loaded && failure.empty()) {
        void *lib = nullptr;
        if (const char *path = getenv("TURBOGPT_NCCL_LIBRARY"))
            lib = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
        for (const char *name : {"libnccl.so.2", "libnccl.so"})
            if (!lib)
                lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
        if (!lib) {
            failure = "NCCL library not found (set TURBOGPT_NCCL_LIBRARY)";
        } else {
            api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
            api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(lib, "ncclCommInitRank"));
            api.CommInitRankConfig =
                reinterpret_cast<decltype(api.CommInitRankConfig)>(dlsym(lib, "ncclCommInitRankConfig"));
            api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(lib, "ncclAllReduce"));
            api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(lib, "ncclAllGather"));
            api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
            api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
            if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.AllGather || !api.CommDestroy)
                failure = "NCCL library lacks a required symbol";
            else
                loaded = true;
        }
    }
    if (!loaded)
        throw std::runtime_error(failure);
    return api;
}
void Nccl::check(int result, const char *what) const {
    if (result != 0)
        throw std::runtime_error(std::string(what) + ": " +
                                 (GetErrorString ? GetErrorString(result) : "NCCL error"));
}

constexpr int ExchangeSms = 4; // CTAs of the gradient all-reduce = SMs the backward GEMMs leave free for it

// ------------------------------------------------------------------------------- setup -------
template <class T> void Engine::allocate(T *&p, size_t n, bool zero) {
    void *raw = nullptr;
    size_t bytes = std::max<size_t>(n * sizeof(T), 16);
    CHECK_CUDA(cudaMalloc(&raw, bytes));
    p = static_cast<T *>(raw);
    allocations.push_back(raw);
    allocated_bytes += bytes;
    if (zero)
        CHECK_CUDA(cudaMemsetAsync(raw, 0, bytes, stream));
}
void Engine::set_device() const { CHECK_CUDA(cudaSetDevice(config.base.device)); }
const void *Engine::weight(int64_t offset) const {
    return act == Dtype::BF16 ? (const void *)(weight_high + offset) : (const void *)(weight_fp32 + offset);
}

Engine::Engine(const TgConfigEx &c) : config(c) {
    try {
        initialize();
    } catch (...) {
        release();
        throw;
    }
}
Engine::~Engine() { release(); }

void Engine::initialize() {
    const TgConfigEx &c = config;
    validate_config(c);
    layout = make_layout(c);
    if (layout.count > (int64_t(1) << 31) - 1)
        throw std::runtime_error("parameter count exceeds signed 32-bit indexing of the engine interface");
    set_device();
    cudaDeviceProp prop{};
    CHECK_CUDA(cudaGetDeviceProperties(&prop, c.base.device));
    if (prop.major != 10)
        throw std::runtime_error("This library is built for sm_100a (B200); device is sm_" +
                                 std::to_string(prop.major) + std::to_string(prop.minor));
    sms = c.base.blocks > 0 ? std::min(c.base.blocks, prop.multiProcessorCount) : prop.multiProcessorCount;
    act = c.precision == TG_PRECISION_FP32 ? Dtype::FP32 : Dtype::BF16;
    tensor_cores = !(c.flags & TG_FLAG_NO_TENSOR_CORES);
    profile = c.flags & TG_FLAG_PROFILE;
    tokens = c.base.batch * c.base.context;
    gemm_sms = sms;
    CHECK_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));

    const int64_t P = layout.count;
    const int W = c.width, Hd = c.hidden, T = c.base.context, depth = c.base.depth;
    const size_t e = dtype_size(act), M = size_t(tokens);
    allocate(weight_high, P);
    allocate(weight_low, P);
    if (act == Dtype::FP32)
        allocate(weight_fp32, P);
    allocate(momentum, P);
    allocate(variance, P);
    allocate(gradient, P);
    allocate(adam_mode, P / 8);
    allocate(x, M);
    allocate(y, M);
    allocate(counters, 1);
    allocate(token_losses, M);
    allocate(loss_history, size_t(MaxLaunchSteps) * T);
    allocate(mean_loss, 1);

    const int wide = c.mlp == TG_MLP_SWIGLU ? 2 * Hd : Hd;
    layers.resize(depth);
    auto bytes = [&](void *&p, size_t elements) {
        uint8_t *raw = nullptr;
        allocate(raw, elements * e, false);
        p = raw;
    };
    for (LayerActivations &a : layers) {
        bytes(a.x, M * W);
        bytes(a.normed1, M * W);
        bytes(a.qkv, M * 3 * W);
        bytes(a.attended, M * W);
        bytes(a.middle, M * W);
        bytes(a.normed2, M * W);
        bytes(a.wide, M * wide);
        bytes(a.activated, M * Hd);
        a.selected = nullptr, a.gates = a.derivatives = a.lse = nullptr;
        allocate(a.stats1, M * 2, false);
        allocate(a.stats2, M * 2, false);
        if (c.attention == TG_ATTENTION_ARGMAX) {
            allocate(a.selected, M * c.heads, false);
            allocate(a.gates, M * c.heads, false);
            allocate(a.derivatives, M * c.heads, false);
        } else {
            allocate(a.lse, M * c.heads, false);
        }
    }
    bytes(final_x, M * W);
    bytes(final_normed, M * W);
    allocate(final_stats, M * 2, false);
    bytes(logits, M * Vocabulary);
    bytes(dhidden[0], M * W);
    bytes(dhidden[1], M * W);
    bytes(dbranch, M * W);
    bytes(dwide, M * wide);
    bytes(dactivated, M * Hd);
    bytes(dqkv, M * 3 * W);
    allocate(attention_scratch,
             std::max<size_t>(size_t(M) * c.heads, flash_attention_backward_scratch_bytes(c.base.batch, T, c.heads) / sizeof(float)),
             false);
    allocate(simt_scratch, SimtScratchBytes / sizeof(float), false);
    norm_blocks = norm_backward_blocks(tokens, sms);
    allocate(norm_partial, size_t(norm_blocks) * 2 * W, false);
    if (W <= 1024 && tokens >= 4096)
        allocate(embedding_partial, size_t(EmbeddingSlices) * Vocabulary * W, false);
    sumsq_blocks = sms * 8;
    allocate(sumsq_partial, sumsq_blocks);

    // Per 8 parameters: 0 = Muon, 1 = AdamW, 2 = AdamW with decay (reference cuda/optim.cuh:5-15:
    // decay on the head only; with AdamW on hidden matrices they decay too; a tied embedding is the head).
    std::vector<uint8_t> mode(P / 8, 1);
    bool any_muon = false;
    for (const TensorInfo &t : layout.tensors) {
        uint8_t m = 1;
        if (t.kind == 3)
            m = 2;
        else if (t.kind == 2) {
            m = c.hidden_optimizer == TG_HIDDEN_MUON ? 0 : 2;
            any_muon |= m == 0;
        }
        int64_t count = int64_t(t.rows) * (t.cols ? t.cols : 1);
        std::fill(mode.begin() + t.offset / 8, mode.begin() + (t.offset + count) / 8, m);
    }
    CHECK_CUDA(cudaMemcpyAsync(adam_mode, mode.data(), mode.size(), cudaMemcpyHostToDevice, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream)); // `mode` is about to go out of scope
    if (any_muon) {
        size_t largest = std::max(size_t(3) * W * W, size_t(Hd) * W) * depth;
        size_t square = size_t(std::min(3 * W, W)) * std::min(3 * W, W);
        square = std::max(square, size_t(std::min(Hd, W)) * std::min(Hd, W)) * depth;
        allocate(muon_x[0], largest, false);
        allocate(muon_x[1], largest, false);
        allocate(muon_a, square, false);
        allocate(muon_b, square, false);
        allocate(muon_sumsq, size_t(depth) * MuonBlocks);
    }
    if (c.world > 1 && !(c.flags & TG_FLAG_NO_COMMUNICATOR)) {
        const Nccl &nccl = Nccl::get();
        Nccl::UniqueId id;
        memcpy(id.internal, c.nccl_id, sizeof(id.internal));
        // The GEMM kernel is one persistent CTA per SM holding all of its shared memory, so a collective
        // kernel cannot share an SM with it: it either waits for a GEMM to end or takes SMs the next GEMM
        // then waits for, with its tiles statically assigned.  The exchange needs little bandwidth
        // (one layer's gradients per ~1.5 ms of backward), so the communicator is limited to
        // ExchangeSms CTAs and the backward GEMMs leave that many SMs free (Engine::gemm_sms).
        if (nccl.CommInitRankConfig) {
            Nccl::Config limits{};
            limits.size = sizeof(limits), limits.magic = 0xcafebeefu, limits.version = 21700;
            limits.blocking = 1, limits.cga_cluster_size = INT32_MIN, limits.min_ctas = 1, limits.max_ctas = ExchangeSms;
            limits.net_name = nullptr;
            nccl.check(nccl.CommInitRankConfig(&comm, c.world, id, c.rank, &limits), "ncclCommInitRankConfig");
        } else {
            nccl.check(nccl.CommInitRank(&comm, c.world, id, c.rank), "ncclCommInitRank");
        }
        int least, greatest;
        CHECK_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest));
        CHECK_CUDA(cudaStreamCreateWithPriority(&exchange_stream, cudaStreamNonBlocking, greatest));
        bucket_events.resize(depth + 2);
        for (cudaEvent_t &ev : bucket_events)
            CHECK_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        CHECK_CUDA(cudaEventCreateWithFlags(&exchange_done, cudaEventDisableTiming));
        if (c.flags & TG_FLAG_BF16_GRADIENT_EXCHANGE)
            allocate(gradient_bf16, P, false);
    }
    CHECK_CUDA(cudaStreamSynchronize(stream));
}

void Engine::release() {
    cudaSetDevice(config.base.device);
    if (stream)
        cudaStreamSynchronize(stream);
    if (exchange_stream)
        cudaStreamSynchronize(exchange_stream);
    if (comm)
        Nccl::get().CommDestroy(comm);
    drop_graph();
    for (auto &t : timed) {
        cudaEventDestroy(t.start);
        cudaEventDestroy(t.stop);
    }
    for (cudaEvent_t ev : event_pool)
        cudaEventDestroy(ev);
    for (cudaEvent_t ev : bucket_events)
        cudaEventDestroy(ev);
    if (exchange_done)
        cudaEventDestroy(exchange_done);
    for (void *p : allocations)
        cudaFree(p);
    release_gemm_workspace(gemm_workspace);
    if (exchange_stream)
        cudaStreamDestroy(exchange_stream);
    if (stream)
        cudaStreamDestroy(stream);
}

// ------------------------------------------------------------------------------- launches ----
template <class F> void Engine::run(Family f, F &&launch) {
    ++launches;
    if (!profile) {
        launch();
        return;
    }
    auto take = [&] {
        if (event_pool.empty()) {
            cudaEvent_t ev;
            CHECK_CUDA(cudaEventCreate(&ev));
            return ev;
        }
        cudaEvent_t ev = event_pool.back();
        event_pool.pop_back();
        return ev;
    };
    Timed t{int(f), take(), take()};
    CHECK_CUDA(cudaEventRecord(t.start, stream));
    launch();
    CHECK_CUDA(cudaEventRecord(t.stop, stream));
    timed.push_back(t);
    if (timed.size() >= 8192)
        flush_profile();
}
void Engine::flush_profile() {
    if (timed.empty())
        return;
    CHECK_CUDA(cudaStreamSynchronize(stream));
    for (Timed &t : timed) {
        float ms = 0;
        CHECK_CUDA(cudaEventElapsedTime(&ms, t.start, t.stop));
        family_ms[t.family] += ms;
        family_launches[t.family] += 1;
        event_pool.push_back(t.start);
        event_pool.push_back(t.stop);
    }
    timed.clear();
}
void Engine::gemm(Family f, GemmArgs g) {
    g.in = act;
    run(f, [&] {
        if (tensor_cores && gemm_tc_supported(g))
            launches += launch_gemm_tc(g, gemm_sms, counters, stream, &gemm_workspace) - 1;
        else
            launch_gemm_simt(g, stream, gemm_simt_scratch_bytes(g) <= SimtScratchBytes ? simt_scratch : nullptr);
    });
}
void Engine::check_device_error() {
    StepCounters host{};
    CHECK_CUDA(cudaMemcpyAsync(&host, counters, sizeof(host), cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
    if (host.error)
        throw std::runtime_error("a device-side wait gave up (code " + std::to_string(host.error) +
                                 "); results of this launch are invalid");
}

// ------------------------------------------------------------------------------- state -------
void Engine::set_weights(const float *w) {
    set_device();
    const int64_t P = layout.count;
    float *staging = act == Dtype::FP32 ? weight_fp32 : gradient; // gradient is free before a step
    CHECK_CUDA(cudaMemcpyAsync(staging, w, P * 4, cudaMemcpyHostToDevice, stream));
    launch_split_weights(staging, weight_high, weight_low, P, stream);
    CHECK_CUDA(cudaMemsetAsync(momentum, 0, P * 4, stream));
    CHECK_CUDA(cudaMemsetAsync(variance, 0, P * 4, stream));
    CHECK_CUDA(cudaMemsetAsync(counters, 0, sizeof(StepCounters), stream));
    step = 0;
    CHECK_CUDA(cudaStreamSynchronize(stream));
}
void Engine::get_weights(float *w) {
    set_device();
    const int64_t P = layout.count;
    launch_join_weights(weight_high, weight_low, gradient, P, stream); // gradient doubles as staging
    CHECK_CUDA(cudaMemcpyAsync(w, gradient, P * 4, cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
}
void Engine::set_data(const uint8_t *bytes, int64_t size) {
    drop_graph();
    set_device();
    if (size <= 8)
        throw std::runtime_error("Dataset needs at least 9 bytes");
    if (size <= config.base.context)
        throw std::runtime_error("Dataset must be longer than the context");
    if (data)
        throw std::runtime_error("Dataset already loaded");
    allocate(data, size_t(size), false);
    data_size = size;
    CHECK_CUDA(cudaMemcpyAsync(data, bytes, size, cudaMemcpyHostToDevice, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
}
void Engine::set_onecycle(const TgOneCycle &s) {
    drop_graph();
    set_device();
    if (schedule || step)
        throw std::runtime_error("Set OneCycle once, before training");
    onecycle_point(s, 0); // validate before allocating
    std::vector<TgStepRates> rates(s.total_steps);
    for (int i = 0; i < s.total_steps; ++i)
        rates[i] = onecycle_point(s, i);
    allocate(schedule, rates.size(), false);
    CHECK_CUDA(cudaMemcpyAsync(schedule, rates.data(), rates.size() * sizeof(TgStepRates), cudaMemcpyHostToDevice,
                               stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
    schedule_steps = s.total_steps;
}

// ------------------------------------------------------------------------------- forward -----
void Engine::forward(bool want_gradient, bool dump_logits) {
    const TgConfigEx &c = config;
    const int B = forward_batch ? forward_batch : c.base.batch, T = c.base.context, M = B * T;
    const int W = c.width, Hd = c.hidden, H = c.heads;
    const int depth = c.base.depth;
    const bool layer_norm = c.norm == TG_NORM_LAYER;
    auto norm = [&](const void *in, int64_t scale, int64_t bias, void *out, float *stats) {
        NormArgs a{c.norm, in, weight_high + scale, layer_norm ? weight_high + bias : nullptr, weight_low + scale,
                   layer_norm ? weight_low + bias : nullptr, out, M, W, stats};
        run(FNorm, [&] { launch_norm(act, a, stream); });
    };
    run(FEmbedding, [&] { launch_embedding(act, weight(layout.embedding), x, layers[0].x, M, W, stream); });
    for (int l = 0; l < depth; ++l) {
        LayerActivations &a = layers[l];
        const LayerOffsets &p = layout.layers[l];
        void *next = l + 1 < depth ? layers[l + 1].x : final_x;
        norm(a.x, p.attention_norm, p.attention_norm_bias, a.normed1, a.stats1);
        GemmArgs qkv;
        qkv.a = a.normed1, qkv.a_row = W, qkv.b = weight(p.qkv), qkv.b_row = W, qkv.c = a.qkv, qkv.ldc = 3 * W;
        qkv.m = M, qkv.n = 3 * W, qkv.k = W, qkv.out = act;
        gemm(FGemmForward, qkv);
        if (c.rope == TG_ROPE_PARTIAL)
            run(FMisc, [&] { launch_rope(act, a.qkv, M, T, W, H, false, stream); });
        if (c.attention == TG_ATTENTION_ARGMAX) {
            ArgmaxAttentionArgs at{a.qkv, a.attended, a.selected, a.gates, a.derivatives, B, T, W, H};
            run(FAttentionForward, [&] { launch_argmax_attention(act, at, stream); });
        } else {
            SoftmaxAttentionArgs at{a.qkv, a.attended, a.lse, B, T, W, H};
            run(FAttentionForward, [&] {
                if (tensor_cores && act == Dtype::BF16 && flash_attention_supported(W, H))
                    launch_flash_attention_forward(a.qkv, a.attended, a.lse, B, T, H, counters, stream);
                else
                    launch_softmax_attention(act, at, stream);
            });
        }
        GemmArgs proj;
        proj.a = a.attended, proj.a_row = W, proj.b = weight(p.attention), proj.b_row = W, proj.c = a.middle;
        proj.ldc = W, proj.m = M, proj.n = W, proj.k = W, proj.out = act;
        proj.epilogue = Epilogue::Residual, proj.r = a.x, proj.ldr = W;
        gemm(FGemmForward, proj);
        norm(a.middle, p.mlp_norm, p.mlp_norm_bias, a.normed2, a.stats2);
        GemmArgs up;
        up.a = a.normed2, up.a_row = W, up.b = weight(p.gate), up.b_row = W, up.c = a.wide, up.m = M, up.k = W;
        up.out = act;
        if (c.mlp == TG_MLP_SWIGLU) { // gate and up are adjacent: one projection computes both
            up.n = 2 * Hd, up.ldc = 2 * Hd;
            gemm(FGemmForward, up);
            run(FActivation, [&] { launch_swiglu(act, a.wide, a.activated, M, Hd, stream); });
        } else {
            up.n = Hd, up.ldc = Hd, up.epilogue = Epilogue::GeluDual, up.c2 = a.activated;
            gemm(FGemmForward, up);
        }
        GemmArgs down;
        down.a = a.activated, down.a_row = Hd, down.b = weight(p.down), down.b_row = Hd, down.c = next;
        down.ldc = W, down.m = M, down.n = W, down.k = Hd, down.out = act;
        down.epilogue = Epilogue::Residual, down.r = a.middle, down.ldr = W;
        gemm(FGemmForward, down);
    }
    norm(final_x, layout.final_norm, layout.final_norm_bias, final_normed, final_stats);
    GemmArgs head;
    head.a = final_normed, head.a_row = W, head.b = weight(layout.head), head.b_row = W, head.c = logits;
    head.ldc = Vocabulary, head.m = M, head.n = Vocabulary, head.k = W, head.out = act;
    const float divisor = float(int64_t(B) * c.world * T);
    // Training steps take the loss and its gradient from the head product's FP32 accumulators (the reference
    // fuses them the same way, cuda/model.cuh:31-58); calls that return logits run the two kernels.
    GemmArgs fused = head;
    fused.in = act, fused.epilogue = Epilogue::CrossEntropy, fused.r = y, fused.c2 = token_losses;
    fused.c = want_gradient ? logits : nullptr, fused.alpha = 1.f / divisor;
    if (tensor_cores && !dump_logits && act == Dtype::BF16 && gemm_tc_supported(fused)) {
        gemm(FGemmForward, fused);
        return;
    }
    gemm(FGemmForward, head);
    CrossEntropyArgs ce{logits, y, token_losses, want_gradient ? logits : nullptr,
                        dump_logits ? logits_fp32 : nullptr, divisor, M};
    run(FCrossEntropy, [&] { launch_cross_entropy(act, ce, stream); });
}

// ------------------------------------------------------------------------------- backward ----
void Engine::exchange_bucket(int64_t begin, int64_t end, int index) {
    if (!comm || end <= begin)
        return;
    const Nccl &nccl = Nccl::get();
    CHECK_CUDA(cudaEventRecord(bucket_events[index], stream));
    CHECK_CUDA(cudaStreamWaitEvent(exchange_stream, bucket_events[index], 0));
    ++launches;
    if (gradient_bf16) {
        launch_cast(Dtype::FP32, gradient + begin, Dtype::BF16, gradient_bf16 + begin, end - begin, exchange_stream);
        nccl.check(nccl.AllReduce(gradient_bf16 + begin, gradient_bf16 + begin, size_t(end - begin), Nccl::Bfloat16,
                                  Nccl::Sum, comm, exchange_stream),
                   "ncclAllReduce");
        launch_cast(Dtype::BF16, gradient_bf16 + begin, Dtype::FP32, gradient + begin, end - begin, exchange_stream);
    } else {
        nccl.check(nccl.AllReduce(gradient + begin, gradient + begin, size_t(end - begin), Nccl::Float32, Nccl::Sum,
                                  comm, exchange_stream),
                   "ncclAllReduce");
    }
}
void Engine::finish_exchange() {
    if (!comm)
        return;
    CHECK_CUDA(cudaEventRecord(exchange_done, exchange_stream));
    CHECK_CUDA(cudaStreamWaitEvent(stream, exchange_done, 0));
}

void Engine::backward() {
    const TgConfigEx &c = config;
    const int W = c.width, Hd = c.hidden, M = tokens, B = c.base.batch, T = c.base.context, H = c.heads;
    const int depth = c.base.depth;
    const bool layer_norm = c.norm == TG_NORM_LAYER;
    const int wide = c.mlp == TG_MLP_SWIGLU ? 2 * Hd : Hd;
    // dW[out, in] = dy^T x: both operands are read "MN-major" (tokens are the contraction).
    auto weight_grad = [&](const void *dy, int out, const void *xin, int in, int64_t offset) {
        GemmArgs g;
        g.a = dy, g.a_row = 1, g.a_col = out, g.b = xin, g.b_row = 1, g.b_col = in;
        g.c = gradient + offset, g.ldc = in, g.m = out, g.n = in, g.k = M, g.out = Dtype::FP32;
        gemm(FGemmWeightGrad, g);
    };
    // dx[M, in] = dy[M, out] W[out, in].
    auto input_grad = [&](const void *dy, int out, int64_t w_offset, int in, void *dx) {
        GemmArgs g;
        g.a = dy, g.a_row = out, g.b = weight(w_offset), g.b_row = 1, g.b_col = in;
        g.c = dx, g.ldc = in, g.m = M, g.n = in, g.k = out, g.out = act;
        return g;
    };
    auto norm_back = [&](const void *xin, const void *dy, int64_t scale, int64_t bias, const void *residual,
                         void *dx, const float *stats) {
        NormBackwardArgs a{c.norm, xin, dy, weight_high + scale, weight_low + scale, residual, dx, norm_partial,
                           gradient + scale, layer_norm ? gradient + bias : nullptr, M, W, norm_blocks, stats};
        run(FNormBackward, [&] { launch_norm_backward(act, a, stream); });
        ++launches; // rows kernel + reduce kernel
    };
    void *dh = dhidden[0], *dh_other = dhidden[1];
    // From the first bucket to the end of backward a collective may be running beside the GEMMs.
    struct Reserve {
        Engine &e;
        explicit Reserve(Engine &engine) : e(engine) {
            if (e.comm && e.sms > 4 * ExchangeSms)
                e.gemm_sms = (e.sms - ExchangeSms) & ~1;
        }
        ~Reserve() { e.gemm_sms = e.sms; }
    } reserve(*this);

    weight_grad(logits, Vocabulary, final_normed, W, layout.head);
    gemm(FGemmInputGrad, input_grad(logits, Vocabulary, layout.head, W, dbranch));
    norm_back(final_x, dbranch, layout.final_norm, layout.final_norm_bias, nullptr, dh, final_stats);
    if (!c.tied) // final norm + head form the first bucket; a tied head waits for the embedding scatter
        exchange_bucket(layout.final_norm, layout.count, depth);
    else
        exchange_bucket(layout.final_norm, layout.final_norm + (layer_norm ? 2 : 1) * W, depth);

    for (int l = depth - 1; l >= 0; --l) {
        LayerActivations &a = layers[l];
        const LayerOffsets &p = layout.layers[l];
        weight_grad(dh, W, a.activated, Hd, p.down);
        GemmArgs dact = input_grad(dh, W, p.down, Hd, c.mlp == TG_MLP_SWIGLU ? dactivated : dwide);
        if (c.mlp == TG_MLP_SWIGLU) {
            gemm(FGemmInputGrad, dact);
            run(FActivation, [&] { launch_swiglu_backward(act, a.wide, dactivated, dwide, M, Hd, stream); });
        } else {
            dact.epilogue = Epilogue::GeluGrad, dact.r = a.wide, dact.ldr = Hd;
            gemm(FGemmInputGrad, dact);
        }
        weight_grad(dwide, wide, a.normed2, W, p.gate);
        gemm(FGemmInputGrad, input_grad(dwide, wide, p.gate, W, dbranch));
        norm_back(a.middle, dbranch, p.mlp_norm, p.mlp_norm_bias, dh, dh_other, a.stats2);
        std::swap(dh, dh_other);

        weight_grad(dh, W, a.attended, W, p.attention);
        gemm(FGemmInputGrad, input_grad(dh, W, p.attention, W, dbranch));
        if (c.attention == TG_ATTENTION_ARGMAX) {
            ArgmaxAttentionBackwardArgs at{a.qkv, dbranch, a.selected, a.gates, a.derivatives, attention_scratch,
                                           dqkv, B, T, W, H};
            run(FAttentionBackward, [&] { launch_argmax_attention_backward(act, at, stream); });
        } else {
            SoftmaxAttentionBackwardArgs at{a.qkv, a.attended, dbranch, a.lse, attention_scratch, dqkv, B, T, W, H};
            run(FAttentionBackward, [&] {
                if (tensor_cores && act == Dtype::BF16 && flash_attention_supported(W, H)) {
                    launch_flash_attention_backward(a.qkv, a.attended, dbranch, a.lse, attention_scratch, dqkv, B, T, H,
                                                    counters, stream);
                    ++launches; // dq kernel + dk/dv kernel
                } else {
                    launch_softmax_attention_backward(act, at, stream);
                }
            });
        }
        if (c.rope == TG_ROPE_PARTIAL)
            run(FMisc, [&] { launch_rope(act, dqkv, M, T, W, H, true, stream); });
        weight_grad(dqkv, 3 * W, a.normed1, W, p.qkv);
        gemm(FGemmInputGrad, input_grad(dqkv, 3 * W, p.qkv, W, dbranch));
        norm_back(a.x, dbranch, p.attention_norm, p.attention_norm_bias, dh, dh_other, a.stats1);
        std::swap(dh, dh_other);
        int64_t layer_end = l + 1 < depth ? layout.layers[l + 1].attention_norm : layout.final_norm;
        exchange_bucket(p.attention_norm, layer_end, l);
    }
    run(FEmbeddingBackward, [&] {
        launch_embedding_backward(act, dh, x, gradient + layout.embedding, M, W, c.tied != 0, embedding_partial,
                                  stream);
    });
    if (embedding_partial)
        ++launches; // slices kernel + sum kernel
    exchange_bucket(layout.embedding, layout.embedding + int64_t(Vocabulary) * W, depth + 1);
    finish_exchange();
}

// ------------------------------------------------------------------------------- optimizer ---
void Engine::muon_family(int64_t first_offset, int rows, int cols) {
    const TgConfigEx &c = config;
    const int depth = c.base.depth;
    const int64_t stride = depth > 1 ? layout.layers[1].qkv - layout.layers[0].qkv : 0;
    const int r = std::min(rows, cols), n = std::max(rows, cols); // orthogonalise the wide orientation
    const int64_t per = int64_t(rows) * cols;
    // Under data parallelism the gradients are identical on every rank after the exchange, so the
    // Newton-Schulz iterations (the expensive part: 15 GEMMs per family) are sharded by layer: rank k
    // orthogonalises layers k*depth/world .. (k+1)*depth/world-1 and the BF16 results are
    // all-gathered; momentum and the weight update run for every layer on every rank, so replicas
    // stay bit-identical and any rank can write a checkpoint.
    const bool sharded = comm && depth % c.world == 0 && depth >= c.world;
    const int mine = sharded ? depth / c.world : depth, first = sharded ? c.rank * mine : 0;
    MuonPrepareArgs prep{gradient + first_offset, momentum + first_offset, muon_x[0], muon_sumsq, sumsq_partial,
                         sumsq_blocks, schedule, counters, c.base.momentum, c.base.clip, rows, cols, depth, stride};
    run(FMuon, [&] { launch_muon_prepare(prep, stream); });
    run(FMuon, [&] { launch_muon_normalize(muon_x[0], muon_sumsq, per, depth, stream); });
    bf16 *cur = muon_x[0] + first * per, *nxt = muon_x[1] + first * per;
    bf16 *a_buffer = muon_a + int64_t(first) * r * r, *b_buffer = muon_b + int64_t(first) * r * r;
    const bool small = muon_newton_schulz_small_supported(r, n); // the reference architecture: one launch, in place
    if (small)
        run(FMuon, [&] { launch_muon_newton_schulz_small(cur, r, n, c.base.ns_steps, mine, stream); });
    for (int it = 0; !small && it < c.base.ns_steps; ++it) {
        GemmArgs a; // A = X X^T
        a.a = cur, a.a_row = n, a.b = cur, a.b_row = n, a.c = a_buffer, a.ldc = r, a.m = r, a.n = r, a.k = n;
        a.batch = mine, a.a_batch = per, a.b_batch = per, a.c_batch = int64_t(r) * r, a.out = Dtype::BF16;
        GemmArgs b; // B = -4.775 A + 2.0315 A A
        b.a = a_buffer, b.a_row = r, b.b = a_buffer, b.b_row = 1, b.b_col = r, b.c = b_buffer, b.ldc = r;
        b.m = r, b.n = r, b.k = r, b.batch = mine, b.a_batch = b.b_batch = b.c_batch = b.r_batch = int64_t(r) * r;
        b.epilogue = Epilogue::Axpby, b.alpha = 2.0315f, b.beta = -4.775f, b.r = a_buffer, b.ldr = r;
        b.out = Dtype::BF16;
        GemmArgs x2; // X' = 3.4445 X + B X
        x2.a = b_buffer, x2.a_row = r, x2.b = cur, x2.b_row = 1, x2.b_col = n, x2.c = nxt, x2.ldc = n;
        x2.m = r, x2.n = n, x2.k = r, x2.batch = mine, x2.a_batch = int64_t(r) * r;
        x2.b_batch = x2.c_batch = x2.r_batch = per;
        x2.epilogue = Epilogue::Axpby, x2.alpha = 1.f, x2.beta = 3.4445f, x2.r = cur, x2.ldr = n;
        x2.out = Dtype::BF16;
        for (GemmArgs *g : {&a, &b, &x2}) {
            run(FMuon, [&] {
                g->in = Dtype::BF16;
                if (tensor_cores && gemm_tc_supported(*g))
                    launches += launch_gemm_tc(*g, sms, counters, stream, &gemm_workspace) - 1;
                else
                    launch_gemm_simt(*g, stream);
            });
        }
        std::swap(cur, nxt);
    }
    bf16 *all = cur - first * per; // the buffer holding every layer's result
    if (sharded) {
        const Nccl &nccl = Nccl::get();
        run(FExchange, [&] {
            nccl.check(nccl.AllGather(cur, all, size_t(mine) * per, Nccl::Bfloat16, comm, stream), "ncclAllGather");
        });
    }
    MuonApplyArgs apply{all, weight_high + first_offset, weight_low + first_offset,
                        weight_fp32 ? weight_fp32 + first_offset : nullptr, schedule, counters, c.base.muon_lr,
                        c.base.weight_decay, rows, cols, depth, stride};
    run(FMuon, [&] { launch_muon_apply(apply, stream); });
}

void Engine::optimize() {
    const TgConfigEx &c = config;
    run(FOptimizer, [&] { launch_sum_squares(gradient, layout.count, sumsq_partial, sumsq_blocks, stream); });
    AdamArgs a{gradient, momentum, variance, weight_high, weight_low, weight_fp32, adam_mode, sumsq_partial,
               sumsq_blocks, schedule, counters, c.base.learning_rate, c.base.beta1, c.base.beta2,
               c.base.weight_decay, c.base.epsilon, c.base.clip, layout.count};
    run(FOptimizer, [&] { launch_adamw(a, sms, stream); });
    if (c.hidden_optimizer == TG_HIDDEN_MUON) {
        const LayerOffsets &p = layout.layers[0];
        const int W = c.width, Hd = c.hidden;
        muon_family(p.qkv, 3 * W, W); // q, k and v orthogonalised as one matrix (reference cuda/optim.cuh:109-117)
        muon_family(p.attention, W, W);
        muon_family(p.gate, Hd, W);
        if (c.mlp == TG_MLP_SWIGLU)
            muon_family(p.up, Hd, W);
        muon_family(p.down, W, Hd);
    }
    run(FMisc, [&] { launch_advance(counters, stream); });
}

// ------------------------------------------------------------------------------- modes -------
void Engine::one_step(RunMode mode) {
    if (mode == RunMode::Train) {
        SampleArgs s{data, data_size, config.base.seed, counters, -1, config.base.batch, config.base.context,
                     config.world, config.rank, x, y};
        run(FSample, [&] { launch_sample(s, stream); });
    }
    if (mode != RunMode::OptimizerOnly) {
        forward(mode != RunMode::Evaluate, mode != RunMode::Train && logits_fp32 != nullptr);
        if (mode == RunMode::Evaluate)
            return;
        if (mode == RunMode::Train)
            run(FMisc, [&] {
                launch_loss_history(token_losses, loss_history, counters, config.base.batch, config.base.context,
                                    stream);
            });
        backward();
        if (mode == RunMode::Gradients)
            return;
    }
    optimize();
}

// The captured step holds raw pointers: it is dropped whenever one of them may change.
void Engine::drop_graph() {
    if (step_graph)
        cudaGraphExecDestroy(step_graph);
    step_graph = nullptr;
}

void Engine::train(int steps) {
    set_device();
    if (!data || steps < 1 || steps > MaxLaunchSteps)
        throw std::runtime_error("Load data first; each invocation permits 1.." + std::to_string(MaxLaunchSteps) +
                                 " steps");
    if (config.world > 1 && !comm)
        throw std::runtime_error("This engine was created without a communicator: it cannot train on its own");
    if (step + uint64_t(steps) > uint64_t(INT32_MAX))
        throw std::runtime_error("Training step count exceeds signed 32-bit indexing");
    if (schedule && step + uint64_t(steps) > uint64_t(schedule_steps))
        throw std::runtime_error("Training would exceed the OneCycle schedule");
    CHECK_CUDA(cudaMemsetAsync(&counters->iteration, 0, sizeof(int), stream));
    // A step reads everything that changes from device memory, so its kernel sequence is captured
    // once (after one eager step has sized every workspace) and replayed as a CUDA graph.
    const bool use_graph = !profile && !comm && !(config.flags & TG_FLAG_NO_GRAPH);
    for (int i = 0; i < steps; ++i) {
        if (!use_graph || !graph_warm) {
            one_step(RunMode::Train);
            graph_warm = true;
            continue;
        }
        if (step_graph && graph_generation != gemm_workspace.generation)
            drop_graph(); // the split-K workspace moved since the capture
        if (!step_graph) {
            graph_generation = gemm_workspace.generation;
            const int64_t before = launches;
            cudaGraph_t graph = nullptr;
            CHECK_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
            try {
                one_step(RunMode::Train);
            } catch (...) {
                cudaStreamEndCapture(stream, &graph);
                if (graph)
                    cudaGraphDestroy(graph);
                throw;
            }
            CHECK_CUDA(cudaStreamEndCapture(stream, &graph));
            cudaError_t status = cudaGraphInstantiate(&step_graph, graph, 0);
            cudaGraphDestroy(graph);
            CHECK_CUDA(status);
            graph_launches = launches - before;
            launches = before;
        }
        CHECK_CUDA(cudaGraphLaunch(step_graph, stream));
        launches += graph_launches;
    }
    last_train_steps = steps;
    losses_reduced = false;
    step += steps;
}

void Engine::training_losses(float *out, int count) {
    if (!out && count)
        throw std::runtime_error("Missing training loss output");
    if (count < 0 || count > last_train_steps)
        throw std::runtime_error("Training loss count exceeds the last launch");
    set_device();
    const int T = config.base.context;
    if (comm && !losses_reduced) { // per-position means of the global batch = mean over ranks
        const Nccl &nccl = Nccl::get();
        nccl.check(nccl.AllReduce(loss_history, loss_history, size_t(last_train_steps) * T, Nccl::Float32, Nccl::Sum,
                                  comm, stream),
                   "ncclAllReduce");
        losses_reduced = true;
        std::vector<float> all(size_t(last_train_steps) * T);
        CHECK_CUDA(cudaMemcpyAsync(all.data(), loss_history, all.size() * 4, cudaMemcpyDeviceToHost, stream));
        CHECK_CUDA(cudaStreamSynchronize(stream));
        for (float &v : all)
            v /= config.world;
        CHECK_CUDA(cudaMemcpyAsync(loss_history, all.data(), all.size() * 4, cudaMemcpyHostToDevice, stream));
    }
    CHECK_CUDA(cudaMemcpyAsync(out, loss_history, size_t(count) * T * sizeof(float), cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
    flush_profile();
    check_device_error();
}

float Engine::train_mean_loss(int steps) {
    train(steps);
    std::vector<float> all(size_t(steps) * config.base.context);
    training_losses(all.data(), steps);
    double sum = 0;
    for (int p = 0; p < config.base.context; ++p)
        sum += all[size_t(steps - 1) * config.base.context + p];
    return float(sum / config.base.context);
}

void Engine::batch(const uint8_t *bx, const uint8_t *by, float *logits_out, float *gradient_out,
                   float *per_position) {
    set_device();
    const int B = config.base.batch, T = config.base.context;
    if (!logits_fp32)
        allocate(logits_fp32, size_t(tokens) * Vocabulary, false);
    CHECK_CUDA(cudaMemcpyAsync(x, bx, tokens, cudaMemcpyHostToDevice, stream));
    CHECK_CUDA(cudaMemcpyAsync(y, by, tokens, cudaMemcpyHostToDevice, stream));
    one_step(gradient_out ? RunMode::Gradients : RunMode::Evaluate);
    if (logits_out)
        CHECK_CUDA(cudaMemcpyAsync(logits_out, logits_fp32, size_t(tokens) * Vocabulary * 4, cudaMemcpyDeviceToHost,
                                   stream));
    if (gradient_out)
        CHECK_CUDA(cudaMemcpyAsync(gradient_out, gradient, layout.count * 4, cudaMemcpyDeviceToHost, stream));
    std::vector<float> losses(tokens);
    CHECK_CUDA(cudaMemcpyAsync(losses.data(), token_losses, size_t(tokens) * 4, cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
    flush_profile();
    check_device_error();
    if (per_position)
        for (int p = 0; p < T; ++p) { // reference cuda/runtime.cu:279-290
            double sum = 0;
            for (int b = 0; b < B; ++b)
                sum += losses[size_t(b) * T + p];
            per_position[p] = float(sum / B);
        }
}

void Engine::predict(const uint8_t *context, float *logits256) {
    if (!context || !logits256)
        throw std::runtime_error("Missing prediction input or output");
    set_device();
    const int T = config.base.context;
    if (!logits_fp32)
        allocate(logits_fp32, size_t(tokens) * Vocabulary, false);
    // One sequence through the forward pass.  The reference fills the whole batch with copies of the
    // context (cuda/runtime.cu:322-351) and reads row T-1 of the first; sequences are independent, so
    // the single row gives the same logits for 1/batch of the work.
    CHECK_CUDA(cudaMemcpyAsync(x, context, T, cudaMemcpyHostToDevice, stream));
    CHECK_CUDA(cudaMemsetAsync(y, 0, T, stream));
    forward_batch = 1;
    try {
        one_step(RunMode::Evaluate);
    } catch (...) {
        forward_batch = 0;
        throw;
    }
    forward_batch = 0;
    CHECK_CUDA(cudaMemcpyAsync(logits256, logits_fp32 + size_t(T - 1) * Vocabulary, Vocabulary * sizeof(float),
                               cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
    check_device_error();
}

void Engine::optimizer_test(const float *g, int steps) {
    set_device();
    if (steps < 1 || steps > 64)
        throw std::runtime_error("steps must be 1..64");
    if (schedule && step + uint64_t(steps) > uint64_t(schedule_steps))
        throw std::runtime_error("Optimizer test would exceed the OneCycle schedule");
    CHECK_CUDA(cudaMemcpyAsync(gradient, g, layout.count * 4, cudaMemcpyHostToDevice, stream));
    for (int i = 0; i < steps; ++i)
        one_step(RunMode::OptimizerOnly);
    step += steps;
    CHECK_CUDA(cudaStreamSynchronize(stream));
    check_device_error();
}

void Engine::sample(uint64_t at_step, uint8_t *bx, uint8_t *by) {
    set_device();
    if (!data)
        throw std::runtime_error("Load data first");
    SampleArgs s{data, data_size, config.base.seed, counters, (long long)at_step, config.base.batch,
                 config.base.context, config.world, config.rank, x, y};
    run(FSample, [&] { launch_sample(s, stream); });
    CHECK_CUDA(cudaMemcpyAsync(bx, x, tokens, cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaMemcpyAsync(by, y, tokens, cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
}

void Engine::set_optimizer_state(const float *m, const float *v, uint64_t at_step) {
    if (!m || !v)
        throw std::runtime_error("Missing optimizer state input");
    set_device();
    CHECK_CUDA(cudaMemcpyAsync(momentum, m, layout.count * 4, cudaMemcpyHostToDevice, stream));
    CHECK_CUDA(cudaMemcpyAsync(variance, v, layout.count * 4, cudaMemcpyHostToDevice, stream));
    StepCounters host{};
    host.step = at_step;
    CHECK_CUDA(cudaMemcpyAsync(counters, &host, sizeof(host), cudaMemcpyHostToDevice, stream));
    step = at_step;
    CHECK_CUDA(cudaStreamSynchronize(stream));
}
void Engine::get_optimizer_state(float *m, float *v, uint64_t *at_step) {
    if (!m || !v || !at_step)
        throw std::runtime_error("Missing optimizer state output");
    set_device();
    CHECK_CUDA(cudaMemcpyAsync(m, momentum, layout.count * 4, cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaMemcpyAsync(v, variance, layout.count * 4, cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
    *at_step = step;
}

// Diagnostic read-back of an activation the last forward pass saved (they are kept for backward).
int64_t Engine::read_activation(int layer, const char *name, float *out, int64_t capacity) {
    set_device();
    const std::string which = name ? name : "";
    const int W = config.width;
    const void *source = nullptr;
    int64_t columns = W;
    if (layer < 0) {
        if (which == "final_x")
            source = final_x;
        else if (which == "final_normed")
            source = final_normed;
    } else if (layer < int(layers.size())) {
        const LayerActivations &a = layers[layer];
        if (which == "x")
            source = a.x;
        else if (which == "normed1")
            source = a.normed1;
        else if (which == "qkv")
            source = a.qkv, columns = 3 * W;
        else if (which == "attended")
            source = a.attended;
        else if (which == "middle")
            source = a.middle;
        else if (which == "normed2")
            source = a.normed2;
        else if (which == "activated")
            source = a.activated, columns = config.hidden;
    }
    if (!source)
        throw std::runtime_error("Unknown activation '" + which + "' for layer " + std::to_string(layer));
    const int64_t count = int64_t(tokens) * columns;
    if (!out)
        return count;
    if (capacity < count)
        throw std::runtime_error("Activation buffer too small");
    if (act == Dtype::FP32) {
        CHECK_CUDA(cudaMemcpyAsync(out, source, count * 4, cudaMemcpyDeviceToHost, stream));
        CHECK_CUDA(cudaStreamSynchronize(stream));
        return count;
    }
    std::vector<uint16_t> raw(count);
    CHECK_CUDA(cudaMemcpyAsync(raw.data(), source, count * 2, cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
    for (int64_t i = 0; i < count; ++i) {
        const uint32_t bits = uint32_t(raw[i]) << 16;
        memcpy(out + i, &bits, 4);
    }
    return count;
}

// One optimizer step on bytes supplied by the caller instead of the resident corpus.
void Engine::train_batch(const uint8_t *bx, const uint8_t *by, float *per_position) {
    set_device();
    if (!bx || !by)
        throw std::runtime_error("Missing batch input");
    if (config.world > 1 && !comm)
        throw std::runtime_error("This engine was created without a communicator: it cannot train on its own");
    if (schedule && step + 1 > uint64_t(schedule_steps))
        throw std::runtime_error("Training would exceed the OneCycle schedule");
    CHECK_CUDA(cudaMemcpyAsync(x, bx, tokens, cudaMemcpyHostToDevice, stream));
    CHECK_CUDA(cudaMemcpyAsync(y, by, tokens, cudaMemcpyHostToDevice, stream));
    CHECK_CUDA(cudaMemsetAsync(&counters->iteration, 0, sizeof(int), stream));
    forward(true, false);
    run(FMisc, [&] {
        launch_loss_history(token_losses, loss_history, counters, config.base.batch, config.base.context, stream);
    });
    backward();
    optimize();
    step += 1;
    last_train_steps = 1;
    losses_reduced = false;
    if (per_position)
        training_losses(per_position, 1);
}
