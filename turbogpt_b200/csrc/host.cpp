// Host-only pieces shared with the reference's host program: configuration checks, the flat
// parameter layout, weight initialisation and the OneCycle schedule.
#include "common.h"
#include <algorithm>
#include <cmath>
#include <random>

void validate_config(const TgConfigEx &c) {
    const TgConfig &b = c.base;
    if (c.struct_size != int(sizeof(TgConfigEx)))
        throw std::runtime_error("TgConfigEx.struct_size does not match this library");
    if (b.depth < 1 || b.depth > MaxDepth)
        throw std::runtime_error("depth must be 1.." + std::to_string(MaxDepth));
    if (b.context < 2 || b.context > 65536)
        throw std::runtime_error("context must be 2..65536");
    if (b.batch < 1 || int64_t(b.batch) * b.context > (int64_t(1) << 24))
        throw std::runtime_error("batch must be at least 1 with batch*context at most 16777216");
    if (b.inflight != 1)
        throw std::runtime_error(b.inflight > 1 && b.inflight <= 256
                                     ? "Experimental overlap requires build.ps1 -Pipeline"
                                     : "inflight must be 1..256");
    if (b.ns_steps < 1 || b.ns_steps > 10)
        throw std::runtime_error("ns_steps must be 1..10");
    if (c.width < 8 || c.width % 8 || c.heads < 1 || c.width % c.heads || (c.width / c.heads) % 2)
        throw std::runtime_error("width must be a multiple of 8 and of heads, with an even head size");
    if (c.hidden < 8 || c.hidden % 8)
        throw std::runtime_error("hidden must be a positive multiple of 8");
    if (c.width > 8192 || c.hidden > 32768)
        throw std::runtime_error("width at most 8192 and hidden at most 32768");
    auto flag = [](int v, int n, const char *name) {
        if (v < 0 || v >= n)
            throw std::runtime_error(std::string("unknown ") + name + " selector");
    };
    flag(c.norm, 2, "norm");
    flag(c.attention, 2, "attention");
    flag(c.mlp, 2, "mlp");
    flag(c.tied, 2, "tied");
    flag(c.rope, 2, "rope");
    flag(c.hidden_optimizer, 2, "hidden_optimizer");
    flag(c.precision, 2, "precision");
    if (c.world < 1 || c.world > 64 || c.rank < 0 || c.rank >= c.world)
        throw std::runtime_error("world must be 1..64 and rank in [0, world)");
    if (c.attention == TG_ATTENTION_SOFTMAX && c.width / c.heads > 256)
        throw std::runtime_error("softmax attention supports head sizes up to 256");
}

Layout make_layout(const TgConfigEx &c) {
    Layout p{};
    int64_t n = 0;
    const int W = c.width, Hd = c.hidden, depth = c.base.depth;
    const float residual_scale = .02f / std::sqrt(2.f * depth);
    auto take = [&](int rows, int cols, int kind, int key, float scale) {
        int64_t offset = n;
        p.tensors.push_back({offset, rows, cols, kind, key, scale});
        n += int64_t(rows) * (cols ? cols : 1);
        return offset;
    };
    p.embedding = take(Vocabulary, W, c.tied ? 3 : 0, 1, .02f);
    for (int l = 0; l < depth; ++l) {
        LayerOffsets &b = p.layers[l];
        b.attention_norm = take(W, 0, 1, -1, 1.f);
        b.attention_norm_bias = c.norm == TG_NORM_LAYER ? take(W, 0, 1, -1, 0.f) : -1;
        b.qkv = take(3 * W, W, 2, 100 + l * 10, .02f);
        b.attention = take(W, W, 2, 101 + l * 10, residual_scale);
        b.mlp_norm = take(W, 0, 1, -1, 1.f);
        b.mlp_norm_bias = c.norm == TG_NORM_LAYER ? take(W, 0, 1, -1, 0.f) : -1;
        // gate and up are adjacent so one projection computes both (reference model.h:27-31).
        b.gate = take(Hd, W, 2, 102 + l * 10, .02f);
        b.up = c.mlp == TG_MLP_SWIGLU ? take(Hd, W, 2, 104 + l * 10, .02f) : -1;
        b.down = take(W, Hd, 2, 103 + l * 10, residual_scale);
    }
    p.final_norm = take(W, 0, 1, -1, 1.f);
    p.final_norm_bias = c.norm == TG_NORM_LAYER ? take(W, 0, 1, -1, 0.f) : -1;
    p.head = c.tied ? p.embedding : take(Vocabulary, W, 3, 3, .02f);
    p.count = n;
    return p;
}

void initialize_weights(const TgConfigEx &c, float *w) {
    Layout p = make_layout(c);
    for (const TensorInfo &t : p.tensors) {
        int64_t count = int64_t(t.rows) * (t.cols ? t.cols : 1);
        if (t.seed_key < 0) {
            std::fill_n(w + t.offset, count, t.init_scale);
            continue;
        }
        // One generator per tensor role keeps common matrices identical across shapes.
        std::mt19937 generator(unsigned(hash_u64(c.base.seed + uint64_t(t.seed_key))));
        std::normal_distribution<float> normal(0, t.init_scale);
        for (int64_t i = 0; i < count; ++i)
            w[t.offset + i] = normal(generator);
    }
}

TgStepRates onecycle_point(const TgOneCycle &s, int step) {
    if (s.total_steps < 1 || step < 0 || step >= s.total_steps ||
        !(s.warmup_fraction > 0 && s.warmup_fraction < 1) ||
        !(s.initial_lr_fraction > 0 && s.initial_lr_fraction < 1) ||
        !(s.final_lr_fraction > 0 && s.final_lr_fraction <= s.initial_lr_fraction) ||
        !(s.low_momentum >= 0 && s.low_momentum < 1) ||
        !(s.high_momentum >= s.low_momentum && s.high_momentum < 1))
        throw std::runtime_error("Invalid OneCycle schedule or step");
    const double warmup = s.warmup_fraction * s.total_steps - 1;
    if (warmup == 0)
        throw std::runtime_error("OneCycle warmup must span at least two steps");
    const bool rising = step <= warmup;
    const double t = rising ? step / warmup : (step - warmup) / (s.total_steps - 1 - warmup);
    const double blend = 0.5 * (1 + std::cos(3.14159265358979323846 * t));
    auto between = [blend](double from, double to) { return to + (from - to) * blend; };
    TgStepRates r;
    r.multiplier = float(rising ? between(s.initial_lr_fraction, 1.0) : between(1.0, s.final_lr_fraction));
    r.momentum = float(rising ? between(s.high_momentum, s.low_momentum)
                              : between(s.low_momentum, s.high_momentum));
    return r;
}
