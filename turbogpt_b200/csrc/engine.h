// The training engine behind the C ABI: device arena, the kernel sequence of one step
// (forward, loss, backward, gradient exchange, optimizer) and its evaluation modes.
#pragma once
#include "kernels.cuh"
#include <memory>
#include <string>
#include <vector>

// Minimal NCCL surface, resolved with dlopen so the library loads without NCCL present.
struct Nccl {
    using Comm = void *;
    struct UniqueId {
        char internal[128];
    };
    int (*GetUniqueId)(UniqueId *) = nullptr;
    int (*CommInitRank)(Comm *, int, UniqueId, int) = nullptr;
    // ncclConfig_t as NCCL 2.17 laid it out; later libraries read `size` and `version` and fill the
    // fields added since with their defaults.
    struct Config {
        size_t size;
        unsigned magic, version;
        int blocking, cga_cluster_size, min_ctas, max_ctas;
        const char *net_name;
    };
    int (*CommInitRankConfig)(Comm *, int, UniqueId, int, Config *) = nullptr; // optional (NCCL >= 2.17)
    int (*AllReduce)(const void *, void *, size_t, int, int, Comm, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, Comm, cudaStream_t) = nullptr;
    int (*CommDestroy)(Comm) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    static const Nccl &get(); // throws when NCCL cannot be loaded
    void check(int result, const char *what) const;
    static constexpr int Float32 = 7, Bfloat16 = 9, Sum = 0;
};

enum Family {
    FSample, FEmbedding, FNorm, FGemmForward, FGemmInputGrad, FGemmWeightGrad, FAttentionForward,
    FAttentionBackward, FActivation, FCrossEntropy, FNormBackward, FEmbeddingBackward, FOptimizer, FMuon,
    FExchange, FMisc, FamilyCount
};
extern const char *const family_names[FamilyCount];

struct LayerActivations { // saved by forward for backward (reference cuda/types.cuh:40-44)
    void *x, *normed1, *qkv, *attended, *middle, *normed2, *wide, *activated; // wide: gate|up, or gelu'(pre-activation)
    int *selected;
    float *gates, *derivatives, *lse;
    float *stats1, *stats2; // per row: mean and 1/sigma of the two norms, saved by forward for backward
};

enum class RunMode { Evaluate, Gradients, Train, OptimizerOnly }; // reference cuda/trainer.cuh:6

struct Engine {
    TgConfigEx config{};
    Layout layout{};
    Dtype act = Dtype::BF16;
    int sms = 0, tokens = 0;
    bool tensor_cores = true, profile = false;
    cudaStream_t stream = nullptr, exchange_stream = nullptr;
    std::vector<void *> allocations;
    size_t allocated_bytes = 0;

    // parameters and optimizer state (flat, layout order)
    bf16 *weight_high = nullptr;
    uint16_t *weight_low = nullptr;
    float *weight_fp32 = nullptr, *momentum = nullptr, *variance = nullptr, *gradient = nullptr;
    uint8_t *adam_mode = nullptr;
    bf16 *gradient_bf16 = nullptr; // staging for BF16 gradient exchange
    // data
    uint8_t *data = nullptr, *x = nullptr, *y = nullptr;
    int64_t data_size = 0;
    // activations
    std::vector<LayerActivations> layers;
    void *final_x = nullptr, *final_normed = nullptr, *logits = nullptr;
    float *final_stats = nullptr;
    void *dhidden[2] = {nullptr, nullptr}, *dbranch = nullptr, *dwide = nullptr, *dactivated = nullptr,
         *dqkv = nullptr;
    float *attention_scratch = nullptr; // dt (arg-max) or delta (softmax)
    float *token_losses = nullptr, *loss_history = nullptr, *norm_partial = nullptr, *sumsq_partial = nullptr,
          *logits_fp32 = nullptr, *mean_loss = nullptr, *embedding_partial = nullptr;
    int norm_blocks = 0, sumsq_blocks = 0;
    StepCounters *counters = nullptr;
    TgStepRates *schedule = nullptr;
    int schedule_steps = 0;
    // Muon scratch
    bf16 *muon_x[2] = {nullptr, nullptr}, *muon_a = nullptr, *muon_b = nullptr;
    float *muon_sumsq = nullptr;
    // host mirrors
    uint64_t step = 0;
    int last_train_steps = 0;
    bool losses_reduced = true;
    // data parallel
    Nccl::Comm comm = nullptr;
    int gemm_sms = 0; // SMs the GEMMs of the current phase may use (fewer while a gradient bucket may be in flight)
    std::vector<cudaEvent_t> bucket_events;
    cudaEvent_t exchange_done = nullptr;
    // profiling
    struct Timed {
        int family;
        cudaEvent_t start, stop;
    };
    std::vector<Timed> timed;
    std::vector<cudaEvent_t> event_pool;
    double family_ms[FamilyCount] = {};
    int64_t family_launches[FamilyCount] = {};
    int64_t launches = 0, graph_launches = 0;
    GemmWorkspace gemm_workspace; // this engine's split-K scratch (never shared with another engine or stream)
    float *simt_scratch = nullptr; // partial tiles of CUDA-core GEMMs that are cut along K (6 MB bounds every shape)
    cudaGraphExec_t step_graph = nullptr; // one captured training step
    bool graph_warm = false;
    int forward_batch = 0; // sequences the next forward pass covers (0: the configured batch)
    uint64_t graph_generation = 0;
    void drop_graph();

    explicit Engine(const TgConfigEx &c);
    ~Engine();
    Engine(const Engine &) = delete;

    template <class T> void allocate(T *&p, size_t n, bool zero = true);
    const void *weight(int64_t offset) const;
    void set_device() const;

    void set_weights(const float *w);
    void get_weights(float *w);
    void set_data(const uint8_t *bytes, int64_t size);
    void set_onecycle(const TgOneCycle &s);
    void train(int steps);
    void training_losses(float *out, int count);
    void batch(const uint8_t *bx, const uint8_t *by, float *logits_out, float *gradient_out, float *per_position);
    void predict(const uint8_t *context, float *logits256);
    void optimizer_test(const float *g, int steps);
    void sample(uint64_t at_step, uint8_t *bx, uint8_t *by);
    void set_optimizer_state(const float *m, const float *v, uint64_t at_step);
    void get_optimizer_state(float *m, float *v, uint64_t *at_step);
    float train_mean_loss(int steps);
    void train_batch(const uint8_t *bx, const uint8_t *by, float *per_position);
    void flush_profile();
    int64_t read_activation(int layer, const char *name, float *out, int64_t capacity);

  private:
    void initialize();
    void release();
    template <class F> void run(Family f, F &&launch);
    void gemm(Family f, GemmArgs g);
    void forward(bool want_gradient, bool dump_logits);
    void backward();
    void exchange_bucket(int64_t begin, int64_t end, int index);
    void finish_exchange();
    void optimize();
    void muon_family(int64_t first_offset, int rows, int cols);
    void one_step(RunMode mode);
    void check_device_error();
};
