// Shared declarations of the engine: configuration, flat parameter layout, error helpers.
#pragma once
#include "../../include/turbogpt_b200.h"
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

using bf16 = __nv_bfloat16;

inline void check_cuda(cudaError_t error, const char *what = nullptr) {
    if (error != cudaSuccess)
        throw std::runtime_error(std::string(what ? what : "CUDA") + ": " + cudaGetErrorString(error));
}
#define CHECK_CUDA(expr) check_cuda((expr), #expr)

// splitmix64 finaliser; defines the data indexing (reference utils.h:13-18) and must be bit-exact.
__host__ __device__ inline uint64_t hash_u64(uint64_t x) {
    x += 0x9e3779b97f4a7c15ULL;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
    return x ^ (x >> 31);
}

constexpr int Vocabulary = 256;
constexpr int MaxDepth = 64;
constexpr int MaxLaunchSteps = 4096; // reference cuda/types.cuh:10

// Offsets of one layer's tensors in the flat parameter array (reference model.h:6-8, with
// LayerNorm biases and without `up` for a GELU MLP; -1 marks an absent tensor).
struct LayerOffsets {
    int64_t attention_norm, attention_norm_bias, qkv, attention, mlp_norm, mlp_norm_bias, gate, up, down;
};
struct TensorInfo {
    int64_t offset;
    int rows, cols;   // cols == 0: vector of `rows` elements
    int kind;         // 0 embedding, 1 norm scale/bias, 2 hidden matrix, 3 head
    int seed_key;     // initialize_weights key (reference model.cpp:17-29); -1: constant
    float init_scale; // normal scale, or the constant for norm tensors
};
struct Layout {
    int64_t embedding, final_norm, final_norm_bias, head, count;
    LayerOffsets layers[MaxDepth];
    std::vector<TensorInfo> tensors;
};

void validate_config(const TgConfigEx &c);           // throws std::runtime_error
Layout make_layout(const TgConfigEx &c);             // reference model.h:12-37 generalised
void initialize_weights(const TgConfigEx &c, float *w); // reference model.cpp:7-31 generalised
TgStepRates onecycle_point(const TgOneCycle &s, int step); // reference optim.h:18-44
void save_checkpoint(const std::string &path, const TgConfigEx &c, const TgCheckpoint &s); // checkpoint.cpp
void load_checkpoint(const std::string &path, const TgConfigEx &c, TgCheckpoint &s);

static_assert(sizeof(TgConfig) == 72 && sizeof(TgOneCycle) == 48 && sizeof(TgStepRates) == 8,
              "struct layouts are part of the ABI (reference tests/bridge.py:7-26)");
static_assert(sizeof(TgConfigEx) == 256, "TgConfigEx layout is mirrored by the ctypes bridge");
