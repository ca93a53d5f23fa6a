// Prints known answers from the reference's own host headers (utils.h, optim.h, model.h,
// model.cpp), compiled where they lie with -I<reference root>.  Used only by
// make_golden.py in the development container; the JSON it prints is committed.
#include "model.h"
#include "optim.h"
#include "utils.h"
#include <cinttypes>
#include <cstdio>
#include <cstring>

int main() {
    std::printf("{\n \"hash_u64\": [");
    const uint64_t keys[] = {0, 1, 2, 3407, 3407 + 16, 0xffffffffffffffffULL, 0x9e3779b97f4a7c15ULL,
                             123456789012345ULL};
    for (size_t i = 0; i < sizeof(keys) / sizeof(*keys); ++i)
        std::printf("%s[\"%" PRIu64 "\", \"%" PRIu64 "\"]", i ? ", " : "", keys[i], hash_u64(keys[i]));
    std::printf("],\n \"parameter_count\": {\"4\": %d, \"8\": %d},\n", parameter_layout(4).count,
                parameter_layout(8).count);
    ParameterLayout p = parameter_layout(4);
    std::printf(" \"layout4\": {\"embedding\": %d, \"l0_qkv\": %d, \"l3_down\": %d, \"final_norm\": %d, \"head\": %d},\n",
                p.embedding, p.layers[0].qkv, p.layers[3].down, p.final_norm, p.head);
    std::printf(" \"sizes\": {\"Config\": %zu, \"OneCycle\": %zu, \"StepRates\": %zu},\n", sizeof(Config),
                sizeof(OneCycle), sizeof(StepRates));
    std::printf(" \"onecycle\": [");
    const int totals[] = {8, 20, 37, 48829};
    bool first = true;
    for (int total : totals) {
        OneCycle s;
        s.total_steps = total;
        const int steps[] = {0, 1, total / 3, int(.3 * total) - 1, int(.3 * total), int(.3 * total) + 1,
                             total - 2, total - 1};
        for (int step : steps) {
            if (step < 0 || step >= total)
                continue;
            StepRates r = onecycle_point(s, step);
            uint32_t a, b;
            std::memcpy(&a, &r.multiplier, 4);
            std::memcpy(&b, &r.momentum, 4);
            std::printf("%s[%d, %d, %u, %u]", first ? "" : ", ", total, step, a, b);
            first = false;
        }
    }
    std::printf("],\n");
    // Initial weights of the shipped configuration (seed 3407): bit patterns of a few entries
    // and a checksum, pinning the mt19937 + normal_distribution + hash_u64 seeding rule.
    Config c;
    c.depth = 4;
    std::vector<float> w = initialize_weights(c);
    uint64_t sum = 0;
    for (float v : w) {
        uint32_t bits;
        std::memcpy(&bits, &v, 4);
        sum = hash_u64(sum ^ bits);
    }
    std::printf(" \"init_weights\": {\"count\": %zu, \"checksum\": \"%" PRIu64 "\", \"first\": [", w.size(), sum);
    const int probe[] = {0, 1, 4095, 4096, 4112, 4113, 21647};
    for (size_t i = 0; i < sizeof(probe) / sizeof(*probe); ++i) {
        uint32_t bits;
        std::memcpy(&bits, &w[probe[i]], 4);
        std::printf("%s[%d, %u]", i ? ", " : "", probe[i], bits);
    }
    std::printf("]}\n}\n");
}
