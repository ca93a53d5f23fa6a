// Test probe (TEST INFRASTRUCTURE ONLY): drives the reference's own checkpoint reader and writer
// (checkpoint.cpp, compiled unmodified where it lies) so the tests can check that files move between
// it and the library's extended format in both directions.
//   ckpt_probe load <file> <depth> <context>         prints: step total_steps sum(weights) sum(momentum)
//   ckpt_probe save <file> <depth> <context> <step>  writes weights[i] = i * 0.001, 40 scheduled steps
#include "checkpoint.h"
#include "model.h"
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>

int main(int argc, char **argv) {
    try {
        if (argc < 5)
            throw std::runtime_error("usage: ckpt_probe load|save <file> <depth> <context> [step]");
        Config config{};
        config.depth = atoi(argv[3]), config.context = atoi(argv[4]);
        if (!strcmp(argv[1], "load")) {
            TrainingState state = load_training_state(argv[2], config);
            double weights = 0, momentum = 0;
            for (float v : state.weights)
                weights += v;
            for (float v : state.momentum)
                momentum += v;
            printf("%llu %d %.17g %.17g\n", (unsigned long long)state.step, state.scheduler.total_steps, weights,
                   momentum);
            return 0;
        }
        TrainingState state;
        const int count = parameter_layout(config.depth).count;
        state.weights.resize(count), state.momentum.assign(count, 0.25f), state.variance.assign(count, 0.5f);
        for (int i = 0; i < count; ++i)
            state.weights[i] = float(i) * .001f;
        state.scheduler = OneCycle{};
        state.scheduler.total_steps = 40;
        state.step = argc > 5 ? strtoull(argv[5], nullptr, 10) : 0;
        state.final_loss_sums.assign(config.context, 0.0);
        save_training_state(argv[2], config, state);
        return 0;
    } catch (const std::exception &error) {
        fprintf(stderr, "%s\n", error.what());
        return 1;
    }
}
