// turbogpt_dp: a data-parallel training host over the C ABI, in the terms of the reference's
// trainer.cpp:39-180 — create, load or initialise, OneCycle, corpus, chunks of tg_train whose
// losses are read back while the next chunk runs, periodic and final checkpoints, --load to
// resume — with one engine per device instead of one engine (config.h:6 selects a single GPU).
//
// One thread per device drives its engine; the engines of one job share an NCCL communicator
// created from one id.  Rank 0 alone logs and writes checkpoints (replicas hold identical weights
// and optimizer state: gradients are summed before every update).  A rank stops only between
// chunks: every rank checks the shared failure flag before it launches the next chunk, so no rank
// is left waiting in a collective that another one will never join.
//
//   turbogpt_dp --data corpus.bin --log-to runs/x [--devices 0,1,2,3] [--tokens N]
//               [--depth L --width W --heads H --hidden F --context T --batch B]
//               [--optimizer adamw|muon] [--learning-rate R] [--chunk N] [--checkpoint-every N]
//               [--load runs/x/model.pt] [--save path] [--seed S] [--bf16-exchange] [--stop-after N]
#include "../../include/turbogpt_b200.h"
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <sys/stat.h>
#include <thread>
#include <vector>

namespace {
using Clock = std::chrono::steady_clock;

struct Options {
    std::string data, log_to, load, save;
    std::vector<int> devices{0};
    long long tokens = 0;
    int depth = 12, width = 768, heads = 12, hidden = 3072, context = 1024, batch = 32;
    int chunk = 20, checkpoint_every = 0, stop_after = 0; // stop_after: leave after that many steps of this run, with a checkpoint
    bool muon = false, bf16_exchange = false;
    float learning_rate = 3e-4f;
    unsigned long long seed = 3407;
};

[[noreturn]] void usage(const std::string &why) {
    fprintf(stderr,
            "%s\nusage: turbogpt_dp --data FILE --log-to DIR [--devices 0,1,..] [--tokens N] [--depth L] [--width W]\n"
            "       [--heads H] [--hidden F] [--context T] [--batch B] [--optimizer adamw|muon] [--learning-rate R]\n"
            "       [--chunk N] [--checkpoint-every N] [--stop-after N] [--load FILE] [--save FILE] [--seed S] [--bf16-exchange]\n",
            why.c_str());
    exit(2);
}

Options parse(int argc, char **argv) {
    Options o;
    for (int i = 1; i < argc; ++i) {
        const std::string flag = argv[i];
        auto value = [&]() -> std::string {
            if (i + 1 >= argc)
                usage("missing value for " + flag);
            return argv[++i];
        };
        if (flag == "--data") o.data = value();
        else if (flag == "--log-to") o.log_to = value();
        else if (flag == "--load") o.load = value();
        else if (flag == "--save") o.save = value();
        else if (flag == "--tokens") o.tokens = atoll(value().c_str());
        else if (flag == "--depth") o.depth = atoi(value().c_str());
        else if (flag == "--width") o.width = atoi(value().c_str());
        else if (flag == "--heads") o.heads = atoi(value().c_str());
        else if (flag == "--hidden") o.hidden = atoi(value().c_str());
        else if (flag == "--context") o.context = atoi(value().c_str());
        else if (flag == "--batch") o.batch = atoi(value().c_str());
        else if (flag == "--chunk") o.chunk = atoi(value().c_str());
        else if (flag == "--checkpoint-every") o.checkpoint_every = atoi(value().c_str());
        else if (flag == "--stop-after") o.stop_after = atoi(value().c_str());
        else if (flag == "--learning-rate") o.learning_rate = float(atof(value().c_str()));
        else if (flag == "--seed") o.seed = strtoull(value().c_str(), nullptr, 10);
        else if (flag == "--bf16-exchange") o.bf16_exchange = true;
        else if (flag == "--optimizer") {
            const std::string kind = value();
            if (kind != "adamw" && kind != "muon")
                usage("--optimizer takes adamw or muon");
            o.muon = kind == "muon";
        } else if (flag == "--devices") {
            o.devices.clear();
            std::stringstream list(value());
            for (std::string item; std::getline(list, item, ',');)
                o.devices.push_back(atoi(item.c_str()));
        } else
            usage("unknown option " + flag);
    }
    if (o.data.empty() || o.log_to.empty())
        usage("--data and --log-to are required");
    if (o.devices.empty() || o.chunk < 1 || o.chunk > 4096)
        usage("--devices needs at least one device; --chunk is 1..4096");
    if (o.save.empty())
        o.save = o.log_to + "/model.pt";
    return o;
}

void check(int status) {
    if (status < 0)
        throw std::runtime_error(tg_error());
}

// Reusable barrier for the rank threads; releases everyone early once a rank has failed.
class Rendezvous {
  public:
    explicit Rendezvous(int count) : count_(count) {}
    void wait(const std::atomic<bool> &failed) {
        std::unique_lock<std::mutex> lock(mutex_);
        const unsigned long long generation = generation_;
        if (++arrived_ == count_) {
            arrived_ = 0;
            ++generation_;
            wake_.notify_all();
            return;
        }
        while (generation == generation_ && !failed.load())
            wake_.wait_for(lock, std::chrono::milliseconds(50));
    }

  private:
    std::mutex mutex_;
    std::condition_variable wake_;
    int count_, arrived_ = 0;
    unsigned long long generation_ = 0;
};

struct Shared {
    Options options;
    TgConfigEx config{}; // rank and device are filled per thread
    std::vector<float> weights, momentum, variance;
    std::vector<double> final_loss_sums;
    std::vector<uint8_t> corpus;
    TgOneCycle schedule{};
    unsigned long long start_step = 0, final_loss_batches = 0;
    double train_seconds = 0;
    int steps = 0;
    std::atomic<bool> failed{false};
    std::mutex error_mutex;
    std::string error;
    void fail(const std::string &message) {
        std::lock_guard<std::mutex> lock(error_mutex);
        if (error.empty())
            error = message;
        failed.store(true);
    }
};

void run_rank(Shared &shared, Rendezvous &meet, int rank) {
    const Options &o = shared.options;
    Engine *engine = nullptr;
    try {
        TgConfigEx config = shared.config;
        config.rank = rank;
        config.base.device = o.devices[rank];
        engine = tg_create_ex(&config);
        if (!engine)
            throw std::runtime_error(tg_error());
        const int context = o.context, world = int(o.devices.size());
        check(tg_set_weights(engine, shared.weights.data()));
        check(tg_set_onecycle(engine, &shared.schedule));
        if (shared.start_step > 0)
            check(tg_set_optimizer_state(engine, shared.momentum.data(), shared.variance.data(), shared.start_step));
        check(tg_set_data(engine, shared.corpus.data(), int64_t(shared.corpus.size())));

        FILE *log = nullptr;
        if (rank == 0) {
            log = fopen((o.log_to + "/train.log").c_str(), shared.start_step ? "a" : "w");
            if (!log)
                throw std::runtime_error("Cannot write " + o.log_to + "/train.log");
            double gigabytes = 0;
            check(tg_memory(engine, &gigabytes));
            fprintf(log, "# %d parameters, %d device(s), global batch %d x %d, %.2f GB per device, steps %llu..%d\n",
                    tg_parameter_count(engine), world, o.batch * world, context, gigabytes, shared.start_step,
                    shared.steps);
        }
        std::vector<float> history;
        std::vector<double> loss_sums = shared.final_loss_sums;
        unsigned long long loss_batches = shared.final_loss_batches;
        const int window_first = shared.steps - std::max(1, (shared.steps + 99) / 100);
        double train_seconds = shared.train_seconds;
        int done = int(shared.start_step), since_checkpoint = 0;
        const long long tokens_per_step = (long long)o.batch * world * context;

        auto checkpoint = [&]() {
            // Every rank reaches this point with the same `done`; rank 0 reads its engine and writes.
            if (rank == 0) {
                uint64_t step = 0;
                check(tg_get_weights(engine, shared.weights.data()));
                check(tg_get_optimizer_state(engine, shared.momentum.data(), shared.variance.data(), &step));
                if (step != uint64_t(done))
                    throw std::runtime_error("Optimizer step changed while saving the checkpoint");
                TgCheckpoint state{};
                state.weights = shared.weights.data(), state.momentum = shared.momentum.data();
                state.variance = shared.variance.data(), state.final_loss_sums = loss_sums.data();
                state.step = step, state.final_loss_batches = loss_batches, state.train_seconds = train_seconds;
                state.scheduler = shared.schedule;
                check(tg_ex_save_checkpoint(o.save.c_str(), &config, &state));
                fprintf(log, "# checkpoint at step %d: %s\n", done, o.save.c_str());
                fflush(log);
            }
            meet.wait(shared.failed);
        };

        const int last = o.stop_after > 0 ? std::min(shared.steps, int(shared.start_step) + o.stop_after) : shared.steps;
        while (done < last && !shared.failed.load()) {
            meet.wait(shared.failed); // everyone launches the chunk, or no one does
            if (shared.failed.load())
                break;
            const int count = std::min(o.chunk, last - done);
            const auto launched = Clock::now();
            check(tg_train(engine, count));
            history.resize(size_t(count) * context);
            check(tg_get_training_losses(engine, history.data(), count)); // global per-position means, on every rank
            const double seconds = std::chrono::duration<double>(Clock::now() - launched).count();
            train_seconds += seconds;
            for (int s = 0; s < count; ++s)
                if (done + s >= window_first) { // final-loss average over the last hundredth of the run
                    for (int p = 0; p < context; ++p)
                        loss_sums[p] += history[size_t(s) * context + p];
                    ++loss_batches;
                }
            done += count;
            since_checkpoint += count;
            if (rank == 0) {
                double mean = 0;
                for (int p = 0; p < context; ++p)
                    mean += history[size_t(count - 1) * context + p];
                mean /= context;
                fprintf(log, "step %d loss %.6f bpb %.6f tokens_per_second %.0f\n", done, mean, mean / 0.6931471805599453,
                        double(tokens_per_step) * count / seconds);
                fflush(log);
                printf("step %d/%d loss %.4f  %.0f tokens/s\n", done, shared.steps, mean,
                       double(tokens_per_step) * count / seconds);
                fflush(stdout);
            }
            if (done == last || (o.checkpoint_every > 0 && since_checkpoint >= o.checkpoint_every)) {
                checkpoint();
                since_checkpoint = 0;
            }
        }
        if (log)
            fclose(log);
    } catch (const std::exception &error) {
        shared.fail("rank " + std::to_string(rank) + ": " + error.what());
    }
    if (engine)
        tg_destroy(engine);
}
} // namespace

int main(int argc, char **argv) {
    Shared shared;
    shared.options = parse(argc, argv);
    const Options &o = shared.options;
    try {
        const int world = int(o.devices.size());
        TgConfig base{};
        base.depth = o.depth, base.context = o.context, base.batch = o.batch, base.device = o.devices[0];
        base.blocks = 0, base.ns_steps = 5;
        base.learning_rate = o.learning_rate, base.muon_lr = 0.02f, base.beta1 = 0.9f, base.beta2 = 0.95f;
        base.momentum = 0.95f, base.weight_decay = 0.1f, base.epsilon = 1e-8f, base.clip = 1.0f;
        base.seed = o.seed, base.inflight = 1;
        tg_ex_gpt_config(&base, o.width, o.heads, o.hidden, &shared.config);
        shared.config.hidden_optimizer = o.muon ? TG_HIDDEN_MUON : TG_HIDDEN_ADAMW;
        shared.config.world = world;
        if (o.bf16_exchange)
            shared.config.flags |= TG_FLAG_BF16_GRADIENT_EXCHANGE;
        const int64_t count = tg_ex_parameter_count(&shared.config);
        if (count < 0)
            throw std::runtime_error(tg_error());

        std::ifstream file(o.data, std::ios::binary);
        if (!file)
            throw std::runtime_error("Cannot open " + o.data);
        shared.corpus.assign(std::istreambuf_iterator<char>(file), std::istreambuf_iterator<char>());
        const long long tokens_per_step = (long long)o.batch * world * o.context;
        const long long tokens = o.tokens > 0 ? o.tokens : (long long)shared.corpus.size();
        const long long steps = (tokens + tokens_per_step - 1) / tokens_per_step;
        if (steps < 4 || steps > 2000000000ll)
            throw std::runtime_error("The run needs between 4 and 2e9 steps; adjust --tokens");
        shared.steps = int(steps);
        shared.schedule = TgOneCycle{};
        shared.schedule.total_steps = shared.steps;
        shared.schedule.warmup_fraction = 0.30, shared.schedule.initial_lr_fraction = 0.04;
        shared.schedule.final_lr_fraction = 0.000004, shared.schedule.low_momentum = 0.85;
        shared.schedule.high_momentum = 0.95;

        shared.weights.resize(size_t(count)), shared.momentum.assign(size_t(count), 0.f);
        shared.variance.assign(size_t(count), 0.f), shared.final_loss_sums.assign(size_t(o.context), 0.0);
        mkdir(o.log_to.c_str(), 0777);
        if (o.load.empty()) {
            check(tg_ex_initialize_weights(&shared.config, shared.weights.data()));
        } else {
            TgCheckpoint state{};
            state.weights = shared.weights.data(), state.momentum = shared.momentum.data();
            state.variance = shared.variance.data(), state.final_loss_sums = shared.final_loss_sums.data();
            check(tg_ex_load_checkpoint(o.load.c_str(), &shared.config, &state));
            if (state.scheduler.total_steps != shared.steps)
                throw std::runtime_error("Checkpoint does not match the source experiment");
            if (state.step >= uint64_t(shared.steps))
                throw std::runtime_error("Checkpoint already reached the requested step count");
            shared.start_step = state.step, shared.final_loss_batches = state.final_loss_batches;
            shared.train_seconds = state.train_seconds;
            shared.schedule = state.scheduler;
        }
        if (world > 1 && tg_ex_nccl_unique_id(shared.config.nccl_id) < 0)
            throw std::runtime_error(tg_error());

        Rendezvous meet(world);
        std::vector<std::thread> ranks;
        for (int rank = 0; rank < world; ++rank)
            ranks.emplace_back(run_rank, std::ref(shared), std::ref(meet), rank);
        for (std::thread &t : ranks)
            t.join();
        if (shared.failed.load())
            throw std::runtime_error(shared.error);
        printf("done: %d steps, checkpoint %s\n", shared.steps, o.save.c_str());
        return 0;
    } catch (const std::exception &error) {
        fprintf(stderr, "turbogpt_dp: %s\n", error.what());
        return 1;
    }
}
