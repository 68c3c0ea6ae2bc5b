// Timing driver for the reference arm of bench.py.
//
// Links the UNMODIFIED libraries of Deyu-Kong/mini-infer (built out of tree from its own
// CMakeLists.txt) and calls its stock public path and nothing of this repository:
//   ModelConfig::load                    (src/model/model_config.cpp)
//   WeightIndex::load + load_weights     (src/model/safetensors_loader.cpp, transformer_model.cpp:189-365)
//   Scheduler::submit / Scheduler::step  (src/scheduler/scheduler.cpp:338-370), the continuous-batching path
// on a model folder with random weights in float16 and seeded synthetic token ids (as the
// reference's own benchmarks make them, benchmarks/common/dataset.h:41-55: ids in [10, vocab)).
//
// Usage: reference_bench MODEL_DIR BATCH PROMPT_LEN STEPS WARMUP [SEED] [PREFILL_BATCH]
//
// BATCH requests are submitted; the scheduler admits PREFILL_BATCH prompts per iteration (default 1: every
// expert of the reference owns a cuBLAS handle, src/layers/moe.cpp:147-150 and mlp.cpp, whose workspaces
// take about 75 GB on a B200 at these sizes before any weight is loaded, and keeps three activation buffers
// of the largest batch it has seen, src/layers/mlp.cpp:243-247, 13 MB per prompt token over all experts; so
// 8 x 2,048 tokens in one prefill would need about 200 GB and even two prompts at once do not fit beside
// the 134 GB that handles and weights hold), and once all are running every iteration is one decode step of
// BATCH tokens.  WARMUP such steps are skipped, STEPS are timed with the scheduler's own clock
// (IterationStats::wall_ms: host clock around the step, which uploads the token ids and reads the sampled
// ids back, so it is end to end).
// Engine::generate_batched_paged (src/core/engine.cpp:348-486) is the other batched path; it runs all prompts
// in one prefill, which at the headline sizes ends in "out of memory" (src/core/tensor.cpp:155) for the
// reason above, and it cannot be linked beside the scheduler: engine.cpp and scheduler.cpp both include
// kernels/sampling_kernel.cu, so one program that names both gets every sampling kernel twice.
// Prints one line "RESULT {json}".
#include <cuda_runtime.h>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <string>
#include <vector>

#include "scheduler/paged_kv_cache.h"
#include "scheduler/request.h"
#include "scheduler/scheduler.h"
#include "model/model_config.h"
#include "model/safetensors_loader.h"
#include "model/transformer_model.h"

using namespace mini_infer;

static uint64_t splitmix64(uint64_t& s) {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static void note(const char* what) {
    size_t free_b = 0, total_b = 0;
    cudaMemGetInfo(&free_b, &total_b);
    std::fprintf(stderr, "[reference_bench] %s: %.1f of %.1f GB of device memory in use\n", what,
                 (total_b - free_b) / 1e9, total_b / 1e9);
}

int main(int argc, char** argv) {
    if (argc < 6) {
        std::fprintf(stderr, "usage: %s MODEL_DIR BATCH PROMPT_LEN STEPS WARMUP [SEED] [PREFILL_BATCH]\n", argv[0]);
        return 2;
    }
    const std::string dir = argv[1];
    const int batch = std::atoi(argv[2]);
    const int prompt_len = std::atoi(argv[3]);
    const int steps = std::atoi(argv[4]);
    const int warmup = std::atoi(argv[5]);
    uint64_t seed = argc > 6 ? std::strtoull(argv[6], nullptr, 10) : 42;
    const std::string mode = "scheduler";
    const int prefill_batch = argc > 7 ? std::atoi(argv[7]) : 1;
    try {
        auto t_load = std::chrono::high_resolution_clock::now();
        ModelConfig cfg = ModelConfig::load(dir + "/config.json");
        WeightIndex idx = WeightIndex::load(dir);
        note("start");
        auto model = std::make_shared<TransformerModel>(cfg, 0);
        note("model built");
        model->load_weights(idx);
        note("weights loaded");
        const int longest = prompt_len + steps + warmup + batch + 8;
        const int blocks_per_seq = (longest + 15) / 16 + 1;
        const int blocks = batch * blocks_per_seq + 16;
        double load_s = std::chrono::duration<double>(std::chrono::high_resolution_clock::now() - t_load).count();

        std::vector<std::vector<int64_t>> prompts(batch);
        for (auto& p : prompts) {
            p.resize(prompt_len);
            for (auto& t : p) t = 10 + static_cast<int64_t>(splitmix64(seed) % static_cast<uint64_t>(cfg.vocab_size - 10));
        }
        double tps = 0.0, call_s = 0.0;
        size_t made = 0;
        auto t0 = std::chrono::high_resolution_clock::now();
        {
            auto kv = std::make_shared<PagedKVCache>(blocks, (int)cfg.num_hidden_layers, (int)cfg.num_key_value_heads,
                                                     (int)cfg.head_dim(), blocks_per_seq, 0);
            SchedulerConfig sc;
            sc.max_num_blocks = blocks;
            sc.max_blocks_per_seq = blocks_per_seq;
            sc.prefill_buckets = {prompt_len};
            sc.max_prefill_batch = prefill_batch;
            sc.max_decode_batch = batch;
            Scheduler sched(model, kv, sc, 0);
            for (auto& p : prompts) sched.submit(std::make_unique<Request>(p, steps + warmup + batch + 4));
            int warm = 0, timed = 0;
            double timed_ms = 0.0;
            for (int it = 0; it < 10 * (steps + warmup + batch) && timed < steps; ++it) {
                IterationStats st = sched.step();
                if (st.num_prefilled != 0 || it < 2) note(st.num_prefilled ? "after an iteration that prefilled" : "after an iteration");
                if (st.num_prefilled != 0 || st.num_waiting != 0 || st.num_decoded != batch) continue;
                if (warm < warmup) { ++warm; continue; }
                timed_ms += st.wall_ms;
                ++timed;
                made += st.num_decoded;
            }
            cudaDeviceSynchronize();
            if (timed != steps) {
                std::fprintf(stderr, "reference_bench: only %d of %d full decode steps ran\n", timed, steps);
                return 4;
            }
            tps = 1000.0 * batch * steps / timed_ms;
        }
        call_s = std::chrono::duration<double>(std::chrono::high_resolution_clock::now() - t0).count();
        cudaError_t err = cudaGetLastError();
        if (err != cudaSuccess) {
            std::fprintf(stderr, "reference_bench: CUDA error after the timed region: %s\n", cudaGetErrorString(err));
            return 3;
        }
        const double ms_per_step = tps > 0 ? 1000.0 * batch / tps : 0.0;
        std::printf("\nRESULT {\"decode_tok_s\": %.3f, \"ms_per_step\": %.4f, \"batch\": %d, \"prompt_len\": %d, "
                    "\"steps\": %d, \"warmup\": %d, \"mode\": \"%s\", \"prefill_batch\": %d, \"generated\": %zu, \"call_seconds\": %.3f, \"load_seconds\": %.1f, "
                    "\"layers\": %ld, \"hidden\": %ld, \"experts\": %ld, \"vocab\": %ld}\n",
                    tps, ms_per_step, batch, prompt_len, steps, warmup, mode.c_str(), prefill_batch, made, call_s, load_s,
                    (long)cfg.num_hidden_layers, (long)cfg.hidden_size, (long)cfg.num_experts, (long)cfg.vocab_size);
        std::fflush(stdout);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "reference_bench: %s\n", e.what());
        return 1;
    }
    return 0;
}
