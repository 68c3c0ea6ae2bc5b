// Timing driver for the reference arm of bench.py.
//
// Links the UNMODIFIED libraries of Deyu-Kong/mini-infer (built out of tree from its own
// CMakeLists.txt) and calls its stock public path and nothing of this repository:
//   ModelConfig::load                    (src/model/model_config.cpp)
//   WeightIndex::load + load_weights     (src/model/safetensors_loader.cpp, transformer_model.cpp:189-365)
//   Engine::generate_batched_paged       (src/core/engine.cpp:348-486)
// on a model folder with random weights in float16 and seeded synthetic token ids (as the
// reference's own benchmarks make them, benchmarks/common/dataset.h:41-55: ids in [10, vocab)).
//
// Usage: reference_bench MODEL_DIR BATCH PROMPT_LEN STEPS WARMUP [SEED]
// One call of generate_batched_paged(prompts, n + 1) runs the prompts and then exactly n decode
// steps of BATCH tokens, and the engine clocks that decode loop itself (host clock around the loop;
// every step uploads its token ids and reads the sampled ids back, so the loop is end to end).
// The driver makes a warm-up call with WARMUP steps, gives the pages back, then a timed call with
// STEPS steps, and prints one line "RESULT {json}" with the engine's own decode_tokens_per_sec().
#include <cuda_runtime.h>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <string>
#include <vector>

#include "core/engine.h"
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

int main(int argc, char** argv) {
    if (argc < 6) {
        std::fprintf(stderr, "usage: %s MODEL_DIR BATCH PROMPT_LEN STEPS WARMUP [SEED]\n", argv[0]);
        return 2;
    }
    const std::string dir = argv[1];
    const int batch = std::atoi(argv[2]);
    const int prompt_len = std::atoi(argv[3]);
    const int steps = std::atoi(argv[4]);
    const int warmup = std::atoi(argv[5]);
    uint64_t seed = argc > 6 ? std::strtoull(argv[6], nullptr, 10) : 42;
    try {
        auto t_load = std::chrono::high_resolution_clock::now();
        ModelConfig cfg = ModelConfig::load(dir + "/config.json");
        WeightIndex idx = WeightIndex::load(dir);
        auto model = std::make_shared<TransformerModel>(cfg, 0);
        model->load_weights(idx);
        const int longest = prompt_len + (steps > warmup ? steps : warmup) + 2;
        const int blocks = batch * ((longest + 15) / 16 + 1) + 16;
        Engine engine(model, longest, 0, blocks);
        engine.set_sampling(SamplingMode::Greedy);
        double load_s = std::chrono::duration<double>(std::chrono::high_resolution_clock::now() - t_load).count();

        std::vector<std::vector<int64_t>> prompts(batch);
        for (auto& p : prompts) {
            p.resize(prompt_len);
            for (auto& t : p) t = 10 + static_cast<int64_t>(splitmix64(seed) % static_cast<uint64_t>(cfg.vocab_size - 10));
        }
        if (warmup > 0) {
            engine.generate_batched_paged(prompts, warmup + 1, {});
            engine.clear_paged_sequences();
        }
        auto t0 = std::chrono::high_resolution_clock::now();
        auto outs = engine.generate_batched_paged(prompts, steps + 1, {});
        cudaDeviceSynchronize();
        double call_s = std::chrono::duration<double>(std::chrono::high_resolution_clock::now() - t0).count();
        cudaError_t err = cudaGetLastError();
        if (err != cudaSuccess) {
            std::fprintf(stderr, "reference_bench: CUDA error after the timed call: %s\n", cudaGetErrorString(err));
            return 3;
        }
        const double tps = engine.decode_tokens_per_sec();
        const double ms_per_step = tps > 0 ? 1000.0 * batch / tps : 0.0;
        size_t made = 0;
        for (auto& o : outs) made += o.size() - prompt_len;
        std::printf("\nRESULT {\"decode_tok_s\": %.3f, \"ms_per_step\": %.4f, \"batch\": %d, \"prompt_len\": %d, "
                    "\"steps\": %d, \"warmup\": %d, \"generated\": %zu, \"call_seconds\": %.3f, \"load_seconds\": %.1f, "
                    "\"layers\": %ld, \"hidden\": %ld, \"experts\": %ld, \"vocab\": %ld}\n",
                    tps, ms_per_step, batch, prompt_len, steps, warmup, made, call_s, load_s,
                    (long)cfg.num_hidden_layers, (long)cfg.hidden_size, (long)cfg.num_experts, (long)cfg.vocab_size);
        std::fflush(stdout);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "reference_bench: %s\n", e.what());
        return 1;
    }
    return 0;
}
