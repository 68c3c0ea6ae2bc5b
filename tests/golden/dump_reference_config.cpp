// Prints what the reference's own configuration parser (src/model/model_config.cpp, ModelConfig::load)
// reads from a config.json, as one JSON object on standard output.  Built against the reference's
// sources by make_config_golden.py; host-only (no CUDA).
#include "model/model_config.h"

#include <cstdio>
#include <string>

int main(int argc, char** argv) {
    if (argc != 2) {
        std::fprintf(stderr, "usage: dump_reference_config CONFIG_JSON\n");
        return 2;
    }
    const mini_infer::ModelConfig c = mini_infer::ModelConfig::load(argv[1]);
    std::printf("{\"hidden_size\": %lld, \"intermediate_size\": %lld, \"num_hidden_layers\": %lld, "
                "\"num_attention_heads\": %lld, \"num_key_value_heads\": %lld, \"vocab_size\": %lld, "
                "\"rms_norm_eps\": %.9g, \"rope_theta\": %.9g, \"max_position_embeddings\": %lld, "
                "\"tie_word_embeddings\": %s, \"hidden_act\": \"%s\", \"has_qkv_bias\": %s, \"head_dim\": %lld, "
                "\"num_experts\": %lld, \"num_experts_per_tok\": %lld, \"moe_intermediate_size\": %lld, "
                "\"shared_expert_intermediate_size\": %lld, \"sliding_window\": %lld, \"is_moe\": %s}\n",
                (long long)c.hidden_size, (long long)c.intermediate_size, (long long)c.num_hidden_layers,
                (long long)c.num_attention_heads, (long long)c.num_key_value_heads, (long long)c.vocab_size,
                (double)c.rms_norm_eps, (double)c.rope_theta, (long long)c.max_position_embeddings,
                c.tie_word_embeddings ? "true" : "false", c.hidden_act.c_str(), c.has_qkv_bias ? "true" : "false",
                (long long)c.head_dim(), (long long)c.num_experts, (long long)c.num_experts_per_tok,
                (long long)c.moe_intermediate_size, (long long)c.shared_expert_intermediate_size,
                (long long)c.sliding_window, c.is_moe() ? "true" : "false");
    return 0;
}
