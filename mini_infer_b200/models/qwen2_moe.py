"""``Qwen2MoeForCausalLM`` described as an arrangement of parts.

Nothing here computes: the function turns ``config.json`` into a
:class:`ModelSpec` whose layers name, by kind and constants, the parts to build.
Layer ``i`` carries the expert block iff the model has experts, ``i`` is not in
``mlp_only_layers`` and ``(i + 1) % decoder_sparse_step == 0``; else the dense
MLP.  Layers at or above ``max_window_layers`` look back ``sliding_window`` keys
when ``use_sliding_window`` is set.  The reference reads none of these four keys:
it makes every layer sparse as soon as the model has experts
(src/model/transformer_model.cpp:141-156) and applies a window whenever
``sliding_window > 0`` (src/model/transformer_model.cpp:169-171).

Checkpoint names follow src/model/weight_mapper.h:73-112 and, for the expert
tensors, src/model/transformer_model.cpp:231-290.
"""

from __future__ import annotations

from typing import Any, Dict

from ..config.model_config import Qwen2MoeConfig
from ..config.registry import register_architecture
from ..config.spec import ModelSpec, PartSpec, default_schedule, prenorm_layer


def build_qwen2_moe(config_json: Dict[str, Any]) -> ModelSpec:
    c = Qwen2MoeConfig.from_json_dict(config_json)
    H = c.hidden_size
    position = PartSpec("rope", {"head_dim": c.head_dim, "theta": c.rope_theta})
    layers = []
    for i in range(c.num_hidden_layers):
        name = f"model.layers.{i}"
        mixer = PartSpec("gqa_attention", {
            "hidden_size": H, "num_heads": c.num_attention_heads, "num_kv_heads": c.num_key_value_heads,
            "head_dim": c.head_dim, "bias": c.qkv_bias, "window": c.layer_window(i), "position": position})
        if c.layer_is_sparse(i):
            ffn = PartSpec("sparse_moe", {
                "hidden_size": H, "num_experts": c.num_experts, "top_k": c.num_experts_per_tok,
                "expert_intermediate_size": c.moe_intermediate_size,
                "shared_intermediate_size": c.shared_expert_intermediate_size,
                "norm_topk_prob": c.norm_topk_prob})
        else:
            ffn = PartSpec("swiglu_mlp", {"hidden_size": H, "intermediate_size": c.intermediate_size})
        norm = PartSpec("rmsnorm", {"size": H, "eps": c.rms_norm_eps})
        layers.append(prenorm_layer(name, mixer, ffn, norm, norm))
    return ModelSpec(
        architecture=c.architecture,
        hidden_size=H,
        vocab_size=c.vocab_size,
        max_context=c.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab_size, "hidden_size": H}),
        layers=tuple(layers),
        schedule=default_schedule(c.num_hidden_layers),
        final_norm=PartSpec("rmsnorm", {"size": H, "eps": c.rms_norm_eps}),
        lm_head=PartSpec("linear", {"vocab_size": c.vocab_size, "hidden_size": H,
                                    "tied_to": "model.embed_tokens.weight" if c.tie_word_embeddings else None}),
    )


register_architecture("Qwen2MoeForCausalLM", build_qwen2_moe,
                      "Qwen2-MoE / Qwen1.5-MoE decoder (GQA attention with biased q/k/v, rotary positions, "
                      "RMSNorm, dense SwiGLU or sparse expert feed-forward with a gated shared expert)")
