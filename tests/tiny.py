"""Tiny Qwen2-MoE configurations for the tests, and helpers shared by them.

A and B are the two tiny configurations of the benchmark description; C adds
what they lack: sliding-window layers, no shared expert, top-1 routing, no
q/k/v bias, a head size that is no multiple of eight.  Between them the three
differ in every size and option.
"""

from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence, Tuple

import torch

import plain_model

CONFIG_A = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
    "max_position_embeddings": 128, "tie_word_embeddings": False, "hidden_act": "silu",
    "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 32,
    "shared_expert_intermediate_size": 64, "norm_topk_prob": True, "decoder_sparse_step": 1,
    "mlp_only_layers": [], "use_sliding_window": False, "sliding_window": 32768, "max_window_layers": 2,
}

CONFIG_B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "vocab_size": 384, "hidden_size": 96, "intermediate_size": 160, "num_hidden_layers": 3,
    "num_attention_heads": 4, "num_key_value_heads": 1, "rms_norm_eps": 1e-5, "rope_theta": 1000000.0,
    "max_position_embeddings": 256, "tie_word_embeddings": True, "hidden_act": "silu",
    "num_experts": 6, "num_experts_per_tok": 3, "moe_intermediate_size": 48,
    "shared_expert_intermediate_size": 96, "norm_topk_prob": False, "decoder_sparse_step": 2,
    "mlp_only_layers": [0], "use_sliding_window": False, "sliding_window": 32768, "max_window_layers": 3,
}

CONFIG_C = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "vocab_size": 301, "hidden_size": 72, "intermediate_size": 100, "num_hidden_layers": 4,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 12, "rms_norm_eps": 3e-6,
    "rope_theta": 50000.0, "max_position_embeddings": 512, "tie_word_embeddings": False,
    "hidden_act": "silu", "qkv_bias": False,
    "num_experts": 5, "num_experts_per_tok": 1, "moe_intermediate_size": 20,
    "shared_expert_intermediate_size": 0, "norm_topk_prob": True, "decoder_sparse_step": 1,
    "mlp_only_layers": [2], "use_sliding_window": True, "sliding_window": 24, "max_window_layers": 2,
}

# A fourth shape for the kernels the tiny models cannot reach: head size 64 (split-KV decode
# kernel), more experts, longer contexts.
CONFIG_D = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "vocab_size": 515, "hidden_size": 128, "intermediate_size": 96, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "max_position_embeddings": 2048, "tie_word_embeddings": False,
    "hidden_act": "silu",
    "num_experts": 12, "num_experts_per_tok": 4, "moe_intermediate_size": 40,
    "shared_expert_intermediate_size": 72, "norm_topk_prob": False, "decoder_sparse_step": 1,
    "mlp_only_layers": [], "use_sliding_window": False, "sliding_window": 0, "max_window_layers": 0,
}

# A fifth shape whose sizes the tensor-core kernels of the bfloat16 path take inside the engine: expert and
# shared widths that are multiples of 64 (grouped products on tcgen05 once a step brings more than
# 8 * experts / top_k tokens), head size 64 (tcgen05 prefill attention, split-KV decode attention), and a
# sliding window on the upper layers so that those kernels meet released pages.
CONFIG_E = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "vocab_size": 777, "hidden_size": 192, "intermediate_size": 320, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 64, "rms_norm_eps": 1e-5,
    "rope_theta": 300000.0, "max_position_embeddings": 4096, "tie_word_embeddings": True,
    "hidden_act": "silu", "qkv_bias": True,
    "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 128,
    "shared_expert_intermediate_size": 64, "norm_topk_prob": True, "decoder_sparse_step": 1,
    "mlp_only_layers": [], "use_sliding_window": True, "sliding_window": 80, "max_window_layers": 1,
}

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D, "E": CONFIG_E}


def make_folder(tmp: str, cfg: dict, seed: int, dtype=torch.float32) -> str:
    """A model folder with seeded random weights, written by the framework's own writer."""
    from mini_infer_b200.weights import write_model_folder
    return write_model_folder(tmp, cfg, seed=seed, dtype=dtype)


def read_weights(folder: str) -> Dict[str, torch.Tensor]:
    """Checkpoint as {name: float32 tensor}, read with the safetensors package (not the engine's reader)."""
    import safetensors.torch as st
    return {k: v.to(torch.float32) for k, v in st.load_file(os.path.join(folder, "model.safetensors")).items()}


def min_routing_gap(cfg: dict, weights, tokens: Sequence[int]) -> float:
    """Smallest gap between the K-th and (K+1)-th router probability over all tokens and layers."""
    rec: dict = {}
    plain_model.forward(cfg, weights, tokens, record=rec)
    K = cfg["num_experts_per_tok"]
    gap = 1.0
    for _, (idx, probs) in rec.get("routing", {}).items():
        s = torch.sort(probs, dim=-1, descending=True).values
        if s.shape[1] > K:
            gap = min(gap, float((s[:, K - 1] - s[:, K]).min()))
    return gap


def pick_tokens(cfg: dict, weights, length: int, seed: int, min_gap: float = 0.0) -> List[int]:
    """Seeded uniform-random token ids; with ``min_gap``, the first seed (counting up) whose
    routing has no nearer tie, so that a bfloat16 engine cannot legitimately route otherwise."""
    for s in range(seed, seed + 200):
        g = torch.Generator().manual_seed(s)
        toks = torch.randint(0, cfg["vocab_size"], (length,), generator=g).tolist()
        if min_gap <= 0.0 or min_routing_gap(cfg, weights, toks) >= min_gap:
            return toks
    raise RuntimeError("no token sequence without a routing near-tie found")
