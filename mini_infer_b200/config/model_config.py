"""Typed model configuration read from a Hugging Face style ``config.json``.

The reference parses the same file into ``struct ModelConfig``
(src/model/model_config.h:51-141, src/model/model_config.cpp:61-178) with
tolerant getters that accept ints, floats and numeric strings
(src/model/model_config.cpp:15-40).  This module keeps that behaviour and adds
the Qwen2-MoE keys the reference silently ignores (``norm_topk_prob``,
``decoder_sparse_step``, ``mlp_only_layers``, ``use_sliding_window``,
``max_window_layers``).

No size or constant of a model lives anywhere else in the package: every part
receives its numbers from an instance of :class:`Qwen2MoeConfig` through the
architecture builder in ``mini_infer_b200.models``.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Dict, Tuple


class ConfigError(ValueError):
    """Raised for an unreadable, incomplete or inconsistent ``config.json``."""


# --------------------------------------------------------------------------- #
# tolerant getters (ints / floats / bools may arrive as strings)
# --------------------------------------------------------------------------- #

def _get_int(j: Dict[str, Any], key: str, default: int) -> int:
    if key not in j or j[key] is None:
        return default
    v = j[key]
    if isinstance(v, bool):
        raise ConfigError(f"config key '{key}' must be an integer, got a boolean")
    if isinstance(v, int):
        return v
    if isinstance(v, float):
        if v != int(v):
            raise ConfigError(f"config key '{key}' must be an integer, got {v!r}")
        return int(v)
    if isinstance(v, str):
        try:
            f = float(v)
        except ValueError as e:
            raise ConfigError(f"config key '{key}' must be an integer, got {v!r}") from e
        if f != int(f):
            raise ConfigError(f"config key '{key}' must be an integer, got {v!r}")
        return int(f)
    raise ConfigError(f"config key '{key}' must be an integer, got {type(v).__name__}")


def _get_float(j: Dict[str, Any], key: str, default: float) -> float:
    if key not in j or j[key] is None:
        return default
    v = j[key]
    if isinstance(v, bool):
        raise ConfigError(f"config key '{key}' must be a number, got a boolean")
    if isinstance(v, (int, float)):
        return float(v)
    if isinstance(v, str):
        try:
            return float(v)
        except ValueError as e:
            raise ConfigError(f"config key '{key}' must be a number, got {v!r}") from e
    raise ConfigError(f"config key '{key}' must be a number, got {type(v).__name__}")


def _get_bool(j: Dict[str, Any], key: str, default: bool) -> bool:
    if key not in j or j[key] is None:
        return default
    v = j[key]
    if isinstance(v, bool):
        return v
    if isinstance(v, int):
        return v != 0
    if isinstance(v, str):
        if v.lower() in ("true", "1"):
            return True
        if v.lower() in ("false", "0"):
            return False
    raise ConfigError(f"config key '{key}' must be a boolean, got {v!r}")


def _get_str(j: Dict[str, Any], key: str, default: str) -> str:
    if key not in j or j[key] is None:
        return default
    v = j[key]
    if not isinstance(v, str):
        raise ConfigError(f"config key '{key}' must be a string, got {type(v).__name__}")
    return v


def _get_int_list(j: Dict[str, Any], key: str) -> Tuple[int, ...]:
    if key not in j or j[key] is None:
        return ()
    v = j[key]
    if not isinstance(v, (list, tuple)):
        raise ConfigError(f"config key '{key}' must be a list of integers")
    out = []
    for x in v:
        if isinstance(x, bool) or not isinstance(x, int):
            raise ConfigError(f"config key '{key}' must be a list of integers, got {x!r}")
        out.append(x)
    return tuple(out)


# --------------------------------------------------------------------------- #
# the typed configuration
# --------------------------------------------------------------------------- #

@dataclass(frozen=True)
class Qwen2MoeConfig:
    """Every ``config.json`` key of ``Qwen2MoeForCausalLM`` that the engine uses.

    Keys and defaults follow src/model/model_config.cpp:68-112,153 of the
    reference; the last block of fields is read by this engine only.
    """

    architecture: str = "Qwen2MoeForCausalLM"
    model_type: str = "qwen2_moe"
    vocab_size: int = 0
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    qkv_bias: bool = True
    # mixture of experts
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    norm_topk_prob: bool = False
    decoder_sparse_step: int = 1
    mlp_only_layers: Tuple[int, ...] = ()
    # sliding window
    use_sliding_window: bool = False
    sliding_window: int = 0
    max_window_layers: int = 0

    # ----- derived -------------------------------------------------------- #
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_is_sparse(self, i: int) -> bool:
        """Layer ``i`` carries the expert block rather than the dense MLP.

        The reference never reads ``decoder_sparse_step`` or ``mlp_only_layers``
        (src/model/transformer_model.cpp:141-156 switches on "has experts" for
        the whole model); the rule here is the one those two keys describe.
        """
        return (self.num_experts > 0
                and i not in self.mlp_only_layers
                and (i + 1) % self.decoder_sparse_step == 0)

    def layer_window(self, i: int) -> int:
        """Keys a query of layer ``i`` may look back over (0 = all of them)."""
        if self.use_sliding_window and self.sliding_window > 0 and i >= self.max_window_layers:
            return self.sliding_window
        return 0

    def to_json_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        d["mlp_only_layers"] = list(self.mlp_only_layers)
        return d

    def save(self, folder: str) -> str:
        os.makedirs(folder, exist_ok=True)
        path = os.path.join(folder, "config.json")
        with open(path, "w") as f:
            json.dump(self.to_json_dict(), f, indent=2)
        return path

    # ----- validation ------------------------------------------------------ #
    def validate(self, where: str = "config") -> None:
        missing = [k for k in ("hidden_size", "num_hidden_layers", "num_attention_heads", "vocab_size")
                   if getattr(self, k) <= 0]
        if missing:
            # src/model/model_config.cpp:157-160
            raise ConfigError(f"ModelConfig: missing required fields in {where}: {', '.join(missing)}")
        if self.head_dim <= 0:
            raise ConfigError(
                f"ModelConfig: head_dim is non-positive (hidden_size={self.hidden_size}, "
                f"num_attention_heads={self.num_attention_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"ModelConfig: head_dim {self.head_dim} must be even (rotary pairs)")
        if self.num_key_value_heads <= 0:
            raise ConfigError("ModelConfig: num_key_value_heads must be positive")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            # src/model/model_config.cpp:173-176
            raise ConfigError(
                "ModelConfig: num_attention_heads not divisible by num_key_value_heads (GQA)")
        if self.hidden_act not in ("silu", "SwiGLU"):
            raise ConfigError(f"ModelConfig: hidden_act '{self.hidden_act}' is not supported (silu only)")
        if self.rms_norm_eps <= 0:
            raise ConfigError("ModelConfig: rms_norm_eps must be positive")
        if self.rope_theta <= 0:
            raise ConfigError("ModelConfig: rope_theta must be positive")
        if self.decoder_sparse_step < 1:
            raise ConfigError("ModelConfig: decoder_sparse_step must be >= 1")
        for i in self.mlp_only_layers:
            if not 0 <= i < self.num_hidden_layers:
                raise ConfigError(
                    f"ModelConfig: mlp_only_layers entry {i} outside [0, {self.num_hidden_layers})")
        if self.num_experts < 0 or self.num_experts_per_tok < 0:
            raise ConfigError("ModelConfig: expert counts must be non-negative")
        any_sparse = any(self.layer_is_sparse(i) for i in range(self.num_hidden_layers))
        any_dense = any(not self.layer_is_sparse(i) for i in range(self.num_hidden_layers))
        if any_sparse:
            if not 1 <= self.num_experts_per_tok <= self.num_experts:
                raise ConfigError(
                    f"ModelConfig: num_experts_per_tok={self.num_experts_per_tok} must lie in "
                    f"[1, num_experts={self.num_experts}]")
            if self.moe_intermediate_size <= 0:
                raise ConfigError("ModelConfig: sparse layers need moe_intermediate_size > 0")
            if self.shared_expert_intermediate_size < 0:
                raise ConfigError("ModelConfig: shared_expert_intermediate_size must be >= 0")
        if any_dense and self.intermediate_size <= 0:
            raise ConfigError("ModelConfig: dense layers need intermediate_size > 0")
        if self.use_sliding_window and self.sliding_window <= 0:
            raise ConfigError("ModelConfig: use_sliding_window needs sliding_window > 0")
        if self.max_window_layers < 0:
            raise ConfigError("ModelConfig: max_window_layers must be >= 0")
        if self.max_position_embeddings <= 0:
            raise ConfigError("ModelConfig: max_position_embeddings must be positive")

    # ----- construction ---------------------------------------------------- #
    @classmethod
    def from_json_dict(cls, j: Dict[str, Any], where: str = "config") -> "Qwen2MoeConfig":
        arch = "Qwen2MoeForCausalLM"
        if isinstance(j.get("architectures"), list) and j["architectures"]:
            arch = j["architectures"][0]
            if not isinstance(arch, str):
                raise ConfigError("config key 'architectures' must be a list of strings")
        hidden = _get_int(j, "hidden_size", 0)
        heads = _get_int(j, "num_attention_heads", 0)
        head_dim = _get_int(j, "head_dim", 0)
        if head_dim == 0 and heads > 0:
            if hidden % heads != 0:
                # src/model/model_config.cpp:169-172
                raise ConfigError("ModelConfig: hidden_size not divisible by num_attention_heads")
            head_dim = hidden // heads
        inter = _get_int(j, "intermediate_size", 0)
        # the number of experts under the names that the reference reads one after the other
        # (src/model/model_config.cpp:95-105)
        n_exp = 0
        for key in ("num_experts", "num_local_experts", "n_routed_experts"):
            if n_exp == 0:
                n_exp = _get_int(j, key, 0)
        moe_inter = _get_int(j, "moe_intermediate_size", 0)
        if n_exp > 0 and moe_inter == 0:
            moe_inter = inter  # src/model/model_config.cpp:108-110
        cfg = cls(
            architecture=arch,
            model_type=_get_str(j, "model_type", "qwen2_moe"),
            vocab_size=_get_int(j, "vocab_size", 0),
            hidden_size=hidden,
            intermediate_size=inter,
            num_hidden_layers=_get_int(j, "num_hidden_layers", 0),
            num_attention_heads=heads,
            num_key_value_heads=_get_int(j, "num_key_value_heads", heads),
            head_dim=head_dim,
            rms_norm_eps=_get_float(j, "rms_norm_eps", 1e-6),
            rope_theta=_get_float(j, "rope_theta", 10000.0),
            max_position_embeddings=_get_int(j, "max_position_embeddings", 32768),
            tie_word_embeddings=_get_bool(j, "tie_word_embeddings", False),
            hidden_act=_get_str(j, "hidden_act", "silu"),
            torch_dtype=_get_str(j, "torch_dtype", "bfloat16"),
            qkv_bias=_get_bool(j, "qkv_bias", True),
            num_experts=n_exp,
            num_experts_per_tok=_get_int(j, "num_experts_per_tok", 0),
            moe_intermediate_size=moe_inter,
            shared_expert_intermediate_size=_get_int(j, "shared_expert_intermediate_size", 0),
            norm_topk_prob=_get_bool(j, "norm_topk_prob", False),
            decoder_sparse_step=_get_int(j, "decoder_sparse_step", 1),
            mlp_only_layers=_get_int_list(j, "mlp_only_layers"),
            use_sliding_window=_get_bool(j, "use_sliding_window", False),
            sliding_window=_get_int(j, "sliding_window", 0),
            max_window_layers=_get_int(j, "max_window_layers", 0),
        )
        cfg.validate(where)
        return cfg


def read_config_json(path_or_folder: str) -> Dict[str, Any]:
    """Return the raw dictionary of ``config.json`` (file path or model folder)."""
    path = path_or_folder
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path) as f:
            j = json.load(f)
    except OSError as e:
        raise ConfigError(f"ModelConfig: cannot open {path}") from e  # model_config.cpp:62-63
    except json.JSONDecodeError as e:
        raise ConfigError(f"ModelConfig: {path} is not valid JSON: {e}") from e
    if not isinstance(j, dict):
        raise ConfigError(f"ModelConfig: {path} must hold a JSON object")
    return j


def architecture_name(j: Dict[str, Any]) -> str:
    archs = j.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json has no 'architectures' entry naming the model class")
    return archs[0]
