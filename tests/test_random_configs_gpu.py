"""Randomly drawn tiny configurations through the engine, against the plain model.

Head sizes in steps of 8 and 16 (12 to 128), any number of heads and groups, widths and vocabularies that
are no power of two, with and without shared expert, bias, tied embeddings, dense layers among the sparse
ones and sliding windows on some layers, at page sizes 4 to 32: each in float32 and bfloat16, in portions of
changing size and mixed with other requests (decode steps are CUDA-graph replays).  A configuration a kernel
cannot take must be refused with an error, never computed wrongly; every one drawn here is taken.
"""

import random

import pytest
import torch

import tiny
import traces
from engine_harness import make_runner, run_and_compare

pytestmark = pytest.mark.gpu
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def draw(seed: int):
    rnd = random.Random(seed)
    d = rnd.choice([12, 16, 24, 32, 48, 64, 80, 96, 128])
    nkv = rnd.choice([1, 2, 3])
    nh = nkv * rnd.choice([1, 2, 4])
    explicit = rnd.random() < 0.3
    H = nh * d if not explicit else rnd.choice([64, 96, 160])
    if not explicit and H > 512:
        d = 32
        H = nh * d
    E = rnd.choice([4, 5, 8, 12, 17])
    K = rnd.randint(1, min(4, E))
    L = rnd.randint(1, 3)
    window = rnd.random() < 0.4
    cfg = {"architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
           "vocab_size": rnd.choice([97, 256, 301, 1000]), "hidden_size": H,
           "intermediate_size": rnd.choice([40, 64, 96, 130]), "num_hidden_layers": L,
           "num_attention_heads": nh, "num_key_value_heads": nkv, "rms_norm_eps": rnd.choice([1e-6, 1e-5]),
           "rope_theta": rnd.choice([1e4, 5e4, 1e6]), "max_position_embeddings": 512,
           "tie_word_embeddings": rnd.random() < 0.4, "hidden_act": "silu",
           "num_experts": E, "num_experts_per_tok": K, "moe_intermediate_size": rnd.choice([16, 32, 40, 64]),
           "shared_expert_intermediate_size": rnd.choice([0, 32, 64, 72]), "norm_topk_prob": rnd.random() < 0.5,
           "decoder_sparse_step": rnd.choice([1, 1, 2]),
           "mlp_only_layers": [0] if (L > 1 and rnd.random() < 0.3) else [],
           "use_sliding_window": window, "sliding_window": rnd.choice([7, 20, 33, 100]) if window else 0,
           "max_window_layers": rnd.randint(0, L) if window else 0}
    if explicit:
        cfg["head_dim"] = d
    if rnd.random() < 0.2:
        cfg["qkv_bias"] = False
    return cfg, rnd.choice([4, 8, 16, 32]), [rnd.randint(1, 150) for _ in range(5)]


@pytest.mark.parametrize("seed", range(8))
def test_a_randomly_drawn_configuration(tmp_path, seed):
    cfg, page, lengths = draw(seed)
    folder = tiny.make_folder(str(tmp_path), cfg, seed=seed + 3, dtype=torch.bfloat16)
    w = tiny.read_weights(folder)
    reqs = {f"q{i}": tiny.pick_tokens(cfg, w, n, seed=77 * (i + 1) + seed) for i, n in enumerate(lengths)}
    for dtype in ("float32", "bfloat16"):
        runner = make_runner(folder, dtype, page_size=page, num_pages=max(48, 400 // page), max_requests=4,
                             max_tokens=512, max_context=512)
        for steps in (traces.portions(reqs, (5, 2, 19, 3, 40, 2)),
                      traces.mixed(reqs, max_live=3, seed=seed, decode_tail=8)):
            run_and_compare(runner, steps, cfg, w, reqs, dtype, TOL[dtype])
        assert runner.graph_replays > 0
        assert runner.cache.used_pages() == [0] * len(runner.cache.pools)
