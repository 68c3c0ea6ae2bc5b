"""The plain implementation itself (CPU): properties that any right reading of the
reference's formulas must have, and agreement of the two Philox implementations."""

import math

import pytest
import torch

import plain_model as pm
import tiny


@pytest.fixture(scope="module", params=["A", "B", "C"])
def model(request, tmp_path_factory):
    cfg = tiny.CONFIGS[request.param]
    folder = tiny.make_folder(str(tmp_path_factory.mktemp("m")), cfg, seed=21, dtype=torch.float32)
    return cfg, tiny.read_weights(folder)


def test_causal_prefix_property(model):
    cfg, w = model
    toks = tiny.pick_tokens(cfg, w, 40, 1)
    full = pm.forward(cfg, w, toks)
    part = pm.forward(cfg, w, toks[:17])
    assert torch.allclose(full[:17], part, atol=2e-6, rtol=0)
    assert full.shape == (40, cfg["vocab_size"])


def test_float64_agrees_with_float32(model):
    cfg, w = model
    toks = tiny.pick_tokens(cfg, w, 24, 2, min_gap=1e-4)
    a = pm.forward(cfg, w, toks)
    b = pm.forward(cfg, w, toks, dtype=torch.float64)
    assert float((a - b.float()).abs().max()) < 2e-5 * float(b.abs().max())


def test_rms_norm_and_rope_basics():
    x = torch.randn(5, 32)
    y = pm.rms_norm(x, torch.ones(32), 0.0)
    assert torch.allclose((y * y).mean(-1), torch.ones(5), atol=1e-5)
    q = torch.randn(7, 3, 16)
    pos = torch.arange(7)
    r = pm.apply_rope(q, pos, 10000.0)
    assert torch.allclose(r[0], q[0], atol=1e-7)                               # position 0: identity
    assert torch.allclose(r.norm(dim=-1), q.norm(dim=-1), atol=1e-5)          # a rotation
    # relative property: <rope(a, p), rope(b, j)> depends on p - j only
    a, b = torch.randn(1, 1, 16), torch.randn(1, 1, 16)
    d1 = (pm.apply_rope(a, torch.tensor([9]), 1e4) * pm.apply_rope(b, torch.tensor([4]), 1e4)).sum()
    d2 = (pm.apply_rope(a, torch.tensor([25]), 1e4) * pm.apply_rope(b, torch.tensor([20]), 1e4)).sum()
    assert abs(float(d1 - d2)) < 1e-4
    inv = pm.rope_inv_freq(16, 10000.0)
    assert inv[0] == 1.0 and abs(float(inv[-1]) - 10000.0 ** (-14 / 16)) < 1e-9


def test_window_masks_exactly_w_keys():
    S, W = 12, 5
    q = torch.zeros(S, 1, 4)
    k = torch.zeros(S, 1, 4)
    v = torch.eye(S)[:, None, :4 * 3].reshape(S, 1, -1)[:, :, :4] * 0 + torch.arange(S, dtype=torch.float32)[:, None, None]
    out = pm.attention_scores_softmax_pv(q, k, v.expand(S, 1, 4).contiguous(), window=W)
    for p in range(S):
        lo = max(0, p - W + 1)
        assert abs(float(out[p, 0, 0]) - (lo + p) / 2) < 1e-5                  # uniform mean over [lo, p]
    same = pm.attention_scores_softmax_pv(q, k, v.expand(S, 1, 4).contiguous(), window=S + 3)
    full = pm.attention_scores_softmax_pv(q, k, v.expand(S, 1, 4).contiguous(), window=0)
    assert torch.equal(same, full)


def test_gqa_head_mapping():
    S, nh, nkv, d = 3, 4, 2, 2
    q = torch.zeros(S, nh, d)
    k = torch.zeros(S, nkv, d)
    v = torch.zeros(S, nkv, d)
    v[:, 0] = 1.0
    v[:, 1] = 2.0
    out = pm.attention_scores_softmax_pv(q, k, v)
    assert torch.allclose(out[:, :2], torch.ones(S, 2, d)) and torch.allclose(out[:, 2:], 2 * torch.ones(S, 2, d))


def test_routing_rules():
    x = torch.randn(9, 16)
    w = torch.randn(6, 16)
    probs, idx, wt = pm.route(x, w, 3, True)
    assert torch.allclose(wt.sum(-1), torch.ones(9), atol=1e-6)
    probs2, idx2, wt2 = pm.route(x, w, 3, False)
    assert torch.equal(idx, idx2) and torch.allclose(wt2, probs.gather(1, idx))
    assert (wt2[:, :-1] >= wt2[:, 1:]).all()                                   # descending probability
    # ties: equal router rows give equal probabilities; the lowest index wins
    w[4] = w[1]
    w[2] = w[1]
    _, idx3, _ = pm.route(x, w, 2, False)
    for t in range(9):
        chosen = idx3[t].tolist()
        for e in (2, 4):
            if e in chosen:
                assert 1 in chosen and chosen.index(1) < chosen.index(e)


def test_moe_equals_dense_sum_over_chosen(model):
    cfg, w = model
    i = next(i for i in range(cfg["num_hidden_layers"]) if pm.layer_is_sparse(cfg, i))
    p = f"model.layers.{i}.mlp."
    x = torch.randn(4, cfg["hidden_size"]) * 0.5
    out, idx, probs = pm.moe_block(x, w, p, cfg["num_experts"], cfg["num_experts_per_tok"],
                                   cfg["norm_topk_prob"], cfg["shared_expert_intermediate_size"] > 0)
    # forcing the same routing reproduces the result; forcing another changes it
    out2, _, _ = pm.moe_block(x, w, p, cfg["num_experts"], cfg["num_experts_per_tok"], cfg["norm_topk_prob"],
                              cfg["shared_expert_intermediate_size"] > 0, forced_idx=idx)
    assert torch.allclose(out, out2)
    other = (idx + 1) % cfg["num_experts"]
    out3, _, _ = pm.moe_block(x, w, p, cfg["num_experts"], cfg["num_experts_per_tok"], cfg["norm_topk_prob"],
                              cfg["shared_expert_intermediate_size"] > 0, forced_idx=other)
    assert not torch.allclose(out, out3)


def test_by_expert_form_agrees_with_the_token_by_token_form(model):
    cfg, w = model
    toks = tiny.pick_tokens(cfg, w, 50, 9)
    a = pm.forward(cfg, w, toks)
    b = pm.forward(cfg, w, toks, by_expert=True)
    assert float((a - b).abs().max()) < 1e-5 * float(a.abs().max())


def test_sampling_rules():
    logits = torch.tensor([0.0, 3.0, 3.0, -1.0, 3.0])
    assert pm.greedy(logits) == 1
    assert pm.sample(logits, 0.0, 1.0, 0.99) == 1
    p = torch.softmax(logits, -1)
    assert pm.sample(logits, 1.0, 1.0, 0.0) == 0
    assert pm.sample(logits, 1.0, 1.0, float(p[0]) + 1e-4) == 1
    assert pm.sample(logits, 1.0, 1.0, 0.999999) == 4
    # nucleus: the three tied maxima hold 0.96 of the mass; top_p = 0.5 keeps all three ties
    for u, want in ((0.0, 1), (0.34, 2), (0.99, 4)):
        assert pm.sample(logits, 1.0, 0.5, u) == want
    # a sharper temperature concentrates the mass
    peaked = torch.tensor([0.0, 1.0, 5.0, 2.0])
    assert pm.sample(peaked, 0.1, 0.9, 0.5) == 2
    counts = [0] * 4
    for n in range(2000):
        counts[pm.sample(peaked, 1.0, 1.0, pm.uniform_for(3, 0, n))] += 1
    freq = torch.tensor(counts) / 2000.0
    assert float((freq - torch.softmax(peaked, -1)).abs().max()) < 0.03


def test_philox_known_answers_and_engine_agreement():
    from mini_infer_b200.sampling import philox4x32, uniform
    # known-answer vectors of the Random123 distribution (kat_vectors, philox4x32 10)
    assert pm.philox4x32((0, 0, 0, 0), (0, 0)) == (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)
    assert pm.philox4x32((0xffffffff,) * 4, (0xffffffff,) * 2) == (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)
    assert pm.philox4x32((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0)) == \
        (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)
    for seed, stream, idx in [(42, 0, 0), (42, 3, 17), (2 ** 40 + 5, 2 ** 33, 2 ** 35 + 1)]:
        assert philox4x32((idx, idx >> 32, stream, stream >> 32), (seed, seed >> 32)) == \
            pm.philox4x32((idx & 0xffffffff, (idx >> 32) & 0xffffffff, stream & 0xffffffff, (stream >> 32) & 0xffffffff),
                          (seed & 0xffffffff, (seed >> 32) & 0xffffffff))
        assert uniform(seed, stream, idx) == pm.uniform_for(seed, stream, idx)
        assert 0.0 <= uniform(seed, stream, idx) < 1.0


def test_generate_is_reproducible(model):
    cfg, w = model
    a = pm.generate(cfg, w, [3, 1, 4, 1, 5], 6, temperature=0.8, top_p=1.0, seed=7, stream=2)
    b = pm.generate(cfg, w, [3, 1, 4, 1, 5], 6, temperature=0.8, top_p=1.0, seed=7, stream=2)
    c = pm.generate(cfg, w, [3, 1, 4, 1, 5], 6, temperature=0.8, top_p=1.0, seed=8, stream=2)
    assert a == b and len(a) == 6 and a != c
