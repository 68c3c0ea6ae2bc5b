"""Parts that are not Qwen2-MoE's, defined here and never in the framework: a mixer with a
fixed-size state of its own, registered, built, loaded with random weights and stepped through the
engine's own step function without a change to the framework's files; a layer named twice in the
schedule; a layer that reads another layer's cache."""

import dataclasses

import pytest
import torch

import tiny
import traces
from engine_harness import run_trace

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _register_toy():
    from mini_infer_b200.config import register_part
    from mini_infer_b200.parts import Mixer, StateNeed, TensorDecl, linear

    class DecayingSumMixer(Mixer):
        """state_t = decay * state_{t-1} + x_t W_in ;  y_t = state_t W_out.
        One state vector per request, carried across steps in the request's state slot."""

        def __init__(self, params, prefix):
            super().__init__(params, prefix)
            self.H, self.S, self.decay = params["hidden_size"], params["state_size"], params["decay"]

        def tensor_decls(self):
            return [TensorDecl(self.prefix + "in.weight", (self.S, self.H)),
                    TensorDecl(self.prefix + "out.weight", (self.H, self.S))]

        def load(self, tensors, rt):
            self.rt = rt
            self.w_in = rt.precision.matrix(tensors[self.prefix + "in.weight"], rt.device)
            self.w_out = rt.precision.matrix(tensors[self.prefix + "out.weight"], rt.device)

        def cache_need(self):
            return StateNeed((self.S,), torch.float32)

        def forward(self, x, ctx, cache):
            state = ctx.states[cache.group]
            u = linear(x, self.w_in, torch.float32)
            out = torch.empty_like(u)
            for b in range(ctx.num_requests):                 # a request's portion runs in order
                lo, hi, slot = ctx.host_q_start[b], ctx.host_q_start[b + 1], ctx.host_state_slot[b]
                s = state[slot]
                for t in range(lo, hi):
                    s = self.decay * s + u[t]
                    out[t] = s
                state[slot] = s
            return linear(out.to(self.rt.act), self.w_out, torch.float32)

    register_part("mixer", "toy_decaying_sum", DecayingSumMixer)
    return DecayingSumMixer


def plain_toy_model(spec, weights, tokens, cfg, forced=None):
    """Plain float32 model for the toy spec: layers with the toy mixer use its recurrence, the rest
    the plain attention; schedule and cache sharing as the spec says."""
    import plain_model as pm
    w = {k: v.float() for k, v in weights.items()}
    ids = torch.tensor(tokens)
    h = w["model.embed_tokens.weight"][ids]
    eps = cfg["rms_norm_eps"]
    kv_of_entry = {}
    for pos, e in enumerate(spec.schedule):
        ls = spec.layers[e.layer]
        p = ls.name + "."
        x = pm.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        if ls.mixer.kind == "toy_decaying_sum":
            u = x @ w[p + "self_attn.in.weight"].T
            s = torch.zeros(u.shape[1])
            rows = []
            for t in range(len(tokens)):
                s = ls.mixer.get("decay") * s + u[t]
                rows.append(s)
            y = torch.stack(rows) @ w[p + "self_attn.out.weight"].T
        else:
            m = ls.mixer
            nh, nkv, d = m.get("num_heads"), m.get("num_kv_heads"), m.get("head_dim")
            S = len(tokens)
            posn = torch.arange(S)
            q = x @ w[p + "self_attn.q_proj.weight"].T + w[p + "self_attn.q_proj.bias"]
            q = pm.apply_rope(q.view(S, nh, d), posn, cfg["rope_theta"])
            if e.cache_from is None:
                k = x @ w[p + "self_attn.k_proj.weight"].T + w[p + "self_attn.k_proj.bias"]
                v = x @ w[p + "self_attn.v_proj.weight"].T + w[p + "self_attn.v_proj.bias"]
                k = pm.apply_rope(k.view(S, nkv, d), posn, cfg["rope_theta"])
                kv_of_entry[pos] = (k, v.view(S, nkv, d))
            k, v = kv_of_entry[e.cache_from if e.cache_from is not None else pos]
            a = pm.attention_scores_softmax_pv(q, k, v, m.get("window"))
            y = a.reshape(S, nh * d) @ w[p + "self_attn.o_proj.weight"].T
        h = h + y
        x = pm.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        if ls.feed_forward.kind == "sparse_moe":
            f = None
            if forced and e.layer in forced:
                f = torch.tensor([forced[e.layer][t] for t in range(len(tokens))])
            y, _, _ = pm.moe_block(x, w, p + "mlp.", cfg["num_experts"], cfg["num_experts_per_tok"],
                                   cfg["norm_topk_prob"], cfg["shared_expert_intermediate_size"] > 0, f)
        else:
            y = pm.swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                              w[p + "mlp.down_proj.weight"])
        h = h + y
    x = pm.rms_norm(h, w["model.norm.weight"], eps)
    return x @ w["lm_head.weight"].T


def build(spec, dtype, seed=4, **runner_kw):
    from mini_infer_b200.engine.loading import _runtime
    from mini_infer_b200.engine.model import Model
    from mini_infer_b200.engine.step import ModelRunner
    from mini_infer_b200.weights import RandomSource
    rt = _runtime(dtype, DEV)
    model = Model(spec)
    src = RandomSource(model.tensor_decls(), seed, torch.bfloat16, "cpu", std=0.05)
    weights = {n: src.read(n) for n in src.names()}
    model.load(src, rt)
    kw = dict(page_size=8, num_pages=40, max_requests=4, max_tokens_per_step=256, max_context=256)
    kw.update(runner_kw)
    return ModelRunner(model, rt, **kw), weights


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_of_its_own(dtype):
    from mini_infer_b200.config import PartSpec, build_model_spec
    _register_toy()
    cfg = tiny.CONFIG_A
    base = build_model_spec(cfg)
    toy_layer = base.layers[1].with_part("mixer", PartSpec(
        "toy_decaying_sum", {"hidden_size": cfg["hidden_size"], "state_size": 24, "decay": 0.9}))
    spec = dataclasses.replace(base, layers=(base.layers[0], toy_layer))
    runner, weights = build(spec, dtype)
    # (a slot per request and a spare one for the rows that fill a captured batch up)
    assert len(runner.state_tensors) == 1 and runner.state_tensors[0].shape == (4 + 1, 24)
    assert [b["mixer"].kind for b in runner.model.bindings] == ["kv", "state"]
    g = torch.Generator().manual_seed(0)
    reqs = {f"t{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()
            for i, n in enumerate([30, 7, 45, 18, 26, 11])}
    tol = 3e-5 if dtype == "float32" else 3e-2
    for steps in (traces.whole(reqs), traces.portions(reqs, (5, 2, 9, 3)),
                  traces.mixed(reqs, max_live=3, seed=1, decode_tail=6)):     # slots are used again
        routing = {}
        got = run_trace(runner, steps, routing)
        # near-ties of the router may go either way: the plain model follows the engine's choice
        ref = {rid: plain_toy_model(spec, weights, toks, cfg, routing.get(rid)) for rid, toks in reqs.items()}
        for (rid, pos), row in got.items():
            scale = float(ref[rid].abs().max())
            assert float((row - ref[rid][pos]).abs().max()) <= tol * scale, (rid, pos)


def test_layer_named_twice_and_shared_cache():
    from mini_infer_b200.config import ScheduleEntry, build_model_spec
    from mini_infer_b200.config.spec import PartSpec
    cfg = tiny.CONFIG_A
    base = build_model_spec(cfg)
    # layer 2: attention without k/v projections of its own, reading the cache of schedule entry 1
    shared_mixer = PartSpec("gqa_attention", dict(base.layers[1].mixer.params, shares_cache=True))
    layer2 = base.layers[1].renamed("model.layers.2").with_part("mixer", shared_mixer)
    spec = dataclasses.replace(base, layers=base.layers + (layer2,),
                               schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0),
                                         ScheduleEntry(2, cache_from=1)))
    runner, weights = build(spec, "float32")
    assert "model.layers.2.self_attn.k_proj.weight" not in weights
    assert runner.model.kv_groups[0].num_layers == 3
    g = torch.Generator().manual_seed(1)
    reqs = {f"s{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate([21, 40, 9])}
    ref = {rid: plain_toy_model(spec, weights, toks, cfg) for rid, toks in reqs.items()}
    for steps in (traces.whole(reqs), traces.mixed(reqs, max_live=3, seed=2, decode_tail=5)):
        got = run_trace(runner, steps)
        for (rid, pos), row in got.items():
            assert float((row - ref[rid][pos]).abs().max()) <= 3e-5 * float(ref[rid].abs().max()), (rid, pos)
