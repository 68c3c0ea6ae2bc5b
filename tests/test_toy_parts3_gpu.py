"""More parts that are nobody's model, defined here and never in the framework, each registered, built,
loaded with random weights and stepped through the engine's own step function, cache manager and
scheduler-facing cuttings without a change to the framework's files:

* a *sandwich* block with four norms (a norm before and after the mixer, a norm before and after the
  feed-forward): another arrangement is another ``Block`` class with other roles;
* a mixer that caches ONE latent row per token instead of keys and values: its cache need describes its
  own tensor per page, and the engine allocates exactly that;
* a mixer with a per-request state that runs inside CUDA-graph replays: its state tensor is static
  memory that the captured pass updates in place.
"""

import dataclasses
import math

import pytest
import torch

import plain_model as pm
import tiny
import traces
from engine_harness import run_trace
from test_toy_parts_gpu import build

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _register():
    from mini_infer_b200.config import register_part
    from mini_infer_b200.parts import Block, Mixer, PagedCacheNeed, StateNeed, TensorDecl, apply_norm, linear, resolve

    class SandwichBlock(Block):
        """``a = x + Norm2(Mixer(Norm1(x)))``;  ``y = a + Norm4(FFN(Norm3(a)))``."""

        roles = {"pre_mixer_norm": "norm", "mixer": "mixer", "post_mixer_norm": "norm",
                 "pre_ffn_norm": "norm", "feed_forward": "feed_forward", "post_ffn_norm": "norm"}

        def forward(self, layer, hidden, pending, ctx, caches):
            x = apply_norm(layer.pre_mixer_norm, hidden, pending)           # hidden += pending; x = norm(hidden)
            y = layer.mixer.forward(x, ctx, caches.get("mixer"))
            y = layer.post_mixer_norm.apply(y, None).float()                # the norm of the part's own output
            x = layer.pre_ffn_norm.apply(hidden, y)                         # hidden += y
            z = layer.feed_forward.forward(x, ctx)
            return layer.post_ffn_norm.apply(z, None).float()               # added by whoever comes next

    @dataclasses.dataclass(frozen=True)
    class LatentNeed(PagedCacheNeed):
        """One row of ``rank`` numbers per token."""
        rank: int
        window: int = 0
        pages_fraction: float = 0.5

        def tensors(self, page_size):
            return [("latent", (page_size, self.rank), torch.float32)]

    class LatentCacheMixer(Mixer):
        """``c_t = x_t W_down`` is all that is cached; ``q_t = x_t W_q``; the output is
        ``(softmax_j<=t(q_t . c_j / sqrt(r)) c_j) W_up``: keys and values are the same latent row."""

        def __init__(self, params, prefix):
            super().__init__(params, prefix)
            self.H, self.r = params["hidden_size"], params["rank"]

        def tensor_decls(self):
            return [TensorDecl(self.prefix + "down.weight", (self.r, self.H)),
                    TensorDecl(self.prefix + "q.weight", (self.r, self.H)),
                    TensorDecl(self.prefix + "up.weight", (self.H, self.r))]

        def load(self, tensors, rt):
            self.rt = rt
            m = rt.precision.matrix
            self.w_down, self.w_q, self.w_up = (m(tensors[self.prefix + n + ".weight"], rt.device)
                                                for n in ("down", "q", "up"))

        def cache_need(self):
            return LatentNeed(self.r)

        def forward(self, x, ctx, cache):
            view = ctx.kv_groups[cache.group]
            pages = view.tensors["latent"][cache.layer_slot]                  # [pages, page_size, r]
            c = linear(x, self.w_down, torch.float32)
            q = linear(x, self.w_q, torch.float32)
            pages.view(-1, self.r)[view.slot_mapping.long()] = c
            out = torch.empty_like(c)
            ps = view.page_size
            for b in range(ctx.num_requests):
                lo, hi, n = ctx.host_q_start[b], ctx.host_q_start[b + 1], ctx.host_kv_len[b]
                table = view.block_table[b, :-(-n // ps)].long()
                keys = pages[table].reshape(-1, self.r)[:n]                    # this request's latent rows
                s = (q[lo:hi] @ keys.T) / math.sqrt(self.r)
                qpos = torch.arange(n - (hi - lo), n, device=s.device)
                s = s.masked_fill(torch.arange(n, device=s.device)[None, :] > qpos[:, None], float("-inf"))
                out[lo:hi] = torch.softmax(s, dim=-1) @ keys
            return linear(out.to(self.rt.act), self.w_up, torch.float32)

    class GraphSafeStateMixer(Mixer):
        """``state = decay * state + x W_in``; ``y = state W_out``.  Decode steps use device tensors only
        (the state rows are gathered and scattered by the step's ``state_slot``), so they may be captured;
        a portion of several tokens runs in order on the host's copy of the batch layout."""

        graph_safe = True

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
            return StateNeed((self.S,))

        def forward(self, x, ctx, cache):
            state = ctx.states[cache.group]
            u = linear(x, self.w_in, torch.float32)
            if ctx.all_decode:
                slots = ctx.state_slot.long()
                s = self.decay * state.index_select(0, slots) + u
                state.index_copy_(0, slots, s)
                out = s
            else:
                out = torch.empty_like(u)
                for b in range(ctx.num_requests):
                    lo, hi, slot = ctx.host_q_start[b], ctx.host_q_start[b + 1], ctx.host_state_slot[b]
                    s = state[slot]
                    for t in range(lo, hi):
                        s = self.decay * s + u[t]
                        out[t] = s
                    state[slot] = s
            return linear(out.to(self.rt.act), self.w_out, torch.float32)

    register_part("block", "toy_sandwich", SandwichBlock)
    register_part("mixer", "toy_latent_cache", LatentCacheMixer)
    register_part("mixer", "toy_graph_safe_state", GraphSafeStateMixer)


def plain(spec, weights, tokens, cfg, forced=None):
    """Plain float32 model of the toy specs of this file."""
    w = {k: v.float() for k, v in weights.items()}
    h = w["model.embed_tokens.weight"][torch.tensor(tokens)]
    eps = cfg["rms_norm_eps"]
    S = len(tokens)
    for e in spec.schedule:
        ls = spec.layers[e.layer]
        p = ls.name + "."
        sandwich = ls.block.kind == "toy_sandwich"
        x = pm.rms_norm(h, w[p + ("pre_mixer_norm.weight" if sandwich else "input_layernorm.weight")], eps)
        kind = ls.mixer.kind
        if kind == "toy_latent_cache":
            r = ls.mixer.get("rank")
            c = x @ w[p + "self_attn.down.weight"].T
            q = x @ w[p + "self_attn.q.weight"].T
            s = (q @ c.T) / math.sqrt(r)
            s = s.masked_fill(torch.arange(S)[None, :] > torch.arange(S)[:, None], float("-inf"))
            y = (torch.softmax(s, -1) @ c) @ w[p + "self_attn.up.weight"].T
        elif kind == "toy_graph_safe_state":
            u = x @ w[p + "self_attn.in.weight"].T
            st, rows = torch.zeros(u.shape[1]), []
            for t in range(S):
                st = ls.mixer.get("decay") * st + u[t]
                rows.append(st)
            y = torch.stack(rows) @ w[p + "self_attn.out.weight"].T
        else:
            m = ls.mixer
            nh, nkv, d = m.get("num_heads"), m.get("num_kv_heads"), m.get("head_dim")
            posn = torch.arange(S)
            q = pm.apply_rope((x @ w[p + "self_attn.q_proj.weight"].T + w[p + "self_attn.q_proj.bias"]).view(S, nh, d),
                              posn, cfg["rope_theta"])
            k = pm.apply_rope((x @ w[p + "self_attn.k_proj.weight"].T + w[p + "self_attn.k_proj.bias"]).view(S, nkv, d),
                              posn, cfg["rope_theta"])
            v = (x @ w[p + "self_attn.v_proj.weight"].T + w[p + "self_attn.v_proj.bias"]).view(S, nkv, d)
            y = pm.attention_scores_softmax_pv(q, k, v, m.get("window")).reshape(S, nh * d) @ w[p + "self_attn.o_proj.weight"].T
        if sandwich:
            y = pm.rms_norm(y, w[p + "post_mixer_norm.weight"], eps)
        h = h + y
        x = pm.rms_norm(h, w[p + ("pre_ffn_norm.weight" if sandwich else "post_attention_layernorm.weight")], eps)
        if ls.feed_forward.kind == "sparse_moe":
            f = None
            if forced and e.layer in forced:
                f = torch.tensor([forced[e.layer][t] for t in range(S)])
            y, _, _ = pm.moe_block(x, w, p + "mlp.", cfg["num_experts"], cfg["num_experts_per_tok"],
                                   cfg["norm_topk_prob"], cfg["shared_expert_intermediate_size"] > 0, f)
        else:
            y = pm.swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        if sandwich:
            y = pm.rms_norm(y, w[p + "post_ffn_norm.weight"], eps)
        h = h + y
    return pm.rms_norm(h, w["model.norm.weight"], eps) @ w["lm_head.weight"].T


def _three_cuttings(runner, spec, weights, cfg, dtype, lengths=(30, 7, 45, 18, 26, 11)):
    g = torch.Generator().manual_seed(2)
    reqs = {f"v{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}
    tol = 3e-5 if dtype == "float32" else 3e-2
    for steps in (traces.whole(reqs), traces.portions(reqs, (5, 2, 9, 3)),
                  traces.mixed(reqs, max_live=3, seed=1, decode_tail=6)):
        routing = {}
        got = run_trace(runner, steps, routing)
        ref = {rid: plain(spec, weights, toks, cfg, routing.get(rid)) for rid, toks in reqs.items()}
        assert len(got) == sum(len(t) for t in reqs.values())
        for (rid, pos), row in got.items():
            assert float((row - ref[rid][pos]).abs().max()) <= tol * float(ref[rid].abs().max()), (rid, pos)
    return reqs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sandwich_block_with_four_norms(dtype):
    from mini_infer_b200.config import LayerPart, LayerSpec, PartSpec, build_model_spec
    _register()
    cfg = tiny.CONFIG_A
    base = build_model_spec(cfg)
    norm = base.layers[0].mixer_norm
    b1 = base.layers[1]
    sandwich = LayerSpec(b1.name, PartSpec("toy_sandwich"), {
        "pre_mixer_norm": LayerPart("norm", norm, "pre_mixer_norm."),
        "mixer": b1.parts["mixer"],
        "post_mixer_norm": LayerPart("norm", norm, "post_mixer_norm."),
        "pre_ffn_norm": LayerPart("norm", norm, "pre_ffn_norm."),
        "feed_forward": b1.parts["feed_forward"],
        "post_ffn_norm": LayerPart("norm", norm, "post_ffn_norm."),
    })
    spec = dataclasses.replace(base, layers=(base.layers[0], sandwich))
    runner, weights = build(spec, dtype)
    assert "model.layers.1.post_ffn_norm.weight" in weights and "model.layers.1.input_layernorm.weight" not in weights
    _three_cuttings(runner, spec, weights, cfg, dtype)
    # a description that lacks a role of the block is refused when the model is built
    broken = LayerSpec(b1.name, PartSpec("toy_sandwich"), {k: v for k, v in sandwich.parts.items() if k != "pre_ffn_norm"})
    with pytest.raises(ValueError, match="missing \\['pre_ffn_norm'\\]"):
        from mini_infer_b200.engine.model import Model
        Model(dataclasses.replace(base, layers=(base.layers[0], broken)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixer_that_caches_one_latent_row_per_token(dtype):
    from mini_infer_b200.config import PartSpec, build_model_spec
    _register()
    cfg = tiny.CONFIG_A
    base = build_model_spec(cfg)
    latent = base.layers[0].with_part("mixer", PartSpec("toy_latent_cache", {"hidden_size": cfg["hidden_size"], "rank": 12}))
    spec = dataclasses.replace(base, layers=(latent, base.layers[1]))
    runner, weights = build(spec, dtype, num_pages=40, page_size=8)
    # two groups: the latent rows (one float32 tensor of [layers, pages, page_size, rank], half the page budget)
    # and the keys and values of the attention layer
    by_name = [sorted(t) for t in runner.kv_tensors]
    assert sorted(by_name) == [["k", "v"], ["latent"]]
    gl = by_name.index(["latent"])
    assert runner.kv_tensors[gl]["latent"].shape == (1, 20, 8, 12) and runner.kv_tensors[gl]["latent"].dtype == torch.float32
    assert runner.cache.pools[gl].num_pages == 20 and runner.cache.pools[1 - gl].num_pages == 40
    _three_cuttings(runner, spec, weights, cfg, dtype, lengths=(30, 7, 45, 18, 26))
    assert runner.cache.used_pages() == [0, 0]
    runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_state_mixer_inside_graph_replays_and_a_failed_step_leaves_no_trace(dtype):
    from mini_infer_b200.config import PartSpec, build_model_spec
    from mini_infer_b200.engine.step import StepEntry
    _register()
    cfg = tiny.CONFIG_A
    base = build_model_spec(cfg)
    toy = base.layers[1].with_part("mixer", PartSpec(
        "toy_graph_safe_state", {"hidden_size": cfg["hidden_size"], "state_size": 20, "decay": 0.8}))
    spec = dataclasses.replace(base, layers=(base.layers[0], toy))
    runner, weights = build(spec, dtype)
    assert runner.cuda_graphs and not runner.can_step_ahead(["x"])
    _three_cuttings(runner, spec, weights, cfg, dtype)
    assert runner.graph_replays > 0                      # the all-decode steps of the mixed trace were replays
    # a step whose forward pass fails: pages cancelled, the requests' state rows as before
    runner.add_request("f")
    runner.step([StepEntry("f", [3, 4, 5], [2])])
    before = [st.clone() for st in runner.state_tensors]
    tokens_before = runner.num_tokens("f")
    part = runner.model.layers[1].feed_forward
    original = part.forward_from_residual

    def failing(*a, **k):
        raise RuntimeError("injected on the host")
    part.forward_from_residual = failing
    try:
        with pytest.raises(RuntimeError, match="injected on the host"):
            runner.step([StepEntry("f", [6, 7], [1])])
    finally:
        part.forward_from_residual = original
    assert all(torch.equal(a, b) for a, b in zip(before, runner.state_tensors))
    assert runner.num_tokens("f") == tokens_before
    res = runner.step([StepEntry("f", [6, 7], [0, 1])])
    if dtype == "float32":                               # (bfloat16 could route a near-tie otherwise)
        ref = plain(spec, weights, [3, 4, 5, 6, 7], cfg)
        assert float((res.logits.float().cpu() - ref[3:5]).abs().max()) <= 3e-5 * float(ref.abs().max())
    runner.release("f")
    runner.cache.check_invariants()


def test_rows_that_fill_a_captured_batch_keep_their_state_to_themselves(monkeypatch):
    """Ten requests decode together through the mixer with a state of its own: the step is filled up to the
    captured size of 12 with rows of no request, whose state goes to the spare slot and nowhere else."""
    from mini_infer_b200.config import PartSpec, build_model_spec
    # a coarse ladder of captured sizes for the test: every size to 8, multiples of 4 above
    from mini_infer_b200.parts.tuning import Tuning
    monkeypatch.setattr(Tuning, "decode_graph_batch", lambda self, n: n if n <= 8 else -(-n // 4) * 4)
    _register()
    cfg = tiny.CONFIG_A
    base = build_model_spec(cfg)
    toy = base.layers[1].with_part("mixer", PartSpec(
        "toy_graph_safe_state", {"hidden_size": cfg["hidden_size"], "state_size": 20, "decay": 0.8}))
    spec = dataclasses.replace(base, layers=(base.layers[0], toy))
    runner, weights = build(spec, "float32", max_requests=12, num_pages=80)
    g = torch.Generator().manual_seed(3)
    reqs = {f"s{i}": torch.randint(0, cfg["vocab_size"], (9 + i,), generator=g).tolist() for i in range(10)}
    steps = traces.decoded_together(reqs, tail=5)
    routing = {}
    got = run_trace(runner, steps, routing)
    assert runner.graph_replays == 5 and {key[0] for key in runner._graphs} == {12}
    for rid, toks in reqs.items():
        ref = plain(spec, weights, toks, cfg, routing.get(rid))
        for pos in range(len(toks) - 6, len(toks)):
            assert float((got[(rid, pos)] - ref[pos]).abs().max()) <= 3e-5 * float(ref.abs().max()), (rid, pos)
    assert not bool(runner.state_tensors[0][12].eq(0).all())      # the spare slot took the filling rows' state
