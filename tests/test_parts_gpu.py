"""Each part alone, built from its PartSpec and random tensors, against the plain function for
the same part - at sizes that none of the tiny models has."""

import pytest
import torch

import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def runtime(dtype):
    from mini_infer_b200.parts.base import Runtime, configure_matmul_exactness, precision_from_name
    configure_matmul_exactness()
    return Runtime(precision_from_name(dtype), torch.device(DEV))


def random_tensors(part, seed, dtype):
    from mini_infer_b200.weights import RandomSource
    src = RandomSource(part.tensor_decls(), seed, dtype, "cpu", std=0.08)
    return {n: src.read(n) for n in src.names()}


def whole_sequence_ctx(S, nkv, d, page_size, act, n_layers=1, prefix_len=0):
    """A StepContext for one request fed tokens [prefix_len, S) with pages in reverse order."""
    from mini_infer_b200.parts.base import KVGroupView, StepContext
    pages = -(-S // page_size)
    order = list(range(pages - 1, -1, -1))
    table = torch.tensor([order], dtype=torch.int32, device=DEV)
    n = S - prefix_len
    pos = torch.arange(prefix_len, S, dtype=torch.int32, device=DEV)
    slot = torch.tensor([order[p // page_size] * page_size + p % page_size for p in range(prefix_len, S)],
                        dtype=torch.int32, device=DEV)
    k = torch.zeros(n_layers, pages, nkv, page_size, d, dtype=act, device=DEV)
    view = KVGroupView(table, slot, page_size, {"k": k, "v": torch.zeros_like(k)})
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return StepContext(num_tokens=n, num_requests=1, max_q_len=n, max_kv_len=S, all_decode=(n == 1),
                       token_ids=i32([0] * n), positions=pos, q_start=i32([0, n]), kv_len=i32([S]),
                       req_of_token=i32([0] * n), state_slot=i32([0]), fresh=i32([1 if prefix_len == 0 else 0]),
                       kv_groups=[view], host_q_start=[0, n], host_kv_len=[S], host_state_slot=[0])


TOL = {"float32": 3e-5, "bfloat16": 2e-2}


def close(got, ref, tol):
    err = float((got.float().cpu() - ref.float().cpu()).abs().max())
    scale = float(ref.abs().max())
    assert err <= tol * scale, f"error {err:.3e}, scale {scale:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from mini_infer_b200.config import PartSpec, part_class
    rt = runtime(dtype)
    part = part_class("norm", "rmsnorm")({"size": 136, "eps": 2e-5}, "n.")
    t = random_tensors(part, 1, rt.act)
    part.load(t, rt)
    h = torch.randn(5, 136, device=DEV)
    d = torch.randn(5, 136, device=DEV)
    ref = pm.rms_norm((h + d).cpu(), t["n.weight"].float(), 2e-5)
    out = part.apply(h, d)
    assert out.dtype == rt.act
    close(out, ref, TOL[dtype] if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,d,window,bias", [(6, 3, 32, 0, True), (4, 1, 64, 20, False), (2, 2, 128, 0, True)])
def test_attention_part_whole_then_tail(dtype, nh, nkv, d, window, bias):
    from mini_infer_b200.config import PartSpec, part_class
    rt = runtime(dtype)
    H, S, theta = 112, 75, 30000.0
    part = part_class("mixer", "gqa_attention")({
        "hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": d, "bias": bias, "window": window,
        "position": PartSpec("rope", {"head_dim": d, "theta": theta})}, "a.")
    t = random_tensors(part, 2, rt.act)
    part.load(t, rt)
    from mini_infer_b200.parts.base import CacheBinding
    x = (torch.randn(S, H, generator=torch.Generator().manual_seed(3)) * 1.0).to(rt.act)
    w = {k: v.float() for k, v in t.items()}
    ref = pm.attention(x.float(), w, "a.", nh, nkv, d, theta, window)
    # whole sequence in one go
    ctx = whole_sequence_ctx(S, nkv, d, 8, rt.act)
    out = part.forward(x.to(DEV), ctx, CacheBinding("kv", 0, 0, True))
    assert out.dtype == torch.float32
    close(out, ref, TOL[dtype])
    # then: first 60 tokens, the rest one at a time from the cache the first call left
    pages = -(-S // 8)
    k = torch.zeros(1, pages, nkv, 8, d, dtype=rt.act, device=DEV)
    v = torch.zeros_like(k)
    part.forward(x[:60].to(DEV), _with_cache(k, v, 8, 0, 60), CacheBinding("kv", 0, 0, True))
    for p in range(60, S):
        c = _with_cache(k, v, 8, p, p + 1)
        o = part.forward(x[p:p + 1].to(DEV), c, CacheBinding("kv", 0, 0, True))
        close(o, ref[p:p + 1], TOL[dtype] * (float(ref.abs().max()) / float(ref[p].abs().max())))


def _with_cache(k, v, ps, lo, hi):
    from mini_infer_b200.parts.base import KVGroupView, StepContext
    pages = k.shape[1]
    order = list(range(pages - 1, -1, -1))
    table = torch.tensor([order], dtype=torch.int32, device=DEV)
    n = hi - lo
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    slot = i32([order[p // ps] * ps + p % ps for p in range(lo, hi)])
    view = KVGroupView(table, slot, ps, {"k": k, "v": v})
    return StepContext(num_tokens=n, num_requests=1, max_q_len=n, max_kv_len=hi, all_decode=(n == 1),
                       token_ids=i32([0] * n), positions=i32(list(range(lo, hi))), q_start=i32([0, n]),
                       kv_len=i32([hi]), req_of_token=i32([0] * n), state_slot=i32([0]),
                       fresh=i32([int(lo == 0)]), kv_groups=[view], host_q_start=[0, n], host_kv_len=[hi],
                       host_state_slot=[0])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu_mlp_part(dtype):
    from mini_infer_b200.config import part_class
    rt = runtime(dtype)
    part = part_class("feed_forward", "swiglu_mlp")({"hidden_size": 88, "intermediate_size": 150}, "m.")
    t = random_tensors(part, 4, rt.act)
    part.load(t, rt)
    x = torch.randn(11, 88).to(rt.act)
    ref = pm.swiglu_mlp(x.float(), t["m.gate_proj.weight"].float(), t["m.up_proj.weight"].float(),
                        t["m.down_proj.weight"].float())
    close(part.forward(x.to(DEV), None), ref, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,K,mI,sI,norm", [(7, 2, 24, 40, True), (16, 5, 36, 0, False), (60, 4, 16, 56, False)])
def test_sparse_moe_part(dtype, E, K, mI, sI, norm):
    from mini_infer_b200.config import part_class
    rt = runtime(dtype)
    H, T = 104, 33
    part = part_class("feed_forward", "sparse_moe")({
        "hidden_size": H, "num_experts": E, "top_k": K, "expert_intermediate_size": mI,
        "shared_intermediate_size": sI, "norm_topk_prob": norm}, "f.")
    t = random_tensors(part, 5, rt.act)
    part.load(t, rt)
    part.keep_routing = True
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(6)).to(rt.act)
    out = part.forward(x.to(DEV), None)
    idx = part.last_routing[0].cpu().long()
    w = {k: v.float() for k, v in t.items()}
    ref, ref_idx, probs = pm.moe_block(x.float(), w, "f.", E, K, norm, sI > 0)
    # rows whose K-th and (K+1)-th probabilities are within rounding may legitimately route
    # otherwise; they are compared with the plain model forced to the engine's choice
    ties = (idx != ref_idx).any(dim=1)
    if ties.any():
        s = torch.sort(probs, dim=-1, descending=True).values
        assert float((s[ties, K - 1] - s[ties, K]).abs().max()) < 1e-5
        ref, _, _ = pm.moe_block(x.float(), w, "f.", E, K, norm, sI > 0, forced_idx=idx)
    close(out, ref, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_deferred_sum_of_the_experts_rows(dtype):
    """The experts' weighted sum may be left to the norm that follows: the same bits as summing first,
    through the framework's RMSNorm (which folds it into its kernel) and through a norm that knows
    nothing of deferred outputs (which is handed the tensor)."""
    from mini_infer_b200.config import part_class
    from mini_infer_b200.parts import Deferred, Norm, WeightedRowSum, apply_norm, resolve
    rt = runtime(dtype)
    H, T = 104, 21
    moe = part_class("feed_forward", "sparse_moe")({
        "hidden_size": H, "num_experts": 6, "top_k": 3, "expert_intermediate_size": 48,
        "shared_intermediate_size": 80, "norm_topk_prob": True}, "f.")
    moe.load(random_tensors(moe, 5, rt.act), rt)
    norm = part_class("norm", "rmsnorm")({"size": H, "eps": 1e-6}, "n.")
    norm.load(random_tensors(norm, 1, rt.act), rt)
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(6)).to(rt.act).to(DEV)
    plain = moe.forward(x, None)
    later = moe.forward_deferred(x, None)
    assert isinstance(later, WeightedRowSum) and isinstance(later, Deferred)
    assert torch.equal(resolve(later), plain) and resolve(plain) is plain
    h0 = torch.randn(T, H, device=DEV)
    h1, h2 = h0.clone(), h0.clone()
    assert norm.accepts_deferred
    assert torch.equal(apply_norm(norm, h1, later), norm.apply(h2, plain)) and torch.equal(h1, h2)

    class PlainNorm(Norm):
        def apply(self, hidden, delta, rows=None):
            assert isinstance(delta, torch.Tensor)
            return hidden + delta

    assert torch.equal(apply_norm(PlainNorm({}, ""), h0, later), h0 + plain)


def test_embedding_and_head_parts():
    from mini_infer_b200.config import part_class
    rt = runtime("bfloat16")
    emb = part_class("embedding", "token_embedding")({"vocab_size": 301, "hidden_size": 40}, "e.")
    t = random_tensors(emb, 7, rt.act)
    emb.load(t, rt)
    ids = torch.tensor([300, 0, 17], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids).cpu(), t["e.weight"].float()[ids.cpu().long()])
    head = part_class("lm_head", "linear")({"vocab_size": 301, "hidden_size": 40, "tied_to": "e.weight"}, "h.")
    assert head.tensor_decls() == []
    head.load({}, rt)
    head.tie(emb.weight)
    x = torch.randn(3, 40).to(rt.act)
    close(head.forward(x.to(DEV)), x.float() @ t["e.weight"].float().T, 1e-2)
