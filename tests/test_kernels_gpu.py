"""Each CUDA kernel alone against a plain float32 PyTorch reference of the same op, at sizes
other than the tiny models' (odd widths, head sizes in steps of 16 and between, vocabularies and
widths that are no power of two), in float32 and bfloat16."""

import math
import random

import pytest
import torch

import plain_model as pm

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def F():
    from mini_infer_b200.ops import functional
    return functional


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, ref, tol, what=""):
    got, ref = got.float().cpu(), ref.float().cpu()
    err = float((got - ref).abs().max())
    scale = max(float(ref.abs().max()), 1e-6)
    assert err <= tol * scale, f"{what}: error {err:.3e} vs scale {scale:.3e} (tolerance {tol:.1e})"


TOL = {torch.float32: 2e-6, torch.bfloat16: 1e-2}


@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16])
def test_embed_gather(wdt):
    table = rnd(1003, 200, dtype=wdt)
    ids = torch.tensor([0, 1002, 5, 5, 77, 400], dtype=torch.int32, device=DEV)
    out = F().embed_gather(ids, table)
    assert out.dtype == torch.float32 and torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("H", [72, 200, 2048 + 8])
@pytest.mark.parametrize("adt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32)])
def test_add_rmsnorm(H, adt, wdt):
    T, eps = 7, 1e-5
    h = rnd(T, H, seed=1)
    d = rnd(T, H, seed=2)
    w = (1 + rnd(H, seed=3) * 0.1).to(wdt)
    ref_h = h + d
    ref = pm.rms_norm(ref_h, w.float(), eps)
    h1 = h.clone()
    out = F().add_rmsnorm(h1, d, w, eps, adt)
    assert out.dtype == adt
    assert torch.allclose(h1, ref_h, atol=0, rtol=0)                          # residual written back exactly
    close(out, ref, 4e-6 if adt == torch.float32 else 8e-3, "add_rmsnorm")
    # without delta, hidden untouched
    h2 = h.clone()
    out2 = F().add_rmsnorm(h2, None, w, eps, adt)
    assert torch.equal(h2, h)
    close(out2, pm.rms_norm(h, w.float(), eps), 4e-6 if adt == torch.float32 else 8e-3)
    # with rows (one of them twice): hidden untouched, rows ordered as asked
    rows = torch.tensor([5, 0, 5, 3], dtype=torch.int32, device=DEV)
    h3 = h.clone()
    out3 = F().add_rmsnorm(h3, d, w, eps, adt, rows=rows)
    assert torch.equal(h3, h) and out3.shape == (4, H)
    close(out3, ref[rows.long()], 4e-6 if adt == torch.float32 else 8e-3)


@pytest.mark.parametrize("adt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,rot", [(5, 1, 24, 24), (4, 2, 64, 32), (3, 3, 16, 16), (2, 1, 128, 128),
                                          (7, 1, 48, 48)])
@pytest.mark.parametrize("T", [9, 70])          # a few tokens; many (one block per token, vector loads)
def test_qkv_post(adt, nh, nkv, d, rot, T):
    ps, pages = 4, 6 if T == 9 else 24
    width = (nh + 2 * nkv) * d
    qkv = rnd(T, width, seed=4)
    bias = rnd(width, seed=5).to(adt if adt == torch.bfloat16 else torch.float32)
    pos = torch.tensor(([0, 1, 2, 3, 17, 18, 400, 4000, 5] * 8)[:T], dtype=torch.int32, device=DEV)
    theta = 1e6
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)
    inv = inv.float().to(DEV)
    slots = torch.tensor(random.Random(0).sample(range(ps * pages), T), dtype=torch.int32, device=DEV)
    kc = torch.zeros(pages, nkv, ps, d, dtype=adt, device=DEV)
    vc = torch.zeros_like(kc)
    q = F().qkv_post(qkv, bias, pos, inv, rot, slots, kc, vc, nh, nkv, d, ps, adt)
    x = qkv + bias.float()
    xq = x[:, :nh * d].view(T, nh, d)
    xk = x[:, nh * d:(nh + nkv) * d].view(T, nkv, d)
    xv = x[:, (nh + nkv) * d:].view(T, nkv, d)

    def rope(t):
        a = pos.float()[:, None] * inv[None, :]
        c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
        h = rot // 2
        y = t.clone()
        y[..., :h] = t[..., :h] * c - t[..., h:rot] * s
        y[..., h:rot] = t[..., h:rot] * c + t[..., :h] * s
        return y
    tol = 3e-6 if adt == torch.float32 else 8e-3
    close(q, rope(xq), tol, "q")
    page, off = slots.long() // ps, slots.long() % ps
    close(kc[page, :, off, :], rope(xk), tol, "k cache")
    close(vc[page, :, off, :], xv, tol, "v cache")
    written = torch.zeros(pages * ps, dtype=torch.bool)
    written[slots.long().cpu()] = True
    flat = kc.permute(0, 2, 1, 3).reshape(pages * ps, -1).float().cpu()
    assert float(flat[~written].abs().max()) == 0.0                           # nothing else touched
    # queries only (a layer that reads another layer's cache), no rotation
    q2 = F().qkv_post(qkv[:, :nh * d].contiguous(), None, pos, None, 0, None, None, None, nh, 0, d, ps, adt)
    close(q2, qkv[:, :nh * d].view(T, nh, d), tol)


@pytest.mark.parametrize("adt", [torch.float32, torch.bfloat16])
def test_swiglu(adt):
    gu = rnd(13, 2 * 70, dtype=adt, scale=2.0)
    out = F().swiglu(gu)
    g, u = gu.float()[:, :70], gu.float()[:, 70:]
    close(out, g / (1 + torch.exp(-g)) * u, 1e-6 if adt == torch.float32 else 8e-3)


def test_moe_combine():
    T, K, H = 6, 3, 100
    y = rnd(T * K, H, seed=1)
    w = rnd(T, K, seed=2).abs()
    perm = torch.randperm(T * K, generator=torch.Generator().manual_seed(1)).to(torch.int32).to(DEV)
    shared = rnd(T, H, seed=3)
    gate = torch.sigmoid(rnd(T, seed=4))
    out = F().moe_combine(y, perm, w, shared, gate)
    ref = (w[:, :, None] * y[perm.long()].view(T, K, H)).sum(1) + gate[:, None] * shared
    close(out, ref, 2e-6)
    out2 = F().moe_combine(y, perm, w, None, None)
    close(out2, (w[:, :, None] * y[perm.long()].view(T, K, H)).sum(1), 2e-6)


@pytest.mark.parametrize("adt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("T,K,H", [(6, 3, 100), (9, 4, 2048), (5, 2, 3584), (3, 8, 8192), (4, 1, 1028)])
@pytest.mark.parametrize("indexed,with_extra", [(True, True), (False, True), (True, False)])
def test_combine_add_rmsnorm_is_the_two_kernels(adt, wdt, T, K, H, indexed, with_extra):
    """The fused kernel adds in the order of moe_combine followed by add_rmsnorm: same bits, in hidden
    and in the normalised rows, for whole steps and for selected rows."""
    y = rnd(T * K, H, seed=1)
    w = rnd(T, K, seed=2).abs()
    perm = torch.randperm(T * K, generator=torch.Generator().manual_seed(1)).to(torch.int32).to(DEV) if indexed else None
    shared = rnd(T, H, seed=3) if with_extra else None
    gate = torch.sigmoid(rnd(T, seed=4)) if with_extra else None
    nw = (1.0 + 0.1 * rnd(H, seed=5)).to(wdt)
    h0 = rnd(T, H, seed=6)
    h_ref, h_got = h0.clone(), h0.clone()
    ref = F().add_rmsnorm(h_ref, F().moe_combine(y, perm, w, shared, gate), nw, 1e-5, adt)
    got = F().combine_add_rmsnorm(h_got, y, perm, w, shared, gate, nw, 1e-5, adt)
    assert torch.equal(got, ref) and torch.equal(h_got, h_ref) and not torch.equal(h_got, h0)
    rows = torch.tensor([T - 1, 0, T - 1], dtype=torch.int32, device=DEV)
    h_ref, h_got = h0.clone(), h0.clone()
    ref = F().add_rmsnorm(h_ref, F().moe_combine(y, perm, w, shared, gate), nw, 1e-5, adt, rows)
    got = F().combine_add_rmsnorm(h_got, y, perm, w, shared, gate, nw, 1e-5, adt, rows)
    assert torch.equal(got, ref) and torch.equal(h_got, h0)


@pytest.mark.parametrize("T,N,K", [(1, 7, 5), (70, 130, 96), (333, 515, 200), (64, 64, 2048), (5, 151936, 72)])
def test_dense_float32_product_and_its_fixed_order(T, N, K):
    """The float32 path's dense product against a float64 product, and the property it exists for: a
    row's result is the same bits whether it is computed alone, among others, or at another place."""
    x, w = rnd(T, K, seed=T), rnd(N, K, seed=N, scale=0.1)
    out = F().dense_f32(x, w)
    ref = (x.double() @ w.double().T).float()
    close(out, ref, 2e-6, "dense_f32")
    alone = F().dense_f32(x[T - 1:].contiguous(), w)
    assert torch.equal(alone[0], out[T - 1])
    shifted = F().dense_f32(torch.cat([rnd(37, K, seed=1), x]), w)
    assert torch.equal(shifted[37:], out)


# --------------------------------------------------------------------------- #
# attention
# --------------------------------------------------------------------------- #

def paged_case(kv_lens, q_lens, nh, nkv, d, ps, adt, seed=0, shuffle=True, extra_pages=3, release_window=0):
    """Random K/V for whole sequences, packed into a paged cache with shuffled pages.  With
    ``release_window`` the pages that a window of that size has passed before this step (as the cache
    manager gives them back: page ``i`` once ``(i + 1) * ps <= kv_len - q_len - window + 1``) are marked -1
    in the table and filled with NaN, so that any read of them shows."""
    g = torch.Generator().manual_seed(seed)
    B = len(kv_lens)
    pages_per = [-(-n // ps) for n in kv_lens]
    total = sum(pages_per) + extra_pages
    order = list(range(total))
    if shuffle:
        random.Random(seed).shuffle(order)
    kc = torch.full((total, nkv, ps, d), 7.0, dtype=adt)          # poison: unused slots must not matter
    vc = torch.full((total, nkv, ps, d), -7.0, dtype=adt)
    max_pages = max(pages_per) + 1
    table = torch.full((B, max_pages), -1, dtype=torch.int32)
    seqs, qs = [], []
    nxt = 0
    for b, n in enumerate(kv_lens):
        k = torch.randn(n, nkv, d, generator=g).to(adt)
        v = torch.randn(n, nkv, d, generator=g).to(adt)
        q = torch.randn(n, nh, d, generator=g).to(adt)
        seqs.append((q, k, v))
        for i in range(pages_per[b]):
            p = order[nxt]
            nxt += 1
            table[b, i] = p
            lo, hi = i * ps, min(n, (i + 1) * ps)
            kc[p, :, :hi - lo] = k[lo:hi].transpose(0, 1)
            vc[p, :, :hi - lo] = v[lo:hi].transpose(0, 1)
        qs.append(q[n - q_lens[b]:])
        if release_window > 0:
            for i in range(pages_per[b]):
                if (i + 1) * ps <= n - q_lens[b] - release_window + 1:
                    kc[int(table[b, i])] = float("nan")
                    vc[int(table[b, i])] = float("nan")
                    table[b, i] = -1
    q_start = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    return {"q": torch.cat(qs).to(DEV), "kc": kc.to(DEV), "vc": vc.to(DEV), "table": table.to(DEV),
            "q_start": q_start.to(DEV), "kv_len": torch.tensor(kv_lens, dtype=torch.int32, device=DEV),
            "seqs": seqs, "q_lens": q_lens}


def plain_attention(case, window=0):
    outs = []
    for (q, k, v), ql in zip(case["seqs"], case["q_lens"]):
        o = pm.attention_scores_softmax_pv(q.float(), k.float(), v.float(), window)
        outs.append(o[len(q) - ql:])
    return torch.cat(outs)


@pytest.mark.parametrize("adt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d", [(6, 2, 16), (3, 3, 24), (4, 1, 40), (8, 2, 64), (2, 2, 128), (2, 1, 256),
                                      (5, 5, 80)])
def test_attention_tiled_ragged(adt, nh, nkv, d):
    case = paged_case(kv_lens=[1, 37, 130, 64, 16], q_lens=[1, 37, 50, 1, 2], nh=nh, nkv=nkv, d=d, ps=16,
                      adt=adt, seed=d)
    out = F().attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"], 50)
    close(out, plain_attention(case), 3e-6 if adt == torch.float32 else 1e-2, "attention")


@pytest.mark.parametrize("ps", [1, 4, 64])
@pytest.mark.parametrize("window", [0, 7, 16, 33])
def test_attention_tiled_windows_and_page_sizes(ps, window):
    case = paged_case(kv_lens=[70, 33, 5], q_lens=[70, 3, 1], nh=4, nkv=2, d=32, ps=ps, adt=torch.float32, seed=ps)
    out = F().attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"], 70,
                        window=window)
    close(out, plain_attention(case, window), 3e-6, f"window {window} page {ps}")


def test_attention_finds_a_far_key_and_respects_the_window_edge():
    """One key among hundreds is made to stand out; it must dominate exactly when it is visible."""
    n, d, ps = 400, 64, 16
    for adt in (torch.float32, torch.bfloat16):
        for far, window, visible in ((3, 0, True), (250, 150, True), (249, 150, False), (399, 1, True)):
            case = paged_case([n], [1], 2, 1, d, ps, adt, seed=far)
            q, k, v = case["seqs"][0]
            k[far] = q[n - 1, 0] * 4.0                              # aligned with the last query: a huge score
            v[far] = 50.0
            page, off = int(case["table"][0, far // ps]), far % ps
            case["kc"][page, :, off] = k[far].to(DEV)
            case["vc"][page, :, off] = v[far].to(DEV)
            out = F().attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"],
                                case["kv_len"], 1, window=window)
            ref = plain_attention(case, window)
            close(out, ref, 3e-6 if adt == torch.float32 else 1e-2, f"far key {far} window {window}")
            assert (float(out[0, 0].float().mean()) > 40.0) == visible
            if mi_decode_ok(d):
                po, pml, splits = decode_scratch(1, 2, n, d)
                out2 = F().decode_attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"],
                                            case["kv_len"], po, pml, splits, window=window)
                close(out2, ref, 3e-6 if adt == torch.float32 else 1e-2, f"decode far key {far}")


def mi_decode_ok(d):
    return F().decode_attention_supported(d)


def decode_scratch(B, nh, max_kv, d):
    splits = -(-max_kv // F().decode_split_size())
    return (torch.empty(B * nh * splits * d, dtype=torch.float32, device=DEV),
            torch.empty(B * nh * splits * 2, dtype=torch.float32, device=DEV), splits)


@pytest.mark.parametrize("adt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d", [(4, 2, 64), (3, 3, 128), (7, 1, 128), (2, 1, 256)])
@pytest.mark.parametrize("window", [0, 100, 5])
def test_decode_attention(adt, nh, nkv, d, window):
    # lengths around the splits' edges: a tail of up to a quarter of a split joins the split before it
    # (1030 = 2 x 512 + 6, 640 = 512 + 128, 161 = 128 + 33), and a window of 5 lies inside such a tail
    kv = [1, 255, 256, 257, 700, 1030, 16, 640, 641, 160, 161]
    case = paged_case(kv, [1] * len(kv), nh, nkv, d, 16, adt, seed=nh)
    po, pml, splits = decode_scratch(len(kv), nh, max(kv), d)
    out = F().decode_attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"],
                               po, pml, splits, window=window)
    ref = plain_attention(case, window)
    close(out, ref, 3e-6 if adt == torch.float32 else 1e-2, "decode attention")
    # a larger split budget than needed (as under a fixed launch shape) changes nothing
    po2, pml2, splits2 = decode_scratch(len(kv), nh, 4096, d)
    out2 = F().decode_attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"],
                                po2, pml2, splits2, window=window)
    assert torch.equal(out, out2)
    # smaller splits (used for one or two requests) agree within rounding
    for split in (128, 256):
        po3, pml3, _ = decode_scratch(len(kv), nh, 4 * 4096, d)
        out3 = F().decode_attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"],
                                    case["kv_len"], po3, pml3, -(-max(kv) // split), window=window, split=split)
        close(out3, ref, 3e-6 if adt == torch.float32 else 1e-2, f"decode attention, splits of {split}")
    tiled = F().attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"], 1,
                          window=window)
    close(out, tiled, 3e-6 if adt == torch.float32 else 1e-2, "decode vs tiled")


@pytest.mark.parametrize("nh,nkv,d", [(4, 2, 64), (2, 2, 128), (6, 1, 128)])
@pytest.mark.parametrize("ps,window", [(16, 0), (4, 0), (16, 70), (64, 130)])
def test_prefill_attention_tensor_cores(nh, nkv, d, ps, window):
    """The mma prefill kernel against the plain attention: portions with and without history, single
    tokens in the same batch, lengths around the 64-query and 64-key tiles."""
    kv = [1, 64, 65, 200, 333, 130, 17]
    ql = [1, 64, 2, 200, 63, 1, 17]
    case = paged_case(kv, ql, nh, nkv, d, ps, torch.bfloat16, seed=d + ps)
    out = F().prefill_attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"],
                                max(ql), window=window)
    ref = plain_attention(case, window)
    close(out, ref, 1e-2, "prefill attention")
    tiled = F().attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"], max(ql),
                          window=window)
    close(out, tiled, 1e-2, "prefill vs tiled")


@pytest.mark.parametrize("nh,nkv,d", [(2, 2, 128), (4, 2, 64), (6, 1, 128)])
@pytest.mark.parametrize("ps,window", [(16, 0), (8, 0), (16, 70), (64, 130), (64, 0), (32, 300)])
def test_prefill_attention_tcgen05(nh, nkv, d, ps, window):
    """The tcgen05 prefill kernel against the plain attention: portions with and without history,
    single tokens in the same batch, lengths around the 128-query and 128-key tiles."""
    assert F().prefill_attention_tc_supported(d, ps)
    kv = [1, 128, 129, 200, 333, 130, 17, 600]
    ql = [1, 128, 2, 200, 63, 1, 17, 600]
    case = paged_case(kv, ql, nh, nkv, d, ps, torch.bfloat16, seed=d + ps)
    out = F().prefill_attention_tc(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"],
                                   max(ql), window=window)
    F().check_tc_status()
    ref = plain_attention(case, window)
    close(out, ref, 1e-2, "prefill attention (tcgen05)")


@pytest.mark.parametrize("ps", [8, 16, 64])
@pytest.mark.parametrize("nh,nkv,d", [(4, 2, 64), (2, 1, 128)])
def test_fast_attention_kernels_skip_released_pages(ps, nh, nkv, d):
    """Behind a sliding window the cache manager gives pages back and the block table holds -1 there.  The
    released pages are full of NaN here: the split-KV decode kernel, the mma.sync prefill kernel and the
    tcgen05 prefill kernel (whose TMA loads skip such pages and count fewer bytes) must never read one.
    A window of 100 releases whole 64-key tiles of the longer histories."""
    window = 100
    kv = [700, 1030, 161, 90, 300, 1]
    case = paged_case(kv, [1] * len(kv), nh, nkv, d, ps, torch.bfloat16, seed=ps, release_window=window)
    assert int((case["table"] == -1).sum()) > 0 and bool(torch.isnan(case["kc"].float()).any())
    po, pml, splits = decode_scratch(len(kv), nh, max(kv), d)
    out = F().decode_attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"],
                               po, pml, splits, window=window)
    close(out, plain_attention(case, window), 1e-2, "decode attention over released pages")
    kv = [600, 333, 200, 130, 900, 64]
    ql = [63, 2, 200, 1, 130, 64]
    case = paged_case(kv, ql, nh, nkv, d, ps, torch.bfloat16, seed=ps + 1, release_window=window)
    assert int((case["table"][:, :2] == -1).sum()) > 0
    ref = plain_attention(case, window)
    out = F().prefill_attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"],
                                max(ql), window=window)
    close(out, ref, 1e-2, "mma.sync prefill attention over released pages")
    out = F().prefill_attention_tc(case["q"], case["kc"], case["vc"], case["table"], case["q_start"],
                                   case["kv_len"], max(ql), window=window)
    F().check_tc_status()
    close(out, ref, 1e-2, "tcgen05 prefill attention over released pages")
    tiled = F().attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"], max(ql),
                          window=window)
    close(tiled, ref, 1e-2, "tiled attention over released pages")


def test_prefill_attention_tcgen05_far_key_and_refusals():
    n, d, ps = 700, 128, 16
    for far, window, visible in ((5, 0, True), (440, 250, True), (439, 250, False)):
        case = paged_case([n], [60], 2, 1, d, ps, torch.bfloat16, seed=far)
        q, k, v = case["seqs"][0]
        k[far] = q[n - 11, 0] * 4.0                             # aligned with the query at position n - 11
        v[far] = 50.0
        page, off = int(case["table"][0, far // ps]), far % ps
        case["kc"][page, :, off] = k[far].to(DEV)
        case["vc"][page, :, off] = v[far].to(DEV)
        out = F().prefill_attention_tc(case["q"], case["kc"], case["vc"], case["table"], case["q_start"],
                                       case["kv_len"], 60, window=window)
        F().check_tc_status()
        close(out, plain_attention(case, window), 1e-2, f"far key {far}, window {window}")
        row = out[60 - 11, 0].float()
        assert (float(row.mean()) > 40.0) == visible
    assert not F().prefill_attention_tc_supported(128, 4)
    assert not F().prefill_attention_tc_supported(128, 128)
    assert not F().prefill_attention_tc_supported(96, 16)
    from mini_infer_b200.ops.library import KernelError
    case = paged_case([20], [20], 2, 1, 128, 4, torch.bfloat16)
    with pytest.raises(KernelError, match="not taken"):
        F().prefill_attention_tc(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"], 20)


def test_prefill_attention_far_key():
    n, d, ps = 700, 128, 16
    for far, window, visible in ((5, 0, True), (440, 250, True), (439, 250, False)):
        case = paged_case([n], [60], 2, 1, d, ps, torch.bfloat16, seed=far)
        q, k, v = case["seqs"][0]
        k[far] = q[n - 11, 0] * 4.0                             # aligned with the query at position n - 11
        v[far] = 50.0
        page, off = int(case["table"][0, far // ps]), far % ps
        case["kc"][page, :, off] = k[far].to(DEV)
        case["vc"][page, :, off] = v[far].to(DEV)
        out = F().prefill_attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"],
                                    60, window=window)
        close(out, plain_attention(case, window), 1e-2, f"far key {far} window {window}")
        row = 60 - 11                                            # the query at position n - 11
        want_visible = visible and (window == 0 or far > (n - 11) - window)
        assert (float(out[row, 0].float().mean()) > 40.0) == want_visible


def test_attention_refuses_bad_shapes():
    from mini_infer_b200.ops.library import KernelError
    case = paged_case([5], [1], 3, 2, 16, 16, torch.float32)
    with pytest.raises(KernelError, match="multiple"):
        F().attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"], 1)
    q = torch.zeros(1, 1, 300, device=DEV)
    kc = torch.zeros(case["kc"].shape[0], 1, 16, 300, device=DEV)      # as many pages as the table names
    with pytest.raises(KernelError, match="head_dim"):
        F().attention(q, kc, kc.clone(), case["table"], case["q_start"], case["kv_len"], 1)
    with pytest.raises(RuntimeError, match="CUDA only"):
        F().swiglu(torch.zeros(2, 4))


# --------------------------------------------------------------------------- #
# mixture of experts
# --------------------------------------------------------------------------- #

@pytest.mark.parametrize("adt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("E,K,norm", [(6, 3, False), (8, 2, True), (60, 4, False), (130, 8, True), (5, 1, True),
                                      (33, 32, False)])
def test_router(adt, wdt, E, K, norm):
    T, H = 19, 200
    x = rnd(T, H, dtype=adt, seed=E)
    wr = rnd(E, H, dtype=wdt, scale=0.3, seed=K)
    wsg = rnd(H, dtype=wdt, scale=0.2, seed=9)
    idx, w, gate, probs = F().moe_router(x, wr, wsg, K, norm, want_probs=True)
    rp, ri, rw = pm.route(x.float().cpu(), wr.float().cpu(), K, norm)
    close(probs, rp, 5e-6, "router probabilities")
    # where the reference's K-th and (K+1)-th probabilities are not within rounding, the choice is the same
    s = torch.sort(rp, dim=-1, descending=True).values
    clear = torch.ones(T, dtype=torch.bool)
    for k in range(min(K, E - 1)):
        clear &= (s[:, k] - s[:, k + 1]) > 2e-7
    assert clear.sum() >= (T // 2 if K <= 8 else 1)
    assert torch.equal(idx.cpu().long()[clear], ri[clear])
    close(w.cpu()[clear], rw[clear], 5e-6, "router weights")
    ref_gate = torch.sigmoid(x.float().cpu() @ wsg.float().cpu())
    close(gate, ref_gate, 5e-6, "shared gate")
    if norm:
        assert torch.allclose(w.sum(-1).cpu(), torch.ones(T), atol=1e-5)


@pytest.mark.parametrize("T,H", [(130, 224), (700, 96), (333, 200), (2050, 64)])
@pytest.mark.parametrize("E,K,gate", [(60, 4, True), (130, 8, False), (5, 2, True), (64, 3, True)])
def test_router_of_many_tokens_on_the_tensor_cores(T, H, E, K, gate):
    """bfloat16 steps of more than 128 tokens take the mma.sync logits kernel when H is a multiple of 32
    (H = 200 stays on the float kernel); both give the float logits of the plain router."""
    x = rnd(T, H, dtype=torch.bfloat16, seed=T)
    wr = rnd(E, H, dtype=torch.bfloat16, scale=0.05, seed=E)      # a flat softmax: the K best stay apart
    wsg = rnd(H, dtype=torch.bfloat16, scale=0.2, seed=9) if gate else None
    idx, w, g, probs = F().moe_router(x, wr, wsg, K, True, want_probs=True)
    rp, ri, rw = pm.route(x.float().cpu(), wr.float().cpu(), K, True)
    close(probs, rp, 5e-6, "router probabilities")
    s = torch.sort(rp, dim=-1, descending=True).values
    clear = torch.ones(T, dtype=torch.bool)
    for k in range(min(K, E - 1)):
        clear &= (s[:, k] - s[:, k + 1]) > 2e-7
    assert clear.sum() >= T // 2
    assert torch.equal(idx.cpu().long()[clear], ri[clear])
    close(w.cpu()[clear], rw[clear], 5e-6, "router weights")
    if gate:
        close(g, torch.sigmoid(x.float().cpu() @ wsg.float().cpu()), 5e-6, "shared gate")
    else:
        assert g is None
    # a token's logits do not depend on its neighbours in the step
    part = F().moe_router(x[129:].contiguous(), wr, wsg, K, True, want_probs=True)[3] if T - 129 > 128 else None
    if part is not None:
        assert torch.equal(part, probs[129:])


def test_router_ties_go_to_the_lowest_index():
    T, H, E = 4, 64, 10
    x = rnd(T, H)
    wr = rnd(E, H, scale=0.2)
    wr[7] = wr[2]
    wr[5] = wr[2]
    wr[2] *= 1.0
    idx, w, _, probs = F().moe_router(x, wr, None, 3, False, want_probs=True)
    for t in range(T):
        chosen = idx[t].tolist()
        for e in (5, 7):
            if e in chosen:
                assert 2 in chosen and chosen.index(2) < chosen.index(e)
        if 7 in chosen:
            assert 5 in chosen and chosen.index(5) < chosen.index(7)
        assert len(set(chosen)) == 3
    from mini_infer_b200.ops.library import KernelError
    with pytest.raises(KernelError, match="experts per token"):
        F().moe_router(x, wr, None, 11, False)


@pytest.mark.parametrize("T", [1, 5, 9, 17, 32])
@pytest.mark.parametrize("N,Kd", [(40, 96), (200, 64), (2048 + 24, 352), (6, 1024)])
def test_dense_skinny(T, N, Kd):
    x = rnd(T, Kd, dtype=torch.bfloat16, seed=T)
    w = rnd(N, Kd, dtype=torch.bfloat16, scale=0.2, seed=N)
    bias = rnd(N, seed=3)
    ref = x.float() @ w.float().t()
    close(F().dense_skinny(x, w), ref, 5e-6, "product")
    close(F().dense_skinny(x, w, bias), ref + bias, 5e-6, "product with bias")
    if N % 2 == 0:
        g, u = ref[:, :N // 2], ref[:, N // 2:]
        out = F().dense_skinny(x, w, swiglu_pair=True)
        assert out.dtype == torch.bfloat16
        close(out, g / (1 + torch.exp(-g)) * u, 8e-3, "SwiGLU pair")
    # the same row gives the same bits whatever stands beside it
    alone = F().dense_skinny(x[:1].contiguous(), w)
    assert torch.equal(alone[0], F().dense_skinny(x, w)[0])


def test_dense_skinny_refuses_what_it_cannot_take():
    from mini_infer_b200.ops.library import KernelError
    w = rnd(16, 40, dtype=torch.bfloat16)
    with pytest.raises(KernelError, match="multiple of 32"):
        F().dense_skinny(rnd(2, 40, dtype=torch.bfloat16), w)
    w = rnd(16, 64, dtype=torch.bfloat16)
    with pytest.raises(KernelError, match="rows"):
        F().dense_skinny(rnd(33, 64, dtype=torch.bfloat16), w)
    assert not F().dense_skinny_takes(rnd(33, 64, dtype=torch.bfloat16), w)
    assert not F().dense_skinny_takes(rnd(3, 64), rnd(16, 64))


@pytest.mark.parametrize("T", [1, 7, 12, 31])
@pytest.mark.parametrize("nh,nkv,d,H,rope", [(4, 2, 16, 64, True), (3, 1, 48, 96, True), (2, 2, 128, 256, True),
                                             (5, 1, 32, 160, False)])
def test_qkv_skinny_equals_product_and_post(T, nh, nkv, d, H, rope):
    ps, pages = 4, 12
    width = (nh + 2 * nkv) * d
    x = rnd(T, H, dtype=torch.bfloat16, seed=T)
    w = rnd(width, H, dtype=torch.bfloat16, scale=0.2, seed=d)
    bias = rnd(width, seed=5)
    pos = torch.tensor([0, 1, 2, 3, 17, 18, 400, 4000, 5] * 4, dtype=torch.int32, device=DEV)[:T].contiguous()
    inv = None
    if rope:
        inv = torch.pow(torch.tensor(1e6, dtype=torch.float64),
                        -2.0 * torch.arange(d // 2, dtype=torch.float64) / d).float().to(DEV)
    slots = torch.tensor(random.Random(1).sample(range(ps * pages), T), dtype=torch.int32, device=DEV)
    if T > 2:
        slots[2] = -1                                                          # a row that is not stored
    assert F().qkv_skinny_supported(H, d, d if rope else 0)
    kc = torch.zeros(pages, nkv, ps, d, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    q = F().qkv_skinny(x, w, bias, pos, inv, slots, kc, vc, nh, nkv, d, ps)
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(kc)
    qkv = x.float() @ w.float().t()
    q2 = F().qkv_post(qkv, bias, pos, inv, d if rope else 0, slots, kc2, vc2, nh, nkv, d, ps, torch.bfloat16)
    # float sums in another order, then one rounding to bfloat16: at most one step apart
    close(q, q2, 8e-3, "q")
    close(kc, kc2, 8e-3, "k cache")
    close(vc, vc2, 8e-3, "v cache")
    assert torch.equal(kc == 0, kc2 == 0) and torch.equal(vc == 0, vc2 == 0)   # the same places written


def test_qkv_skinny_refuses_partial_rotation():
    assert not F().qkv_skinny_supported(64, 32, 16)
    assert not F().qkv_skinny_supported(64, 24, 24)
    assert not F().qkv_skinny_supported(40, 32, 32)


@pytest.mark.parametrize("adt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("T,E,K,norm", [(1, 6, 3, False), (8, 60, 4, False), (19, 8, 2, True), (32, 130, 8, True),
                                        (128, 60, 4, False), (77, 9, 3, True)])
def test_route_small_equals_router_and_permute(adt, wdt, T, E, K, norm):
    H = 200
    x = rnd(T, H, dtype=adt, seed=E)
    wr = rnd(E, H, dtype=wdt, scale=0.3, seed=K)
    wsg = rnd(H, dtype=wdt, scale=0.2, seed=9)
    ticket = torch.zeros(1 + T, dtype=torch.int32, device=DEV)
    # the two-kernel router sums a logit in the same order for steps of up to 32 tokens
    parts = [F().moe_router(x[i:i + 32].contiguous(), wr, wsg, K, norm, want_probs=True) for i in range(0, T, 32)]
    idx, w, gate, probs = (torch.cat([p[j] for p in parts]) for j in range(4))
    offsets, sorted_token, inv_perm = F().moe_permute(idx, E)
    for _ in range(3):                                                         # the ticket is left at zero
        got = F().moe_route_small(x, wr, wsg, K, norm, ticket, want_probs=True)
        for a, b in zip(got, (idx, w, gate, probs, offsets, sorted_token, inv_perm)):
            assert torch.equal(a, b)
        assert int(ticket.abs().sum()) == 0
    got = F().moe_route_small(x, wr, None, K, norm, ticket)
    assert got[2] is None and torch.equal(got[0], idx) and torch.equal(got[6], inv_perm)
    got = F().moe_route_small(x, wr, wsg, K, norm, ticket, permute=False)
    assert got[4] is None and torch.equal(got[0], idx) and torch.equal(got[1], w) and torch.equal(got[2], gate)
    assert int(ticket.abs().sum()) == 0
    from mini_infer_b200.ops.library import KernelError
    with pytest.raises(KernelError, match="tokens"):
        n = F().route_small_max_tokens() + 1
        F().moe_route_small(rnd(n, H, dtype=adt), wr, wsg, K, norm, torch.zeros(1 + n, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("adt,wdt,ndt", [(torch.float32, torch.float32, torch.float32),
                                         (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                         (torch.bfloat16, torch.float32, torch.bfloat16),
                                         (torch.bfloat16, torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("T,H,E,K,gated,with_delta", [(1, 2048, 60, 4, True, True), (8, 2048, 60, 4, True, True),
                                                      (5, 104, 6, 3, False, True), (3, 3584, 64, 8, True, False),
                                                      (8, 8192, 9, 2, True, True), (2, 1028, 130, 8, False, True)])
def test_norm_and_route_in_one_launch(adt, wdt, ndt, T, H, E, K, gated, with_delta):
    """Residual addition, RMSNorm and routing of the smallest steps in one kernel against the separate
    kernels: the same residual stream; the same normalised rows bit for bit where the norm's own kernel
    adds in the same order (widths from 1024), within rounding otherwise; the routing of those rows."""
    hidden = rnd(T, H, seed=T)
    delta = rnd(T, H, seed=H) if with_delta else None
    nw = (1.0 + 0.1 * rnd(H, seed=5)).to(ndt)
    wr = rnd(E, H, dtype=wdt, scale=0.05, seed=K)
    wsg = rnd(H, dtype=wdt, scale=0.05, seed=9) if gated else None
    ticket = torch.zeros(1 + T, dtype=torch.int32, device=DEV)
    h_ref = hidden.clone()
    x_ref = F().add_rmsnorm(h_ref, delta, nw, 1e-5, adt)
    r_idx, r_w, r_gate, r_probs, _, _, _ = F().moe_route_small(x_ref, wr, wsg, K, True, ticket, want_probs=True, permute=False)
    for _ in range(2):
        h = hidden.clone()
        x, idx, w, gate, probs = F().moe_norm_route_small(h, delta, nw, 1e-5, adt, wr, wsg, K, True, want_probs=True)
        assert x.dtype == adt
        assert torch.equal(h, h_ref)
        if H >= 1024:
            assert torch.equal(x, x_ref)
        else:
            close(x, x_ref, 3e-6 if adt == torch.float32 else 8e-3, "normalised rows")
        close(probs, r_probs, 2e-5 if H >= 1024 else 2e-3, "router probabilities")
        s = torch.sort(r_probs, dim=-1, descending=True).values
        clear = torch.ones(T, dtype=torch.bool, device=DEV)
        for k in range(min(K, E - 1)):
            clear &= (s[:, k] - s[:, k + 1]) > (1e-5 if H >= 1024 else 1e-3)
        assert torch.equal(idx[clear], r_idx[clear])
        close(w[clear], r_w[clear], 2e-5 if H >= 1024 else 2e-3, "router weights")
        if gated:
            close(gate, r_gate, 2e-5 if H >= 1024 else 2e-3, "shared gate")
        else:
            assert gate is None
    from mini_infer_b200.ops.library import KernelError
    with pytest.raises(KernelError, match="multiple of 4"):
        F().moe_norm_route_small(rnd(2, 102), None, rnd(102), 1e-5, torch.float32, rnd(4, 102), None, 2, True)
    # a router whose rows do not fit the shared memory of a cluster's blocks is refused, and the question
    # that parts ask first says so
    assert F().norm_route_small_takes(H, E, gated, wdt)
    assert not F().norm_route_small_takes(8192, 512, True, torch.float32)
    assert not F().norm_route_small_takes(102, 4, False, torch.float32)
    with pytest.raises(KernelError, match="shared memory"):
        F().moe_norm_route_small(rnd(1, 8192), None, rnd(8192), 1e-5, torch.float32, rnd(512, 8192), None, 2, True)


@pytest.mark.parametrize("T,E,K", [(1, 8, 2), (37, 6, 3), (300, 60, 4), (2048, 60, 4), (5, 130, 8), (700, 9, 3),
                                   (2100, 7, 1), (4099, 60, 4), (3001, 130, 8), (513, 64, 8)])
def test_permute(T, E, K):
    g = torch.Generator().manual_seed(T)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    if K == 1:
        idx[idx == 3] = 4                                        # an expert nobody is routed to
    idx = idx.to(DEV)
    offsets, sorted_token, inv_perm = F().moe_permute(idx, E)
    flat = idx.flatten().cpu().long()
    counts = torch.bincount(flat, minlength=E)
    assert offsets.cpu().tolist() == [0] + counts.cumsum(0).tolist()
    order = torch.sort(flat, stable=True).indices                            # stable: token order inside an expert
    assert sorted_token.cpu().tolist() == (order // K).tolist()
    inv = torch.empty(T * K, dtype=torch.long)
    inv[order] = torch.arange(T * K)
    assert inv_perm.cpu().tolist() == inv.tolist()


@pytest.mark.parametrize("adt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,K,H,I", [(1, 8, 2, 64, 32), (45, 6, 3, 96, 48), (130, 12, 4, 200, 70), (9, 60, 4, 128, 24)])
def test_grouped_gemm_plain(adt, T, E, K, H, I):
    g = torch.Generator().manual_seed(E)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    offsets, sorted_token, inv_perm = F().moe_permute(idx, E)
    x = rnd(T, H, dtype=adt, seed=1)
    wgu = rnd(E, 2 * I, H, dtype=adt, scale=0.2, seed=2)
    wd = rnd(E, H, I, dtype=adt, scale=0.2, seed=3)
    act = F().grouped_gemm_plain(x, sorted_token, wgu, offsets, T * K, True, adt)
    xs = x.float()[sorted_token.long()]
    expert_of_row = torch.repeat_interleave(torch.arange(E, device=DEV), (offsets[1:] - offsets[:-1]).long())
    ref_act = torch.empty(T * K, I, device=DEV)
    for r in range(T * K):
        e = int(expert_of_row[r])
        gte = xs[r] @ wgu[e, :I].float().T
        up = xs[r] @ wgu[e, I:].float().T
        ref_act[r] = gte / (1 + torch.exp(-gte)) * up
    close(act, ref_act, 3e-6 if adt == torch.float32 else 1e-2, "gate/up product")
    y = F().grouped_gemm_plain(act, None, wd, offsets, T * K, False, torch.float32)
    ref_y = torch.stack([act[r].float() @ wd[int(expert_of_row[r])].float().T for r in range(T * K)])
    close(y, ref_y, 3e-6 if adt == torch.float32 else 1e-2, "down product")


@pytest.mark.parametrize("T,E,K,H,I", [(1, 8, 2, 64, 32), (8, 60, 4, 256, 96), (64, 12, 4, 128, 72), (37, 6, 3, 96, 40),
                                       (200, 5, 1, 64, 24)])
def test_grouped_gemm_skinny_equals_plain(T, E, K, H, I):
    """The decode-sized tensor-core product against the plain kernel: 0, 1, 8, 9, 16 and more rows
    per expert; feature counts that are no multiple of the 16-row tile."""
    g = torch.Generator().manual_seed(T + E)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    offsets, sorted_token, inv_perm = F().moe_permute(idx, E)
    x = rnd(T, H, dtype=torch.bfloat16, seed=1)
    wgu = rnd(E, 2 * I, H, dtype=torch.bfloat16, scale=0.2, seed=2)
    wd = rnd(E, H, I, dtype=torch.bfloat16, scale=0.2, seed=3)
    assert F().grouped_gemm_skinny_supported(H)
    act = F().grouped_gemm_skinny(x, sorted_token, wgu, offsets, T * K, True)
    ref = F().grouped_gemm_plain(x, sorted_token, wgu, offsets, T * K, True, torch.float32)
    close(act, ref, 6e-3, "gate/up product")
    if F().grouped_gemm_skinny_supported(I):
        y = F().grouped_gemm_skinny(act, None, wd, offsets, T * K, False)
        ref_y = F().grouped_gemm_plain(act, None, wd, offsets, T * K, False, torch.float32)
        close(y, ref_y, 2e-5, "down product")
    from mini_infer_b200.ops.library import KernelError
    with pytest.raises(KernelError, match="multiple of 32"):
        F().grouped_gemm_skinny(x[:, :48].contiguous(), sorted_token, wgu[:, :, :48].contiguous(), offsets, T * K, True)


@pytest.mark.parametrize("T,E,K,H,I", [(1, 8, 2, 64, 32), (8, 60, 4, 256, 96), (32, 12, 4, 128, 160), (19, 6, 3, 96, 64),
                                       (32, 5, 5, 64, 64), (128, 60, 4, 128, 64), (70, 3, 2, 64, 96),
                                       (3, 60, 4, 64, 32), (8, 300, 8, 64, 32), (2, 64, 8, 96, 64), (5, 130, 6, 64, 32)])
def test_grouped_gemm_skinny_by_pair_equals_sorted(T, E, K, H, I):
    # few pairs beside many experts (4 T K <= E) launch block rows only for the experts that were chosen;
    # with more than 32 pairs their list is found in several rounds
    g = torch.Generator().manual_seed(E + T)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    offsets, sorted_token, inv_perm = F().moe_permute(idx, E)
    x = rnd(T, H, dtype=torch.bfloat16, seed=1)
    w1 = rnd(E, 2 * I, H, dtype=torch.bfloat16, scale=0.2, seed=2)
    w2 = rnd(E, H, I, dtype=torch.bfloat16, scale=0.2, seed=3)
    act_sorted = F().grouped_gemm_skinny(x, sorted_token, w1, offsets, T * K, True)
    y_sorted = F().grouped_gemm_skinny(act_sorted, None, w2, offsets, T * K, False)
    act = F().grouped_gemm_skinny_pairs(x, idx, w1, True)
    y = F().grouped_gemm_skinny_pairs(act, idx, w2, False)
    if T > 8:
        # the same sums in the same order, only the rows stand elsewhere
        assert torch.equal(act, act_sorted[inv_perm.long()])
        assert torch.equal(y, y_sorted[inv_perm.long()])
    else:
        # the smallest steps split the inner dimension over the warps: float sums in another order
        close(act, act_sorted[inv_perm.long()], 8e-3, "activation")
        close(y, y_sorted[inv_perm.long()], 1e-2, "second product")
        e_of = idx.flatten().long()
        gu = torch.einsum("nh,nfh->nf", x.float()[torch.arange(T * K, device=DEV) // K], w1.float()[e_of])
        close(act, torch.nn.functional.silu(gu[:, :I]) * gu[:, I:], 8e-3, "activation against the plain formula")
    wts = rnd(T, K, seed=4).abs()
    assert torch.equal(F().moe_combine(y, None, wts, None, None),
                       F().moe_combine(y[inv_perm.long().argsort()].contiguous(), inv_perm, wts, None, None))
    from mini_infer_b200.ops.library import KernelError
    with pytest.raises(KernelError, match="tokens"):
        F().grouped_gemm_skinny_pairs(rnd(129, H, dtype=torch.bfloat16),
                                      torch.zeros(129, K, dtype=torch.int32, device=DEV), w1, True)


@pytest.mark.parametrize("T,E,K,H,I", [(300, 6, 3, 128, 64), (2048, 60, 4, 256, 192), (1000, 12, 2, 192, 320),
                                       (129, 4, 1, 64, 128), (512, 8, 8, 2048, 1408), (3000, 3, 1, 64, 192),
                                       (700, 5, 2, 128, 64)])
def test_grouped_gemm_tensor_core_equals_plain(T, E, K, H, I):
    """The tcgen05 grouped product, in each of its forms (one block per tile or persistent, row tiles
    of 128, 160 and 256), against the plain kernel: experts with 0, 1, 127, 128, 129 and thousands of
    rows; feature counts that are and are not multiples of the 128-column tile.  All forms add in the
    same order, so they agree to the bit."""
    g = torch.Generator().manual_seed(T + E)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    if E > 2 and K < E:
        idx[idx == 1] = 0 if K == 1 else idx[idx == 1]          # K == 1: expert 1 gets no rows at all
    idx = idx.to(DEV)
    offsets, sorted_token, inv_perm = F().moe_permute(idx, E)
    x = rnd(T, H, dtype=torch.bfloat16, seed=1)
    wgu = rnd(E, 2 * I, H, dtype=torch.bfloat16, scale=0.1, seed=2)
    wd = rnd(E, H, I, dtype=torch.bfloat16, scale=0.1, seed=3)
    assert F().grouped_gemm_tc_supported(H) and F().grouped_gemm_tc_supported(I)
    xs = F().gather_rows(x, sorted_token)
    assert torch.equal(xs, x[sorted_token.long()])
    ref = F().grouped_gemm_plain(x, sorted_token, wgu, offsets, T * K, True, torch.float32)
    first = None
    for form in (None,) + tuple(F().TC_FORMS):
        act = F().grouped_gemm_tc(xs, wgu, offsets, True, form)
        F().check_tc_status()
        close(act, ref, 6e-3, f"gate/up product, form {form}")
        y = F().grouped_gemm_tc(act, wd, offsets, False, form)
        F().check_tc_status()
        ref_y = F().grouped_gemm_plain(act, None, wd, offsets, T * K, False, torch.float32)
        close(y, ref_y, 2e-5, f"down product, form {form}")
        if first is None:
            first = (act, y)
        else:
            assert torch.equal(act, first[0]) and torch.equal(y, first[1]), form


def test_a_bounded_wait_that_runs_out_is_reported_and_the_next_call_is_right():
    """Every mbarrier wait of the tcgen05 kernels gives up after a bound instead of hanging the device.  The
    test makes one run out: the producer leaves out the loads of one k block and the waits get a short
    limit, so the MMA warp's wait for that data (or the epilogue's wait for the accumulators) ends, the
    kernel frees its tensor memory and returns by itself, and the status word names the wait.  The same
    call without the fault is then right: nothing was left behind."""
    from mini_infer_b200.ops.library import KernelError
    T, E, K, H, I = 96, 3, 2, 256, 64
    g = torch.Generator().manual_seed(3)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    offsets, sorted_token, _ = F().moe_permute(idx, E)
    x = rnd(T, H, dtype=torch.bfloat16, seed=1)
    wgu = rnd(E, 2 * I, H, dtype=torch.bfloat16, scale=0.1, seed=2)
    xs = F().gather_rows(x, sorted_token)
    ref = F().grouped_gemm_plain(x, sorted_token, wgu, offsets, T * K, True, torch.float32)
    F().check_tc_status()
    F().grouped_gemm_tc_inject_wait_fault(skip_k_block=1, wait_limit=20000)
    F().grouped_gemm_tc(xs, wgu, offsets, True, form=0)
    with pytest.raises(KernelError, match=r"a wait ran out \(code [23]"):
        F().check_tc_status()
    act = F().grouped_gemm_tc(xs, wgu, offsets, True, form=0)           # the fault held for one launch only
    F().check_tc_status()
    close(act, ref, 6e-3, "the call after the fault")


def test_grouped_gemm_tensor_core_refuses_what_it_cannot_take():
    from mini_infer_b200.ops.library import KernelError
    x = rnd(40, 64, dtype=torch.bfloat16)
    w = rnd(2, 32, 64, dtype=torch.bfloat16)
    offsets = torch.tensor([0, 15, 40], dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="no form"):
        F().grouped_gemm_tc(x, w, offsets, False, 7)
    with pytest.raises(KernelError, match="multiple of 64"):
        F().grouped_gemm_tc(rnd(40, 48, dtype=torch.bfloat16), rnd(2, 32, 48, dtype=torch.bfloat16), offsets, False)


# --------------------------------------------------------------------------- #
# sampling
# --------------------------------------------------------------------------- #

def test_greedy_rows_lowest_index_wins():
    V = 151_937                                                              # no power of two, not even
    logits = rnd(5, V)
    logits[1, 100] = 50.0
    logits[1, 99_000] = 50.0
    logits[2, V - 1] = 60.0
    logits[3, 0] = 60.0
    out = F().sample_rows(logits).cpu().tolist()
    ref = [pm.greedy(logits[r].cpu()) for r in range(5)]
    assert out == ref and out[1] == 100 and out[2] == V - 1 and out[3] == 0


@pytest.mark.parametrize("V", [301, 5000, 151_936])
def test_temperature_and_nucleus_rows(V):
    R = 24
    logits = rnd(R, V, scale=3.0, seed=V)
    temps = torch.tensor([0.0, 0.7, 1.0, 1.3] * 6)
    tops = torch.tensor([1.0] * 8 + [0.9] * 8 + [0.3] * 8)
    us = torch.tensor([pm.uniform_for(5, r, r) for r in range(R)], dtype=torch.float32)
    us[4], us[5] = 0.0, 0.99999994
    out = F().sample_rows(logits, temps.to(DEV), tops.to(DEV), us.to(DEV)).cpu().tolist()
    for r in range(R):
        ref = pm.sample(logits[r].cpu(), float(temps[r]), float(tops[r]), float(us[r]))
        if out[r] != ref:
            # Only a draw that lands within rounding of a boundary of the cumulative sum may fall on either
            # side of it: every boundary between the two tokens must lie within 1e-5 of the draw (so no mass
            # to speak of lies between them), and the engine's token must belong to the nucleus.
            cdf, keep = pm.nucleus_cdf(logits[r].cpu(), float(temps[r]), float(tops[r]))
            lo, hi = sorted((out[r], ref))
            draw = float(us[r]) * float(cdf[-1])
            assert bool(keep[out[r]]), (r, out[r], ref)
            assert float((cdf[lo:hi] - draw).abs().max()) < 1e-5 * float(cdf[-1]), (r, out[r], ref)


def test_sampling_frequencies_follow_the_distribution():
    logits = torch.tensor([[0.0, 1.0, 5.0, 2.0, 4.0]], device=DEV).repeat(4000, 1)
    us = torch.tensor([pm.uniform_for(9, 1, n) for n in range(4000)], dtype=torch.float32, device=DEV)
    t = torch.ones(4000, device=DEV)
    out = F().sample_rows(logits, t, torch.ones(4000, device=DEV), us)
    freq = torch.bincount(out.cpu().long(), minlength=5).float() / 4000
    assert float((freq - torch.softmax(logits[0].cpu(), -1)).abs().max()) < 0.03
    out2 = F().sample_rows(logits, t, torch.full((4000,), 0.8, device=DEV), us)   # nucleus {2, 4}
    assert set(out2.cpu().tolist()) == {2, 4}


# --------------------------------------------------------------------------- #
# debug mode: indices checked on the host before a kernel can follow them
# --------------------------------------------------------------------------- #

def test_debug_bounds_mode_names_the_bad_index(monkeypatch):
    """With the debug switch on, an index outside its buffer raises before the launch and names the tensor,
    the place and the value; nothing runs.  (No bad index ever reaches the device in this test.)"""
    from mini_infer_b200.ops.library import KernelError
    f = F()
    monkeypatch.setattr(f, "DEBUG_BOUNDS", True)
    table = rnd(50, 16)
    ids = torch.tensor([3, 49, 50], dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match=r"embed_gather ids: element 2 is 50, outside \[0, 50\)"):
        f.embed_gather(ids, table)
    case = paged_case([40, 9], [3, 1], 4, 2, 64, 8, torch.bfloat16)
    f.attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], case["kv_len"], 3)     # a good call passes
    bad = case["table"].clone()
    bad[0, 2] = case["kc"].shape[0]                                    # one past the last page
    with pytest.raises(KernelError, match="request 0 reads page entry 2"):
        f.attention(case["q"], case["kc"], case["vc"], bad, case["q_start"], case["kv_len"], 3)
    with pytest.raises(KernelError, match="request 0 reads page entry 2"):
        f.prefill_attention_tc(case["q"], case["kc"], case["vc"], bad, case["q_start"], case["kv_len"], 3)
    long = torch.tensor([40, 200], dtype=torch.int32, device=DEV)      # longer than the table can hold
    with pytest.raises(KernelError, match="request 1: kv_len 200"):
        f.attention(case["q"], case["kc"], case["vc"], case["table"], case["q_start"], long, 3)
    x = rnd(6, 64, dtype=torch.bfloat16)
    w = rnd(3, 32, 64, dtype=torch.bfloat16)
    off = torch.tensor([0, 4, 3, 6], dtype=torch.int32, device=DEV)    # not rising
    with pytest.raises(KernelError, match="do not rise from 0 to 6"):
        f.grouped_gemm_plain(x, None, w, off, 6, False, torch.float32)
    idx = torch.tensor([[0, 3]], dtype=torch.int32, device=DEV)        # expert 3 of 3
    with pytest.raises(KernelError, match="expert indices: element 1 is 3"):
        f.moe_permute(idx, 3)
    dec = paged_case([700], [1], 2, 1, 64, 16, torch.bfloat16)
    po, pml, _ = decode_scratch(1, 2, 700, 64)
    with pytest.raises(KernelError, match="1 splits of 512 keys cannot hold"):
        f.decode_attention(dec["q"], dec["kc"], dec["vc"], dec["table"], dec["q_start"], dec["kv_len"], po, pml, 1)
    assert f.debug_checks_run > 0


def test_dependent_launch_gives_the_same_bits():
    """A chain of decode-sized kernels launched as programmatic dependents of one another (each waits for
    the kernels before it at its first line), eagerly and replayed from a CUDA graph, against the same
    chain launched plainly."""
    T, H, N = 5, 1024, 640
    hidden0 = rnd(T, H, seed=1)
    delta = rnd(T, H, seed=2)
    nw = (1.0 + 0.1 * rnd(H, seed=3)).to(torch.bfloat16)
    w1 = rnd(N, H, dtype=torch.bfloat16, scale=0.05, seed=4)
    w2 = rnd(H, N, dtype=torch.bfloat16, scale=0.05, seed=5)

    def chain(hidden):
        x = F().add_rmsnorm(hidden, delta, nw, 1e-6, torch.bfloat16)
        y = F().dense_skinny(x, w1, None, False)
        z = F().dense_skinny(y.to(torch.bfloat16), w2, None, False)
        x2 = F().add_rmsnorm(hidden, z, nw, 1e-6, torch.bfloat16)
        return x2, F().sample_rows(F().dense_skinny(x2, w1, None, False))

    h = hidden0.clone()
    want_x, want_tok = chain(h)
    want_h = h.clone()
    with F().dependent_launch(True):
        h = hidden0.clone()
        got_x, got_tok = chain(h)
        torch.cuda.synchronize()
        assert torch.equal(got_x, want_x) and torch.equal(got_tok, want_tok) and torch.equal(h, want_h)
        static_h = hidden0.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            chain(static_h)                                     # warm-up outside the capture
            static_h.copy_(hidden0)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                gx, gt = chain(static_h)
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            static_h.copy_(hidden0)
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(gx, want_x) and torch.equal(gt, want_tok) and torch.equal(static_h, want_h)
