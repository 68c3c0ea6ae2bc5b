"""The entry point that allocates nothing, called through its exported C symbol.

``mi_attn_decode_noalloc`` is for callers of the library that cannot allocate device memory
(in a latency-critical loop where cudaMalloc's device synchronisation is not acceptable, under a
device-memory budget fixed at start-up, in a host without an allocator to hand scratch from): it keeps the decode kernel's per-split partials in an array built into the library.
The test loads the shared library with ctypes, calls the symbol directly, twice in a row on
different inputs (the array keeps the first call's contents), and compares each result with the
existing entry point ``mi_attn_decode`` given caller scratch, and with the plain attention of
``tests/plain_model.py`` over the keys and values unpacked from the pages.  It is collected last so that a run
that stops at the first failure has already run every other test, and it passes alone in a fresh
process as well.
"""

import ctypes
import random

import pytest
import torch

import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _lib():
    from mini_infer_b200.csrc.build import build
    lib = ctypes.CDLL(build())
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.mi_attn_decode_noalloc.argtypes = [P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, F, P]
    lib.mi_attn_decode_noalloc.restype = I
    lib.mi_attn_decode.argtypes = [P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P]
    lib.mi_attn_decode.restype = I
    lib.mi_attn_decode_noalloc_capacity.restype = ctypes.c_uint
    lib.mi_attn_decode_split_size.restype = I
    lib.mi_last_error.restype = ctypes.c_char_p
    return lib


def _case(seed, kv_lens, nh, nkv, d, ps, dtype):
    g = torch.Generator().manual_seed(seed)
    B = len(kv_lens)
    pages_per = [-(-n // ps) for n in kv_lens]
    total = sum(pages_per) + 2
    order = list(range(total))
    random.Random(seed).shuffle(order)
    kc = torch.randn(total, nkv, ps, d, generator=g).to(dtype)
    vc = torch.randn(total, nkv, ps, d, generator=g).to(dtype)
    table = torch.full((B, max(pages_per) + 1), -1, dtype=torch.int32)
    nxt = 0
    for b, n in enumerate(pages_per):
        for i in range(n):
            table[b, i] = order[nxt]
            nxt += 1
    q = torch.randn(B, nh, d, generator=g).to(dtype)
    return (q.to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV),
            torch.arange(B + 1, dtype=torch.int32, device=DEV), torch.tensor(kv_lens, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, 1), (torch.float32, 0)])
def test_no_alloc_entry_point_matches_the_existing_one_twice_in_a_row(dtype, code):
    lib = _lib()
    nh, nkv, d, ps = 4, 2, 128, 16
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    split = lib.mi_attn_decode_split_size()
    for seed, kv_lens in ((1, [700, 3, 256, 1025]), (2, [40, 513, 90, 300])):      # two calls in a row
        q, kc, vc, table, q_start, kv_len = _case(seed, kv_lens, nh, nkv, d, ps, dtype)
        B = len(kv_lens)
        splits = -(-max(kv_lens) // split)
        scale = d ** -0.5
        out_a = torch.zeros_like(q)
        out_b = torch.zeros_like(q)
        rc = lib.mi_attn_decode_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), code, table.data_ptr(),
                                        q_start.data_ptr(), kv_len.data_ptr(), out_a.data_ptr(), B, nh, nkv, d, ps,
                                        table.shape[1], splits, 0, scale, stream)
        assert rc == 0, lib.mi_last_error()
        part_o = torch.empty(B * nh * splits * d, dtype=torch.float32, device=DEV)
        part_ml = torch.empty(B * nh * splits * 2, dtype=torch.float32, device=DEV)
        rc = lib.mi_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), code, table.data_ptr(),
                                q_start.data_ptr(), kv_len.data_ptr(), out_b.data_ptr(), part_o.data_ptr(),
                                part_ml.data_ptr(), B, nh, nkv, d, ps, table.shape[1], splits, 0, scale, stream)
        assert rc == 0, lib.mi_last_error()
        torch.cuda.synchronize()
        err = float((out_a.float() - out_b.float()).abs().max())
        tol = (3e-6 if dtype == torch.float32 else 1e-2) * float(out_b.float().abs().max())
        assert err <= tol, f"call with seed {seed}: {err} > {tol}"
        assert float(out_a.float().abs().max()) > 0.0
        # and against the plain attention over the unpacked pages
        for b, n in enumerate(kv_lens):
            pages = table[b, :-(-n // ps)].long()
            k = kc[pages].float().transpose(1, 2).reshape(-1, nkv, d)[:n].cpu()      # [n, nkv, d]
            v = vc[pages].float().transpose(1, 2).reshape(-1, nkv, d)[:n].cpu()
            q_all = torch.zeros(n, nh, d)
            q_all[n - 1] = q[b].float().cpu()
            ref = pm.attention_scores_softmax_pv(q_all, k, v, 0)[n - 1]
            err = float((out_a[b].float().cpu() - ref).abs().max())
            assert err <= (3e-6 if dtype == torch.float32 else 1e-2) * float(ref.abs().max()), (seed, b, err)


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib = _lib()
    cap = lib.mi_attn_decode_noalloc_capacity()
    assert cap == 4 << 20
    q, kc, vc, table, q_start, kv_len = _case(3, [10, 10], 4, 2, 128, 16, torch.bfloat16)
    out = torch.zeros_like(q)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    too_many_splits = cap // (2 * 4 * 130 * 4) + 1
    rc = lib.mi_attn_decode_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), 1, table.data_ptr(),
                                    q_start.data_ptr(), kv_len.data_ptr(), out.data_ptr(), 2, 4, 2, 128, 16,
                                    table.shape[1], too_many_splits, 0, 0.1, stream)
    assert rc == -2
    assert b"built-in array holds" in lib.mi_last_error()
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0                       # nothing ran
