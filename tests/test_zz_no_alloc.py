"""The allocation-free decode attention entry point, called through its exported C symbol.

Some users of the library's C interface cannot allocate device memory while serving: they
gave all of it to their page pool at start-up, or they must not take the device-wide stall
that cudaMalloc and cudaFree cause.  ``tk_attention_decode_noalloc`` keeps the kernels'
scratch in a static device array inside the library instead.  This test calls it the way
such a user would (ctypes on the shared library, raw pointers, no PyTorch op in between)
and checks its output against the ordinary entry point, twice in a row, because the
second call finds the first call's leftovers in the shared array.

The file is named so that pytest collects it last.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _load():
    from tokamak_b200.csrc.build import ensure_built
    lib = ctypes.CDLL(str(ensure_built()))
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.tk_attention_decode_noalloc.argtypes = [P, P, P, P, P, P, P, P, P, P,
                                                I, I, I, I, I, I, I, I, I, I, F, P]
    lib.tk_attention_decode_noalloc.restype = I
    lib.tk_attention_decode_noalloc_capacity_floats.restype = ctypes.c_longlong
    lib.tk_noalloc_error_string.argtypes = [I]
    lib.tk_noalloc_error_string.restype = ctypes.c_char_p
    return lib


def _case(seed: int, kv_lens, hq=8, hkv=2, d=128, page=16):
    """Random queries and a paged cache with shuffled tables; unwritten cache slots are NaN."""
    gen = torch.Generator().manual_seed(seed)
    n = len(kv_lens)
    max_pages = max(-(-l // page) for l in kv_lens)
    num_pages = n * max_pages + 3
    table = torch.randperm(num_pages, generator=gen)[: n * max_pages].view(n, max_pages).to(torch.int32)
    kc = torch.full((num_pages, hkv, page, d), float("nan"), dtype=torch.bfloat16)
    vc = torch.full_like(kc, float("nan"))
    for r, l in enumerate(kv_lens):
        for p in range(l):
            pg = int(table[r, p // page])
            kc[pg, :, p % page] = torch.randn(hkv, d, generator=gen).bfloat16()
            vc[pg, :, p % page] = torch.randn(hkv, d, generator=gen).bfloat16()
    q = torch.randn(n, hq, d, generator=gen).bfloat16()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    # float64 attention written out here, so that the check leans on no other path of the engine
    truth = torch.zeros(n, hq, d, dtype=torch.float64)
    for r, l in enumerate(kv_lens):
        rows = [(int(table[r, p // page]), p % page) for p in range(l)]
        keys = torch.stack([kc[pg, :, o] for pg, o in rows]).double()       # [l, hkv, d]
        vals = torch.stack([vc[pg, :, o] for pg, o in rows]).double()
        for h in range(hq):
            scores = (keys[:, h // (hq // hkv)] @ q[r, h].double()) * d ** -0.5
            truth[r, h] = torch.softmax(scores, 0) @ vals[:, h // (hq // hkv)]
    return dict(truth=truth, q=q.to(DEV), kc=kc.to(DEV), vc=vc.to(DEV), table=table.to(DEV), items=i32(list(range(n))),
                positions=i32([l - 1 for l in kv_lens]), tok_req=i32(list(range(n))),
                req_slot=i32(list(range(n))), hq=hq, hkv=hkv, d=d, page=page, n=n,
                max_pages=max_pages, num_pages=num_pages)


def _call_noalloc(lib, c, n_splits, scale):
    out = torch.full_like(c["q"], float("nan"))
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    rc = lib.tk_attention_decode_noalloc(
        c["q"].data_ptr(), out.data_ptr(), c["kc"].data_ptr(), c["vc"].data_ptr(), c["items"].data_ptr(),
        c["positions"].data_ptr(), c["tok_req"].data_ptr(), c["req_slot"].data_ptr(),
        c["table"].data_ptr(), err.data_ptr(), c["n"], c["n"], c["hq"], c["hkv"], c["d"], c["page"],
        c["max_pages"], c["num_pages"], 0, n_splits, scale, torch.cuda.current_stream().cuda_stream)
    return rc, out, err


def _call_ordinary(c, n_splits, scale):
    from tokamak_b200.csrc import ops
    out = torch.full_like(c["q"], float("nan"))
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.attention_decode(c["q"], out, c["kc"], c["vc"], c["items"], c["positions"], c["tok_req"],
                         c["req_slot"], c["table"], err, scale=scale, window=None, n_splits=n_splits)
    return out, err


def test_noalloc_decode_matches_the_ordinary_entry_point_twice_in_a_row():
    lib = _load()
    assert lib.tk_attention_decode_noalloc_capacity_floats() == 1 << 20
    # first call: many splits, long contexts; second call: other shapes, fewer splits, so that
    # it reads a region of the array which the first call filled with other values; third call:
    # one split, which stores its result itself and uses neither array
    for seed, kv_lens, n_splits in ((1, [700, 1, 33, 2048], 9), (2, [90, 515, 16], 2), (4, [300, 40], 1)):
        c = _case(seed, kv_lens)
        scale = c["d"] ** -0.5
        rc, got, err = _call_noalloc(lib, c, n_splits, scale)
        assert rc == 0, lib.tk_noalloc_error_string(rc).decode()
        want, err2 = _call_ordinary(c, n_splits, scale)
        torch.cuda.synchronize()
        assert err.tolist()[0] == 0 and err2.tolist()[0] == 0
        assert torch.isfinite(got.float()).all()
        # the same kernel with the same order of sums: every bit agrees
        assert torch.equal(got, want)
        # and both are right: against float64 attention, within what bfloat16 outputs allow
        torch.testing.assert_close(got.double().cpu(), c["truth"], rtol=2e-2, atol=2e-2)


def test_noalloc_decode_rejects_what_does_not_fit():
    lib = _load()
    c = _case(3, [40, 40])
    # 2 items * 8 heads * n_splits * 130 floats > 2^20  for n_splits = 600
    rc, out, _ = _call_noalloc(lib, c, 600, 1.0)
    assert rc == -2
    assert b"more scratch" in lib.tk_noalloc_error_string(rc)
    torch.cuda.synchronize()
    assert torch.isnan(out.float()).all()          # nothing was launched
    # more (token, kv head) pairs than the library holds arrival counters for (4,096)
    # (2,100 tokens x 2 heads = 4,200), while the scratch would fit (2,100 * 2 * 2 * 66 floats)
    many = _case(5, [3] * 2100, hq=2, hkv=2, d=64)
    rc, out, _ = _call_noalloc(lib, many, 2, 1.0)
    assert rc == -2
    torch.cuda.synchronize()
    assert torch.isnan(out.float()).all()
    # with one split neither limit applies: the kernel needs no scratch and no counters
    rc, out, err = _call_noalloc(lib, many, 1, many["d"] ** -0.5)
    torch.cuda.synchronize()
    assert rc == 0 and err.tolist()[0] == 0
    torch.testing.assert_close(out.double().cpu(), many["truth"], rtol=2e-2, atol=2e-2)
