"""Each kernel alone against a plain PyTorch reference, at sizes other than the engine's."""

from __future__ import annotations

import math

import random

import pytest
import torch

from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def err_word():
    return torch.zeros(4, dtype=torch.int32, device=DEV)


# ----------------------------------------------------------------------------- small kernels

@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_gather_and_bad_token(dtype):
    from tokamak_b200.csrc import ops
    table = torch.randn(1000, 200, device=DEV).to(dtype)
    ids = torch.tensor([0, 999, 17, 17, 500], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 200, device=DEV)
    err = err_word()
    ops.embed_gather(table, ids, out, err)
    torch.testing.assert_close(out, table[ids.long()].float(), rtol=0, atol=0)
    assert err.tolist() == [0, 0, 0, 0]
    bad = torch.tensor([3, 1000], dtype=torch.int32, device=DEV)
    ops.embed_gather(table, bad, out[:2], err)
    assert err.tolist()[:3] == [1, 1, 1000] and out[1].abs().sum() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [80, 320, 4096, 5120])
def test_add_rmsnorm(dtype, hidden):
    from tokamak_b200.csrc import ops
    n, eps = 37, 1e-5
    resid = torch.randn(n, hidden, device=DEV) * 3
    delta = torch.randn(n, hidden, device=DEV).to(dtype)
    w = 1 + 0.1 * torch.randn(hidden, device=DEV)
    want_sum = resid.double() + delta.double()
    want = plain.rms_norm(want_sum, w.double(), eps)
    r = resid.clone()
    out = torch.empty(n, hidden, device=DEV, dtype=dtype)
    ops.add_rmsnorm(r, delta, w, out, eps)
    torch.testing.assert_close(r.double(), want_sum, rtol=1e-6, atol=1e-6)      # the sum is a 32-bit sum
    torch.testing.assert_close(out.double(), want, **tol(dtype))
    # without a pending branch, and on chosen rows only
    r2 = resid.clone()
    ops.add_rmsnorm(r2, None, w, out, eps)
    torch.testing.assert_close(out.double(), plain.rms_norm(resid.double(), w.double(), eps), **tol(dtype))
    assert torch.equal(r2, resid)
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32, device=DEV)
    out3 = torch.empty(4, hidden, device=DEV, dtype=dtype)
    r3 = resid.clone()
    ops.add_rmsnorm(r3, delta, w, out3, eps, rows)
    torch.testing.assert_close(out3.double(), want[rows.long()], **tol(dtype))
    assert torch.equal(r3, resid)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    from tokamak_b200.csrc import ops
    n, inter = 19, 333
    gu = (torch.randn(n, 2 * inter, device=DEV) * 4).to(dtype)
    out = torch.empty(n, inter, device=DEV, dtype=dtype)
    ops.swiglu(gu, out)
    g, u = gu[:, :inter].double(), gu[:, inter:].double()
    torch.testing.assert_close(out.double(), g * torch.sigmoid(g) * u, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter,block", [(192, 64), (320, 64), (45, 9), (96, 24)])
def test_swiglu_gate_and_up_in_blocks(dtype, inter, block):
    """Rows that hold ``block`` gate values, then the ``block`` up values of the same outputs."""
    from tokamak_b200.csrc import ops
    n = 7
    g = (torch.randn(n, inter, device=DEV) * 3).to(dtype)
    u = torch.randn(n, inter, device=DEV).to(dtype)
    gu = torch.stack((g.view(n, inter // block, block), u.view(n, inter // block, block)), dim=2).reshape(n, 2 * inter)
    out = torch.empty(n, inter, device=DEV, dtype=dtype)
    ops.swiglu(gu.contiguous(), out, block=block)
    torch.testing.assert_close(out.double(), g.double() * torch.sigmoid(g.double()) * u.double(), **tol(dtype))
    parts = torch.stack((0.25 * gu.float(), 0.75 * gu.float()))
    out2 = torch.empty_like(out)
    ops.swiglu(parts, out2, block=block)
    torch.testing.assert_close(out2.double(), out.double(), **tol(dtype))


@pytest.mark.parametrize("shape", [(3, 317, 96), (130, 70, 33), (1, 1, 1), (64, 64, 16), (65, 129, 1000)])
def test_gemm_f32_is_true_float32_and_row_independent(shape):
    from tokamak_b200.csrc import ops
    m, n, k = shape
    a = torch.randn(m, k, device=DEV)
    w = torch.randn(n, k, device=DEV)
    out = ops.gemm_f32(a, w)
    want = a.double() @ w.double().T
    torch.testing.assert_close(out.double(), want, rtol=1e-5, atol=1e-5 * math.sqrt(k))
    # a row's result does not depend on the other rows of the batch: bit-equal
    one = ops.gemm_f32(a[m // 2:m // 2 + 1].contiguous(), w)
    assert torch.equal(one[0], out[m // 2])


def test_gemm_f32_keeps_what_reduced_precision_would_lose():
    from tokamak_b200.csrc import ops
    a = torch.tensor([[1.0, 2.0 ** -12]], device=DEV)
    w = torch.tensor([[1.0, 1.0]], device=DEV)
    assert ops.gemm_f32(a, w).item() == 1.0 + 2.0 ** -12        # TF32 or bf16 operands would give 1.0


# ----------------------------------------------------------------------------- rope + cache write

def make_tables(n_reqs, max_pages, num_pages, seed):
    """A shuffled, non-monotonic assignment of distinct pages to request rows."""
    gen = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_pages, generator=gen)[: n_reqs * max_pages]
    return perm.view(n_reqs, max_pages).to(torch.int32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page", [(6, 2, 48, 8), (4, 4, 128, 16), (7, 1, 16, 4)])
def test_rope_kv_write(dtype, hq, hkv, d, page):
    from tokamak_b200.csrc import ops
    eps, theta = 1e-6, 1e6
    q_lens = [5, 1, 9]
    starts = [0, 40001, 13]                      # one request far out, to test the angle's accuracy
    n = sum(q_lens)
    max_pages = max((s + l + page - 1) // page for s, l in zip(starts, q_lens))
    num_pages = 3 * max_pages + 5
    table = torch.zeros(3, max_pages, dtype=torch.int32)
    gen = torch.Generator().manual_seed(0)
    free = torch.randperm(num_pages, generator=gen).tolist()
    positions, tok_req = [], []
    for r, (s, l) in enumerate(zip(starts, q_lens)):
        for p in range(s, s + l):
            positions.append(p); tok_req.append(r)
        for pi in range(s // page, (s + l - 1) // page + 1):
            table[r, pi] = free.pop()
    qkv = torch.randn(n, (hq + 2 * hkv) * d, device=DEV).to(dtype)
    qw = 1 + 0.1 * torch.randn(d, device=DEV)
    kw = 1 + 0.1 * torch.randn(d, device=DEV)
    inv_freq = (1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV)
    kc = torch.full((num_pages, hkv, page, d), float("nan"), device=DEV, dtype=dtype)
    vc = torch.full_like(kc, float("nan"))
    q_out = torch.empty(n, hq, d, device=DEV, dtype=dtype)
    err = err_word()
    pos_t = torch.tensor(positions, dtype=torch.int32, device=DEV)
    rot = ops.rope_table(pos_t, inv_freq)
    ops.rope_kv(qkv, q_out, kc, vc, pos_t, torch.tensor(tok_req, dtype=torch.int32, device=DEV),
                torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV), table.to(DEV), qw, kw, rot,
                err, n_q_heads=hq, n_kv_heads=hkv, head_dim=d, rotary_dim=d, eps=eps)
    assert err.tolist()[0] == 0
    x = qkv.double().cpu()
    q = x[:, : hq * d].view(n, hq, d)
    k = x[:, hq * d:(hq + hkv) * d].view(n, hkv, d)
    v = x[:, (hq + hkv) * d:].view(n, hkv, d)
    cos, sin = plain.rope_tables(torch.tensor(positions), d, theta, torch.float64)
    q_want = plain.apply_rope(plain.rms_norm(q, qw.double().cpu(), eps), cos, sin)
    k_want = plain.apply_rope(plain.rms_norm(k, kw.double().cpu(), eps), cos, sin)
    t = dict(rtol=3e-5, atol=3e-5) if dtype == torch.float32 else tol(dtype)
    torch.testing.assert_close(q_out.double().cpu(), q_want, **t)
    written = torch.zeros(num_pages, page, dtype=torch.bool)
    for i, (p, r) in enumerate(zip(positions, tok_req)):
        pg = int(table[r, p // page])
        torch.testing.assert_close(kc[pg, :, p % page].double().cpu(), k_want[i], **t)
        torch.testing.assert_close(vc[pg, :, p % page].double().cpu(), v[i], rtol=0, atol=0)
        written[pg, p % page] = True
    # nothing else was touched
    untouched = lambda c: c.float().cpu().permute(0, 2, 1, 3)[~written]
    assert torch.isnan(untouched(kc)).all() and torch.isnan(untouched(vc)).all()


def test_rope_kv_reports_a_page_outside_the_pool():
    from tokamak_b200.csrc import ops
    d = 16
    qkv = torch.randn(1, 3 * d, device=DEV)
    kc = torch.zeros(4, 1, 4, d, device=DEV); vc = torch.zeros_like(kc)
    err = err_word()
    one = lambda v: torch.tensor([v], dtype=torch.int32, device=DEV)
    ops.rope_kv(qkv, torch.empty(1, 1, d, device=DEV), kc, vc, one(2), one(0), one(0),
                torch.tensor([[9]], dtype=torch.int32, device=DEV), None, None, None, err,
                n_q_heads=1, n_kv_heads=1, head_dim=d, rotary_dim=0, eps=0.0)
    assert err.tolist()[0] == 2 and kc.abs().sum() == 0


# ----------------------------------------------------------------------------- attention

def attention_reference(q, k_all, v_all, positions, tok_req, scale, window):
    """float64 attention per token over its request's keys [lo, pos]."""
    n, hq, d = q.shape
    out = torch.zeros(n, hq, d, dtype=torch.float64)
    for t in range(n):
        r, pos = tok_req[t], positions[t]
        lo = max(0, pos - window + 1) if window else 0
        k = k_all[r][lo:pos + 1].double()        # [keys, hkv, d]
        v = v_all[r][lo:pos + 1].double()
        group = hq // k.shape[1]
        for h in range(hq):
            s = (k[:, h // group] @ q[t, h].double()) * scale
            out[t, h] = torch.softmax(s, 0) @ v[:, h // group]
    return out


def fill_cache(k_all, v_all, table, num_pages, page, dtype):
    hkv, d = k_all[0].shape[1:]
    kc = torch.full((num_pages, hkv, page, d), float("nan"), dtype=dtype)
    vc = torch.full_like(kc, float("nan"))
    for r, (k, v) in enumerate(zip(k_all, v_all)):
        for p in range(k.shape[0]):
            pg = int(table[r, p // page])
            kc[pg, :, p % page] = k[p].to(dtype)
            vc[pg, :, p % page] = v[p].to(dtype)
    return kc.to(DEV), vc.to(DEV)


def run_attention(fn, q, kc, vc, positions, tok_req, table, scale, window):
    err = err_word()
    out = torch.empty_like(q)
    n_reqs = table.shape[0]
    fn(q, out, kc, vc, torch.tensor(positions, dtype=torch.int32, device=DEV),
       torch.tensor(tok_req, dtype=torch.int32, device=DEV),
       torch.arange(n_reqs, dtype=torch.int32, device=DEV), table.to(DEV), err, scale=scale, window=window)
    assert err.tolist()[0] == 0
    return out


ATTN_SHAPES = [(4, 2, 16, 16, None), (6, 1, 32, 8, None), (5, 5, 48, 16, 24), (8, 2, 128, 16, None),
               (3, 3, 80, 4, 7), (32, 8, 128, 16, None), (2, 1, 256, 16, None)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page,window", ATTN_SHAPES)
def test_attention_mixed_batch(dtype, hq, hkv, d, page, window):
    """Portions, single tokens and a whole prompt in one batch over shuffled pages; pages
    that no request owns are NaN and must never be read."""
    from tokamak_b200.csrc import ops
    kv_lens = [37, 1, 150, 64, 3 * page + 1]
    q_lens = [37, 1, 1, 9, 2]                      # whole prompt, first token, decode, portion, two tokens
    max_pages = max(-(-l // page) for l in kv_lens)
    num_pages = len(kv_lens) * max_pages + 7
    table = make_tables(len(kv_lens), max_pages, num_pages, seed=d)
    gen = torch.Generator().manual_seed(d + hq)
    k_all = [torch.randn(l, hkv, d, generator=gen) for l in kv_lens]
    v_all = [torch.randn(l, hkv, d, generator=gen) for l in kv_lens]
    if dtype == torch.bfloat16:
        k_all = [k.bfloat16().float() for k in k_all]; v_all = [v.bfloat16().float() for v in v_all]
    kc, vc = fill_cache(k_all, v_all, table, num_pages, page, dtype)
    positions, tok_req = [], []
    for r, (kl, ql) in enumerate(zip(kv_lens, q_lens)):
        positions += list(range(kl - ql, kl)); tok_req += [r] * ql
    q = torch.randn(len(positions), hq, d, generator=gen).to(dtype)
    scale = d ** -0.5
    out = run_attention(ops.attention_plain, q.to(DEV), kc, vc, positions, tok_req, table, scale, window)
    want = attention_reference(q.float(), k_all, v_all, positions, tok_req, scale, window)
    torch.testing.assert_close(out.double().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("where", ["first", "far", "page_edge", "last", "window_edge", "just_outside"])
def test_attention_finds_the_one_key_that_matters(dtype, where):
    """One key among hundreds is made to dominate the softmax; the output must be its value.
    Random inputs would hide a key that is skipped at a page's edge or at the window's edge."""
    from tokamak_b200.csrc import ops
    hq, hkv, d, page = 4, 2, 64, 16
    kv_len, window = 700, None
    target = {"first": 0, "far": 123, "page_edge": 16 * 20 - 1, "last": kv_len - 1,
              "window_edge": kv_len - 100, "just_outside": kv_len - 101}[where]
    if where in ("window_edge", "just_outside"):
        window = 100
    gen = torch.Generator().manual_seed(3)
    k = torch.randn(kv_len, hkv, d, generator=gen) * 0.1
    v = torch.randn(kv_len, hkv, d, generator=gen)
    q = torch.randn(1, hq, d, generator=gen) * 0.1
    direction = torch.randn(d, generator=gen)
    direction /= direction.norm()
    q[0, :] += 40.0 * direction
    k[target, :] += 40.0 * direction
    if dtype == torch.bfloat16:
        k, v, q = k.bfloat16().float(), v.bfloat16().float(), q.bfloat16().float()
    max_pages = -(-kv_len // page)
    table = make_tables(1, max_pages, max_pages + 9, seed=1)
    kc, vc = fill_cache([k], [v], table, max_pages + 9, page, dtype)
    out = run_attention(ops.attention_plain, q.to(dtype).to(DEV), kc, vc, [kv_len - 1], [0], table,
                        1.0, window).double().cpu()
    want = attention_reference(q, [k], [v], [kv_len - 1], [0], 1.0, window)
    torch.testing.assert_close(out, want, **tol(dtype))
    group = hq // hkv
    hit = torch.stack([v[target, h // group] for h in range(hq)]).double()
    if where == "just_outside":
        assert (out[0] - hit).abs().max() > 0.1            # the key is outside the window: not seen
    else:
        torch.testing.assert_close(out[0], hit, rtol=5e-2, atol=5e-2)


# ----------------------------------------------------------------------------- sampling

def sample_rows(logits, temps, top_ks, top_ps, seeds, counters):
    from tokamak_b200.csrc import ops
    n = logits.shape[0]
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV).contiguous(), torch.tensor(temps, dtype=torch.float32, device=DEV),
               torch.tensor(top_ks, dtype=torch.int32, device=DEV),
               torch.tensor(top_ps, dtype=torch.float32, device=DEV),
               torch.tensor(seeds, dtype=torch.int64, device=DEV),
               torch.tensor(counters, dtype=torch.int32, device=DEV), out)
    return out.tolist()


def test_sample_greedy_takes_the_first_maximum():
    logits = torch.randn(6, 5003)
    logits[2, 77] = 50.0; logits[2, 4000] = 50.0
    logits[3, 5002] = 60.0
    got = sample_rows(logits, [0.0] * 6, [0] * 6, [1.0] * 6, [0] * 6, [0] * 6)
    assert got == logits.argmax(-1).tolist() and got[2] == 77 and got[3] == 5002


def test_philox_matches_the_plain_generator():
    from tokamak_b200.csrc import ops
    for seed, counter in [(0, 0), (1, 5), (2 ** 40 + 17, 123456), (2 ** 62 - 1, 2 ** 31)]:
        want = plain.philox4x32_10((counter, 0, 0, 0), (seed & 0xFFFFFFFF, seed >> 32))[0]
        assert ops.philox_u32(seed, counter) == want


@pytest.mark.parametrize("vocab", [317, 5003, 151936])
def test_sample_draws_match_the_plain_sampler(vocab):
    gen = torch.Generator().manual_seed(vocab)
    n = 48
    logits = torch.randn(n, vocab, generator=gen) * 3
    temps = [0.8 if i % 3 else 1.3 for i in range(n)]
    top_ks = [0, 50, 0, 7][0:4] * (n // 4)
    top_ps = [1.0, 1.0, 0.9, 0.5] * (n // 4)
    seeds = [1000 + i for i in range(n)]
    counters = [i * 3 for i in range(n)]
    got = sample_rows(logits, temps, top_ks, top_ps, seeds, counters)
    miss = 0
    for i in range(n):
        want = plain.sample_token(logits[i], temps[i], top_ks[i], top_ps[i], seeds[i], counters[i])
        probs = plain.filtered_probs(logits[i], temps[i], top_ks[i], top_ps[i])
        assert probs[got[i]] > 0, f"row {i}: token {got[i]} is outside the kept set"
        miss += got[i] != want
    assert miss == 0


@pytest.mark.parametrize("rows,vocab", [(1, 151936), (5, 151936), (20, 151936), (3, 40001), (12, 33000), (70, 20000)])
def test_sample_rows_shared_by_several_blocks(rows, vocab):
    """A row is shared by a cluster of 8, 4 or 2 blocks where the batch leaves SMs free (or by one block): the
    slices' maxima, histograms and sums meet in one block, and the token is the plain sampler's, whichever
    slice it lies in; greedy rows take the first maximum also when its like lies in another slice."""
    gen = torch.Generator().manual_seed(rows * 1000 + vocab)
    logits = torch.randn(rows, vocab, generator=gen) * 3
    temps = [[0.7, 1.0, 0.0, 1.4][i % 4] for i in range(rows)]
    top_ks = [[0, 40, 0, 0, 3][i % 5] for i in range(rows)]
    top_ps = [[1.0, 0.95, 1.0, 0.6, 1.0, 0.9][i % 6] for i in range(rows)]
    seeds = [77 + 13 * i for i in range(rows)]
    counters = [5 * i + 1 for i in range(rows)]
    for i in range(rows):
        if temps[i] == 0.0:          # two equal maxima far apart: the first one counts
            logits[i, vocab // 7] = 40.0
            logits[i, vocab - 3] = 40.0
    got = sample_rows(logits, temps, top_ks, top_ps, seeds, counters)
    for i in range(rows):
        if temps[i] == 0.0:
            assert got[i] == vocab // 7
            continue
        want = plain.sample_token(logits[i], temps[i], top_ks[i], top_ps[i], seeds[i], counters[i])
        assert got[i] == want, (i, got[i], want)
    # tokens drawn from all over the row: every slice gets to draw
    spread = sample_rows(logits[:1].repeat(64, 1) * 0.05, [1.0] * 64, [0] * 64, [1.0] * 64, list(range(64)), [0] * 64)
    assert len({t * 8 // vocab for t in spread}) >= 6


def test_sample_support_sets_and_distribution():
    """top-k and top-p keep the right sets; draws follow the probabilities."""
    vocab = 64
    logits = torch.linspace(4, -4, vocab)[None].repeat(4000, 1)
    seeds = list(range(4000))
    got_k = sample_rows(logits, [1.0] * 4000, [5] * 4000, [1.0] * 4000, seeds, [0] * 4000)
    assert set(got_k) == {0, 1, 2, 3, 4}
    probs = plain.filtered_probs(logits[0], 1.0, top_p=0.6)
    got_p = sample_rows(logits, [1.0] * 4000, [0] * 4000, [0.6] * 4000, seeds, [1] * 4000)
    assert set(got_p) == set(torch.nonzero(probs > 0).flatten().tolist())
    got = torch.tensor(sample_rows(logits, [1.0] * 4000, [0] * 4000, [1.0] * 4000, seeds, [2] * 4000))
    freq = torch.bincount(got, minlength=vocab).double() / 4000
    want = torch.softmax(logits[0].double(), 0)
    assert (freq - want).abs().max() < 0.03


# ----------------------------------------------------------------------------- split-K decode kernel

def run_decode(q, kc, vc, items, positions, tok_req, table, scale, window, n_splits):
    from tokamak_b200.csrc import ops
    err = err_word()
    out = torch.full_like(q, float("nan"))
    args = (q, out, kc, vc, torch.tensor(items, dtype=torch.int32, device=DEV),
            torch.tensor(positions, dtype=torch.int32, device=DEV),
            torch.tensor(tok_req, dtype=torch.int32, device=DEV),
            torch.arange(table.shape[0], dtype=torch.int32, device=DEV), table.to(DEV), err)
    if n_splits > 0:
        ops.attention_decode(*args, scale=scale, window=window, n_splits=n_splits)
    else:           # the kernel that deals the key tiles out evenly, over -n_splits blocks
        ops.attention_decode_balanced(*args, scale=scale, window=window, blocks=-n_splits)
    assert err.tolist()[0] == 0
    return out


@pytest.mark.parametrize("n_splits", [1, 3, 8, 33, -1, -2, -7, -37, -296, -512])
@pytest.mark.parametrize("hq,hkv,d,page,window", [(8, 2, 128, 16, None), (32, 8, 128, 16, None),
                                                    (6, 1, 64, 16, None), (16, 1, 64, 32, None),
                                                    (4, 4, 128, 16, 24), (14, 2, 64, 16, 7),
                                                    (5, 5, 128, 64, 100)])
def test_attention_decode_split_k(hq, hkv, d, page, window, n_splits):
    """Single next tokens at many lengths over shuffled pages; the last page of every request
    is only partly filled and everything unwritten is NaN, so a key beyond the end, or a page
    that the request does not own, shows as NaN in the result."""
    kv_lens = [1, 15, 16, 17, 700, 2041, 33]
    max_pages = max(-(-l // page) for l in kv_lens)
    num_pages = len(kv_lens) * max_pages + 5
    table = make_tables(len(kv_lens), max_pages, num_pages, seed=hq + d)
    gen = torch.Generator().manual_seed(hq * 7 + d)
    k_all = [torch.randn(l, hkv, d, generator=gen).bfloat16().float() for l in kv_lens]
    v_all = [torch.randn(l, hkv, d, generator=gen).bfloat16().float() for l in kv_lens]
    kc, vc = fill_cache(k_all, v_all, table, num_pages, page, torch.bfloat16)
    # the decoded tokens sit among other tokens of the batch: rows 1, 3, 5, ... of q
    n = 2 * len(kv_lens)
    items = [2 * r + 1 for r in range(len(kv_lens))]
    positions = [0] * n
    tok_req = [0] * n
    for r, l in enumerate(kv_lens):
        positions[2 * r + 1] = l - 1
        tok_req[2 * r + 1] = r
    q = torch.randn(n, hq, d, generator=gen).bfloat16()
    scale = d ** -0.5
    out = run_decode(q.to(DEV), kc, vc, items, positions, tok_req, table, scale, window, n_splits)
    want = attention_reference(q.float()[items], k_all, v_all, [positions[i] for i in items],
                               [tok_req[i] for i in items], scale, window)
    torch.testing.assert_close(out[items].double().cpu(), want, **tol(torch.bfloat16))
    assert torch.isnan(out[[i - 1 for i in items]].float()).all()       # other rows are not touched
    if n_splits < 0:
        # the counters are back at zero and the scratch may hold anything: a second call gives the same bits
        again = run_decode(q.to(DEV), kc, vc, items, positions, tok_req, table, scale, window, n_splits)
        assert torch.equal(again[items], out[items])


@pytest.mark.parametrize("where", ["first", "far", "page_edge", "last", "window_edge", "just_outside"])
def test_attention_decode_finds_the_one_key_that_matters(where):
    hq, hkv, d, page = 8, 2, 128, 16
    kv_len, window = 1500, None
    target = {"first": 0, "far": 123, "page_edge": 16 * 40 - 1, "last": kv_len - 1,
              "window_edge": kv_len - 200, "just_outside": kv_len - 201}[where]
    if where in ("window_edge", "just_outside"):
        window = 200
    gen = torch.Generator().manual_seed(11)
    k = torch.randn(kv_len, hkv, d, generator=gen) * 0.1
    v = torch.randn(kv_len, hkv, d, generator=gen)
    q = torch.randn(1, hq, d, generator=gen) * 0.1
    direction = torch.randn(d, generator=gen)
    direction /= direction.norm()
    q[0, :] += 40.0 * direction
    k[target, :] += 40.0 * direction
    k, v, q = k.bfloat16().float(), v.bfloat16().float(), q.bfloat16().float()
    max_pages = -(-kv_len // page)
    table = make_tables(1, max_pages, max_pages + 9, seed=2)
    kc, vc = fill_cache([k], [v], table, max_pages + 9, page, torch.bfloat16)
    want = attention_reference(q, [k], [v], [kv_len - 1], [0], 1.0, window)
    for n_splits in (-11, 5):       # the kernel that deals the tiles out evenly (11 blocks), the one with 5 splits
        out = run_decode(q.bfloat16().to(DEV), kc, vc, [0], [kv_len - 1], [0], table, 1.0, window,
                         n_splits=n_splits).double().cpu()
        torch.testing.assert_close(out, want, **tol(torch.bfloat16))
    hit = torch.stack([v[target, h // (hq // hkv)] for h in range(hq)]).double()
    if where == "just_outside":
        assert (out[0] - hit).abs().max() > 0.1
    else:
        torch.testing.assert_close(out[0], hit, rtol=5e-2, atol=5e-2)


# ----------------------------------------------------------------------------- flash prefill kernels

def zero_rest_of_last_pages(kc, vc, table, kv_lens, page):
    """What the cache-writing kernel guarantees to kernels that load whole pages: behind a
    request's last position its page holds zeros, never stale values."""
    for r, l in enumerate(kv_lens):
        if l % page:
            pg = int(table[r, (l - 1) // page])
            kc[pg, :, l % page:] = 0
            vc[pg, :, l % page:] = 0


def run_prefill(kernel, q, out, kc, vc, q_lens, kv_lens, q_start, table, scale, window):
    """kernel: "mma" (mma.sync, 64-token tiles), "tc" (tcgen05, the work list balanced for this
    device) or "tc_parts" (the same with every block of tokens cut into as many parts as allowed)."""
    from tokamak_b200.csrc import ops
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    err = err_word()
    slots = list(range(len(q_lens)))
    if kernel == "mma":
        tiles = [(r, t) for r in range(len(q_lens)) for t in range(-(-q_lens[r] // 64))][::-1]
        ops.attention_prefill(q, out, kc, vc, i32([x for rt in tiles for x in rt]), i32(q_start), i32(q_lens),
                              i32(kv_lens), i32(slots), table.to(DEV), err, scale=scale, window=window)
    else:
        sms = ops.sm_count(torch.device(DEV)) if kernel == "tc" else 1 << 20
        records, n_parts, n_split = ops.prefill_tc_records(q_start, q_lens, kv_lens, slots, heads=q.shape[1], sms=sms)
        if kernel == "tc_parts":
            assert n_split > 0 or max(kv_lens) < 2 * ops.PREFILL_TC_MIN_PART * ops.PREFILL_TC_KEYS
        items = ops.PrefillItems(torch.from_numpy(records).to(DEV), n_parts, n_split)
        ops.attention_prefill_tc(q, out, kc, vc, items, table.to(DEV), err, scale=scale, window=window)
    torch.cuda.synchronize()
    assert err.tolist()[0] == 0, err.tolist()


@pytest.mark.parametrize("kernel", ["mma", "tc", "tc_parts"])
@pytest.mark.parametrize("hq,hkv,d,page,window", [(8, 2, 128, 16, None), (4, 4, 64, 16, None),
                                                    (6, 1, 64, 8, None), (8, 8, 128, 32, 50),
                                                    (3, 1, 128, 16, 200), (10, 5, 64, 4, 9),
                                                    (4, 2, 128, 64, None), (2, 1, 64, 128, 300)])
def test_attention_prefill_portions(kernel, hq, hkv, d, page, window):
    """Whole prompts and portions that continue a request, with lengths around the tile sizes
    and the page edges; cache slots that no request has written are NaN."""
    from tokamak_b200.csrc import ops
    if kernel != "mma" and not ops.prefill_tc_kernel_takes(hq, hkv, d, page):
        pytest.skip("page size not taken by the tcgen05 kernel")
    kv_lens = [2, 64, 65, 300, 129, 1000, 47, 256, 385, 1500]
    q_lens = [2, 64, 65, 37, 128, 130, 3, 256, 129, 700]      # whole prompts and portions
    n_reqs = len(kv_lens)
    max_pages = max(-(-l // page) for l in kv_lens)
    num_pages = n_reqs * max_pages + 5
    table = make_tables(n_reqs, max_pages, num_pages, seed=d + hq)
    gen = torch.Generator().manual_seed(5 * hq + d)
    k_all = [torch.randn(l, hkv, d, generator=gen).bfloat16().float() for l in kv_lens]
    v_all = [torch.randn(l, hkv, d, generator=gen).bfloat16().float() for l in kv_lens]
    kc, vc = fill_cache(k_all, v_all, table, num_pages, page, torch.bfloat16)
    if kernel != "mma":
        zero_rest_of_last_pages(kc, vc, table, kv_lens, page)
    positions, tok_req, q_start = [], [], []
    for r, (kl, ql) in enumerate(zip(kv_lens, q_lens)):
        q_start.append(len(positions))
        positions += list(range(kl - ql, kl)); tok_req += [r] * ql
    n = len(positions)
    q = torch.randn(n, hq, d, generator=gen).bfloat16()
    out = torch.full_like(q, float("nan")).to(DEV)
    scale = d ** -0.5
    run_prefill(kernel, q.to(DEV), out, kc, vc, q_lens, kv_lens, q_start, table, scale, window)
    want = attention_reference(q.float(), k_all, v_all, positions, tok_req, scale, window)
    torch.testing.assert_close(out.double().cpu(), want, **tol(torch.bfloat16))


def causal_attention_float64(q, k, v, first_pos, scale, window):
    """float64 attention of a request's new tokens (positions first_pos ..) over its keys, all heads at once."""
    n, hq, d = q.shape
    group = hq // k.shape[1]
    kk = k.double().repeat_interleave(group, dim=1)          # [keys, hq, d]
    vv = v.double().repeat_interleave(group, dim=1)
    s = torch.einsum("nhd,khd->hnk", q.double(), kk) * scale
    pos = torch.arange(first_pos, first_pos + n).view(1, n, 1)
    key = torch.arange(k.shape[0]).view(1, 1, -1)
    mask = key <= pos
    if window:
        mask = mask & (key >= pos - window + 1)
    s = s.masked_fill(~mask, float("-inf"))
    return torch.einsum("hnk,khd->nhd", torch.softmax(s, dim=-1), vv)


@pytest.mark.parametrize("kernel", ["tc", "tc_parts"])
@pytest.mark.parametrize("hq,hkv,d,page,window", [(16, 4, 64, 16, None), (16, 16, 128, 32, 300)])
def test_attention_prefill_more_items_than_blocks(kernel, hq, hkv, d, page, window):
    """The persistent kernel with two to three items per block: items run on into each other (the
    queries' second buffer, the ring and the score buffers carry over), are dealt out by the
    counter, and, cut into parts, are added up by parts that other blocks ran."""
    from tokamak_b200.csrc import ops
    q_lens = [1024, 1000, 700, 1024, 515, 900]
    kv_lens = [q + extra for q, extra in zip(q_lens, [0, 300, 0, 1024, 77, 0])]
    n_reqs = len(q_lens)
    assert sum(-(-q // ops.PREFILL_TC_ROWS) for q in q_lens) * hq > 2 * ops.sm_count(torch.device(DEV))
    max_pages = max(-(-l // page) for l in kv_lens)
    num_pages = n_reqs * max_pages + 3
    table = make_tables(n_reqs, max_pages, num_pages, seed=7 + hq)
    gen = torch.Generator().manual_seed(11 * hq + d)
    k_all = [torch.randn(l, hkv, d, generator=gen).bfloat16().float() for l in kv_lens]
    v_all = [torch.randn(l, hkv, d, generator=gen).bfloat16().float() for l in kv_lens]
    kc = torch.full((num_pages, hkv, page, d), float("nan"), dtype=torch.bfloat16)
    vc = torch.full_like(kc, float("nan"))
    for r in range(n_reqs):                      # whole pages at a time
        for pg in range(-(-kv_lens[r] // page)):
            rows = slice(pg * page, min((pg + 1) * page, kv_lens[r]))
            kc[int(table[r, pg]), :, :rows.stop - rows.start] = k_all[r][rows].transpose(0, 1).bfloat16()
            vc[int(table[r, pg]), :, :rows.stop - rows.start] = v_all[r][rows].transpose(0, 1).bfloat16()
    kc, vc = kc.to(DEV), vc.to(DEV)
    zero_rest_of_last_pages(kc, vc, table, kv_lens, page)
    q_start = [sum(q_lens[:r]) for r in range(n_reqs)]
    q = torch.randn(sum(q_lens), hq, d, generator=gen).bfloat16()
    out = torch.full_like(q, float("nan")).to(DEV)
    scale = d ** -0.5
    for _ in range(2):                           # the second call finds the counters as the first left them
        out.fill_(float("nan"))
        run_prefill(kernel, q.to(DEV), out, kc, vc, q_lens, kv_lens, q_start, table, scale, window)
    got = out.double().cpu()
    for r in range(n_reqs):
        want = causal_attention_float64(q[q_start[r]:q_start[r] + q_lens[r]].float(), k_all[r], v_all[r],
                                        kv_lens[r] - q_lens[r], scale, window)
        torch.testing.assert_close(got[q_start[r]:q_start[r] + q_lens[r]], want, **tol(torch.bfloat16))


@pytest.mark.parametrize("seed", range(24))
def test_attention_prefill_random_batches(seed):
    """Random batches of whole prompts and portions, head counts, head sizes, page sizes and windows
    through the tcgen05 kernel, with the work list as the engine makes it and with every block of
    tokens cut into parts."""
    from tokamak_b200.csrc import ops
    rng = random.Random(100 + seed)
    hq, hkv = rng.choice([(4, 2), (8, 1), (6, 6), (5, 5), (16, 4)])
    d = rng.choice([64, 128])
    page = rng.choice([8, 16, 32, 64, 128])
    window = rng.choice([None, None, 37, 300, 1000])
    n_reqs = rng.randint(1, 5)
    q_lens = [rng.choice([2, 3, 63, 64, 65, 127, 128, 129, 255, 256, 257, rng.randint(2, 900)]) for _ in range(n_reqs)]
    kv_lens = [q + rng.choice([0, 0, 1, 63, 64, 200, rng.randint(0, 1500)]) for q in q_lens]
    max_pages = max(-(-l // page) for l in kv_lens)
    num_pages = n_reqs * max_pages + 2
    table = make_tables(n_reqs, max_pages, num_pages, seed=seed)
    gen = torch.Generator().manual_seed(seed)
    k_all = [torch.randn(l, hkv, d, generator=gen).bfloat16().float() for l in kv_lens]
    v_all = [torch.randn(l, hkv, d, generator=gen).bfloat16().float() for l in kv_lens]
    kc = torch.full((num_pages, hkv, page, d), float("nan"), dtype=torch.bfloat16)
    vc = torch.full_like(kc, float("nan"))
    for r in range(n_reqs):
        for pg in range(-(-kv_lens[r] // page)):
            rows = slice(pg * page, min((pg + 1) * page, kv_lens[r]))
            kc[int(table[r, pg]), :, :rows.stop - rows.start] = k_all[r][rows].transpose(0, 1).bfloat16()
            vc[int(table[r, pg]), :, :rows.stop - rows.start] = v_all[r][rows].transpose(0, 1).bfloat16()
    kc, vc = kc.to(DEV), vc.to(DEV)
    zero_rest_of_last_pages(kc, vc, table, kv_lens, page)
    q_start = [sum(q_lens[:r]) for r in range(n_reqs)]
    q = torch.randn(sum(q_lens), hq, d, generator=gen).bfloat16()
    scale = d ** -0.5
    want = [causal_attention_float64(q[q_start[r]:q_start[r] + q_lens[r]].float(), k_all[r], v_all[r],
                                     kv_lens[r] - q_lens[r], scale, window) for r in range(n_reqs)]
    for kernel in ("tc", "tc_parts"):
        if kernel == "tc_parts" and max(kv_lens) < 2 * ops.PREFILL_TC_MIN_PART * ops.PREFILL_TC_KEYS:
            continue
        out = torch.full_like(q, float("nan")).to(DEV)
        run_prefill(kernel, q.to(DEV), out, kc, vc, q_lens, kv_lens, q_start, table, scale, window)
        got = out.double().cpu()
        for r in range(n_reqs):
            torch.testing.assert_close(got[q_start[r]:q_start[r] + q_lens[r]], want[r], **tol(torch.bfloat16))


@pytest.mark.parametrize("kernel", ["mma", "tc", "tc_parts"])
@pytest.mark.parametrize("where", ["first", "far", "page_edge", "diagonal", "window_edge", "just_outside"])
def test_attention_prefill_finds_the_one_key_that_matters(kernel, where):
    """The last query of a 100-token portion at the end of 1,300 tokens must find one key."""
    hq, hkv, d, page = 4, 2, 128, 16
    kv_len, q_len, window = 1300, 100, None
    target = {"first": 0, "far": 123, "page_edge": 16 * 30 - 1, "diagonal": kv_len - 1,
              "window_edge": kv_len - 300, "just_outside": kv_len - 301}[where]
    if where in ("window_edge", "just_outside"):
        window = 300
    gen = torch.Generator().manual_seed(21)
    k = torch.randn(kv_len, hkv, d, generator=gen) * 0.1
    v = torch.randn(kv_len, hkv, d, generator=gen)
    q = torch.randn(q_len, hq, d, generator=gen) * 0.1
    direction = torch.randn(d, generator=gen)
    direction /= direction.norm()
    q[-1, :] += 40.0 * direction
    k[target, :] += 40.0 * direction
    k, v, q = k.bfloat16().float(), v.bfloat16().float(), q.bfloat16().float()
    max_pages = -(-kv_len // page)
    table = make_tables(1, max_pages, max_pages + 9, seed=4)
    kc, vc = fill_cache([k], [v], table, max_pages + 9, page, torch.bfloat16)
    if kernel != "mma":
        zero_rest_of_last_pages(kc, vc, table, [kv_len], page)
    out = torch.empty(q_len, hq, d, dtype=torch.bfloat16, device=DEV)
    run_prefill(kernel, q.bfloat16().to(DEV), out, kc, vc, [q_len], [kv_len], [0], table, 1.0, window)
    positions = list(range(kv_len - q_len, kv_len))
    want = attention_reference(q, [k], [v], positions, [0] * q_len, 1.0, window)
    out = out.double().cpu()
    torch.testing.assert_close(out, want, **tol(torch.bfloat16))
    hit = torch.stack([v[target, h // (hq // hkv)] for h in range(hq)]).double()
    if where == "just_outside":
        assert (out[-1] - hit).abs().max() > 0.1
    else:
        torch.testing.assert_close(out[-1], hit, rtol=5e-2, atol=5e-2)


def test_rope_kv_clears_the_rest_of_a_page_begun_in_this_step():
    from tokamak_b200.csrc import ops
    hq, hkv, d, page = 2, 2, 16, 8
    # request 0 brings 11 tokens from position 0 (pages 0 and 1 begun now: slots 3.. of page 1 cleared);
    # request 1 brings 2 tokens at positions 9, 10 (its page was begun earlier: nothing cleared)
    q_lens, kv_lens = [11, 2], [11, 11]
    positions = list(range(11)) + [9, 10]
    tok_req = [0] * 11 + [1] * 2
    table = torch.tensor([[3, 1], [0, 2]], dtype=torch.int32)
    qkv = torch.randn(13, (hq + 2 * hkv) * d, device=DEV)
    kc = torch.full((4, hkv, page, d), 7.0, device=DEV)
    vc = torch.full_like(kc, 7.0)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    err = err_word()
    ops.rope_kv(qkv, torch.empty(13, hq, d, device=DEV), kc, vc, i32(positions), i32(tok_req), i32([0, 1]),
                table.to(DEV), None, None, None, err, n_q_heads=hq, n_kv_heads=hkv, head_dim=d, rotary_dim=0,
                eps=0.0, req_q_len=i32(q_lens), req_kv_len=i32(kv_lens))
    assert err.tolist()[0] == 0
    assert (vc[1, :, 3:] == 0).all() and (kc[1, :, 3:] == 0).all()        # request 0, page 1, slots 3..7
    assert (vc[2, :, 3:] == 7).all() and (vc[2, :, :1] == 7).all()        # request 1: untouched around its tokens
    assert (vc[3] != 7).all() and (vc[0] == 7).all()


# ----------------------------------------------------------------------------- tcgen05 matrix product

@pytest.mark.parametrize("tokens,n_out,k,splits,cluster", [
    (8, 300, 512, 1, 0), (8, 256, 4096, 4, 0), (1, 128, 64, 1, 0), (64, 1000, 1536, 3, 0), (16, 384, 96, 2, 2),
    (33, 130, 200, 5, 5), (8, 4096, 4096, 8, 8), (64, 640, 12288, 8, 4), (8, 512, 12288, 16, 8),
    (16, 300, 4096, 6, 3)])
def test_gemm_tcgen05_swapped_partials(tokens, n_out, k, splits, cluster):
    """The weight as the 128-row operand: partials over K splits sum to x @ W^T, whether the
    caller adds them up or the thread-block cluster does."""
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(tokens + n_out)
    x = torch.randn(tokens, k, generator=gen).bfloat16()
    w = torch.randn(n_out, k, generator=gen).bfloat16()
    err = err_word()
    parts = ops.gemm_tc_swapped(w.to(DEV), x.to(DEV), err, splits, cluster=cluster)
    torch.cuda.synchronize()
    assert err.tolist()[0] == 0, err.tolist()
    assert parts.shape[0] == (splits // cluster if cluster > 1 else splits)
    want = x.double() @ w.double().T
    got = parts.double().sum(0).cpu()
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-3 * (k ** 0.5) / 8)


@pytest.mark.parametrize("tokens,inter,k,splits", [(8, 192, 512, 2), (1, 64, 64, 1), (64, 640, 1536, 6),
                                                    (33, 128, 200, 1), (16, 12288, 4096, 8), (5, 320, 4096, 8)])
def test_gemm_tcgen05_swapped_with_gated_activation(tokens, inter, k, splits):
    """The decode product of a stacked gate/up weight (rows alternating in blocks of 64) whose
    cluster stores silu(gate) * up itself, against the separate product and formula."""
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(tokens + inter)
    x = torch.randn(tokens, k, generator=gen).bfloat16()
    wg = (torch.randn(inter, k, generator=gen) * (2.0 / k ** 0.5)).bfloat16()
    wu = (torch.randn(inter, k, generator=gen) / k ** 0.5).bfloat16()
    b = ops.SWIGLU_TILE_BLOCK
    w = torch.stack((wg.view(inter // b, b, k), wu.view(inter // b, b, k)), dim=1).reshape(2 * inter, k).contiguous()
    err = err_word()
    got = ops.gemm_tc_swapped(w.to(DEV), x.to(DEV), err, splits, cluster=splits, swiglu=True)
    torch.cuda.synchronize()
    assert err.tolist()[0] == 0, err.tolist()
    assert got.shape == (tokens, inter) and got.dtype == torch.bfloat16
    g, u = x.double() @ wg.double().T, x.double() @ wu.double().T
    want = g * torch.sigmoid(g) * u
    torch.testing.assert_close(got.double().cpu(), want, rtol=1e-2, atol=1e-2)
    # the same sums through the float32 partials and the separate activation kernel: bit-equal
    sums = ops.gemm_tc_swapped(w.to(DEV), x.to(DEV), err, splits, cluster=splits)
    two = torch.empty(tokens, inter, device=DEV, dtype=torch.bfloat16)
    ops.swiglu(sums, two, block=b)
    assert torch.equal(two, got)


@pytest.mark.parametrize("tokens,n_out,k", [(256, 256, 64), (300, 384, 320), (77, 200, 96), (1000, 1304, 1032),
                                            (2048, 512, 4096), (513, 256, 12288)])
def test_gemm_tcgen05_pairs_of_sms(tokens, n_out, k):
    """The persistent product on pairs of SMs (cta_group::2): ragged token, output and inner sizes,
    several tiles per pair (both accumulators in turn) and more pairs than tiles."""
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(tokens + n_out + k)
    x = torch.randn(tokens, k, generator=gen).bfloat16()
    w = (torch.randn(n_out, k, generator=gen) / k ** 0.5).bfloat16()
    err = err_word()
    got = ops.gemm_pair(x.to(DEV), w.to(DEV), err)
    torch.cuda.synchronize()
    assert err.tolist()[0] == 0, err.tolist()
    want = x.double() @ w.double().T
    torch.testing.assert_close(got.double().cpu(), want, rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("tokens,inter,k", [(256, 128, 256), (700, 320, 1536), (2048, 1024, 4096), (65, 64, 72)])
def test_gemm_tcgen05_pairs_with_gated_activation(tokens, inter, k):
    """The same product storing silu(gate) * up of a stacked gate/up weight in blocks of 64."""
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(tokens + inter)
    x = torch.randn(tokens, k, generator=gen).bfloat16()
    wg = (torch.randn(inter, k, generator=gen) * (2.0 / k ** 0.5)).bfloat16()
    wu = (torch.randn(inter, k, generator=gen) / k ** 0.5).bfloat16()
    b = ops.SWIGLU_TILE_BLOCK
    w = torch.stack((wg.view(inter // b, b, k), wu.view(inter // b, b, k)), dim=1).reshape(2 * inter, k).contiguous()
    err = err_word()
    got = ops.gemm_pair(x.to(DEV), w.to(DEV), err, swiglu=True)
    torch.cuda.synchronize()
    assert err.tolist()[0] == 0, err.tolist()
    assert got.shape == (tokens, inter)
    g, u = x.double() @ wg.double().T, x.double() @ wu.double().T
    torch.testing.assert_close(got.double().cpu(), g * torch.sigmoid(g) * u, rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("tokens,hidden,k,splits", [(8, 256, 512, 4), (1, 128, 64, 1), (33, 640, 1536, 8), (64, 4096, 4096, 8)])
def test_gemm_tcgen05_swapped_residual_and_owed_norm(tokens, hidden, k, splits):
    """A product that ends a residual branch adds its sums to the residual stream itself and hands
    on bf16(residual * norm weight) with the tiles' sums of squares; the product after it (plain,
    and with the gated activation) multiplies its sums by the owed rsqrt(mean square + eps).  Both
    against the formulas: x + delta, then weight * x * rsqrt(mean(x^2) + eps), then the product."""
    from tokamak_b200.csrc import ops
    eps = 1e-5
    gen = torch.Generator().manual_seed(tokens + hidden)
    a = torch.randn(tokens, k, generator=gen).bfloat16()
    w1 = (torch.randn(hidden, k, generator=gen) / k ** 0.5).bfloat16()
    resid = torch.randn(tokens, hidden, generator=gen)
    norm_w = 1 + 0.1 * torch.randn(hidden, generator=gen)
    err = err_word()
    r_dev = resid.to(DEV)
    xb, sums = ops.gemm_tc_swapped(w1.to(DEV), a.to(DEV), err, splits, cluster=splits,
                                   residual_norm=(r_dev, norm_w.to(DEV)))
    torch.cuda.synchronize()
    assert err.tolist()[0] == 0, err.tolist()
    r_want = resid.double() + a.double() @ w1.double().T
    torch.testing.assert_close(r_dev.double().cpu(), r_want, rtol=1e-5, atol=1e-4 * k ** 0.5)
    torch.testing.assert_close(xb.double().cpu(), r_want * norm_w.double(), rtol=1e-2, atol=1e-2)
    assert sums.shape == (hidden // 128, tokens)
    torch.testing.assert_close(sums.double().sum(0).cpu(), (r_want ** 2).sum(1), rtol=1e-4, atol=1e-4)
    normed = plain.rms_norm(r_want, norm_w.double(), eps)
    # the product after the norm: plain sums ...
    w2 = (torch.randn(384, hidden, generator=gen) / hidden ** 0.5).bfloat16()
    y = ops.gemm_tc_swapped(w2.to(DEV), xb, err, 2, cluster=2, colscale=(sums, hidden, eps))
    torch.testing.assert_close(y[0].double().cpu(), normed @ w2.double().T, rtol=2e-2, atol=2e-2)
    y1 = ops.gemm_tc_swapped(w2.to(DEV), xb, err, 1, colscale=(sums, hidden, eps))      # a single block per tile
    torch.testing.assert_close(y1[0].double().cpu(), normed @ w2.double().T, rtol=2e-2, atol=2e-2)
    # ... and with the gated activation
    b = ops.SWIGLU_TILE_BLOCK
    wg = (torch.randn(128, hidden, generator=gen) * (2.0 / hidden ** 0.5)).bfloat16()
    wu = (torch.randn(128, hidden, generator=gen) / hidden ** 0.5).bfloat16()
    wgu = torch.stack((wg.view(-1, b, hidden), wu.view(-1, b, hidden)), dim=1).reshape(256, hidden).contiguous()
    act = ops.gemm_tc_swapped(wgu.to(DEV), xb, err, 2, cluster=2, swiglu=True, colscale=(sums, hidden, eps))
    g, u = normed @ wg.double().T, normed @ wu.double().T
    torch.testing.assert_close(act.double().cpu(), g * torch.sigmoid(g) * u, rtol=3e-2, atol=3e-2)
    torch.cuda.synchronize()
    assert err.tolist()[0] == 0, err.tolist()


@pytest.mark.parametrize("tokens,hq,hkv,k,splits,page,owed", [(8, 4, 2, 512, 4, 16, False), (1, 2, 1, 64, 1, 8, True),
                                                              (33, 5, 1, 1536, 6, 16, True), (64, 8, 8, 320, 5, 4, False)])
def test_gemm_tcgen05_swapped_with_norm_rotation_and_page_write(tokens, hq, hkv, k, splits, page, owed):
    """The q|k|v product of few tokens whose epilogue does the per-head norm, the rotation and the
    page write (heads of 128): against the formulas, and the cache against the separate kernel's
    rules: values raw, nothing else touched except the cleared rest of a page begun in this step."""
    from tokamak_b200.csrc import ops
    d, eps, theta = 128, 1e-6, 1e6
    gen = torch.Generator().manual_seed(tokens + k)
    # every token its own request: request r has start[r] earlier positions; some begin a page now
    starts = [(7 * r * r + (0 if r % 3 else page * r)) % 5000 for r in range(tokens)]
    starts[0] = 40000                                              # far out: the angle's accuracy
    max_pages = max(s // page for s in starts) + 1
    num_pages = tokens + 3
    pages = torch.randperm(num_pages, generator=gen).tolist()
    table = torch.full((tokens, max_pages), -1, dtype=torch.int32)
    for r, s in enumerate(starts):
        table[r, s // page] = pages[r]
    x = torch.randn(tokens, k, generator=gen).bfloat16()
    w = (torch.randn((hq + 2 * hkv) * d, k, generator=gen) / k ** 0.5).bfloat16()
    qw = 1 + 0.1 * torch.randn(d, generator=gen)
    kw = 1 + 0.1 * torch.randn(d, generator=gen)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    pos_t = i32(starts)
    inv_freq = (1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV)
    rot = ops.rope_table(pos_t, inv_freq)
    kc = torch.full((num_pages, hkv, page, d), 7.0, device=DEV, dtype=torch.bfloat16)
    vc = torch.full_like(kc, 7.0)
    q_out = torch.empty(tokens, hq, d, device=DEV, dtype=torch.bfloat16)
    err = err_word()
    colscale, scale = None, torch.ones(tokens, dtype=torch.float64)
    if owed:       # the input's norm scale is still owed: sums of squares in three tiles
        sums = torch.rand(3, tokens, generator=gen) * k
        colscale = (sums.to(DEV), k, 1e-5)
        scale = torch.rsqrt(sums.double().sum(0) / k + 1e-5)
    ops.gemm_qkv_rope(w.to(DEV), x.to(DEV), err, splits, q_out, kc, vc, pos_t, i32(list(range(tokens))),
                      i32(list(range(tokens))), table.to(DEV), qw.to(DEV), kw.to(DEV), rot, n_q_heads=hq,
                      n_kv_heads=hkv, eps=eps, colscale=colscale, req_q_len=i32([1] * tokens),
                      req_kv_len=i32([s + 1 for s in starts]))
    torch.cuda.synchronize()
    assert err.tolist()[0] == 0, err.tolist()
    y = (x.double() @ w.double().T) * scale[:, None]
    q = y[:, : hq * d].view(tokens, hq, d)
    kk = y[:, hq * d:(hq + hkv) * d].view(tokens, hkv, d)
    v = y[:, (hq + hkv) * d:].view(tokens, hkv, d)
    cos, sin = plain.rope_tables(torch.tensor(starts), d, theta, torch.float64)
    q_want = plain.apply_rope(plain.rms_norm(q, qw.double(), eps), cos, sin)
    k_want = plain.apply_rope(plain.rms_norm(kk, kw.double(), eps), cos, sin)
    t = dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(q_out.double().cpu(), q_want, **t)
    kc_h, vc_h = kc.double().cpu(), vc.double().cpu()
    for r, s in enumerate(starts):
        pg, slot = pages[r], s % page
        torch.testing.assert_close(kc_h[pg, :, slot], k_want[r], **t)
        torch.testing.assert_close(vc_h[pg, :, slot], v[r], **t)
        assert (kc_h[pg, :, :slot] == 7).all() and (vc_h[pg, :, :slot] == 7).all()      # earlier tokens stay
        rest = 0.0 if slot == 0 else 7.0               # a page begun by this token is cleared behind it
        assert (kc_h[pg, :, slot + 1:] == rest).all() and (vc_h[pg, :, slot + 1:] == rest).all()
    for pg in pages[tokens:]:
        assert (kc_h[pg] == 7).all() and (vc_h[pg] == 7).all()
    # the same through the product and the separate kernel: the same cache and queries up to rounding
    kc2 = torch.full_like(kc, 7.0); vc2 = torch.full_like(kc, 7.0); q2 = torch.empty_like(q_out)
    sums2 = ops.gemm_tc_swapped(w.to(DEV), x.to(DEV), err, splits, cluster=splits, colscale=colscale)
    ops.rope_kv(sums2, q2, kc2, vc2, pos_t, i32(list(range(tokens))), i32(list(range(tokens))), table.to(DEV),
                qw.to(DEV), kw.to(DEV), rot, err, n_q_heads=hq, n_kv_heads=hkv, head_dim=d, rotary_dim=d, eps=eps,
                req_q_len=i32([1] * tokens), req_kv_len=i32([s + 1 for s in starts]))
    assert torch.equal(vc2, vc)
    torch.testing.assert_close(q2.float(), q_out.float(), rtol=8e-3, atol=1e-5)       # one bfloat16 step
    torch.testing.assert_close(kc2.float(), kc.float(), rtol=8e-3, atol=1e-5)
    # without norms and rotation the sums pass through
    ops.gemm_qkv_rope(w.to(DEV), x.to(DEV), err, splits, q_out, kc, vc, pos_t, i32(list(range(tokens))),
                      i32(list(range(tokens))), table.to(DEV), None, None, None, n_q_heads=hq, n_kv_heads=hkv,
                      eps=0.0, colscale=colscale)
    torch.cuda.synchronize()
    assert err.tolist()[0] == 0, err.tolist()
    torch.testing.assert_close(q_out.double().cpu(), q, **t)
    # a page outside the pool is reported, not written
    bad = table.clone(); bad[0, starts[0] // page] = num_pages
    ops.gemm_qkv_rope(w.to(DEV), x.to(DEV), err, splits, q_out, kc, vc, pos_t, i32(list(range(tokens))),
                      i32(list(range(tokens))), bad.to(DEV), None, None, None, n_q_heads=hq, n_kv_heads=hkv, eps=0.0)
    torch.cuda.synchronize()
    assert err.tolist()[0] == 2, err.tolist()


@pytest.mark.parametrize("tokens", [1, 8, 64])
def test_gemm_tcgen05_swapped_at_the_real_vocabulary(tokens):
    """The head product of Qwen3: 151,936 rows (1,187 row tiles) over 4,096, planned as the engine
    plans it, against a float64 product computed on the device in slices."""
    from tokamak_b200.csrc import ops
    n_out, k = 151936, 4096
    gen = torch.Generator(device=DEV).manual_seed(tokens)
    x = torch.randn(tokens, k, generator=gen, device=DEV).bfloat16()
    w = (torch.randn(n_out, k, generator=gen, device=DEV) * 0.02).bfloat16()
    splits, stages, cluster = ops.swapped_gemm_plan(n_out, k, tokens)
    err = err_word()
    parts = ops.gemm_tc_swapped(w, x, err, splits, max_stages=stages, cluster=cluster)
    torch.cuda.synchronize()
    assert err.tolist()[0] == 0, err.tolist()
    got = parts.double().sum(0)
    for lo in range(0, n_out, 16384):
        want = x.double() @ w[lo:lo + 16384].double().T
        torch.testing.assert_close(got[:, lo:lo + 16384], want, rtol=1e-4, atol=2e-3)


def test_the_tcgen05_probes_run_and_give_sane_clocks():
    """The measurement aids of csrc/tcgen05_probe.cu: they end by themselves, report no wait that ran
    out, and what they measure lies where a product and a softmax tile can lie."""
    from tokamak_b200.csrc import ops
    one = ops.probe_mma_issue(0, 64)
    assert len(one) == 1 and 8.0 < one[0]["issue_clk"] <= one[0]["done_clk"] < 2000.0
    two = ops.probe_mma_issue(3, 128)
    assert len(two) == 2 and all(32.0 < r["done_clk"] < 4000.0 for r in two)     # 64 clocks of tensor time each
    step = ops.probe_mma_issue(4, 64)
    assert 16.0 < step[0]["done_clk"] < 2000.0
    with pytest.raises(ops.KernelError):
        ops.probe_mma_issue(2, 256)          # two accumulators of 256 columns and the A operand do not fit
    alone = ops.probe_softmax_tile(0, 1)
    beside = ops.probe_softmax_tile(0, 2)
    assert 512.0 < alone["tile"] < 20000.0       # 64 exponentials of a warp take the unit 512 clocks
    assert beside["tile"] > 0.9 * alone["tile"]
    with pytest.raises(ops.KernelError):
        ops.probe_softmax_tile(99, 1)


def test_a_bounded_wait_that_runs_out_is_reported_and_leaves_the_engine_usable():
    """No correct launch makes a barrier wait of the tcgen05 kernels run out, so a kernel made for
    this test does: one block waits, with the kernels' own bounded wait and a limit of 1,024
    polls, for a barrier that nobody arrives at, and reports as they would.  The step function
    raises the error once, with its code, and the next step is clean."""
    import tiny_configs
    from helpers import model_folder, random_tokens
    from tokamak_b200.csrc import ops
    from tokamak_b200.engine.replay import build_core
    from tokamak_b200.engine.step import StepEntry, StepError
    err = err_word()
    ops.wait_probe(1024, err)
    torch.cuda.synchronize()
    word = err.tolist()
    assert word[0] == 5 and word[3] == 1024, word
    with pytest.raises(ops.KernelError):
        ops.wait_probe(1 << 20, err)                       # a probe stays short
    core = build_core(model_folder("A", "float32"), "float32", max_tokens=128, page_size=16)
    toks = random_tokens(tiny_configs.TINY_A["vocab_size"], 20, seed=3)
    clean = core.step.run([StepEntry("a", toks, [19])]).cpu()
    core.step.free("a")
    ops.wait_probe(1024, core.step.buffers.result[:4])     # as if a kernel of the next step had given up
    with pytest.raises(StepError, match="kernel error 5 .*bounded wait"):
        core.step.run([StepEntry("b", toks, [19])])
    core.step.free("b")
    again = core.step.run([StepEntry("c", toks, [19])]).cpu()
    assert torch.equal(again, clean)


def test_step_state_kernels_alone():
    """The kernels that open a step and the sampler that reads the slot records, on hand-made
    buffers: updates are applied under their masks and cleared, fed tokens and positions come
    from the records, bad slots and missing tokens are reported, and the sampler draws what the
    array-driven sampler draws and moves the record on."""
    from tokamak_b200.csrc import ops
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    bits = lambda f: torch.tensor([f], dtype=torch.float32).view(torch.int32).item()
    max_slots, max_tab = 6, 40
    records = torch.zeros(max_slots, 8, dtype=torch.int32, device=DEV)
    records[:, 7] = -1
    tables = torch.full((2, max_slots, 5), -1, dtype=torch.int32, device=DEV)
    ctl = torch.zeros(2 + 9 * max_slots + 2 * max_tab, dtype=torch.int32, device=DEV)
    upd = ops.UpdateBuffers(ctl, max_slots, max_tab, records, tables)
    err = err_word()
    # two record writes (slot 4 in full, slot 1 sampling words only) and three table writes
    rec = [4 | (0xFF << 16), 0, 0, 11, 22, bits(0.5), 7, bits(0.9), -1,
           1 | (0x7E << 16), 99, 3, 33, 44, bits(1.5), 0, bits(1.0), 99]
    tab = [0 * 30 + 4 * 5 + 0, 17, 1 * 30 + 4 * 5 + 2, 9, 0 * 30 + 1 * 5 + 1, -1]
    records[1] = i32([40, 0, 0, 0, 0, 0, 0, 123])
    ctl[:2 + len(rec) + len(tab)] = i32([2, 3] + rec + tab)
    token_ids = i32([50, 51, 52, 53])
    ops.step_begin(upd, token_ids, i32([0, 3]), i32([3, 41]), i32([4, 1]), i32([0, 1]), err)
    torch.cuda.synchronize()
    assert err.tolist()[0] == 0 and ctl[:2].tolist() == [0, 0]
    assert records[4].tolist() == [3, 0, 11, 22, bits(0.5), 7, bits(0.9), -1]
    assert records[1].tolist() == [41, 3, 33, 44, bits(1.5), 0, bits(1.0), 123]     # position, last token kept
    assert token_ids.tolist() == [50, 51, 52, 123]                                   # request 1 was fed
    assert tables[0, 4, 0] == 17 and tables[1, 4, 2] == 9 and tables[0, 1, 1] == -1
    assert int((tables != -1).sum()) == 2
    # a step described by the records alone
    records[4, 7] = 77
    tok, pos, kvl = (torch.zeros(3, dtype=torch.int32, device=DEV) for _ in range(3))
    ops.decode_begin(upd, i32([1, 4]), 2, 64, tok, pos, kvl, err)
    torch.cuda.synchronize()
    assert err.tolist()[0] == 0
    assert tok.tolist()[:2] == [123, 77] and pos.tolist()[:2] == [41, 3] and kvl.tolist()[:2] == [42, 4]
    assert records[1, 0] == 42 and records[4, 0] == 4
    # faults: a slot outside the records, a request that has sampled nothing yet, a position at the limit
    for slots, limit, code in (([9], 64, 4), ([0], 64, 1), ([1], 42, 3)):
        e = err_word()
        ops.decode_begin(upd, i32(slots), 1, limit, tok, pos, kvl, e)
        torch.cuda.synchronize()
        assert e.tolist()[0] == code, (slots, e.tolist())
    # the sampler with records against the sampler with arrays
    gen = torch.Generator().manual_seed(5)
    logits = (torch.randn(2, 317, generator=gen) * 3).to(DEV)
    records[1] = i32([0, 3, 33, 44, bits(1.5), 0, bits(1.0), -1])
    records[4] = i32([0, 9, 11, 22, bits(0.5), 7, bits(0.9), -1])
    out_a, out_b = torch.zeros(2, dtype=torch.int32, device=DEV), torch.zeros(2, dtype=torch.int32, device=DEV)
    ops.sample_slots(logits, records, i32([1, 4]), out_a, err)
    seeds = torch.tensor([33 | (44 << 32), 11 | (22 << 32)], dtype=torch.int64, device=DEV)
    ops.sample(logits, torch.tensor([1.5, 0.5], device=DEV), i32([0, 7]), torch.tensor([1.0, 0.9], device=DEV),
               seeds, i32([3, 9]), out_b)
    torch.cuda.synchronize()
    assert out_a.tolist() == out_b.tolist()
    assert records[1, 1] == 4 and records[4, 1] == 10 and records[1, 7] == out_a[0] and records[4, 7] == out_a[1]


@pytest.mark.parametrize("tokens,hidden,k0,inter,vocab,heads", [(5, 384, 200, 320, 1000, (2, 1)), (64, 1024, 512, 1536, 777, (4, 2)),
                                                                 (17, 4096, 4096, 12288, 2048, (32, 8)), (1, 256, 64, 64, 130, (1, 1))])
def test_chain_of_products_in_one_kernel(tokens, hidden, k0, inter, vocab, heads):
    """Products queued in a ProductChain and launched as one persistent kernel (output product with
    the residual sum and the next norm prepared, gate/up with the activation, down with the
    residual sum, q|k|v with norms, rotation and cache write, and a plain product with an owed
    norm scale, each fed by the one before) against the same products launched one by one, and
    the first of them against float64."""
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(tokens + hidden)
    rnd = lambda *shape, s=1.0: (torch.randn(*shape, generator=gen) * s)
    hq, hkv = heads
    d, page, eps = 128, 16, 1e-6
    x0 = rnd(tokens, k0).bfloat16().to(DEV)
    w_o = rnd(hidden, k0, s=k0 ** -0.5).bfloat16().to(DEV)
    w_gu = rnd(2 * inter, hidden, s=hidden ** -0.5).bfloat16().to(DEV)
    w_d = rnd(hidden, inter, s=inter ** -0.5).bfloat16().to(DEV)
    w_qkv = rnd((hq + 2 * hkv) * d, hidden, s=hidden ** -0.5).bfloat16().to(DEV)
    w_head = rnd(vocab, hidden, s=hidden ** -0.5).bfloat16().to(DEV)
    n1, n2 = (1 + 0.1 * rnd(hidden)).to(DEV), (1 + 0.1 * rnd(hidden)).to(DEV)
    qn, kn = (1 + 0.1 * rnd(d)).to(DEV), (1 + 0.1 * rnd(d)).to(DEV)
    resid0 = rnd(tokens, hidden).to(DEV)
    positions = torch.arange(tokens, dtype=torch.int32, device=DEV) + 3
    tok_req = torch.zeros(tokens, dtype=torch.int32, device=DEV)
    slot = torch.zeros(1, dtype=torch.int32, device=DEV)
    n_pages = -(-(tokens + 3) // page) + 2
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).flip(0).view(1, n_pages).contiguous()
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV)
    rope = ops.rope_table(positions, inv_freq)

    plan = lambda w: ops.swapped_gemm_plan(w.shape[0], w.shape[1], tokens)
    new_cache = lambda: torch.zeros(n_pages, hkv, page, d, dtype=torch.bfloat16, device=DEV)

    def chained_run():
        err = err_word()
        resid, kc, vc = resid0.clone(), new_cache(), new_cache()
        q = torch.zeros(tokens, hq, d, dtype=torch.bfloat16, device=DEV)
        c = ops.ProductChain(tokens, err)
        s, st, cl = plan(w_o)
        xb1, ss1 = ops.gemm_tc_swapped(w_o, x0, err, s, max_stages=st, cluster=cl, residual_norm=(resid, n1), chain=c)
        s, st, cl = plan(w_gu)
        act = ops.gemm_tc_swapped(w_gu, xb1, err, s, max_stages=st, cluster=cl, swiglu=True,
                                  colscale=(ss1, hidden, eps), chain=c)
        s, st, cl = plan(w_d)
        xb2, ss2 = ops.gemm_tc_swapped(w_d, act, err, s, max_stages=st, cluster=cl, residual_norm=(resid, n2), chain=c)
        s, st, cl = plan(w_qkv)
        ops.gemm_qkv_rope(w_qkv, xb2, err, s, q, kc, vc, positions, tok_req, slot, table, qn, kn, rope,
                          n_q_heads=hq, n_kv_heads=hkv, eps=eps, max_stages=st, colscale=(ss2, hidden, eps), chain=c)
        s, st, cl = plan(w_head)
        logits = ops.gemm_tc_swapped(w_head, xb2, err, s, max_stages=st, cluster=cl, colscale=(ss2, hidden, eps), chain=c)
        assert len(c.phases) == 5
        before = ops.LAUNCHES
        ops.flush_chains()
        assert ops.LAUNCHES == before + 1 and not c.phases           # one kernel for the five products
        torch.cuda.synchronize()
        assert err.tolist()[0] == 0, err.tolist()
        return dict(resid=resid, xb1=xb1, ss1=ss1, act=act, xb2=xb2, ss2=ss2, q=q, k=kc, v=vc, logits=logits)

    C = chained_run()

    def close(name, got, want, tol):
        got, want = got.float(), want.float()
        scale = float(want.abs().max()) + 1e-6
        worst = float((got - want).abs().max())
        assert worst <= tol * scale, (name, worst, scale)

    # Every link again as a kernel of its own, fed with what the chain produced before it: the k
    # ranges are cut at other places, so float32 sums come in another order (a few 1e-6 of the
    # largest value) and a bfloat16 result may land on the neighbouring value
    F32, B16 = 2e-5, 1.6e-2
    err = err_word()
    resid = resid0.clone()
    s, st, cl = plan(w_o)
    xb1, ss1 = ops.gemm_tc_swapped(w_o, x0, err, s, max_stages=st, cluster=cl, residual_norm=(resid, n1))
    close("xb1", C["xb1"], xb1, B16); close("ss1", C["ss1"].sum(0), ss1.sum(0), F32)
    s, st, cl = plan(w_gu)
    act = ops.gemm_tc_swapped(w_gu, C["xb1"], err, s, max_stages=st, cluster=cl, swiglu=True, colscale=(C["ss1"], hidden, eps))
    close("act", C["act"], act, B16)
    s, st, cl = plan(w_d)
    xb2, ss2 = ops.gemm_tc_swapped(w_d, C["act"], err, s, max_stages=st, cluster=cl, residual_norm=(resid, n2))
    close("resid", C["resid"], resid, F32); close("xb2", C["xb2"], xb2, B16); close("ss2", C["ss2"].sum(0), ss2.sum(0), F32)
    kc, vc, q = new_cache(), new_cache(), torch.zeros(tokens, hq, d, dtype=torch.bfloat16, device=DEV)
    s, st, cl = plan(w_qkv)
    ops.gemm_qkv_rope(w_qkv, C["xb2"], err, s, q, kc, vc, positions, tok_req, slot, table, qn, kn, rope,
                      n_q_heads=hq, n_kv_heads=hkv, eps=eps, max_stages=st, colscale=(C["ss2"], hidden, eps))
    close("q", C["q"], q, B16); close("k", C["k"], kc, B16); close("v", C["v"], vc, B16)
    assert float(C["k"].float().abs().sum()) > 0
    s, st, cl = plan(w_head)
    logits = ops.gemm_tc_swapped(w_head, C["xb2"], err, s, max_stages=st, cluster=cl, colscale=(C["ss2"], hidden, eps))
    close("logits", C["logits"].sum(0), logits.sum(0), F32)
    torch.cuda.synchronize()
    assert err.tolist()[0] == 0
    chained = {"xb1": C["xb1"].float(), "ss1": C["ss1"].sum(0)}
    # and the first link against float64: what resid + x0 W_o^T gives under the norm weight, and its squares
    want = resid0.double() + x0.double() @ w_o.double().T
    torch.testing.assert_close(chained["xb1"].double(), (want * n1.double()), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(chained["ss1"].double(), (want * want).sum(-1), rtol=1e-4, atol=1e-3)
    # twice in a row: the counters of the first launch are back at zero, and the result is the same to the bit
    again = chained_run()
    assert all(torch.equal(again[n], C[n]) for n in C)
