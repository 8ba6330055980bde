"""The plain implementation against logits that the reference's own model code produced."""

from __future__ import annotations

import hashlib
from pathlib import Path

import pytest
import torch
from safetensors import safe_open

import tiny_configs
from helpers import model_folder
from plain import qwen3_plain as plain

GOLDEN = Path(__file__).resolve().parent / "golden"


def _digest(tensors):
    h = hashlib.sha256()
    for name in sorted(tensors):
        h.update(name.encode())
        h.update(tensors[name].to(torch.float32).contiguous().numpy().tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("tag", ["A", "B"])
def test_plain_matches_reference_golden(tag):
    folder = model_folder(tag, "float32")
    cfg, w = plain.load_folder(folder)
    with safe_open(str(GOLDEN / f"tiny_{tag}.safetensors"), framework="pt") as f:
        golden = f.get_tensor("logits")
        ids = f.get_tensor("token_ids").tolist()
        digest = f.metadata()["weights_sha256"]
    assert _digest(w) == digest, "seeded weights changed: regenerate tests/golden (see make_golden.py)"
    got32 = plain.forward_logits(cfg, w, ids, torch.float32)
    got64 = plain.forward_logits(cfg, w, ids, torch.float64)
    # the reference's own tolerance between its ways of computing is 1e-4 (tests/unit/test_model.py:108)
    torch.testing.assert_close(got32, golden, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(got64.float(), golden, rtol=1e-4, atol=1e-4)


def test_rms_norm_formula():
    x = torch.randn(3, 7, dtype=torch.float64)
    w = torch.randn(7, dtype=torch.float64)
    y = plain.rms_norm(x, w, 1e-5)
    want = w * x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5)
    torch.testing.assert_close(y, want)


def test_rope_properties():
    # identity at position 0, norm preserved, dot product depends on the distance only
    # (the properties the reference checks, tests/unit/test_layers.py:30-68)
    d = 16
    q = torch.randn(1, 2, d, dtype=torch.float64)
    k = torch.randn(1, 2, d, dtype=torch.float64)
    cos0, sin0 = plain.rope_tables(torch.tensor([0]), d, 1e4, torch.float64)
    torch.testing.assert_close(plain.apply_rope(q, cos0, sin0), q)
    def rot(x, p):
        c, s = plain.rope_tables(torch.tensor([p]), d, 1e4, torch.float64)
        return plain.apply_rope(x, c, s)
    torch.testing.assert_close(rot(q, 5).norm(), q.norm())
    a = (rot(q, 7) * rot(k, 3)).sum()
    b = (rot(q, 14) * rot(k, 10)).sum()
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)


def test_attention_is_causal_and_windowed():
    T, d = 9, 8
    q = torch.randn(T, 2, d, dtype=torch.float64)
    k = torch.randn(T, 1, d, dtype=torch.float64)
    v = torch.randn(T, 1, d, dtype=torch.float64)
    full = plain.causal_attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[6:] += 1.0
    v2[6:] -= 2.0
    torch.testing.assert_close(plain.causal_attention(q, k2, v2)[:6], full[:6])
    win = plain.causal_attention(q, k, v, window=3)
    k3, v3 = k.clone(), v.clone()
    k3[:4] += 5.0
    v3[:4] += 5.0
    torch.testing.assert_close(plain.causal_attention(q, k3, v3, window=3)[6:], win[6:])
    torch.testing.assert_close(win[:3], full[:3])


def test_sampler_plain():
    logits = torch.tensor([0.1, 2.0, -1.0, 2.0, 0.5])
    assert plain.sample_token(logits, 0.0) == 1                      # first of the equal maxima
    p = plain.filtered_probs(logits, 1.0, top_k=2)
    assert (p > 0).tolist() == [False, True, False, True, False]
    p = plain.filtered_probs(torch.tensor([3.0, 1.0, 0.0, -2.0]), 1.0, top_p=0.5)
    assert (p > 0).tolist() == [True, False, False, False]           # the best token always stays
    draws = {plain.sample_token(logits, 0.8, seed=3, token_index=i) for i in range(200)}
    assert draws <= {0, 1, 2, 3, 4} and len(draws) >= 3
    assert plain.sample_token(logits, 0.8, seed=3, token_index=5) == \
        plain.sample_token(logits, 0.8, seed=3, token_index=5)
    us = [plain.uniform_for(11, i) for i in range(2000)]
    assert 0.45 < sum(us) / len(us) < 0.55 and min(us) >= 0.0 and max(us) < 1.0
