"""Helpers of the tests: model folders made in temporary folders, token streams, comparisons."""

from __future__ import annotations

import functools
import tempfile
from pathlib import Path

import torch

import tiny_configs
from plain import qwen3_plain as plain

_TMP = []


def model_folder(tag: str, dtype: str) -> Path:
    """A temporary folder holding tiny configuration ``tag`` with weights stored in ``dtype``."""
    return _model_folder(tag, dtype)


@functools.lru_cache(maxsize=None)
def _model_folder(tag: str, dtype: str) -> Path:
    from tokamak_b200.weights import write_random_model

    raw, init, _page = tiny_configs.ALL[tag]
    tmp = tempfile.TemporaryDirectory(prefix=f"tk_tiny_{tag}_{dtype}_")
    _TMP.append(tmp)
    write_random_model(tmp.name, raw, dtype=dtype, **init)
    return Path(tmp.name)


def random_tokens(vocab: int, length: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=gen).tolist()


@functools.lru_cache(maxsize=None)
def _plain_logits_cached(folder: str, tokens: tuple) -> torch.Tensor:
    cfg, w = plain.load_folder(folder)
    return plain.forward_logits(cfg, w, list(tokens), torch.float64)


def plain_logits(folder, tokens) -> torch.Tensor:
    """Float64 logits [T, V] of the plain implementation for a whole sequence."""
    return _plain_logits_cached(str(folder), tuple(int(t) for t in tokens))


# Tolerances.  float32: the engine and the float64 truth differ by rounding of 32-bit
# sums only.  bfloat16: activations are rounded to 8 bits of mantissa between kernels; the
# error of a row of logits is judged against the spread (standard deviation) of that row, as
# a root mean square over the vocabulary and as a maximum.  The limits are set by what
# bfloat16 itself costs, measured once at the Qwen3-8B layer sizes (two layers, 150 tokens,
# vocabulary 2048): a plain PyTorch pipeline that rounds where the reference's bfloat16 model
# rounds is off by 1.45e-2 (rms) and 7.6e-2 (max) of the row's spread; this engine, which keeps
# the residual stream and the rotation in float32, by 1.1e-2 and 6.1e-2.  A wrong key, page or
# mask shows as an error of the order of the spread itself.
F32_ATOL, F32_RTOL = 2e-4, 2e-4
BF16_RMS_TO_ROW = 2e-2
BF16_MAX_TO_ROW = 1e-1


def assert_logits_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    got = got.detach().to("cpu", torch.float64)
    want = want.to(torch.float64)
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    if dtype == "float32":
        err = (got - want).abs()
        bound = F32_ATOL + F32_RTOL * want.abs()
        bad = err > bound
        if bad.any():
            idx = torch.nonzero(bad)[0].tolist()
            raise AssertionError(f"{what}: first mismatch at row {idx[0]} col {idx[1]}: "
                                 f"{got[idx[0], idx[1]]:.6f} vs {want[idx[0], idx[1]]:.6f}; "
                                 f"max err {err.max():.3e}")
    else:
        spread = want.std(dim=-1, keepdim=True).clamp_min(1e-6)
        rel = (got - want).abs() / spread
        rms = rel.pow(2).mean(dim=-1).sqrt()
        worst = int(rms.argmax())
        assert rms[worst] <= BF16_RMS_TO_ROW, (
            f"{what}: row {worst} is off by {rms[worst]:.3e} (rms) of the row's spread "
            f"(limit {BF16_RMS_TO_ROW})")
        mx = rel.amax(dim=-1)
        worst = int(mx.argmax())
        assert mx[worst] <= BF16_MAX_TO_ROW, (
            f"{what}: row {worst} is off by {mx[worst]:.3e} (max) of the row's spread "
            f"(limit {BF16_MAX_TO_ROW})")
