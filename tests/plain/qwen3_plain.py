"""Plain, slow implementation of the Qwen3 dense decoder and of the sampler.

Whole sequences, no cache, no batching, one function for each part, written from
the formulas of WeichunK/tokamak (each function cites the file and lines that it
restates) and sharing no code with the engine.  ``tests/golden/`` holds logits
that the reference's own model code produced on a tiny random model on the CPU;
``tests/test_plain.py`` compares this file with them.

Everything runs on the CPU in the dtype of ``compute_dtype`` (float64 by
default, so that the result can serve as the truth for both the float32 and the
bfloat16 engine).
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch


# ----------------------------------------------------------------------------- loading

def load_folder(model_dir):
    """config.json as a dict and every tensor of the folder's safetensors files, by name."""
    from safetensors import safe_open

    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    tensors = {}
    for file in sorted(model_dir.glob("*.safetensors")):
        with safe_open(str(file), framework="pt", device="cpu") as f:
            for name in f.keys():
                tensors[name] = f.get_tensor(name)
    return cfg, tensors


def rope_theta_of(cfg):
    """src/tokamak/config.py:129-157: rope_parameters dict first, flat rope_theta second."""
    rp = cfg.get("rope_parameters")
    if isinstance(rp, dict) and rp.get("rope_theta") is not None:
        return float(rp["rope_theta"])
    return float(cfg["rope_theta"])


# ----------------------------------------------------------------------------- parts

def rms_norm(x, weight, eps):
    """src/tokamak/model/layers.py:28-33: x * rsqrt(mean(x^2) + eps), then times the weight."""
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return weight.to(x.dtype) * (x * torch.rsqrt(variance + eps))


def rope_tables(positions, head_dim, theta, dtype):
    """src/tokamak/model/layers.py:45-58.

    inv_freq and the angles are float32 in the reference (inv_freq from a float32
    arange, angle = float32 position times inv_freq); they are formed the same way
    here and only then widened, so that the angles are the reference's.
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = positions.to(torch.float32).unsqueeze(-1) * inv_freq          # [T, d/2] float32
    emb = torch.cat((freqs, freqs), dim=-1).to(torch.float64)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x):
    """src/tokamak/model/layers.py:61-63."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def apply_rope(x, cos, sin):
    """src/tokamak/model/layers.py:81-89; x is [T, heads, d], tables are [T, d]."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def causal_attention(q, k, v, window=None):
    """Softmax(q k^T / sqrt(d) + mask) v with grouped heads.

    q [T, Hq, d]; k, v [T, Hkv, d].  Query head h reads kv head h // (Hq / Hkv)
    (src/tokamak/kernels/paged_attention.py:78-80), scale d ** -0.5
    (paged_attention.py:277), the query at position p sees keys 0..p
    (src/tokamak/model/step_context.py:93-96), and with a window only the last
    `window` of them, itself included (src/tokamak/model/attention_policy.py:52-61).
    """
    T, Hq, d = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    scale = d ** -0.5
    rows = torch.arange(T)[:, None]
    cols = torch.arange(T)[None, :]
    mask = cols <= rows
    if window is not None:
        mask &= cols >= (rows - window + 1)
    out = torch.empty_like(q)
    for h in range(Hq):
        kh = k[:, h // group, :]
        vh = v[:, h // group, :]
        scores = (q[:, h, :] @ kh.T) * scale
        scores = scores.masked_fill(~mask, float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        out[:, h, :] = probs @ vh
    return out


def swiglu_mlp(x, w_gate, w_up, w_down):
    """src/tokamak/model/layers.py:103: down(silu(gate(x)) * up(x))."""
    g = x @ w_gate.T
    u = x @ w_up.T
    return (g * torch.sigmoid(g) * u) @ w_down.T


def attention_block(x, positions, w, prefix, cfg, dtype, window=None):
    """src/tokamak/model/transformer.py:67-86 for one sequence."""
    Hq = cfg["num_attention_heads"]
    Hkv = cfg.get("num_key_value_heads") or Hq
    d = cfg.get("head_dim") or cfg["hidden_size"] // Hq
    eps = cfg["rms_norm_eps"]
    T = x.shape[0]
    q = (x @ w[prefix + "q_proj.weight"].to(dtype).T).view(T, Hq, d)
    k = (x @ w[prefix + "k_proj.weight"].to(dtype).T).view(T, Hkv, d)
    v = (x @ w[prefix + "v_proj.weight"].to(dtype).T).view(T, Hkv, d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "k_norm.weight"], eps)
    cos, sin = rope_tables(positions, d, rope_theta_of(cfg), dtype)
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    o = causal_attention(q, k, v, window=window)
    return o.reshape(T, Hq * d) @ w[prefix + "o_proj.weight"].to(dtype).T


def layer_window(cfg, layer_idx):
    """Window of a layer: layers at or beyond max_window_layers when use_sliding_window is set."""
    if not cfg.get("use_sliding_window"):
        return None
    if layer_idx < int(cfg.get("max_window_layers") or 0):
        return None
    return int(cfg["sliding_window"])


def decoder_layer(x, positions, w, layer_idx, cfg, dtype):
    """src/tokamak/model/transformer.py:107-108: two pre-norm residual branches."""
    p = f"model.layers.{layer_idx}."
    eps = cfg["rms_norm_eps"]
    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    x = x + attention_block(h, positions, w, p + "self_attn.", cfg, dtype,
                            window=layer_window(cfg, layer_idx))
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    x = x + swiglu_mlp(h, w[p + "mlp.gate_proj.weight"].to(dtype),
                       w[p + "mlp.up_proj.weight"].to(dtype),
                       w[p + "mlp.down_proj.weight"].to(dtype))
    return x


def forward_logits(cfg, w, token_ids, compute_dtype=torch.float64):
    """Logits [T, vocab] of one whole sequence (src/tokamak/model/transformer.py:138-176)."""
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    x = w["model.embed_tokens.weight"].to(compute_dtype)[ids]
    for layer_idx in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, positions, w, layer_idx, cfg, compute_dtype)
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return x @ head.to(compute_dtype).T


# ----------------------------------------------------------------------------- sampling

_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85
_MASK32 = 0xFFFFFFFF


def philox4x32_10(counter, key):
    """Philox4x32 with ten rounds on Python integers; counter is 4 words, key is 2 words."""
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for _ in range(10):
        p0 = _PHILOX_M0 * c0
        p1 = _PHILOX_M1 * c2
        hi0, lo0 = p0 >> 32, p0 & _MASK32
        hi1, lo1 = p1 >> 32, p1 & _MASK32
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & _MASK32, lo1, (hi0 ^ c3 ^ k1) & _MASK32, lo0
        k0 = (k0 + _PHILOX_W0) & _MASK32
        k1 = (k1 + _PHILOX_W1) & _MASK32
    return c0, c1, c2, c3


def uniform_for(seed, token_index):
    """The uniform in [0, 1) that decides the token_index-th sampled token of a request."""
    words = philox4x32_10((token_index & _MASK32, 0, 0, 0), (seed & _MASK32, (seed >> 32) & _MASK32))
    return words[0] / 2.0 ** 32


def filtered_probs(logits, temperature, top_k=0, top_p=1.0):
    """src/tokamak/sampling/sampler.py:17-39,64-84 on one row, in float64.

    logits / T in float32 as the reference forms them; top-k keeps values >= the
    k-th largest; top-p drops a token iff the mass before it, in descending
    order, already reached top_p.  Values tied with a threshold are kept.
    """
    z = (torch.as_tensor(logits, dtype=torch.float32) / np.float32(temperature)).to(torch.float64)
    V = z.shape[0]
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        kth = torch.topk(z, top_k).values[-1]
        keep &= z >= kth
    if top_p < 1.0:
        zk = z.masked_fill(~keep, float("-inf"))
        probs = torch.softmax(zk, dim=-1)
        order = torch.argsort(zk, descending=True, stable=True)
        sorted_p = probs[order]
        before = torch.cumsum(sorted_p, dim=0) - sorted_p
        kept_sorted = before < top_p
        smallest_kept = zk[order][kept_sorted].min()
        keep &= z >= smallest_kept
    zf = z.masked_fill(~keep, float("-inf"))
    return torch.softmax(zf, dim=-1)


def sample_token(logits, temperature, top_k=0, top_p=1.0, seed=0, token_index=0):
    """Greedy for temperature 0 (lowest index among equal maxima), else an inverse-CDF draw."""
    logits = torch.as_tensor(logits, dtype=torch.float32)
    if temperature == 0.0:
        return int(torch.argmax(logits).item())
    probs = filtered_probs(logits, temperature, top_k, top_p)
    cdf = torch.cumsum(probs, dim=0)
    u = uniform_for(seed, token_index)
    target = u * float(cdf[-1])
    idx = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True).item())
    return min(idx, probs.shape[0] - 1)


def greedy_generate(cfg, w, prompt, max_new_tokens, compute_dtype=torch.float64):
    """Greedy continuation by recomputing the whole sequence for every token."""
    tokens = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        logits = forward_logits(cfg, w, tokens, compute_dtype)[-1]
        nxt = int(torch.argmax(logits.to(torch.float32)).item())
        out.append(nxt)
        tokens.append(nxt)
    return out
