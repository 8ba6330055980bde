"""Each part of a layer alone against the plain functions, the schedule as data, and toy parts
that are registered, built and stepped from the test alone: a mixer with state of its own, a
feed-forward with routing and another position encoding."""

from __future__ import annotations

import json
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import traces
from helpers import assert_logits_close, random_tokens
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"


def runtime(dtype):
    from tokamak_b200.parts.base import Runtime
    return Runtime(device=torch.device("cuda", 0), dtype=dtype)


def tol(dtype):
    return dict(rtol=3e-5, atol=3e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)


# ----------------------------------------------------------------------------- single parts

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from tokamak_b200.parts.norm import RMSNorm, RMSNormSpec
    spec = RMSNormSpec(dim=200, eps=1e-5)
    assert RMSNorm.expected_tensors(spec, "n.weight")["n.weight"].shape == (200,)
    w = 1 + 0.1 * torch.randn(200, device=DEV)
    part = RMSNorm(spec, "n.weight", {"n.weight": w}, runtime(dtype))
    resid = torch.randn(9, 200, device=DEV)
    delta = torch.randn(9, 200, device=DEV).to(dtype)
    want_sum = resid.double() + delta.double()
    out = part.add_norm(resid, delta)
    assert out.dtype == dtype
    torch.testing.assert_close(resid.double(), want_sum, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(out.double(), plain.rms_norm(want_sum, w.double(), 1e-5), **tol(dtype))


def test_position_parts():
    from tokamak_b200.parts.position import NoPosition, NoPositionSpec, RopeNeox, RopeSpec
    from types import SimpleNamespace
    rope = RopeNeox(RopeSpec(head_dim=48, theta=50000.0), {}, runtime(torch.float32))
    positions = [0, 1, 7, 300, 40001]
    step = SimpleNamespace(positions=torch.tensor(positions, dtype=torch.int32, device=DEV), scratch={})
    table, rotary_dim = rope.rotary_table(step)
    assert rotary_dim == 48 and table.shape == (5, 24, 2)
    assert rope.rotary_table(step)[0] is table                      # made once per step
    cos, sin = plain.rope_tables(torch.tensor(positions), 48, 50000.0, torch.float64)
    torch.testing.assert_close(table[..., 0].double().cpu(), cos[:, :24], rtol=0, atol=2e-6)
    torch.testing.assert_close(table[..., 1].double().cpu(), sin[:, :24], rtol=0, atol=2e-6)
    assert NoPosition(NoPositionSpec(), {}, runtime(torch.float32)).rotary_table(step) == (None, 0)
    with pytest.raises(ValueError):
        RopeNeox(RopeSpec(head_dim=15, theta=1e4), {}, runtime(torch.float32))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter", [136, 192])       # stacked gate/up as two halves, and in blocks of 64
def test_swiglu_part(dtype, inter):
    from types import SimpleNamespace
    from tokamak_b200.parts.base import sum_parts
    from tokamak_b200.parts.feedforward import SwiGLU, SwiGLUSpec
    spec = SwiGLUSpec(hidden_size=72, intermediate_size=inter)
    names = SwiGLU.expected_tensors(spec, "mlp.")
    assert names["mlp.down_proj.weight"].shape == (72, inter)
    tensors = {n: (0.1 * torch.randn(r.shape, device=DEV)).to(dtype) for n, r in names.items()}
    part = SwiGLU(spec, "mlp.", tensors, runtime(dtype))
    x = torch.randn(11, 72, device=DEV).to(dtype)
    want = plain.swiglu_mlp(x.double(), tensors["mlp.gate_proj.weight"].double(),
                            tensors["mlp.up_proj.weight"].double(), tensors["mlp.down_proj.weight"].double())
    got = part.forward(x, None)                      # the path of many tokens
    torch.testing.assert_close(got.double(), want, **tol(dtype))
    step = SimpleNamespace(err=torch.zeros(4, dtype=torch.int32, device=DEV))
    got = sum_parts(part.forward(x, step))           # the path of few tokens (the decode products in bfloat16)
    assert step.err.tolist()[0] == 0
    torch.testing.assert_close(got.double(), want, **tol(dtype))


class _Harness:
    """A cache and a step function around one part, so that the part can be stepped alone."""

    def __init__(self, need, dtype, page=8, pool_tokens=256, max_seq_len=256):
        from tokamak_b200.cache.device import DeviceCache, plan_groups
        from tokamak_b200.cache.manager import CacheManager
        from tokamak_b200.engine.step import StepFunction
        kv, st = plan_groups({"c": need}, pool_tokens, page)
        self.manager = CacheManager(kv, st, 4)
        self.cache = DeviceCache(self.manager, dtype, torch.device("cuda", 0), max_seq_len)
        self.step = StepFunction(None, self.cache, 256, max_seq_len)

    def batch(self, entries):
        from tokamak_b200.engine.step import StepEntry
        return self.step.build([StepEntry(r, [0] * n, []) for r, n in entries])

    def done(self, entries):
        from tokamak_b200.engine.step import StepEntry
        self.step.finish([StepEntry(r, [0] * n, []) for r, n in entries])
        self.step.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv,d,window", [(6, 2, 32, None), (4, 1, 64, 9), (3, 3, 16, None)])
def test_attention_part_alone_in_portions(dtype, hq, hkv, d, window):
    """The attention mixer stepped in portions equals the plain attention block on the whole input."""
    from tokamak_b200.parts.attention import Attention, AttentionSpec
    from tokamak_b200.parts.base import sum_parts
    from tokamak_b200.parts.position import RopeSpec
    hidden, T = 40, 37
    spec = AttentionSpec(hidden_size=hidden, num_heads=hq, num_kv_heads=hkv, head_dim=d,
                         position=RopeSpec(d, 1e4), qk_norm_eps=1e-6, window=window)
    names = Attention.expected_tensors(spec, "a.")
    tensors = {}
    for n, r in names.items():
        t = torch.randn(r.shape, device=DEV)
        tensors[n] = (1 + 0.1 * t) if r.role == "vector" else (0.15 * t).to(dtype)
    part = Attention(spec, "a.", tensors, runtime(dtype))
    x = torch.randn(T, hidden, device=DEV).to(dtype)
    cfg = {"num_attention_heads": hq, "num_key_value_heads": hkv, "head_dim": d, "hidden_size": hidden,
           "rms_norm_eps": 1e-6, "rope_theta": 1e4}
    w64 = {k: v.double().cpu() for k, v in tensors.items()}
    want = plain.attention_block(x.double().cpu(), torch.arange(T), w64, "a.", cfg, torch.float64,
                                 window=window)
    h = _Harness(part.cache_need(), dtype)
    got, pos = [], 0
    for n in (5, 1, 16, 2, 13):
        b = h.batch([("r", n)])
        got.append(sum_parts(part.forward(x[pos:pos + n].contiguous(), b, h.cache.view("c"))).to(dtype))
        h.done([("r", n)])
        pos += n
    torch.testing.assert_close(torch.cat(got).double().cpu(), want, **tol(dtype))


def test_schedule_names_a_block_twice_and_shares_a_cache():
    """The order of layers is data: block b0 runs twice with caches of its own, and block b1,
    built without key and value projections, reads the cache that the first call wrote."""
    from tokamak_b200.cache.device import DeviceCache, plan_groups
    from tokamak_b200.cache.manager import CacheManager
    from tokamak_b200.engine.step import StepEntry, StepFunction
    from tokamak_b200.models.decoder import DecoderModel, LayerCall, ModelSpec
    from tokamak_b200.parts.attention import AttentionSpec
    from tokamak_b200.parts.block import PreNormBlockSpec
    from tokamak_b200.parts.embedding import EmbeddingSpec, HeadSpec
    from tokamak_b200.parts.feedforward import SwiGLUSpec
    from tokamak_b200.parts.norm import RMSNormSpec
    from tokamak_b200.parts.position import RopeSpec
    from tokamak_b200.weights import random_tensors

    H, V, d, hq, hkv, inter, eps = 48, 97, 16, 4, 2, 80, 1e-6
    norm = RMSNormSpec(H, eps)

    def block(name, own_kv):
        return PreNormBlockSpec(
            name=name, norm1=norm, norm2=norm,
            mixer=AttentionSpec(H, hq, hkv, d, RopeSpec(d, 1e4), qk_norm_eps=eps, own_kv=own_kv),
            feed_forward=SwiGLUSpec(H, inter), norm1_name=f"{name}.n1", mixer_prefix=f"{name}.attn.",
            norm2_name=f"{name}.n2", ffn_prefix=f"{name}.mlp.")

    spec = ModelSpec(embedding=EmbeddingSpec(V, H, "embed"), blocks=(block("b0", True), block("b1", False)),
                     schedule=(LayerCall("b0", "first"), LayerCall("b1", "first"), LayerCall("b0", "second")),
                     final_norm=norm, final_norm_name="final", head=HeadSpec(V, H, tied=True))
    expected = DecoderModel.expected_tensors(spec)
    assert "b1.attn.k_proj.weight" not in expected and "b0.attn.k_proj.weight" in expected
    tensors = random_tensors(expected, seed=9, std=0.08, dtype=torch.float32, device="cuda")
    model = DecoderModel(spec, tensors, runtime(torch.float32))
    needs = model.cache_needs()
    assert set(needs) == {"first", "second"}
    kv, st = plan_groups(needs, 128, 8)
    assert len(kv) == 1 and sorted(kv[0].cache_keys) == ["first", "second"]      # one group, two slabs
    cache = DeviceCache(CacheManager(kv, st, 2), torch.float32, torch.device("cuda", 0), 128)
    step = StepFunction(model, cache, 128, 128)
    ids = random_tokens(V, 30, seed=1)
    got = torch.cat([step.run([StepEntry("r", ids[:11], list(range(11)))]),
                     step.run([StepEntry("r", ids[11:], list(range(19)))])]).double().cpu()

    # the same computation with the plain functions
    w = {k: v.double().cpu() for k, v in tensors.items()}
    cfg = {"num_attention_heads": hq, "num_key_value_heads": hkv, "head_dim": d, "hidden_size": H,
           "rms_norm_eps": eps, "rope_theta": 1e4}
    pos = torch.arange(30)
    x = w["embed"][torch.tensor(ids)]
    cos, sin = plain.rope_tables(pos, d, 1e4, torch.float64)

    def mlp(x, name):
        h = plain.rms_norm(x, w[f"{name}.n2"], eps)
        return x + plain.swiglu_mlp(h, w[f"{name}.mlp.gate_proj.weight"], w[f"{name}.mlp.up_proj.weight"],
                                    w[f"{name}.mlp.down_proj.weight"])

    def b0(x):
        h = plain.rms_norm(x, w["b0.n1"], eps)
        return mlp(x + plain.attention_block(h, pos, w, "b0.attn.", cfg, torch.float64), "b0")

    # first call of b0: remember its keys and values for b1
    h0 = plain.rms_norm(x, w["b0.n1"], eps)
    k0 = plain.apply_rope(plain.rms_norm((h0 @ w["b0.attn.k_proj.weight"].T).view(30, hkv, d),
                                         w["b0.attn.k_norm.weight"], eps), cos, sin)
    v0 = (h0 @ w["b0.attn.v_proj.weight"].T).view(30, hkv, d)
    x = b0(x)
    h1 = plain.rms_norm(x, w["b1.n1"], eps)
    q1 = plain.apply_rope(plain.rms_norm((h1 @ w["b1.attn.q_proj.weight"].T).view(30, hq, d),
                                         w["b1.attn.q_norm.weight"], eps), cos, sin)
    a1 = plain.causal_attention(q1, k0, v0).reshape(30, hq * d) @ w["b1.attn.o_proj.weight"].T
    x = mlp(x + a1, "b1")
    x = b0(x)
    want = plain.rms_norm(x, w["final"], eps) @ w["embed"].T
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)


# ----------------------------------------------------------------------------- a toy architecture

@dataclass(frozen=True)
class DecaySumSpec:
    """A mixer with state of its own: s_t = decay * s_{t-1} + x_t, y_t = s_t W^T."""
    hidden_size: int
    decay: float
    kind: str = "toy_decay_sum"


class DecaySum:
    def __init__(self, spec, prefix, tensors, rt):
        self.spec, self.rt = spec, rt
        self.w = tensors[prefix + "mix.weight"]

    @staticmethod
    def expected_tensors(spec, prefix):
        from tokamak_b200.parts.base import TensorReq
        return {prefix + "mix.weight": TensorReq((spec.hidden_size, spec.hidden_size))}

    def cache_need(self):
        from tokamak_b200.cache.manager import StateNeed
        return StateNeed((self.spec.hidden_size,), "float32")

    def forward(self, h, step, cache_view):
        from tokamak_b200.parts.base import linear
        records = cache_view.records                       # [max_slots, hidden] float32
        out = torch.empty_like(h, dtype=torch.float32)
        for start, n, slot in zip(step.host_q_start, step.host_q_len, step.host_slot):
            s = records[slot]
            for t in range(start, start + n):              # a toy: one token at a time
                s = self.spec.decay * s + h[t].float()
                out[t] = s
            records[slot] = s
        return linear(out.to(h.dtype), self.w)


TOY_CONFIG = {"architectures": ["ToyDecayForCausalLM"], "vocab_size": 131, "hidden_size": 56,
              "heads": 2, "head_dim": 16, "inter": 72, "eps": 1e-6, "theta": 10000.0, "decay": 0.8,
              "max_position_embeddings": 256}


def _toy_architecture():
    """An architecture of one attention block and one decay-sum block, described from outside."""
    from tokamak_b200.config import Architecture
    from tokamak_b200.models.decoder import LayerCall, ModelSpec
    from tokamak_b200.parts.attention import AttentionSpec
    from tokamak_b200.parts.block import PreNormBlockSpec
    from tokamak_b200.parts.embedding import EmbeddingSpec, HeadSpec
    from tokamak_b200.parts.feedforward import SwiGLUSpec
    from tokamak_b200.parts.norm import RMSNormSpec
    from tokamak_b200.parts.position import RopeSpec

    @dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int
        hidden_size: int
        heads: int
        head_dim: int
        inter: int
        eps: float
        theta: float
        decay: float
        max_position_embeddings: int
        architecture: str = "ToyDecayForCausalLM"
        eos_token_ids: tuple = ()

    def parse_config(raw, eos_token_ids=None):
        return ToyConfig(**{k: raw[k] for k in TOY_CONFIG if k != "architectures"},
                         eos_token_ids=tuple(eos_token_ids or ()))

    def model_spec(cfg):
        H, norm = cfg.hidden_size, RMSNormSpec(cfg.hidden_size, cfg.eps)
        ffn = SwiGLUSpec(H, cfg.inter)
        attn = AttentionSpec(H, cfg.heads, cfg.heads, cfg.head_dim, RopeSpec(cfg.head_dim, cfg.theta),
                             qk_norm_eps=cfg.eps)
        blocks = (
            PreNormBlockSpec("l0", norm, attn, norm, ffn, "l0.n1", "l0.attn.", "l0.n2", "l0.mlp."),
            PreNormBlockSpec("l1", norm, DecaySumSpec(H, cfg.decay), norm, ffn, "l1.n1", "l1.", "l1.n2",
                             "l1.mlp."),
        )
        return ModelSpec(EmbeddingSpec(cfg.vocab_size, H, "embed"), blocks,
                         (LayerCall("l0", "l0"), LayerCall("l1", "l1")), norm, "final",
                         HeadSpec(cfg.vocab_size, H, tied=False, name="head"))

    return Architecture("ToyDecayForCausalLM", parse_config, model_spec)


def _toy_plain_logits(folder, ids):
    cfg, w = plain.load_folder(folder)
    w = {k: v.double() for k, v in w.items()}
    c = {"num_attention_heads": cfg["heads"], "num_key_value_heads": cfg["heads"], "head_dim": cfg["head_dim"],
         "hidden_size": cfg["hidden_size"], "rms_norm_eps": cfg["eps"], "rope_theta": cfg["theta"]}
    T, eps = len(ids), cfg["eps"]
    x = w["embed"][torch.tensor(ids)]
    mlp = lambda x, n: x + plain.swiglu_mlp(plain.rms_norm(x, w[f"{n}.n2"], eps), w[f"{n}.mlp.gate_proj.weight"],
                                            w[f"{n}.mlp.up_proj.weight"], w[f"{n}.mlp.down_proj.weight"])
    x = x + plain.attention_block(plain.rms_norm(x, w["l0.n1"], eps), torch.arange(T), w, "l0.attn.", c,
                                  torch.float64)
    x = mlp(x, "l0")
    h = plain.rms_norm(x, w["l1.n1"], eps)
    s = torch.zeros(cfg["hidden_size"], dtype=torch.float64)
    states = []
    for t in range(T):
        s = cfg["decay"] * s + h[t]
        states.append(s)
    x = mlp(x + torch.stack(states) @ w["l1.mix.weight"].T, "l1")
    return plain.rms_norm(x, w["final"], eps) @ w["head"].T


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    """Nothing in the framework's files knows this mixer or this architecture: the test registers
    both, writes a model folder with the framework's writer, and replays it whole, in portions
    and mixed with other requests through the ordinary engine; slots of ended requests are
    handed to new ones, whose state must start from zero."""
    from tokamak_b200.config import register_architecture
    from tokamak_b200.engine.replay import build_core, run_step
    from tokamak_b200.parts.base import MIXERS
    from tokamak_b200.weights import write_random_model

    MIXERS.register("toy_decay_sum")(DecaySum)
    register_architecture(_toy_architecture())
    try:
        folder = write_random_model(tmp_path / "toy", TOY_CONFIG, seed=3, std=0.08, dtype="float32")
        assert json.loads((folder / "config.json").read_text())["architectures"] == ["ToyDecayForCausalLM"]
        reqs = {f"t{i}": random_tokens(131, n, seed=50 + i) for i, n in enumerate([9, 40, 23, 64, 31, 17])}
        truth = {rid: _toy_plain_logits(folder, ids) for rid, ids in reqs.items()}
        for builder, kw in ((traces.whole, {}), (traces.portions, {}),
                            (traces.mixed, {"max_tokens": 192, "max_live": 3, "seed": 2})):
            core = build_core(folder, "float32", 192, page_size=16, max_live=3)
            assert len(core.manager.state_groups) == 1 and len(core.manager.kv_groups) == 1
            records, rows = builder(reqs, **kw)
            for rec in records:
                out = run_step(core, rec)
                got = torch.from_numpy(out)
                want = torch.stack([truth[rid][p] for rid, p in rows[rec["step"]]])
                assert_logits_close(got, want, "float32", f"toy {builder.__name__} step {rec['step']}")
            assert not core.manager.live_requests()
    finally:
        MIXERS.unregister("toy_decay_sum")


# ----------------------------------------------------------------------------- more toy parts

@dataclass(frozen=True)
class ScaledPartialRopeSpec:
    """A position encoding of the test's own: only the first ``rotary_dim`` elements of a head
    are rotated, at angle (position / factor) * theta ** (-2j / rotary_dim)."""
    rotary_dim: int
    theta: float
    factor: float
    kind: str = "toy_scaled_partial_rope"


class ScaledPartialRope:
    GRAPH_SAFE = True          # tensor operations on the step's device tensors only

    def __init__(self, spec, tensors, rt):
        self.spec = spec
        j = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float32, device=rt.device)
        self.inv_freq = 1.0 / (spec.theta ** (j / spec.rotary_dim))

    @staticmethod
    def expected_tensors(spec):
        return {}

    def rotary_table(self, step):
        key = ("toy_rope", self.spec)
        if key not in step.scratch:
            ang = (step.positions.float() / self.spec.factor)[:, None] * self.inv_freq[None, :]
            step.scratch[key] = torch.stack((ang.cos(), ang.sin()), dim=-1).contiguous()
        return step.scratch[key], self.spec.rotary_dim


@dataclass(frozen=True)
class Top1ExpertsSpec:
    """A feed-forward with routing: float32 router logits, the best expert of every token runs
    (a SwiGLU of its own), scaled by the router's softmax probability of that expert."""
    hidden_size: int
    intermediate_size: int
    num_experts: int
    kind: str = "toy_top1_experts"


class Top1Experts:
    def __init__(self, spec, prefix, tensors, rt):
        self.spec = spec
        self.router = tensors[prefix + "router.weight"]                 # float32 (role "vector")
        self.w = [{n: tensors[f"{prefix}experts.{e}.{n}.weight"] for n in ("gate", "up", "down")}
                  for e in range(spec.num_experts)]

    @staticmethod
    def expected_tensors(spec, prefix):
        from tokamak_b200.parts.base import TensorReq
        h, i = spec.hidden_size, spec.intermediate_size
        out = {prefix + "router.weight": TensorReq((spec.num_experts, h), role="vector")}
        for e in range(spec.num_experts):
            out[f"{prefix}experts.{e}.gate.weight"] = TensorReq((i, h))
            out[f"{prefix}experts.{e}.up.weight"] = TensorReq((i, h))
            out[f"{prefix}experts.{e}.down.weight"] = TensorReq((h, i))
        return out

    def forward(self, h, step):
        from tokamak_b200.parts.base import linear
        logits = h.float() @ self.router.t()                            # router logits in 32-bit
        prob, choice = torch.softmax(logits, dim=-1).max(dim=-1)
        out = torch.zeros_like(h, dtype=torch.float32)
        for e, w in enumerate(self.w):
            rows = (choice == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            x = h[rows]
            g, u = linear(x, w["gate"]).float(), linear(x, w["up"]).float()
            y = linear((g * torch.sigmoid(g) * u).to(h.dtype), w["down"]).float()
            out[rows] = y * prob[rows, None]
        return out.to(h.dtype)


ROUTED_CONFIG = {"architectures": ["ToyRoutedForCausalLM"], "vocab_size": 97, "hidden_size": 40,
                 "heads": 4, "kv_heads": 2, "head_dim": 24, "rotary_dim": 12, "factor": 4.0, "inter": 48,
                 "experts": 3, "eps": 1e-5, "theta": 500.0, "max_position_embeddings": 256}


def _routed_architecture():
    from tokamak_b200.config import Architecture
    from tokamak_b200.models.decoder import LayerCall, ModelSpec
    from tokamak_b200.parts.attention import AttentionSpec
    from tokamak_b200.parts.block import PreNormBlockSpec
    from tokamak_b200.parts.embedding import EmbeddingSpec, HeadSpec
    from tokamak_b200.parts.feedforward import SwiGLUSpec
    from tokamak_b200.parts.norm import RMSNormSpec

    @dataclass(frozen=True)
    class Config:
        vocab_size: int
        hidden_size: int
        heads: int
        kv_heads: int
        head_dim: int
        rotary_dim: int
        factor: float
        inter: int
        experts: int
        eps: float
        theta: float
        max_position_embeddings: int
        architecture: str = "ToyRoutedForCausalLM"
        eos_token_ids: tuple = ()

    def parse_config(raw, eos_token_ids=None):
        return Config(**{k: raw[k] for k in ROUTED_CONFIG if k != "architectures"},
                      eos_token_ids=tuple(eos_token_ids or ()))

    def model_spec(cfg):
        H, norm = cfg.hidden_size, RMSNormSpec(cfg.hidden_size, cfg.eps)
        pos = ScaledPartialRopeSpec(cfg.rotary_dim, cfg.theta, cfg.factor)
        attn = AttentionSpec(H, cfg.heads, cfg.kv_heads, cfg.head_dim, pos, qk_norm_eps=cfg.eps)
        ffn0 = Top1ExpertsSpec(H, cfg.inter, cfg.experts) if cfg.experts else SwiGLUSpec(H, cfg.inter)
        blocks = (
            PreNormBlockSpec("l0", norm, attn, norm, ffn0, "l0.n1", "l0.attn.", "l0.n2",
                             "l0.moe." if cfg.experts else "l0.mlp."),
            PreNormBlockSpec("l1", norm, attn, norm, SwiGLUSpec(H, cfg.inter), "l1.n1", "l1.attn.", "l1.n2",
                             "l1.mlp."),
        )
        return ModelSpec(EmbeddingSpec(cfg.vocab_size, H, "embed"), blocks,
                         (LayerCall("l0", "l0"), LayerCall("l1", "l1")), norm, "final",
                         HeadSpec(cfg.vocab_size, H, tied=True, name="head"))

    return Architecture("ToyRoutedForCausalLM", parse_config, model_spec)


def _routed_plain_logits(folder, ids):
    cfg, w = plain.load_folder(folder)
    w = {k: v.double() for k, v in w.items()}
    T, eps, d, rot = len(ids), cfg["eps"], cfg["head_dim"], cfg["rotary_dim"]
    ang = (torch.arange(T, dtype=torch.float64) / cfg["factor"])[:, None] * \
        (1.0 / cfg["theta"] ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot))[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def rope(x):                                    # [T, heads, d]: the first `rot` elements rotate by halves
        a, b, rest = x[..., :rot // 2], x[..., rot // 2:rot], x[..., rot:]
        return torch.cat((a * cos - b * sin, b * cos + a * sin, rest), dim=-1)

    def attn(x, n):
        q = (x @ w[f"{n}.attn.q_proj.weight"].T).view(T, cfg["heads"], d)
        k = (x @ w[f"{n}.attn.k_proj.weight"].T).view(T, cfg["kv_heads"], d)
        v = (x @ w[f"{n}.attn.v_proj.weight"].T).view(T, cfg["kv_heads"], d)
        q = rope(plain.rms_norm(q, w[f"{n}.attn.q_norm.weight"], eps))
        k = rope(plain.rms_norm(k, w[f"{n}.attn.k_norm.weight"], eps))
        return plain.causal_attention(q, k, v).reshape(T, -1) @ w[f"{n}.attn.o_proj.weight"].T

    x = w["embed"][torch.tensor(ids)]
    x = x + attn(plain.rms_norm(x, w["l0.n1"], eps), "l0")
    h = plain.rms_norm(x, w["l0.n2"], eps)
    if cfg["experts"]:
        prob, choice = torch.softmax(h @ w["l0.moe.router.weight"].T, dim=-1).max(dim=-1)
        y = torch.stack([plain.swiglu_mlp(h[t:t + 1], w[f"l0.moe.experts.{int(e)}.gate.weight"],
                                          w[f"l0.moe.experts.{int(e)}.up.weight"],
                                          w[f"l0.moe.experts.{int(e)}.down.weight"])[0] * prob[t]
                         for t, e in enumerate(choice)])
    else:
        choice = torch.zeros(T, dtype=torch.long)
        y = plain.swiglu_mlp(h, w["l0.mlp.gate_proj.weight"], w["l0.mlp.up_proj.weight"],
                             w["l0.mlp.down_proj.weight"])
    x = x + y
    x = x + attn(plain.rms_norm(x, w["l1.n1"], eps), "l1")
    x = x + plain.swiglu_mlp(plain.rms_norm(x, w["l1.n2"], eps), w["l1.mlp.gate_proj.weight"],
                             w["l1.mlp.up_proj.weight"], w["l1.mlp.down_proj.weight"])
    return plain.rms_norm(x, w["final"], eps) @ w["embed"].T, choice


def test_toy_routed_feed_forward_and_toy_position_encoding(tmp_path):
    """A feed-forward with routing and a position encoding that rotates a part of the head at
    scaled positions, both defined here, are registered, chosen layer by layer by a toy
    architecture, built from a folder that the framework's writer made, and replayed whole, in
    portions and mixed through the ordinary engine.  No file of the framework knows them."""
    from tokamak_b200.config import register_architecture
    from tokamak_b200.engine.replay import build_core, run_step
    from tokamak_b200.parts.base import FEED_FORWARDS, POSITIONS
    from tokamak_b200.weights import write_random_model

    FEED_FORWARDS.register("toy_top1_experts")(Top1Experts)
    POSITIONS.register("toy_scaled_partial_rope")(ScaledPartialRope)
    register_architecture(_routed_architecture())
    try:
        folder = write_random_model(tmp_path / "routed", ROUTED_CONFIG, seed=11, std=0.3, dtype="float32")
        reqs = {f"m{i}": random_tokens(97, n, seed=70 + i) for i, n in enumerate([12, 33, 64, 21, 47])}
        truth, used = {}, set()
        for rid, ids in reqs.items():
            truth[rid], choice = _routed_plain_logits(folder, ids)
            used |= set(choice.tolist())
        assert used == {0, 1, 2}, "the workload should reach every expert"
        for builder, kw in ((traces.whole, {}), (traces.tail_one_by_one, {}), (traces.portions, {}),
                            (traces.mixed, {"max_tokens": 192, "max_live": 3, "seed": 5})):
            core = build_core(folder, "float32", 192, page_size=16, max_live=3)
            records, rows = builder(reqs, **kw)
            for rec in records:
                out = run_step(core, rec)
                if out is None:
                    continue
                got = torch.from_numpy(out)
                want = torch.stack([truth[rid][p] for rid, p in rows[rec["step"]]])
                assert_logits_close(got, want, "float32", f"routed {builder.__name__} step {rec['step']}")
            assert not core.manager.live_requests()
    finally:
        FEED_FORWARDS.unregister("toy_top1_experts")
        POSITIONS.unregister("toy_scaled_partial_rope")


# ----------------------------------------------------------------------------- toys through generate

def _plain_greedy(logits_fn, prompt, n_new):
    """Greedy continuation under a plain logits function of whole sequences."""
    seq = list(prompt)
    for _ in range(n_new):
        out = logits_fn(seq)
        logits = out[0] if isinstance(out, tuple) else out
        seq.append(int(logits[-1].argmax()))
    return seq[len(prompt):]


def test_toy_stateful_mixer_and_routed_feed_forward_through_generate(tmp_path):
    """The toys meet the whole engine: several requests through ``LLM.generate`` with launch-ahead,
    portions, more requests than slots (slots are handed on) and a pool small enough to preempt.

    The decay-sum mixer plans on the host (``step.host_*``) and the routed feed-forward reads a
    routing decision back, so neither declares ``GRAPH_SAFE``: their models must run every step
    kernel by kernel, and the tokens must be the plain implementation's.  A model whose parts all
    declare it (the toy rotation is plain tensor arithmetic on device tensors) is replayed from
    CUDA graphs by the same engine and must be right as well."""
    from tokamak_b200 import LLM, SamplingParams
    from tokamak_b200.config import register_architecture, unregister_architecture
    from tokamak_b200.parts.base import FEED_FORWARDS, MIXERS, POSITIONS
    from tokamak_b200.weights import write_random_model

    MIXERS.register("toy_decay_sum")(DecaySum)
    FEED_FORWARDS.register("toy_top1_experts")(Top1Experts)
    POSITIONS.register("toy_scaled_partial_rope")(ScaledPartialRope)
    register_architecture(_toy_architecture())
    register_architecture(_routed_architecture())
    try:
        cases = [
            ("toy", TOY_CONFIG, 131, lambda f: (lambda ids: _toy_plain_logits(f, ids)), False),
            ("routed", ROUTED_CONFIG, 97, lambda f: (lambda ids: _routed_plain_logits(f, ids)), False),
            ("rope_only", dict(ROUTED_CONFIG, experts=0), 97,
             lambda f: (lambda ids: _routed_plain_logits(f, ids)), True),
        ]
        for name, raw, vocab, plain_of, safe in cases:
            folder = write_random_model(tmp_path / name, raw, seed=21, std=0.3 if name != "toy" else 0.08,
                                        dtype="float32")
            llm = LLM(folder, dtype="float32", max_seq_len=64, block_size=8, kv_pool_tokens=112,
                      max_batch_size=3, max_num_batched_tokens=40, prefill_chunk=16)
            assert llm.core.step.graph_safe is safe
            prompts = [random_tokens(vocab, n, seed=90 + n) for n in (21, 9, 30, 14, 26)]
            outs = llm.generate(prompt_token_ids=prompts,
                                sampling_params=SamplingParams(temperature=0.0, max_new_tokens=22))
            stats = llm.last_stats
            assert stats["preemptions"] > 0 and stats["mixed_steps"] > 0 and stats["decode_steps"] > 5, stats
            logits_fn = plain_of(folder)
            for prompt, out in zip(prompts, outs):
                assert out.output_token_ids == _plain_greedy(logits_fn, prompt, 22), (name, len(prompt))
            assert (llm.core.step.graph_replays > 0) is safe, name
            llm.cache_manager.check_invariants()
            assert llm.cache_manager.num_free_slots == 3
    finally:
        MIXERS.unregister("toy_decay_sum")
        FEED_FORWARDS.unregister("toy_top1_experts")
        POSITIONS.unregister("toy_scaled_partial_rope")
        unregister_architecture("ToyDecayForCausalLM")
        unregister_architecture("ToyRoutedForCausalLM")


# ---- an embedding, a head and an absolute position encoding of the test's own ---------------

@dataclass(frozen=True)
class ScaledEmbeddingSpec:
    vocab_size: int
    hidden_size: int
    scale: float
    name: str = "tok.weight"
    kind: str = "toy_scaled_embedding"


class ScaledEmbedding:
    GRAPH_SAFE = True

    def __init__(self, spec, tensors, rt):
        self.spec, self.weight = spec, tensors[spec.name]

    @staticmethod
    def expected_tensors(spec):
        from tokamak_b200.parts.base import TensorReq
        return {spec.name: TensorReq((spec.vocab_size, spec.hidden_size))}

    def forward(self, step):
        return self.weight[step.token_ids.long()].float() * self.spec.scale


@dataclass(frozen=True)
class CappedHeadSpec:
    """logits = cap * tanh((h W^T + b) / cap)."""
    vocab_size: int
    hidden_size: int
    cap: float
    kind: str = "toy_capped_head"


class CappedHead:
    GRAPH_SAFE = True

    def __init__(self, spec, embedding, tensors, rt):
        self.spec, self.weight, self.bias = spec, tensors["out.weight"], tensors["out.bias"]

    @staticmethod
    def expected_tensors(spec):
        from tokamak_b200.parts.base import TensorReq
        return {"out.weight": TensorReq((spec.vocab_size, spec.hidden_size)),
                "out.bias": TensorReq((spec.vocab_size,), role="vector")}

    def forward(self, h, step=None):
        from tokamak_b200.parts.base import linear, sum_parts
        logits = sum_parts(linear(h, self.weight, out_dtype=torch.float32), torch.float32) + self.bias
        return self.spec.cap * torch.tanh(logits / self.spec.cap)


@dataclass(frozen=True)
class LearnedPositionsSpec:
    """An absolute encoding: row ``position`` of a learned table is added to the embedded token."""
    max_positions: int
    hidden_size: int
    kind: str = "toy_learned_positions"


class LearnedPositions:
    GRAPH_SAFE = True

    def __init__(self, spec, tensors, rt):
        self.table = tensors["pos.weight"]

    @staticmethod
    def expected_tensors(spec):
        from tokamak_b200.parts.base import TensorReq
        return {"pos.weight": TensorReq((spec.max_positions, spec.hidden_size))}

    def add_to_embedding(self, resid, step):
        resid += self.table[step.positions.long()].float()


ABS_CONFIG = {"architectures": ["ToyAbsoluteForCausalLM"], "vocab_size": 83, "hidden_size": 48, "heads": 3,
              "head_dim": 16, "inter": 56, "eps": 1e-6, "cap": 6.0, "max_position_embeddings": 96}


def _absolute_architecture():
    from tokamak_b200.config import Architecture
    from tokamak_b200.models.decoder import LayerCall, ModelSpec
    from tokamak_b200.parts.attention import AttentionSpec
    from tokamak_b200.parts.block import PreNormBlockSpec
    from tokamak_b200.parts.feedforward import SwiGLUSpec
    from tokamak_b200.parts.norm import RMSNormSpec
    from tokamak_b200.parts.position import NoPositionSpec

    @dataclass(frozen=True)
    class Config:
        vocab_size: int
        hidden_size: int
        heads: int
        head_dim: int
        inter: int
        eps: float
        cap: float
        max_position_embeddings: int
        architecture: str = "ToyAbsoluteForCausalLM"
        eos_token_ids: tuple = ()

    def parse_config(raw, eos_token_ids=None):
        return Config(**{k: raw[k] for k in ABS_CONFIG if k != "architectures"})

    def model_spec(cfg):
        H, norm = cfg.hidden_size, RMSNormSpec(cfg.hidden_size, cfg.eps)
        attn = AttentionSpec(H, cfg.heads, cfg.heads, cfg.head_dim, NoPositionSpec(), qk_norm_eps=None)
        blocks = (PreNormBlockSpec("l0", norm, attn, norm, SwiGLUSpec(H, cfg.inter), "l0.n1", "l0.attn.",
                                   "l0.n2", "l0.mlp."),)
        return ModelSpec(ScaledEmbeddingSpec(cfg.vocab_size, H, H ** 0.5), blocks, (LayerCall("l0", "l0"),),
                         norm, "final", CappedHeadSpec(cfg.vocab_size, H, cfg.cap),
                         embedding_position=LearnedPositionsSpec(cfg.max_position_embeddings, H))

    return Architecture("ToyAbsoluteForCausalLM", parse_config, model_spec)


def _absolute_plain_logits(folder, ids):
    cfg, w = plain.load_folder(folder)
    w = {k: v.double() for k, v in w.items()}
    T, H, d, heads, eps = len(ids), cfg["hidden_size"], cfg["head_dim"], cfg["heads"], cfg["eps"]
    x = w["tok.weight"][torch.tensor(ids)] * H ** 0.5 + w["pos.weight"][:T]
    h = plain.rms_norm(x, w["l0.n1"], eps)
    q = (h @ w["l0.attn.q_proj.weight"].T).view(T, heads, d)
    k = (h @ w["l0.attn.k_proj.weight"].T).view(T, heads, d)
    v = (h @ w["l0.attn.v_proj.weight"].T).view(T, heads, d)
    x = x + plain.causal_attention(q, k, v).reshape(T, -1) @ w["l0.attn.o_proj.weight"].T
    x = x + plain.swiglu_mlp(plain.rms_norm(x, w["l0.n2"], eps), w["l0.mlp.gate_proj.weight"],
                             w["l0.mlp.up_proj.weight"], w["l0.mlp.down_proj.weight"])
    logits = plain.rms_norm(x, w["final"], eps) @ w["out.weight"].T + w["out.bias"]
    return cfg["cap"] * torch.tanh(logits / cfg["cap"])


def test_toy_embedding_head_and_absolute_positions(tmp_path):
    """Embedding and head are registry roles like the other parts, and a position encoding may
    sit at the embedding instead of inside the mixers: an architecture with a scaled embedding, a
    learned absolute position table and a biased, soft-capped head is described by the test
    alone, replayed in portions and mixed, and generated from with CUDA graphs."""
    from tokamak_b200 import LLM, SamplingParams
    from tokamak_b200.config import ConfigError, register_architecture, unregister_architecture
    from tokamak_b200.engine.replay import build_core, run_step
    from tokamak_b200.parts.base import EMBEDDINGS, HEADS, POSITIONS
    from tokamak_b200.weights import write_random_model

    EMBEDDINGS.register("toy_scaled_embedding")(ScaledEmbedding)
    HEADS.register("toy_capped_head")(CappedHead)
    POSITIONS.register("toy_learned_positions")(LearnedPositions)
    register_architecture(_absolute_architecture())
    try:
        folder = write_random_model(tmp_path / "abs", ABS_CONFIG, seed=5, std=0.2, dtype="float32")
        reqs = {f"a{i}": random_tokens(83, n, seed=30 + i) for i, n in enumerate([11, 40, 64, 25])}
        truth = {rid: _absolute_plain_logits(folder, ids) for rid, ids in reqs.items()}
        for builder, kw in ((traces.portions, {}), (traces.mixed, {"max_tokens": 192, "max_live": 3, "seed": 8})):
            core = build_core(folder, "float32", 192, page_size=16, max_live=3)
            records, rows = builder(reqs, **kw)
            for rec in records:
                out = run_step(core, rec)
                if out is None:
                    continue
                want = torch.stack([truth[rid][p] for rid, p in rows[rec["step"]]])
                assert_logits_close(torch.from_numpy(out), want, "float32", f"absolute {builder.__name__}")
        llm = LLM(folder, dtype="float32", block_size=16, max_batch_size=4)
        assert llm.core.step.graph_safe
        prompts = [random_tokens(83, n, seed=60 + n) for n in (7, 19, 33)]
        outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(temperature=0.0, max_new_tokens=20))
        for prompt, out in zip(prompts, outs):
            assert out.output_token_ids == _plain_greedy(lambda ids: _absolute_plain_logits(folder, ids), prompt, 20)
        assert llm.core.step.graph_replays > 0
        # the architecture lists no engine options: a window is refused with the reason
        with pytest.raises(ConfigError, match="does not take the engine option 'window'"):
            LLM(folder, dtype="float32", attention_policy="window:8")
    finally:
        EMBEDDINGS.unregister("toy_scaled_embedding")
        HEADS.unregister("toy_capped_head")
        POSITIONS.unregister("toy_learned_positions")
        unregister_architecture("ToyAbsoluteForCausalLM")
