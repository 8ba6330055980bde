"""The attention mixer: grouped-query attention over paged keys and values."""

from __future__ import annotations

import contextlib
from dataclasses import dataclass

import torch

from ..cache.manager import KVPagesNeed
from ..csrc import ops
from .base import (MIXERS, POSITIONS, SWAPPED_GEMM_MAX_TOKENS, OwedNorm, Runtime, TensorReq, chain_of,
                   graph_safe, linear, tensor_bytes)


@dataclass(frozen=True)
class AttentionSpec:
    """Sizes and constants of one attention mixer.

    ``qk_norm_eps`` of ``None`` switches the per-head norm of q and k off;
    ``window`` of ``None`` means every earlier key is seen; ``own_kv=False``
    describes a layer without key and value projections that reads the pages
    another layer wrote (the schedule names which).
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: object                       # a position spec (kind, ...)
    qk_norm_eps: float | None = None
    window: int | None = None
    own_kv: bool = True
    softmax_scale: float | None = None     # default head_dim ** -0.5
    kind: str = "attention"


@MIXERS.register("attention")
class Attention:
    """Projections, per-head q/k norm, rotation, page write and attention
    (src/tokamak/model/transformer.py:22-86 with the step context's
    store-then-attend order, src/tokamak/model/step_context.py:88).

    The q, k and v matrices are stacked into one ``[(Hq + 2 Hkv) d, H]`` operand.
    """

    def __init__(self, spec: AttentionSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads are not a multiple of "
                             f"{spec.num_kv_heads} key/value heads")
        if spec.head_dim > 256 or spec.head_dim % 4:
            raise ValueError(f"head_dim {spec.head_dim} is not taken by the attention kernels: "
                             f"they need a multiple of 4 up to 256")
        self.spec = spec
        self.rt = rt
        mats = [tensors[prefix + "q_proj.weight"]]
        if spec.own_kv:
            mats += [tensors[prefix + "k_proj.weight"], tensors[prefix + "v_proj.weight"]]
        self.w_qkv = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        self.w_o = tensors[prefix + "o_proj.weight"]
        self.q_norm_w = tensors.get(prefix + "q_norm.weight") if spec.qk_norm_eps is not None else None
        self.k_norm_w = tensors.get(prefix + "k_norm.weight") if spec.qk_norm_eps is not None else None
        self.position = POSITIONS.get(spec.position.kind)(spec.position, tensors, rt)
        if not hasattr(self.position, "rotary_table"):
            raise ValueError(f"position encoding {spec.position.kind!r} does not rotate queries and keys "
                             f"(no rotary_table); give it the model's embedding_position seat instead")
        self.scale = spec.softmax_scale if spec.softmax_scale is not None else spec.head_dim ** -0.5
        self.prefill_heads = spec.num_heads      # work items per block of prompt tokens (see parts/base.py)

    @staticmethod
    def expected_tensors(spec: AttentionSpec, prefix: str) -> dict[str, TensorReq]:
        h, d = spec.hidden_size, spec.head_dim
        out = {
            prefix + "q_proj.weight": TensorReq((spec.num_heads * d, h)),
            prefix + "o_proj.weight": TensorReq((h, spec.num_heads * d)),
        }
        if spec.own_kv:
            out[prefix + "k_proj.weight"] = TensorReq((spec.num_kv_heads * d, h))
            out[prefix + "v_proj.weight"] = TensorReq((spec.num_kv_heads * d, h))
        if spec.qk_norm_eps is not None:
            out[prefix + "q_norm.weight"] = TensorReq((d,), role="vector")
            if spec.own_kv:
                out[prefix + "k_norm.weight"] = TensorReq((d,), role="vector")
        out.update(POSITIONS.get(spec.position.kind).expected_tensors(spec.position))
        return out

    def cache_need(self) -> KVPagesNeed:
        return KVPagesNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def GRAPH_SAFE(self) -> bool:
        return graph_safe(self.position)

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_qkv, self.w_o, self.q_norm_w, self.k_norm_w)

    TAKES_OWED_NORM = True     # the q|k|v product pays an owed norm scale in its epilogue
    TAKES_THEN_NORM = True     # the output product can add itself to the residual stream

    def forward(self, h, step, cache_view, then_norm=None):
        spec = self.spec
        n = h.shape[0]
        q = torch.empty((n, spec.num_heads, spec.head_dim), dtype=h.dtype, device=h.device)
        table, rotary_dim = self.position.rotary_table(step)
        if (h.dtype == torch.bfloat16 and n <= SWAPPED_GEMM_MAX_TOKENS and spec.own_kv
                and spec.head_dim == ops.QKV_ROPE_HEAD_DIM and rotary_dim in (0, spec.head_dim)
                and spec.hidden_size % 8 == 0 and cache_view.k.dtype == torch.bfloat16):
            # few tokens and heads that are whole tiles: norm, rotation and page write ride in
            # the product's epilogue
            splits, stages, _ = ops.swapped_gemm_plan(self.w_qkv.shape[0], spec.hidden_size, n)
            colscale, x = ((h.sumsq, h.dim, h.eps), h.xb) if isinstance(h, OwedNorm) else (None, h)
            ops.gemm_qkv_rope(self.w_qkv, x, step.err, splits, q, cache_view.k, cache_view.v, step.positions,
                              step.tok_req, step.req_slot, cache_view.table, self.q_norm_w, self.k_norm_w,
                              table, n_q_heads=spec.num_heads, n_kv_heads=spec.num_kv_heads,
                              eps=spec.qk_norm_eps or 0.0, max_stages=stages, colscale=colscale,
                              req_q_len=step.req_q_len, req_kv_len=step.req_kv_len, chain=chain_of(step))
        else:
            self._project_and_rotate(h, q, table, rotary_dim, step, cache_view)
        out = torch.empty_like(q)
        paged_attention(q, out, cache_view, step, scale=self.scale, window=spec.window)
        return linear(out.view(n, spec.num_heads * spec.head_dim), self.w_o, err=step.err, then_norm=then_norm,
                      chain=chain_of(step))

    def _project_and_rotate(self, h, q, table, rotary_dim, step, cache_view) -> None:
        """The q|k|v product, then norm, rotation and page write in a kernel of their own."""
        spec = self.spec
        qkv = linear(h, self.w_qkv, err=step.err)
        ops.rope_kv(qkv, q, cache_view.k if spec.own_kv else None,
                    cache_view.v if spec.own_kv else None,
                    step.positions, step.tok_req, step.req_slot, cache_view.table,
                    self.q_norm_w, self.k_norm_w, table, step.err,
                    n_q_heads=spec.num_heads, n_kv_heads=spec.num_kv_heads, head_dim=spec.head_dim,
                    rotary_dim=rotary_dim, eps=spec.qk_norm_eps or 0.0, write_kv=spec.own_kv,
                    req_q_len=step.req_q_len, req_kv_len=step.req_kv_len)


_SIDE: dict = {}


def _side_stream(device: torch.device):
    """A second stream of the device and the two events that fork to it and join from it."""
    entry = _SIDE.get(device)
    if entry is None:
        entry = (torch.cuda.Stream(device), torch.cuda.Event(), torch.cuda.Event())
        _SIDE[device] = entry
    return entry


def paged_attention(q: torch.Tensor, out: torch.Tensor, cache_view, step, *, scale: float,
                    window: int | None) -> None:
    """Attention of every token of the step over the pages of its own request.

    Chooses the kernels.  bfloat16 with a head_dim the tiled kernels take: single next
    tokens go to the split-K decode kernel, portions of prompts to the tcgen05 flash
    prefill kernel (or to the mma.sync one for page sizes it does not take).  float32,
    and every other shape, runs on the general kernel.
    """
    ops.flush_chains()     # q and the pages may come from a product that is still queued: launch it on this stream
    n, hq, d = q.shape
    hkv, page = cache_view.k.shape[1], cache_view.k.shape[2]
    bf16 = q.dtype == torch.bfloat16
    n_dec = step.decode_items.numel()
    n_pf = step.prefill_items.numel()
    dec_tiled = bf16 and n_dec > 0 and ops.decode_kernel_takes(hq, hkv, d, page)
    pf_tiled = bf16 and n_pf > 0 and ops.prefill_kernel_takes(hq, hkv, d, page)
    # In a mixed step the two kernels touch different tokens.  One portion against a long context
    # is few blocks (one per pair of 128-row query tiles and head), so the decode kernel runs
    # beside it on a second stream instead of after it.
    beside = dec_tiled and pf_tiled and not torch.cuda.is_current_stream_capturing()
    if beside:
        side, fork, join = _side_stream(q.device)
        fork.record()
        side.wait_event(fork)
    if dec_tiled:
        with torch.cuda.stream(side) if beside else contextlib.nullcontext():
            if ops.decode_uses_balanced(q.device, n_dec, hkv, step.max_kv_len):
                ops.attention_decode_balanced(q, out, cache_view.k, cache_view.v, step.decode_items, step.positions,
                                              step.tok_req, step.req_slot, cache_view.table, step.err, scale=scale,
                                              window=window,
                                              blocks=ops.decode_balanced_blocks(q.device, n_dec, hkv, step.max_kv_len))
            else:
                ops.attention_decode(q, out, cache_view.k, cache_view.v, step.decode_items, step.positions,
                                     step.tok_req, step.req_slot, cache_view.table, step.err, scale=scale,
                                     window=window, n_splits=ops.decode_splits(n_dec, hkv, step.max_kv_len))
            if beside:
                join.record()
    if pf_tiled and ops.prefill_tc_kernel_takes(hq, hkv, d, page):
        ops.attention_prefill_tc(q, out, cache_view.k, cache_view.v, step.prefill_tc,
                                 cache_view.table, step.err, scale=scale, window=window)
    elif pf_tiled:
        ops.attention_prefill(q, out, cache_view.k, cache_view.v, step.prefill_tiles,
                              step.req_q_start, step.req_q_len, step.req_kv_len, step.req_slot,
                              cache_view.table, step.err, scale=scale, window=window)
    if beside:
        torch.cuda.current_stream().wait_event(join)
    dec_rest = n_dec > 0 and not dec_tiled
    pf_rest = n_pf > 0 and not pf_tiled
    if dec_rest or pf_rest:
        items = None if (dec_rest and pf_rest) else (step.decode_items if dec_rest else step.prefill_items)
        ops.attention_plain(q, out, cache_view.k, cache_view.v, step.positions, step.tok_req,
                            step.req_slot, cache_view.table, step.err, scale=scale, window=window,
                            items=items)
