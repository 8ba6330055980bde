"""Python entry points of the CUDA kernels: argument checks, then one C call each.

Every function takes CUDA tensors and launches on PyTorch's current stream, so
the calls can be recorded into a CUDA graph like any other stream work.  There
is no CPU path: a tensor that is not on a CUDA device is an error.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import numpy as np
import torch

from .lib import library

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    """A kernel launch failed or refused its arguments."""


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Every launch asks for it, so the fast accessor is used where
    this torch has it (no Stream object is built)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


LAUNCHES = 0     # kernels of this library launched (or recorded into a graph) so far
_ACTIVE_CHAINS: list = []      # product chains with queued products (see ProductChain)


def _check(code: int, what: str) -> None:
    global LAUNCHES
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}")
    LAUNCHES += 1


def _lib():
    """The library, for a wrapper that is about to launch: products that are still queued in a
    chain are launched first, so that no kernel reads a result that does not exist yet."""
    if _ACTIVE_CHAINS:
        flush_chains()
    return library()


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _want(t: torch.Tensor, dtype: torch.dtype | None, name: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (the engine has no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"unsupported element type {dtype}; the kernels take float32 and bfloat16")


def embed_gather(table: torch.Tensor, ids: torch.Tensor, resid: torch.Tensor, err: torch.Tensor) -> None:
    """resid[t] = float32(table[ids[t]])."""
    _want(table, None, "table"); _want(ids, torch.int32, "ids"); _want(resid, torch.float32, "resid")
    n = ids.numel()
    vocab, hidden = table.shape
    if resid.shape[-1] != hidden or resid.numel() < n * hidden:
        raise KernelError("resid is too small for the tokens")
    _check(_lib().tk_embed_gather(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(),
                                     resid.data_ptr(), n, hidden, vocab, err.data_ptr(), _stream()),
           "embed_gather")


class UpdateBuffers:
    """Device side of the update list that the kernels opening a step apply (``step_state.cu``):
    the list itself, the engine's slot records and the flat block tables it writes into."""

    def __init__(self, ctl: torch.Tensor, max_rec: int, max_tab: int, records: torch.Tensor,
                 tables: torch.Tensor):
        _want(ctl, torch.int32, "ctl"); _want(records, torch.int32, "records"); _want(tables, torch.int32, "tables")
        if ctl.numel() < 2 + 9 * max_rec + 2 * max_tab:
            raise KernelError("the update list is too small for its limits")
        if records.dim() != 2 or records.shape[1] != library().tk_slot_words():
            raise KernelError(f"slot records must be [slots, {library().tk_slot_words()}]")
        self.ctl, self.max_rec, self.max_tab, self.records, self.tables = ctl, max_rec, max_tab, records, tables

    def args(self) -> tuple:
        return (self.ctl.data_ptr(), self.max_rec, self.max_tab, self.records.data_ptr(),
                self.records.shape[0], self.tables.data_ptr(), self.tables.numel())


def step_begin(upd: UpdateBuffers, token_ids: torch.Tensor, req_q_start: torch.Tensor,
               req_kv_len: torch.Tensor, req_slot: torch.Tensor, req_fed: torch.Tensor | None,
               err: torch.Tensor) -> None:
    """Open a step laid out by the host: apply the pending updates, put the last sampled token of
    every request marked in ``req_fed`` at its place in ``token_ids``, and note in each request's
    record that the cache will hold ``req_kv_len`` positions."""
    for name, t in (("token_ids", token_ids), ("req_q_start", req_q_start), ("req_kv_len", req_kv_len),
                    ("req_slot", req_slot)):
        _want(t, torch.int32, name)
    n = req_slot.numel()
    if req_q_start.numel() < n or req_kv_len.numel() < n or (req_fed is not None and req_fed.numel() < n):
        raise KernelError("a per-request array is shorter than the batch")
    _check(_lib().tk_step_begin(*upd.args(), token_ids.data_ptr(), req_q_start.data_ptr(),
                                   req_kv_len.data_ptr(), req_slot.data_ptr(), _ptr(req_fed), n,
                                   token_ids.numel(), err.data_ptr(), _stream()), "step_begin")


def decode_begin(upd: UpdateBuffers, dec_slots: torch.Tensor, n_reqs: int, max_positions: int,
                 token_ids: torch.Tensor, positions: torch.Tensor, req_kv_len: torch.Tensor,
                 err: torch.Tensor) -> None:
    """Open a step of single next tokens from the slot records alone: token, position and cache
    length of the request in slot ``dec_slots[r]`` go to row ``r`` and its record moves on."""
    for name, t in (("dec_slots", dec_slots), ("token_ids", token_ids), ("positions", positions),
                    ("req_kv_len", req_kv_len)):
        _want(t, torch.int32, name)
        if t.numel() < n_reqs:
            raise KernelError(f"{name} is shorter than the batch")
    _check(_lib().tk_decode_begin(*upd.args(), dec_slots.data_ptr(), n_reqs, max_positions,
                                     token_ids.data_ptr(), positions.data_ptr(), req_kv_len.data_ptr(),
                                     err.data_ptr(), _stream()), "decode_begin")


SAMPLING_MAX_VOCAB = 1 << 21      # the pieces of the first histograms of sampling.cu hold vocab / 8 masses
SAMPLING_MAX_ROWS = 65535


def _sampling_takes(rows: int, vocab: int) -> None:
    if vocab > SAMPLING_MAX_VOCAB or rows > SAMPLING_MAX_ROWS:
        raise KernelError(f"the sampling kernel takes up to {SAMPLING_MAX_ROWS} rows of up to {SAMPLING_MAX_VOCAB} "
                          f"logits, got {rows} x {vocab}")


def sample_slots(logits: torch.Tensor, records: torch.Tensor, row_slot: torch.Tensor,
                 out_tokens: torch.Tensor, err: torch.Tensor) -> None:
    """One token per row of float32 logits, with the parameters, seed and counter of the slot
    record ``records[row_slot[r]]``; the token is also written into the record and its counter
    advanced (see sampling.cu)."""
    _want(logits, torch.float32, "logits"); _want(records, torch.int32, "records")
    _want(row_slot, torch.int32, "row_slot"); _want(out_tokens, torch.int32, "out_tokens")
    rows, vocab = logits.shape
    if row_slot.numel() < rows or out_tokens.numel() < rows:
        raise KernelError("a per-row sampling tensor is shorter than the batch")
    _sampling_takes(rows, vocab)
    _check(_lib().tk_sample_slots(logits.data_ptr(), logits.stride(0), records.data_ptr(),
                                     row_slot.data_ptr(), records.shape[0], out_tokens.data_ptr(), rows, vocab,
                                     err.data_ptr(), _stream()), "sample_slots")


def wait_probe(limit: int, err: torch.Tensor) -> None:
    """Test aid: one block waits on a barrier that nobody arrives at, gives up after ``limit``
    polls and reports it through the error word exactly as the tcgen05 kernels would."""
    _want(err, torch.int32, "err")
    _check(_lib().tk_wait_probe(int(limit), err.data_ptr(), _stream()), "wait_probe")


def probe_mma_issue(mode: int, n: int, reps: int = 96) -> list[dict]:
    """Measurement aid (csrc/tcgen05_probe.cu): what ``reps`` tcgen05.mma of M 128 x N ``n`` x K 16
    cost the issuing thread.  ``mode`` 0: both operands in shared memory; 1: A in tensor memory;
    2 / 3: the same with two issuing threads; 4: eight of N ``n`` from shared memory, then four of
    N 128 with A in tensor memory, as the prefill attention kernel issues them.  Per issuing thread:
    clocks and nanoseconds per product until issued and until done."""
    out = torch.zeros(8, dtype=torch.int64, device="cuda")
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    _check(_lib().tk_probe_mma_issue(int(mode), int(n), int(reps), out.data_ptr(), err.data_ptr(), _stream()),
           "probe_mma_issue")
    torch.cuda.synchronize()
    if int(err[0]) != 0:
        raise KernelError(f"probe_mma_issue: a bounded wait ran out (code {int(err[0])})")
    host = out.tolist()
    threads = 2 if mode in (2, 3) else 1
    return [{"issue_clk": host[4 * i] / reps, "done_clk": host[4 * i + 1] / reps,
             "issue_ns": host[4 * i + 2] / reps, "done_ns": host[4 * i + 3] / reps} for i in range(threads)]


def probe_softmax_tile(variant: int, warpgroups: int, tiles: int = 400) -> dict:
    """Measurement aid (csrc/tcgen05_probe.cu): clocks per 64-key tile of one softmax warp, with
    ``warpgroups`` warps on every scheduler (1 or 2), in one of the loop's forms (0: as the prefill
    attention kernel has it; 1: four chains for the maximum; 2: the second half of the scores
    loaded under the first half's maximum; 3: both; 4 / 5 / 6: one, two, all four of every four
    exponentials by a polynomial on the multiply-add pipe)."""
    out = torch.zeros(16, dtype=torch.int32, device="cuda")
    _check(_lib().tk_probe_softmax_tile(int(variant), int(warpgroups), int(tiles), sm_count(out.device),
                                        out.data_ptr(), _stream()), "probe_softmax_tile")
    torch.cuda.synchronize()
    h = [int(x) & 0xFFFFFFFF for x in out.tolist()]
    names = ["load", "maximum", "exponentials_store", "store_arrived", "fence"]
    res = {k: h[i] / tiles for i, k in enumerate(names)}
    res["tile"] = h[5] / tiles
    return res


def add_rmsnorm(resid: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor,
                out: torch.Tensor, eps: float, rows: torch.Tensor | None = None) -> None:
    """x = resid (+ delta), written back unless ``rows`` is given; out = weight * x * rsqrt(mean x^2 + eps).

    ``delta`` is the branch output in the activation type, or a 3-D float32 tensor of partial
    sums ``[parts, tokens, hidden]`` (from a split-K product) that the kernel adds up."""
    _want(resid, torch.float32, "resid"); _want(weight, torch.float32, "weight"); _want(out, None, "out")
    hidden = resid.shape[-1]
    if weight.numel() != hidden or out.shape[-1] != hidden:
        raise KernelError("norm width mismatch")
    parts, n_parts, part_stride = None, 0, 0
    if delta is not None and delta.dim() == 3:
        _want(delta, torch.float32, "delta partial sums")
        if delta.shape[1:] != resid.shape:
            raise KernelError("partial sums and resid differ in shape")
        parts, n_parts, part_stride, delta = delta, delta.shape[0], delta.stride(0), None
    elif delta is not None:
        _want(delta, out.dtype, "delta")
        if delta.shape != resid.shape:
            raise KernelError("delta and resid differ in shape")
    if rows is not None:
        _want(rows, torch.int32, "rows")
        n_rows = rows.numel()
    else:
        n_rows = resid.numel() // hidden
    if out.numel() < n_rows * hidden:
        raise KernelError("out is too small")
    _check(_lib().tk_add_rmsnorm(resid.data_ptr(), _ptr(delta), _ptr(parts), n_parts, part_stride,
                                    weight.data_ptr(), out.data_ptr(), _ptr(rows), n_rows, hidden,
                                    float(eps), dtype_code(out.dtype), _stream()), "add_rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out[t, j] = silu(gate[t, j]) * up[t, j]; a row of ``gate_up`` holds ``block`` gate values,
    then the ``block`` up values of the same outputs, and so on (``block = 0``: all I gate values,
    then all up values).  ``gate_up`` may be float32 partial sums ``[parts, tokens, 2I]`` that the
    kernel adds up first."""
    _want(gate_up, None, "gate_up"); _want(out, None, "out")
    parts, n_parts, part_stride = None, 0, 0
    if gate_up.dim() == 3:
        _want(gate_up, torch.float32, "gate_up partial sums")
        parts, n_parts, part_stride = gate_up, gate_up.shape[0], gate_up.stride(0)
        n, two_i = gate_up.shape[1:]
        gate_up = None
    else:
        if gate_up.dtype != out.dtype:
            raise KernelError("gate_up and out differ in element type")
        n, two_i = gate_up.shape
    if two_i % 2 or out.shape != (n, two_i // 2):
        raise KernelError("swiglu shape mismatch")
    block = block or two_i // 2
    if (two_i // 2) % block:
        raise KernelError("the gate/up block must divide the intermediate size")
    _check(_lib().tk_swiglu(_ptr(gate_up), _ptr(parts), n_parts, part_stride, out.data_ptr(), n,
                               two_i // 2, block, dtype_code(out.dtype), _stream()), "swiglu")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """``[tokens, len(inv_freq), 2]`` float32: (cos, sin) of ``float(position) * inv_freq[j]``."""
    _want(positions, torch.int32, "positions"); _want(inv_freq, torch.float32, "inv_freq")
    n, half = positions.numel(), inv_freq.numel()
    table = torch.empty((n, half, 2), dtype=torch.float32, device=positions.device)
    _check(_lib().tk_rope_table(positions.data_ptr(), inv_freq.data_ptr(), table.data_ptr(), n, 2 * half,
                                   _stream()), "rope_table")
    return table


def rope_kv(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor | None,
            v_cache: torch.Tensor | None, positions: torch.Tensor, tok_req: torch.Tensor,
            req_slot: torch.Tensor, block_table: torch.Tensor, q_norm_w: torch.Tensor | None,
            k_norm_w: torch.Tensor | None, table: torch.Tensor | None, err: torch.Tensor, *,
            n_q_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int, eps: float,
            write_kv: bool = True, req_q_len: torch.Tensor | None = None,
            req_kv_len: torch.Tensor | None = None) -> None:
    """Per-head norm of q and k, rotation, and the write of k and v into their pages.

    ``qkv`` is ``[tokens, (Hq + 2 Hkv) d]`` in the activation type, or float32 partial sums
    ``[parts, tokens, (Hq + 2 Hkv) d]`` that the kernel adds up.  With ``req_q_len`` and
    ``req_kv_len`` the last token of every request also clears the rest of a page begun in
    this step (the tcgen05 attention kernel loads whole pages and relies on it)."""
    _want(qkv, None, "qkv"); _want(q_out, None, "q_out")
    parts, n_parts = None, 0
    if qkv.dim() == 3:
        _want(qkv, torch.float32, "qkv partial sums")
        parts, n_parts = qkv, qkv.shape[0]
        n, row = qkv.shape[1:]
        qkv = None
    else:
        if qkv.dtype != q_out.dtype:
            raise KernelError("qkv and q_out differ in element type")
        n, row = qkv.shape
    need = (n_q_heads + (2 * n_kv_heads if write_kv else 0)) * head_dim
    if row < need:
        raise KernelError(f"qkv rows hold {row} values, {need} needed")
    for name, t in (("positions", positions), ("tok_req", tok_req), ("req_slot", req_slot),
                    ("block_table", block_table)):
        _want(t, torch.int32, name)
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("table", table)):
        if t is not None:
            _want(t, torch.float32, name)
    if head_dim % 4 or rotary_dim % 4 or rotary_dim > head_dim:
        raise KernelError(f"head_dim {head_dim} and rotary_dim {rotary_dim} must be multiples of 4 "
                          f"with rotary_dim <= head_dim")
    if q_norm_w is not None and q_norm_w.numel() != head_dim:
        raise KernelError("q_norm weight does not match head_dim")
    if k_norm_w is not None and k_norm_w.numel() != head_dim:
        raise KernelError("k_norm weight does not match head_dim")
    if table is not None and table.shape != (n, rotary_dim // 2, 2):
        raise KernelError(f"the rotation table must be [{n}, {rotary_dim // 2}, 2], got {tuple(table.shape)}")
    if table is None and rotary_dim != 0:
        raise KernelError("rotary_dim without a rotation table")
    if write_kv:
        _want(k_cache, q_out.dtype, "k_cache"); _want(v_cache, q_out.dtype, "v_cache")
        num_pages, hkv, page_size, d = k_cache.shape
        if hkv != n_kv_heads or d != head_dim or v_cache.shape != k_cache.shape:
            raise KernelError("cache pages do not match the heads")
    else:
        num_pages, page_size = 0, 1
    _check(_lib().tk_rope_kv(_ptr(qkv), _ptr(parts), n_parts, q_out.data_ptr(), _ptr(k_cache), _ptr(v_cache),
                                positions.data_ptr(), tok_req.data_ptr(), req_slot.data_ptr(),
                                block_table.data_ptr(), _ptr(req_q_len), _ptr(req_kv_len),
                                _ptr(q_norm_w), _ptr(k_norm_w), _ptr(table),
                                err.data_ptr(), n, req_slot.numel(), n_q_heads, n_kv_heads, head_dim,
                                rotary_dim, row, page_size, block_table.shape[1], num_pages,
                                1 if write_kv else 0, float(eps), dtype_code(q_out.dtype), _stream()),
           "rope_kv")


def attention_plain(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    positions: torch.Tensor, tok_req: torch.Tensor, req_slot: torch.Tensor,
                    block_table: torch.Tensor, err: torch.Tensor, *, scale: float,
                    window: int | None = None, items: torch.Tensor | None = None) -> None:
    """Paged attention of a mixed batch; q and out are [N, Hq, d].

    ``items`` restricts the work to the listed token indices (rows of q and out)."""
    _want(q, None, "q"); _want(out, q.dtype, "out")
    _want(k_cache, q.dtype, "k_cache"); _want(v_cache, q.dtype, "v_cache")
    n, hq, d = q.shape
    num_pages, hkv, page_size, dk = k_cache.shape
    if dk != d or v_cache.shape != k_cache.shape or out.shape != q.shape:
        raise KernelError("attention shape mismatch")
    if hq % hkv:
        raise KernelError(f"{hq} query heads are not a multiple of {hkv} key/value heads")
    if d > 256:
        raise KernelError(f"head_dim {d} is beyond the kernels' limit of 256")
    _check(_lib().tk_attention_plain(q.data_ptr(), out.data_ptr(), k_cache.data_ptr(),
                                        v_cache.data_ptr(), positions.data_ptr(), tok_req.data_ptr(),
                                        req_slot.data_ptr(), block_table.data_ptr(), _ptr(items),
                                        err.data_ptr(), n if items is None else items.numel(),
                                        req_slot.numel(), hq, hkv, d, page_size,
                                        block_table.shape[1], num_pages, int(window or 0),
                                        float(scale), dtype_code(q.dtype), _stream()),
           "attention_plain")


def decode_splits(n_items: int, n_kv_heads: int, max_kv_len: int) -> int:
    """How many key splits the decode kernel gets.

    Two blocks of three stages fit an SM, or three blocks of two stages (the kernel takes two
    stages when its grid is larger than two blocks per SM), so up to 444 run at a time.  A second,
    partly filled wave costs as much as the first (measured at Qwen3-8B head sizes with two
    blocks to an SM: batch 8 takes 30 us with 4 splits = 256 blocks and 43 us with 5), so the
    splits are chosen to stay within one wave.  A block keeps at least eight 16-key tiles, and a
    multiple of four, so that each of its four warps has the same number (one sequence of 4,096
    keys: 9.6 us with 16 splits, 10.1 with 18, 8.8 with 32).  Where three blocks per SM do not
    give more blocks than two per SM hold, the splits are those of two per SM."""
    tiles = max(1, -(-max_kv_len // 16))
    pairs = max(1, n_items * n_kv_heads)

    def splits_for(slots: int) -> int:
        most = max(1, min(slots // pairs, 128))
        per_split = max(8, -(-(-(-tiles // most)) // 4) * 4)
        return max(1, min(-(-tiles // per_split), most))

    wide = splits_for(444)
    return wide if pairs * wide > 296 else splits_for(296)


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     items: torch.Tensor, positions: torch.Tensor, tok_req: torch.Tensor,
                     req_slot: torch.Tensor, block_table: torch.Tensor, err: torch.Tensor, *,
                     scale: float, window: int | None, n_splits: int,
                     scratch: torch.Tensor | None = None) -> None:
    """Split-K paged attention for the single next tokens listed in ``items`` (bfloat16 only)."""
    _want(q, torch.bfloat16, "q"); _want(out, torch.bfloat16, "out")
    _want(k_cache, torch.bfloat16, "k_cache"); _want(v_cache, torch.bfloat16, "v_cache")
    _want(items, torch.int32, "items")
    n, hq, d = q.shape
    num_pages, hkv, page_size, dk = k_cache.shape
    if not decode_kernel_takes(hq, hkv, d, page_size):
        raise KernelError(f"the split-K decode kernel does not take heads {hq}/{hkv}, head_dim {d}, "
                          f"page size {page_size}")
    n_items = items.numel()
    counters = _decode_counters(q.device, n_items * hkv)
    need = n_items * hq * n_splits * (d + 2)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    else:
        _want(scratch, torch.float32, "scratch")
        if scratch.numel() < need:
            raise KernelError(f"scratch holds {scratch.numel()} floats, {need} needed")
    _check(_lib().tk_attention_decode(q.data_ptr(), out.data_ptr(), k_cache.data_ptr(),
                                         v_cache.data_ptr(), scratch.data_ptr(), counters.data_ptr(),
                                         items.data_ptr(),
                                         positions.data_ptr(), tok_req.data_ptr(), req_slot.data_ptr(),
                                         block_table.data_ptr(), err.data_ptr(), n_items,
                                         req_slot.numel(), hq, hkv, d, page_size, block_table.shape[1],
                                         num_pages, int(window or 0), n_splits, float(scale), _stream()),
           "attention_decode")


# Which decode attention kernel the mixer uses: "balanced" deals the key tiles of all (token, kv head)
# pairs out evenly over two blocks per SM; "split" gives every pair the same number of splits; "auto"
# takes the balanced kernel where there are more pairs than blocks that run at a time (equal splits
# would run as a full wave and a partly filled one) or where a block gets some 320 tiles or more, so
# that its one or two merged parts weigh little.  Inside the decode step at the Qwen3-8B head sizes:
# batch 64, context 4,096: 6,700 against 6,300 tokens/s; batch 8, context 32,768: 895 against 864;
# batch 8, context 16,384: 1,313 against 1,327; batch 8, context 4,096: 2,010 against 2,090.
DECODE_ATTENTION = os.environ.get("TOKAMAK_B200_DECODE_ATTENTION", "auto")
DECODE_BALANCED_MAX_ITEMS = 1024
DECODE_BALANCED_MAX_BLOCKS = 512
_SM_COUNT: dict = {}
_BALANCED_SCRATCH: dict = {}


def decode_balanced_blocks(device: torch.device, n_items: int, n_kv_heads: int, max_kv_len: int) -> int:
    """Blocks of the balanced decode kernel: two per SM, fewer where that would leave a block with
    less than eight 16-key tiles (``max_kv_len`` bounds the longest context)."""
    sms = _SM_COUNT.get(device)
    if sms is None:
        sms = _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    tiles = n_items * n_kv_heads * max(1, -(-max_kv_len // 16))
    return max(1, min(2 * sms, DECODE_BALANCED_MAX_BLOCKS, tiles // 8))


def decode_uses_balanced(device: torch.device, n_items: int, n_kv_heads: int, max_kv_len: int) -> bool:
    """Whether the mixer should take the balanced decode kernel for this many single tokens whose
    longest context is at most ``max_kv_len``."""
    if DECODE_ATTENTION == "split" or n_items > DECODE_BALANCED_MAX_ITEMS:
        return False
    if DECODE_ATTENTION == "balanced":
        return True
    decode_balanced_blocks(device, 1, 1, 16)           # makes sure the SM count is known
    blocks = 2 * _SM_COUNT[device]
    pairs = n_items * n_kv_heads
    if pairs > blocks:
        return True
    # Fewer pairs than that: equal splits fill the SMs three blocks deep (batch 8 at contexts of
    # 16,384 and 32,768: 1,369 and 911 tokens/s against 1,325 and 891 with the tiles dealt out),
    # unless there are too many pairs to split at all and a long context to stream
    return decode_splits(n_items, n_kv_heads, max_kv_len) == 1 and pairs * -(-max_kv_len // 16) >= 320 * blocks


def attention_decode_balanced(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                              items: torch.Tensor, positions: torch.Tensor, tok_req: torch.Tensor,
                              req_slot: torch.Tensor, block_table: torch.Tensor, err: torch.Tensor, *,
                              scale: float, window: int | None, blocks: int) -> None:
    """Paged attention for the single next tokens listed in ``items`` (bfloat16 only), the key tiles of
    all (token, kv head) pairs dealt out evenly over ``blocks`` blocks."""
    _want(q, torch.bfloat16, "q"); _want(out, torch.bfloat16, "out")
    _want(k_cache, torch.bfloat16, "k_cache"); _want(v_cache, torch.bfloat16, "v_cache")
    _want(items, torch.int32, "items")
    n, hq, d = q.shape
    num_pages, hkv, page_size, dk = k_cache.shape
    n_items = items.numel()
    if (not decode_kernel_takes(hq, hkv, d, page_size) or n_items > DECODE_BALANCED_MAX_ITEMS
            or not 1 <= blocks <= DECODE_BALANCED_MAX_BLOCKS):
        raise KernelError(f"the balanced decode kernel does not take heads {hq}/{hkv}, head_dim {d}, "
                          f"page size {page_size}, {n_items} tokens, {blocks} blocks")
    lib = _lib()
    need = lib.tk_attention_decode_balanced_scratch_floats(blocks, d)
    scratch = _BALANCED_SCRATCH.get(q.device)
    if scratch is None or scratch.numel() < need:
        if scratch is not None:
            _RETIRED_COUNTERS.append(scratch)        # captured graphs still hold its address
        scratch = _BALANCED_SCRATCH[q.device] = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=q.device)
    counters = _decode_counters(q.device, n_items * hkv)
    _check(lib.tk_attention_decode_balanced(q.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                            scratch.data_ptr(), counters.data_ptr(), items.data_ptr(),
                                            positions.data_ptr(), tok_req.data_ptr(), req_slot.data_ptr(),
                                            block_table.data_ptr(), err.data_ptr(), n_items, req_slot.numel(),
                                            hq, hkv, d, page_size, block_table.shape[1], num_pages,
                                            int(window or 0), blocks, float(scale), _stream()),
           "attention_decode_balanced")


def attention_prefill(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      tiles: torch.Tensor, req_q_start: torch.Tensor, req_q_len: torch.Tensor,
                      req_kv_len: torch.Tensor, req_slot: torch.Tensor, block_table: torch.Tensor,
                      err: torch.Tensor, *, scale: float, window: int | None) -> None:
    """Paged flash attention for the 64-token query tiles listed in ``tiles`` (bfloat16 only).

    ``tiles`` is int32 ``[n_tiles, 2]``: the request's row in the per-request arrays and the
    index of the tile within the tokens that the request brings to this step."""
    _want(q, torch.bfloat16, "q"); _want(out, torch.bfloat16, "out")
    _want(k_cache, torch.bfloat16, "k_cache"); _want(v_cache, torch.bfloat16, "v_cache")
    _want(tiles, torch.int32, "tiles")
    n, hq, d = q.shape
    num_pages, hkv, page_size, dk = k_cache.shape
    if not prefill_kernel_takes(hq, hkv, d, page_size) or dk != d:
        raise KernelError(f"the flash prefill kernel does not take heads {hq}/{hkv}, head_dim {d}")
    _check(_lib().tk_attention_prefill(q.data_ptr(), out.data_ptr(), k_cache.data_ptr(),
                                          v_cache.data_ptr(), tiles.data_ptr(), req_q_start.data_ptr(),
                                          req_q_len.data_ptr(), req_kv_len.data_ptr(),
                                          req_slot.data_ptr(), block_table.data_ptr(), err.data_ptr(),
                                          tiles.numel() // 2, req_slot.numel(), hq, hkv, d, page_size,
                                          block_table.shape[1], num_pages, int(window or 0),
                                          float(scale), _stream()), "attention_prefill")


PREFILL_TC_ROWS = 256     # query tokens per item of the tcgen05 prefill kernel (two tiles of 128)
PREFILL_TC_KEYS = 64      # keys per tile
PREFILL_TC_RECORD = 12    # int32 fields of an item record
PREFILL_TC_MAX_PARTS = 64
PREFILL_TC_MIN_PART = 8   # key tiles: shorter parts cost more in hand-overs than they balance


@dataclass
class PrefillItems:
    """Work list of :func:`attention_prefill_tc`, made by :func:`prefill_tc_records` and uploaded by
    the caller: ``records`` int32 ``[n, PREFILL_TC_RECORD]`` on the device, and how many parts of cut
    token blocks and how many cut token blocks it holds (sizes of the scratch memory)."""
    records: torch.Tensor
    n_parts: int
    n_split: int


def prefill_tc_records(q_start, q_len, kv_len, slots, *, heads: int, sms: int,
                       parts: int | None = None) -> tuple[np.ndarray, int, int]:
    """Item records of the tcgen05 prefill kernel for the requests that bring more than one token.

    The tokens of a request are cut into blocks of :data:`PREFILL_TC_ROWS`; block ``b`` visits the
    64-key tiles ``0 .. (pos0 + rows - 1) // 64`` (``pos0 = kv_len - q_len + 256 b``; a window
    shortens the walk inside the kernel).  Every block is one item per query head.  The kernel deals
    items out longest first to one thread block per SM.  Where there are fewer items than half the
    SMs (one short portion against a long context), every block is cut along its keys into parts of
    equal length (at least :data:`PREFILL_TC_MIN_PART` tiles each), as many as keep all items in one
    round over the SMs; the kernel adds the parts up.  Measured on a B200: a cut costs a part about
    as much as writing its rows out, and the part that adds up a few microseconds more, so with a
    round of items or more to deal out, cutting loses.  ``heads`` is the number of query heads the
    list is balanced for (the kernel takes any).

    Returns ``(records, n_parts, n_split)``: int32 ``[n, PREFILL_TC_RECORD]`` with the fields
    ``tok0, rows, pos0, slot, kt_begin, kt_end, part, n_parts, poff, split, merger`` longest first, the total
    number of parts of cut blocks, and the number of cut blocks."""
    blocks = []
    for r in range(len(q_len)):
        if q_len[r] <= 1:
            continue
        base = kv_len[r] - q_len[r]
        for b in range(-(-q_len[r] // PREFILL_TC_ROWS)):
            rows = min(PREFILL_TC_ROWS, q_len[r] - PREFILL_TC_ROWS * b)
            pos0 = base + PREFILL_TC_ROWS * b
            blocks.append((q_start[r] + PREFILL_TC_ROWS * b, rows, pos0, slots[r],
                           (pos0 + rows - 1) // PREFILL_TC_KEYS + 1))
    # cutting pays only where the SMs would otherwise stand idle: with fewer items than half the SMs,
    # every block is cut into as many parts as keeps all items in one round over the SMs
    n_items = len(blocks) * max(1, heads)
    parts_all = min(max(1, sms) // n_items, PREFILL_TC_MAX_PARTS) if n_items else 1
    if parts is not None:
        parts_all = parts        # a measurement's own choice
    records, poff, split = [], 0, 0
    for tok0, rows, pos0, slot, n_kt in blocks:
        n_cut = max(1, min(parts_all, n_kt // PREFILL_TC_MIN_PART))
        for i in range(n_cut):
            records.append((tok0, rows, pos0, slot, n_kt * i // n_cut, n_kt * (i + 1) // n_cut, i, n_cut,
                            poff if n_cut > 1 else 0, split if n_cut > 1 else 0, 0, 0))
        if n_cut > 1:
            poff += n_cut
            split += 1
    records.sort(key=lambda rec: rec[4] - rec[5])          # longest first; equal lengths keep their order
    out = np.asarray(records, dtype=np.int32).reshape(-1, PREFILL_TC_RECORD)
    # the part of a cut block that comes last in the list adds the parts up: the kernel hands items
    # out in list order, so all the others are running or done when it gets there
    last_of = {}
    for i, rec in enumerate(records):
        if rec[7] > 1:
            last_of[rec[9]] = i
    for i in last_of.values():
        out[i, 10] = 1
    return out, poff, split


_PREFILL_TC_WS: dict = {}


def _prefill_tc_workspace(device: torch.device, part_slots: int, counters: int, head_dim: int) -> dict:
    """Counters (zero between launches) and scratch of the tcgen05 prefill kernel, one set per device."""
    ws = _PREFILL_TC_WS.get(device)
    if ws is None:
        ws = _PREFILL_TC_WS[device] = {"sched": torch.zeros(2, dtype=torch.int32, device=device),
                                       "count": torch.zeros(1024, dtype=torch.int32, device=device),
                                       "o": None, "ml": None}
    if ws["count"].numel() < counters:
        ws["count"] = torch.zeros(max(counters, 2 * ws["count"].numel()), dtype=torch.int32, device=device)
    floats = part_slots * 128 * head_dim
    if floats > 0 and (ws["o"] is None or ws["o"].numel() < floats):
        ws["o"] = torch.empty(floats, dtype=torch.float32, device=device)
        ws["ml"] = torch.empty(part_slots * 128 * 2, dtype=torch.float32, device=device)
    return ws


def attention_prefill_tc(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         items: PrefillItems, block_table: torch.Tensor, err: torch.Tensor, *,
                         scale: float, window: int | None) -> None:
    """Paged flash attention on tcgen05 for the work list ``items`` (see :func:`prefill_tc_records`),
    a persistent kernel that deals the items out to one block per SM.  Loads whole pages: the cache
    must have been written by :func:`rope_kv` with ``req_q_len`` and ``req_kv_len`` given.  One call
    at a time per device: the calls share counters and scratch."""
    _want(q, torch.bfloat16, "q"); _want(out, torch.bfloat16, "out")
    _want(k_cache, torch.bfloat16, "k_cache"); _want(v_cache, torch.bfloat16, "v_cache")
    _want(items.records, torch.int32, "items.records")
    n, hq, d = q.shape
    num_pages, hkv, page_size, dk = k_cache.shape
    if not prefill_tc_kernel_takes(hq, hkv, d, page_size) or dk != d:
        raise KernelError(f"the tcgen05 prefill kernel does not take heads {hq}/{hkv}, head_dim {d}, "
                          f"page size {page_size}")
    if items.records.dim() != 2 or items.records.shape[1] != PREFILL_TC_RECORD:
        raise KernelError(f"item records want {PREFILL_TC_RECORD} fields, got shape {tuple(items.records.shape)}")
    ws = _prefill_tc_workspace(q.device, items.n_parts * hq * 2, items.n_split * hq * 2, d)
    part_o = ws["o"].data_ptr() if items.n_parts > 0 else 0
    part_ml = ws["ml"].data_ptr() if items.n_parts > 0 else 0
    _check(_lib().tk_attention_prefill_tc(q.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                          items.records.data_ptr(), block_table.data_ptr(), err.data_ptr(),
                                          ws["sched"].data_ptr(), part_o, part_ml, ws["count"].data_ptr(),
                                          n, items.records.shape[0], hq, hkv, d, page_size,
                                          block_table.shape[1], num_pages, int(window or 0),
                                          float(scale), _stream()), "attention_prefill_tc")


def sm_count(device: torch.device) -> int:
    """Streaming multiprocessors of the device."""
    sms = _SM_COUNT.get(device)
    if sms is None:
        sms = _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return sms


def prefill_tc_kernel_takes(n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Shapes of the tcgen05 prefill kernel."""
    return bool(library().tk_attention_prefill_tc_takes(n_q_heads, n_kv_heads, head_dim, page_size))


def prefill_kernel_takes(n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Shapes of the tensor-core prefill kernel; everything else goes to the general kernel."""
    return head_dim in (64, 128) and n_q_heads % n_kv_heads == 0 and page_size >= 1


_DECODE_COUNTERS: dict = {}
_RETIRED_COUNTERS: list = []


def _decode_counters(device: torch.device, n: int) -> torch.Tensor:
    """Arrival counters of the decode kernel: zero between calls, one buffer per device.  A call
    that needs more than the buffer holds gets a larger one; the smaller one is kept alive for
    good, because CUDA graphs captured earlier still hold its address."""
    buf = _DECODE_COUNTERS.get(device)
    if buf is None or buf.numel() < n:
        if buf is not None:
            _RETIRED_COUNTERS.append(buf)
        buf = torch.zeros(max(65536, n), dtype=torch.int32, device=device)
        _DECODE_COUNTERS[device] = buf
    return buf


def decode_kernel_takes(n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Shapes of the tensor-core decode kernel; everything else goes to the general kernel."""
    return (head_dim in (64, 128) and page_size % 16 == 0 and n_q_heads % n_kv_heads == 0
            and n_q_heads // n_kv_heads <= 16)


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T in true float32 (FFMA, ascending k)."""
    _want(a, torch.float32, "a"); _want(w, torch.float32, "w")
    m, k = a.shape
    n, kw = w.shape
    if k != kw:
        raise KernelError(f"inner sizes differ: {k} and {kw}")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    else:
        _want(out, torch.float32, "out")
        if out.shape != (m, n):
            raise KernelError("out has the wrong shape")
    _check(_lib().tk_gemm_f32(a.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, k, k, n,
                                 _stream()), "gemm_f32")
    return out


SWIGLU_TILE_BLOCK = 64     # gate/up rows alternate in blocks of this many for the fused activation


def gemm_tc_swapped(weight: torch.Tensor, x: torch.Tensor, err: torch.Tensor, n_splits: int,
                    out: torch.Tensor | None = None, max_stages: int = 0, cluster: int = 0,
                    swiglu: bool = False, colscale: tuple | None = None,
                    residual_norm: tuple | None = None, chain: "ProductChain | None" = None):
    """``x @ weight^T`` on tcgen05, the weight being the 128-row operand (for few tokens: every
    weight byte is streamed once by TMA), as float32 partial sums ``[parts, tokens, N_out]`` for
    the caller to add up.  ``parts = n_splits``, or ``n_splits / cluster`` with ``cluster`` in
    2..8 (a divisor of ``n_splits``): that many consecutive splits of a tile form a thread-block
    cluster that adds its partials up itself.

    ``swiglu=True``: the weight is a stacked gate/up matrix whose rows alternate in blocks of
    ``SWIGLU_TILE_BLOCK`` (gate rows, then the up rows of the same outputs); all splits form one
    cluster and the result is bfloat16 ``[tokens, N_out / 2] = silu(gate) * up``.

    ``colscale=(sumsq, dim, eps)`` with ``sumsq`` float32 ``[tiles, tokens]``: every token's sums
    are multiplied by ``rsqrt(sum over tiles / dim + eps)`` (all splits in one cluster): ``x``
    then holds activations whose RMS scale is still owed.

    ``residual_norm=(resid, norm_weight)`` (all splits in one cluster, ``N_out`` a multiple of
    128): the sums are added to the float32 residual stream ``resid [tokens, N_out]`` in place and
    ``(xb, sumsq)`` is returned: ``xb = bf16(resid * norm_weight)`` and the tiles' sums of squares
    ``[N_out / 128, tokens]``, ready to be the ``x`` and ``colscale`` of the next product.

    ``chain``: a :class:`ProductChain`; a product whose result is a single part is queued in it
    instead of launched (the result tensors are returned all the same, to be filled at the flush)."""
    _want(weight, torch.bfloat16, "weight"); _want(x, torch.bfloat16, "x")
    n_out, k = weight.shape
    tokens, kx = x.shape
    if k != kx or k % 8:
        raise KernelError(f"inner sizes {k} and {kx} must agree and be a multiple of 8")
    if tokens > 256:
        raise KernelError("the swapped product takes at most 256 tokens")
    if cluster > 1 and (cluster > 8 or n_splits % cluster):
        raise KernelError("a cluster holds 2..8 splits and must divide their count")
    bn = 16
    while bn < tokens:
        bn *= 2
    parts = n_splits // cluster if cluster > 1 else n_splits
    cs_ptr, cs_n, cs_inv, cs_eps = None, 0, 0.0, 0.0
    if colscale is not None:
        sumsq, dim, eps = colscale
        _want(sumsq, torch.float32, "colscale sums")
        if parts != 1 or sumsq.dim() != 2 or sumsq.shape[1] != tokens:
            raise KernelError("colscale wants one cluster and sums of squares [tiles, tokens]")
        cs_ptr, cs_n, cs_inv, cs_eps = sumsq.data_ptr(), sumsq.shape[0], 1.0 / dim, float(eps)
    epilogue, resid_ptr, w_ptr, xb, sums_out, result = 0, None, None, None, None, None
    if residual_norm is not None:
        resid, norm_w = residual_norm
        _want(resid, torch.float32, "resid"); _want(norm_w, torch.float32, "norm weight")
        if swiglu or parts != 1 or n_out % 128 or resid.shape != (tokens, n_out) or norm_w.numel() != n_out:
            raise KernelError("residual_norm wants one cluster, N_out a multiple of 128 and resid [tokens, N_out]")
        xb = torch.empty((tokens, n_out), dtype=torch.bfloat16, device=x.device)
        sums_out = torch.empty((n_out // 128, tokens), dtype=torch.float32, device=x.device)
        epilogue, resid_ptr, w_ptr, result = 2, resid.data_ptr(), norm_w.data_ptr(), (xb, sums_out)
        out_ptr = None
    elif swiglu:
        if n_out % (2 * SWIGLU_TILE_BLOCK) or parts != 1:
            raise KernelError("the fused activation wants rows in blocks of 64 gate + 64 up and one cluster")
        if out is None:
            out = torch.empty((tokens, n_out // 2), dtype=torch.bfloat16, device=x.device)
        epilogue, out_ptr, result = 1, out.data_ptr(), out
    else:
        if out is None:
            out = torch.empty((parts, tokens, n_out), dtype=torch.float32, device=x.device)
        out_ptr, result = out.data_ptr(), out
    def alone():
        _check(library().tk_gemm_bf16_tcgen05(weight.data_ptr(), x.data_ptr(), out_ptr, err.data_ptr(),
                                              n_out, tokens, k, k, k, bn, n_splits, max_stages,
                                              cluster if cluster > 1 else 0, epilogue, cs_ptr, cs_n, cs_inv, cs_eps,
                                              resid_ptr, w_ptr, _ptr(xb), _ptr(sums_out), _stream()),
               "gemm_tc_swapped")

    if chain is not None and parts == 1 and ProductChain.takes(tokens, n_out):
        a = _ChainPhaseArgs()
        a.w, a.x, a.ld_w, a.ld_x, a.rows, a.k, a.epilogue = weight.data_ptr(), x.data_ptr(), k, k, n_out, k, epilogue
        a.out, a.colscale_parts, a.n_colscale_parts = out_ptr, cs_ptr, cs_n
        a.colscale_inv_dim, a.colscale_eps = cs_inv, cs_eps
        a.resid, a.norm_w, a.xb_out, a.sumsq_out = resid_ptr, w_ptr, _ptr(xb), _ptr(sums_out)
        chain.add(a, alone, (weight, x, result, colscale, residual_norm))
        return result
    flush_chains()
    alone()
    return result


QKV_ROPE_HEAD_DIM = 128    # the head size whose heads are whole 128-row tiles of the swapped product


# ---- chains of decode products ---------------------------------------------------------------------

CHAIN_MAX_TOKENS = 64
# Whether the parts queue their decode products into chains ("on") or launch every product as a kernel
# of its own ("off").  Measured at the Qwen3-8B sizes, batch 8: 4.9 ms a step chained against 3.8 ms
# with one kernel per product, so the default is "off"; gemm_chain.cu says where the time goes.
CHAIN_POLICY = os.environ.get("TOKAMAK_B200_CHAIN", "off")


class _ChainPhaseArgs(__import__("ctypes").Structure):
    """``TkChainPhaseArgs`` of gemm_chain.cu."""
    import ctypes as _c
    _fields_ = [("w", _c.c_void_p), ("x", _c.c_void_p), ("ld_w", _c.c_longlong), ("ld_x", _c.c_longlong),
                ("rows", _c.c_int), ("k", _c.c_int), ("epilogue", _c.c_int), ("n_colscale_parts", _c.c_int),
                ("out", _c.c_void_p), ("colscale_parts", _c.c_void_p),
                ("colscale_inv_dim", _c.c_float), ("colscale_eps", _c.c_float),
                ("resid", _c.c_void_p), ("norm_w", _c.c_void_p), ("xb_out", _c.c_void_p), ("sumsq_out", _c.c_void_p),
                ("q_out", _c.c_void_p), ("k_cache", _c.c_void_p), ("v_cache", _c.c_void_p),
                ("positions", _c.c_void_p), ("tok_req", _c.c_void_p), ("req_slot", _c.c_void_p),
                ("block_table", _c.c_void_p), ("req_q_len", _c.c_void_p), ("req_kv_len", _c.c_void_p),
                ("q_norm_w", _c.c_void_p), ("k_norm_w", _c.c_void_p), ("rope_table", _c.c_void_p),
                ("n_reqs", _c.c_int), ("n_q_heads", _c.c_int), ("n_kv_heads", _c.c_int), ("page_size", _c.c_int),
                ("max_pages", _c.c_int), ("num_pages", _c.c_int), ("eps", _c.c_float), ("reserved", _c.c_int)]
    del _c


_CHAIN_WORKSPACES: dict = {}
_CHAIN_MAX_TILES = 2048          # most 128-row tiles of one product (a head of 262,144 rows)


def _chain_workspace(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Scratch for the parts of tiles and the (zero) counters of the chain kernel, one per device."""
    ws = _CHAIN_WORKSPACES.get(device)
    if ws is None:
        lib = library()
        scratch = torch.empty(lib.tk_gemm_chain_scratch_floats(CHAIN_MAX_TOKENS), dtype=torch.float32, device=device)
        counters = torch.zeros(lib.tk_gemm_chain_counter_ints(_CHAIN_MAX_TILES), dtype=torch.int32, device=device)
        ws = _CHAIN_WORKSPACES[device] = (scratch, counters)
    return ws


def reset_workspaces() -> None:
    """Put the counters that kernels expect at zero back to zero (after a kernel reported an error
    and may have left them otherwise)."""
    for _, counters in _CHAIN_WORKSPACES.values():
        counters.zero_()
    for buf in _DECODE_COUNTERS.values():
        buf.zero_()
    for ws in _PREFILL_TC_WS.values():
        ws["sched"].zero_()
        ws["count"].zero_()


class ProductChain:
    """Decode products whose launch is put off so that consecutive ones run as ONE persistent
    kernel (gemm_chain.cu): the weights of the next product stream in while the sums of the one
    before are added up and stored.

    :func:`gemm_tc_swapped` and :func:`gemm_qkv_rope` take a chain; with one, a product that ends
    in a single part is queued instead of launched, and its result tensors are returned at once,
    not yet computed.  :meth:`flush` launches what is queued; every other kernel wrapper of this
    module calls it first, so a kernel of this library never reads a result that is still queued.
    Code that reads such a tensor in any other way must call :meth:`flush` itself.
    """

    def __init__(self, tokens: int, err: torch.Tensor):
        self.tokens = tokens
        self.err = err
        self.phases: list[tuple[_ChainPhaseArgs, object]] = []     # (arguments, launch on its own)
        self.keep: list = []
        self.max_phases = library().tk_gemm_chain_max_phases()

    @staticmethod
    def takes(tokens: int, n_out: int) -> bool:
        return 1 <= tokens <= CHAIN_MAX_TOKENS and -(-n_out // 128) <= _CHAIN_MAX_TILES

    def add(self, args: _ChainPhaseArgs, alone, keep: tuple) -> None:
        if len(self.phases) == self.max_phases:
            self.flush()
        if not self.phases:
            self.stream = _stream()
        self.phases.append((args, alone))
        self.keep.append(keep)               # operands stay allocated until the launch
        if self not in _ACTIVE_CHAINS:
            _ACTIVE_CHAINS.append(self)

    def flush(self) -> None:
        if not self.phases:
            return
        phases, self.phases, self.keep = self.phases, [], []
        if _stream() != self.stream:
            raise KernelError("queued products are being launched on another stream than they were queued on; "
                              "call ops.flush_chains() before changing the stream")
        if len(phases) == 1:
            phases[0][1]()                     # a single product: the kernel tuned for it
            return
        arr = (_ChainPhaseArgs * len(phases))(*[a for a, _ in phases])
        scratch, counters = _chain_workspace(self.err.device)
        _check(library().tk_gemm_chain(arr, len(phases), self.tokens, self.err.data_ptr(), scratch.data_ptr(),
                                       counters.data_ptr(), _CHAIN_MAX_TILES, _stream()), "gemm_chain")


def flush_chains() -> None:
    chains = list(_ACTIVE_CHAINS)
    _ACTIVE_CHAINS.clear()
    for chain in chains:
        chain.flush()


def gemm_qkv_rope(weight: torch.Tensor, x: torch.Tensor, err: torch.Tensor, n_splits: int, q_out: torch.Tensor,
                  k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor, tok_req: torch.Tensor,
                  req_slot: torch.Tensor, block_table: torch.Tensor, q_norm_w: torch.Tensor | None,
                  k_norm_w: torch.Tensor | None, table: torch.Tensor | None, *, n_q_heads: int, n_kv_heads: int,
                  eps: float, max_stages: int = 0, colscale: tuple | None = None,
                  req_q_len: torch.Tensor | None = None, req_kv_len: torch.Tensor | None = None,
                  chain: "ProductChain | None" = None) -> None:
    """The stacked q|k|v projection of few tokens with :func:`rope_kv`'s work in its epilogue, for
    heads of 128 elements: ``weight`` is ``[(Hq + 2 Hkv) 128, K]``, ``x`` ``[tokens, K]``; ``q_out``
    receives the normed and rotated queries, the keys and values go to their pages.  All
    ``n_splits`` (at most 8) blocks of a head form one cluster.  ``colscale`` as in
    :func:`gemm_tc_swapped`; ``table`` is the rotation table ``[tokens, 64, 2]`` or None."""
    _want(weight, torch.bfloat16, "weight"); _want(x, torch.bfloat16, "x"); _want(q_out, torch.bfloat16, "q_out")
    _want(k_cache, torch.bfloat16, "k_cache"); _want(v_cache, torch.bfloat16, "v_cache")
    d = QKV_ROPE_HEAD_DIM
    n_out, k = weight.shape
    tokens, kx = x.shape
    if k != kx or k % 8:
        raise KernelError(f"inner sizes {k} and {kx} must agree and be a multiple of 8")
    if n_out != (n_q_heads + 2 * n_kv_heads) * d:
        raise KernelError(f"the weight has {n_out} rows, {(n_q_heads + 2 * n_kv_heads) * d} needed for heads of {d}")
    if tokens > 256 or not 1 <= n_splits <= 8:
        raise KernelError("the swapped product takes at most 256 tokens and 8 splits in a cluster")
    if q_out.shape != (tokens, n_q_heads, d):
        raise KernelError(f"q_out must be [{tokens}, {n_q_heads}, {d}]")
    num_pages, hkv, page_size, dk = k_cache.shape
    if hkv != n_kv_heads or dk != d or v_cache.shape != k_cache.shape:
        raise KernelError("cache pages do not match the heads")
    for name, t in (("positions", positions), ("tok_req", tok_req), ("req_slot", req_slot),
                    ("block_table", block_table)):
        _want(t, torch.int32, name)
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("table", table)):
        if t is not None:
            _want(t, torch.float32, name)
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w)):
        if t is not None and t.numel() != d:
            raise KernelError(f"{name} does not match head_dim {d}")
    if table is not None and table.shape != (tokens, d // 2, 2):
        raise KernelError(f"the rotation table must be [{tokens}, {d // 2}, 2], got {tuple(table.shape)}")
    if (req_q_len is None) != (req_kv_len is None):
        raise KernelError("req_q_len and req_kv_len come together")
    cs_ptr, cs_n, cs_inv, cs_eps = None, 0, 0.0, 0.0
    if colscale is not None:
        sumsq, dim, cs_eps = colscale
        _want(sumsq, torch.float32, "colscale sums")
        if sumsq.dim() != 2 or sumsq.shape[1] != tokens:
            raise KernelError("colscale wants sums of squares [tiles, tokens]")
        cs_ptr, cs_n, cs_inv, cs_eps = sumsq.data_ptr(), sumsq.shape[0], 1.0 / dim, float(cs_eps)
    bn = 16
    while bn < tokens:
        bn *= 2
    def alone():
        _check(library().tk_gemm_qkv_rope(weight.data_ptr(), x.data_ptr(), err.data_ptr(), tokens, k, k, k, bn,
                                          n_splits, max_stages, cs_ptr, cs_n, cs_inv, cs_eps,
                                          q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                          positions.data_ptr(), tok_req.data_ptr(), req_slot.data_ptr(),
                                          block_table.data_ptr(), _ptr(req_q_len), _ptr(req_kv_len),
                                          _ptr(q_norm_w), _ptr(k_norm_w), _ptr(table), req_slot.numel(),
                                          n_q_heads, n_kv_heads, page_size, block_table.shape[1], num_pages,
                                          float(eps), _stream()), "gemm_qkv_rope")

    if chain is not None and ProductChain.takes(tokens, n_out):
        a = _ChainPhaseArgs()
        a.w, a.x, a.ld_w, a.ld_x, a.rows, a.k, a.epilogue = weight.data_ptr(), x.data_ptr(), k, k, n_out, k, 3
        a.colscale_parts, a.n_colscale_parts, a.colscale_inv_dim, a.colscale_eps = cs_ptr, cs_n, cs_inv, cs_eps
        a.q_out, a.k_cache, a.v_cache = q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
        a.positions, a.tok_req, a.req_slot = positions.data_ptr(), tok_req.data_ptr(), req_slot.data_ptr()
        a.block_table, a.req_q_len, a.req_kv_len = block_table.data_ptr(), _ptr(req_q_len), _ptr(req_kv_len)
        a.q_norm_w, a.k_norm_w, a.rope_table = _ptr(q_norm_w), _ptr(k_norm_w), _ptr(table)
        a.n_reqs, a.n_q_heads, a.n_kv_heads, a.page_size = req_slot.numel(), n_q_heads, n_kv_heads, page_size
        a.max_pages, a.num_pages, a.eps = block_table.shape[1], num_pages, float(eps)
        chain.add(a, alone, (weight, x, q_out, colscale, table, q_norm_w, k_norm_w, positions))
        return
    flush_chains()
    alone()


def swapped_gemm_plan(n_out: int, k: int, tokens: int = 8) -> tuple[int, int, int]:
    """(K splits, pipeline stages, cluster size) of the swapped product.

    About 2.5 to 3 blocks per SM, each with at least four 64-wide k blocks, so that several
    blocks share an SM and one block's start-up hides behind another's streaming; the splits of
    a tile (at most 8) form one cluster that adds its partials up, so the consumer sees a single
    part.  Rings of three stages; four where the grid is short enough that its blocks still all
    fit: with at most 16 tokens a single split or up to about 2.7 blocks per SM (three such
    blocks fit an SM), with more tokens (larger stages) up to two blocks per SM.  Measured on
    the Qwen3-8B decode step: 16 splits in two clusters, deeper rings and other block counts were
    all slower, and so were four stages for the long gate/up grid, and for the q|k|v and head
    products at 32 and 64 tokens (head at 64 tokens: 195 us with three stages, 212 with four)."""
    tiles = -(-n_out // 128)
    k_blocks = -(-k // 64)
    splits = max(1, min(round(448 / tiles), max(1, k_blocks // 4), 8))
    if tokens <= 16:
        stages = 4 if splits == 1 or tiles * splits <= 400 else 3
    else:
        stages = 4 if tiles * splits <= 296 else 3
    return splits, stages, splits


# Which products of many tokens run on the engine's own kernel for pairs of SMs: "all" of them,
# only the gate/up product with the "fused" activation, or none ("off": the library everywhere).
PAIR_GEMM_POLICY = os.environ.get("TOKAMAK_B200_PAIR_GEMM", "all")
PAIR_GEMM_MIN_TILES = 96     # below this the grid of SM pairs is too empty and the library is faster


def pair_gemm_takes(tokens: int, n_out: int, k: int, fused: bool = False) -> bool:
    """Whether :func:`gemm_pair` is the product to use: the policy allows it, there are enough
    256 x 256 tiles to keep the 74 pairs of SMs busy, and its TMA maps and 16-byte stores can
    address the sizes."""
    if PAIR_GEMM_POLICY == "off" or (PAIR_GEMM_POLICY == "fused" and not fused):
        return False
    tiles = -(-tokens // 256) * -(-n_out // 256)
    return tiles >= PAIR_GEMM_MIN_TILES and k % 8 == 0 and n_out % 8 == 0


def gemm_pair(x: torch.Tensor, weight: torch.Tensor, err: torch.Tensor, swiglu: bool = False) -> torch.Tensor:
    """``x @ weight^T`` for many tokens on pairs of SMs (tcgen05.mma.cta_group::2, persistent grid);
    bfloat16 ``[tokens, N_out]``.  ``swiglu=True``: the weight is a stacked gate/up matrix whose rows
    alternate in blocks of ``SWIGLU_TILE_BLOCK``; the result is ``[tokens, N_out / 2] = silu(gate) * up``."""
    _want(weight, torch.bfloat16, "weight"); _want(x, torch.bfloat16, "x")
    n_out, k = weight.shape
    tokens, kx = x.shape
    if k != kx or k % 8:
        raise KernelError(f"inner sizes {k} and {kx} must agree and be a multiple of 8")
    if swiglu and n_out % (2 * SWIGLU_TILE_BLOCK):
        raise KernelError("the fused activation wants rows in blocks of 64 gate + 64 up")
    width = n_out // 2 if swiglu else n_out
    if width % 8:
        raise KernelError("the output width must be a multiple of 8")
    out = torch.empty((tokens, width), dtype=torch.bfloat16, device=x.device)
    _check(_lib().tk_gemm_bf16_pair(x.data_ptr(), weight.data_ptr(), out.data_ptr(), err.data_ptr(), tokens,
                                       n_out, k, k, k, width, 1 if swiglu else 0, _stream()), "gemm_pair")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seed: torch.Tensor, counter: torch.Tensor, out_tokens: torch.Tensor) -> None:
    """One token per row of float32 logits; see sampling.cu for the exact rule."""
    _want(logits, torch.float32, "logits"); _want(temperature, torch.float32, "temperature")
    _want(top_k, torch.int32, "top_k"); _want(top_p, torch.float32, "top_p")
    _want(seed, torch.int64, "seed"); _want(counter, torch.int32, "counter")
    _want(out_tokens, torch.int32, "out_tokens")
    rows, vocab = logits.shape
    for t in (temperature, top_k, top_p, seed, counter, out_tokens):
        if t.numel() < rows:
            raise KernelError("a per-row sampling tensor is shorter than the batch")
    _sampling_takes(rows, vocab)
    _check(_lib().tk_sample(logits.data_ptr(), logits.stride(0), temperature.data_ptr(),
                               top_k.data_ptr(), top_p.data_ptr(), seed.data_ptr(), counter.data_ptr(),
                               out_tokens.data_ptr(), rows, vocab, _stream()), "sample")


_TIMELINE_FILES = ("gemm_tcgen05", "gemm_chain", "attention_decode", "attention_prefill_tc", "sampling", "step_state",
                   "elementwise")


def timeline_start(capacity: int = 1 << 20) -> torch.Tensor:
    """Hand the kernels a buffer for their time stamps (a library built with -DTK_TIMELINE only,
    see timeline.cuh) and return it; :func:`timeline_read` decodes it."""
    import ctypes
    lib = library()
    if not hasattr(lib, "tk_timeline_set_gemm_tcgen05"):
        raise KernelError("the library was built without -DTK_TIMELINE (set TOKAMAK_B200_NVCC_FLAGS)")
    buf = torch.zeros(1 + 2 * capacity, dtype=torch.int64, device="cuda")
    for name in _TIMELINE_FILES:
        fn = getattr(lib, "tk_timeline_set_" + name)
        fn.argtypes = [ctypes.c_void_p, ctypes.c_uint]
        fn.restype = ctypes.c_int
        code = fn(buf.data_ptr(), capacity)
        if code != 0:
            raise KernelError(f"timeline_set_{name}: CUDA error {code}")
    return buf


def timeline_read(buf: torch.Tensor) -> list[tuple[int, int, int, int, int]]:
    """(time in ns, kernel, phase, SM, block) records in the order of time; clears the buffer."""
    torch.cuda.synchronize()
    host = buf.cpu()
    n = min(int(host[0]), (host.numel() - 1) // 2)
    out = []
    for i in range(n):
        t, rec = int(host[1 + 2 * i]), int(host[2 + 2 * i]) & 0xFFFFFFFFFFFFFFFF
        out.append((t, (rec >> 56) & 0xFF, (rec >> 48) & 0xFF, (rec >> 32) & 0xFFFF, rec & 0xFFFFFFFF))
    buf.zero_()
    return sorted(out)


def philox_u32(seed: int, counter: int) -> int:
    """First word of the generator's block for (seed, counter), computed on the host."""
    import ctypes
    out = (ctypes.c_uint * 4)()
    library().tk_philox_u32(seed & 0xFFFFFFFFFFFFFFFF, counter & 0xFFFFFFFF, out)
    return int(out[0])
