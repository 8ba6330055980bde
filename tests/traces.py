"""Builders of replay traces and the check of their results against the plain implementation.

A trace is a list of step records as ``bin/trace_run`` reads them.  Every builder
also returns, per step, which (request, position) each wanted row stands for.
"""

from __future__ import annotations

import random

import numpy as np
import torch

from helpers import assert_logits_close, plain_logits


def whole(requests: dict) -> tuple[list, dict]:
    """Each request alone and whole: one step with every position wanted."""
    records, rows = [], {}
    for step, (rid, toks) in enumerate(requests.items()):
        records.append({"step": step, "entries": [{"id": rid, "tokens": toks,
                                                   "want": list(range(len(toks)))}], "end": [rid]})
        rows[step] = [(rid, p) for p in range(len(toks))]
    return records, rows


def tail_one_by_one(requests: dict, tail: int = 32) -> tuple[list, dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    records, rows = [], {}
    step = 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        records.append({"step": step, "entries": [{"id": rid, "tokens": toks[:head],
                                                   "want": [head - 1]}], "end": []})
        rows[step] = [(rid, head - 1)]
        step += 1
        for p in range(head, len(toks)):
            last = p == len(toks) - 1
            records.append({"step": step, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                            "end": [rid] if last else []})
            rows[step] = [(rid, p)]
            step += 1
        if head == len(toks):
            records[-1]["end"] = [rid]
    return records, rows


def portions(requests: dict, sizes=(7, 2, 16, 1, 3, 2, 33, 5, 2, 64, 2, 9)) -> tuple[list, dict]:
    """One request at a time, in portions of changing size, down to two tokens and one."""
    records, rows = [], {}
    step = 0
    for k, (rid, toks) in enumerate(requests.items()):
        pos = 0
        i = k  # start the size cycle at a different place for every request
        while pos < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - pos)
            i += 1
            last = pos + n == len(toks)
            records.append({"step": step, "entries": [{"id": rid, "tokens": toks[pos:pos + n],
                                                       "want": list(range(n))}],
                            "end": [rid] if last else []})
            rows[step] = [(rid, pos + j) for j in range(n)]
            pos += n
            step += 1
    return records, rows


def mixed(requests: dict, max_tokens: int, max_live: int = 4, seed: int = 0,
          round_to: int = 64) -> tuple[list, dict]:
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others.

    A request is fed in portions of random size up to about two thirds of its length and
    one token at a time after that; now and then a live request sits a step out.  A new
    request starts as soon as the lengths of the live ones, each rounded up to ``round_to``,
    leave room under ``max_tokens``, so the pool is full most of the time and pages of
    ended requests are used again at once.
    """
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict = {}      # rid -> [tokens, fed]
    records, rows = [], {}
    step = 0
    rounded = lambda n: -(-n // round_to) * round_to
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting[0]
            held = sum(rounded(len(t)) for t, _ in live.values())
            if held + rounded(len(toks)) > max_tokens:
                break
            waiting.pop(0)
            live[rid] = [toks, 0]
        entries, ended, wanted = [], [], []
        for rid in list(live):
            toks, fed = live[rid]
            if len(live) > 1 and rng.random() < 0.15:
                continue
            left = len(toks) - fed
            if fed >= (2 * len(toks)) // 3:
                n = 1
            else:
                n = min(left, rng.choice([1, 2, 2, 3, 5, 8, 13, 17, 24, 31]))
            entries.append({"id": rid, "tokens": toks[fed:fed + n], "want": list(range(n))})
            wanted.extend((rid, fed + j) for j in range(n))
            live[rid][1] = fed + n
            if fed + n == len(toks):
                ended.append(rid)
                del live[rid]
        if not entries:
            continue
        records.append({"step": step, "entries": entries, "end": ended})
        rows[step] = wanted
        step += 1
    return records, rows


def check(results: dict, rows: dict, requests: dict, folder, dtype: str, what: str) -> int:
    """Compare every wanted row of every step with the plain implementation; returns rows checked."""
    checked = 0
    for step in sorted(rows):
        got = torch.from_numpy(np.asarray(results[step]))
        want = torch.stack([plain_logits(folder, requests[rid])[p] for rid, p in rows[step]])
        for i, (rid, p) in enumerate(rows[step]):
            assert_logits_close(got[i:i + 1], want[i:i + 1], dtype,
                                f"{what}: step {step}, request {rid!r}, position {p}")
        checked += len(rows[step])
    return checked
