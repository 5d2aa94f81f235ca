"""The generation loop above the step function.

Requests (token-id prompts of unequal lengths) are cut into batches that fit the
cache; a batch starts together with one prefill step and then decodes one token
per live sequence per step; a sequence ends at a stop token (which is not
emitted), at ``max_tokens`` new tokens, or when the cache's longest sequence is
reached; ended sequences give their slot back at once and the rest go on; when a
batch is done the next one starts in the freed slots.

The reference's loop for its single sequence: ``if next == eos: break; if count
>= max_tokens: break; append; forward; sample`` (src/runtime/session.zig:1524-1566).
Here the forward after the last appended token is not run.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from ..kernels import PAGE_TOKENS
from ..sampling import SamplingParams
from .batch import StepEntry


@dataclass
class GenerationStats:
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    prompt_tokens: int = 0
    new_tokens: int = 0
    prefill_steps: int = 0
    decode_steps: int = 0
    batches: int = 0


@dataclass
class GenerationResult:
    tokens: List[List[int]]
    finish_reasons: List[str]          # "stop", "length" or "context"
    stats: GenerationStats


def _pages(n: int) -> int:
    return (n + PAGE_TOKENS - 1) // PAGE_TOKENS


def plan_batches(prompt_lens: Sequence[int], max_tokens: int, capacity_tokens: int, max_batch: int,
                 max_seq_len: int) -> List[List[int]]:
    """Cuts the requests, in their order, into batches whose worst-case cache use
    (prompt plus the tokens that may be fed back, rounded up to pages) fits the
    cache and whose size fits ``max_batch``."""
    cap_pages = capacity_tokens // PAGE_TOKENS
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, n in enumerate(prompt_lens):
        if n <= 0:
            raise ValueError(f"request {i}: empty prompt (there is no tokenizer to supply a first token)")
        if n > max_seq_len:
            raise ValueError(f"request {i}: prompt of {n} tokens exceeds the longest sequence ({max_seq_len})")
        # the last generated token is never fed back, so it needs no place
        need = _pages(min(max_seq_len, n + max(0, max_tokens - 1)))
        if need > cap_pages:
            raise ValueError(f"request {i}: {n} prompt + {max_tokens} new tokens do not fit the cache "
                             f"({cap_pages * PAGE_TOKENS} tokens)")
        if cur and (used + need > cap_pages or len(cur) >= max_batch):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


@dataclass
class _Row:
    request: int
    slot: int
    length: int                       # tokens in the cache
    out: List[int] = field(default_factory=list)
    reason: str = ""


class BatchDecisions:
    """The loop's decisions for one batch, free of any GPU work: given the token
    sampled for every live row, which rows emit it, which end and why."""

    def __init__(self, max_tokens: int, stop_ids: Sequence[int], max_seq_len: int, include_stop: bool = False):
        self.max_tokens = int(max_tokens)
        self.stop = set(int(s) for s in stop_ids)
        self.max_seq_len = int(max_seq_len)
        self.include_stop = include_stop

    def goes_on_unless_stopped(self, row: _Row) -> bool:
        """Whether ``row`` will be live after the token of the step in flight, whatever
        that token is, as long as it is no stop token (``row.length`` counts the token
        that step feeds)."""
        return len(row.out) + 1 < self.max_tokens and row.length + 1 <= self.max_seq_len

    def apply(self, rows: List[_Row], sampled: Sequence[int]) -> Tuple[List[_Row], List[_Row]]:
        """Returns (rows that go on and feed their new token, rows that ended)."""
        live, ended = [], []
        for row, tok in zip(rows, sampled):
            tok = int(tok)
            if tok in self.stop:
                if self.include_stop:
                    row.out.append(tok)
                row.reason = "stop"
                ended.append(row)
                continue
            if len(row.out) >= self.max_tokens:
                row.reason = "length"
                ended.append(row)
                continue
            row.out.append(tok)
            if len(row.out) >= self.max_tokens:
                row.reason = "length"          # nothing more is wanted: do not feed it
                ended.append(row)
            elif row.length + 1 > self.max_seq_len:
                row.reason = "context"
                ended.append(row)
            else:
                live.append(row)
        return live, ended


def generate(engine, prompts: Sequence[Sequence[int]], max_tokens: int = 256,
             sampling: Optional[SamplingParams] = None, stop_token_ids: Optional[Sequence[int]] = None,
             include_stop: bool = False,
             on_token: Optional[Callable[[int, int], None]] = None,
             on_logits: Optional[Callable] = None) -> GenerationResult:
    """Generates up to ``max_tokens`` tokens for every prompt.  ``on_token(request,
    token)`` is called for every emitted token as soon as its step is done.
    ``on_logits(requests, positions, logits)`` is called after every step with the
    step's rows: their request numbers, the position of the token each row is choosing,
    and the fp32 logits [rows, vocab] it chooses from (``engine.last_logits``, still on
    the device; the tensor is overwritten by the next step).  With it, steps run one at
    a time: a queued step would overwrite the logits before the host has seen them.

    ``engine`` needs: config.eos_token_ids, max_tokens, max_batch, max_seq_len,
    new_sequence(), release(slot), prefill_sample(slots, prompts, params, requests)
    and decode_sample(slots, tokens, params, requests), both returning one token id
    per row on the host.  If it also has decode_launch(slots, tokens or None, params,
    requests) -> handle (queues a step; None feeds the tokens the step before sampled
    for the same rows) and decode_fetch(handle) -> token ids, steps are queued one
    ahead."""
    sampling = sampling or SamplingParams()
    if stop_token_ids is None:
        stop_token_ids = tuple(getattr(engine.config, "eos_token_ids", ()))
    if max_tokens < 0:
        raise ValueError("max_tokens must be >= 0")
    stats = GenerationStats()
    n = len(prompts)
    tokens: List[List[int]] = [[] for _ in range(n)]
    reasons: List[str] = ["" for _ in range(n)]
    if max_tokens == 0:
        return GenerationResult(tokens, ["length"] * n, stats)
    decide = BatchDecisions(max_tokens, stop_token_ids, engine.max_seq_len, include_stop)
    batches = plan_batches([len(p) for p in prompts], max_tokens, engine.max_tokens, engine.max_batch,
                           engine.max_seq_len)
    for batch in batches:
        stats.batches += 1
        rows = [_Row(request=i, slot=engine.new_sequence(), length=0) for i in batch]
        try:
            t0 = time.perf_counter()
            sampled = engine.prefill_sample([r.slot for r in rows], [prompts[r.request] for r in rows],
                                            sampling, [r.request for r in rows])
            for r in rows:
                r.length = len(prompts[r.request])
            stats.prefill_ms += (time.perf_counter() - t0) * 1e3
            stats.prefill_steps += 1
            stats.prompt_tokens += sum(r.length for r in rows)
            if on_logits is not None:
                on_logits([r.request for r in rows], [r.length for r in rows], engine.last_logits)
            def settle(rows_, sampled_):
                """Applies one step's tokens: emits, frees the rows that ended; returns the live rows."""
                before = [len(r.out) for r in rows_]
                live, ended = decide.apply(rows_, sampled_)
                for r, b in zip(rows_, before):
                    if on_token is not None and len(r.out) > b:
                        for tok in r.out[b:]:
                            on_token(r.request, tok)
                for r in ended:
                    engine.release(r.slot)
                    r.slot = -1
                    tokens[r.request], reasons[r.request] = r.out, r.reason
                return live

            rows = settle(rows, sampled)
            launch = getattr(engine, "decode_launch", None) if on_logits is None else None
            if launch is None:
                # one step at a time: feed, wait, decide
                while rows:
                    t0 = time.perf_counter()
                    sampled = engine.decode_sample([r.slot for r in rows], [r.out[-1] for r in rows], sampling,
                                                   [r.request for r in rows])
                    for r in rows:
                        r.length += 1
                    stats.decode_ms += (time.perf_counter() - t0) * 1e3
                    stats.decode_steps += 1
                    if on_logits is not None:
                        on_logits([r.request for r in rows], [r.length for r in rows], engine.last_logits)
                    rows = settle(rows, sampled)
            else:
                # One step ahead: while the device runs a step, the next one is already queued with
                # the tokens it is about to sample (they stay on the device), and the host reads the
                # tokens of the step before.  A step is queued ahead only if every row goes on
                # unless it meets a stop token; when one does, the queued step has computed that
                # row for nothing (its slot is freed all the same) and the rows that go on take
                # their tokens from it.  After any change of the rows the next step is fed from the
                # host again.
                t0 = time.perf_counter()
                cur = None
                while rows:
                    if cur is None:
                        cur = launch([r.slot for r in rows], [r.out[-1] for r in rows], sampling,
                                     [r.request for r in rows])
                        for r in rows:
                            r.length += 1
                    ahead = None
                    if all(decide.goes_on_unless_stopped(r) for r in rows):
                        ahead = launch([r.slot for r in rows], None, sampling, [r.request for r in rows])
                    sampled = engine.decode_fetch(cur)
                    stats.decode_steps += 1
                    was = rows
                    rows = settle(rows, sampled)
                    cur = None
                    if ahead is None:
                        continue
                    for r in rows:
                        r.length += 1                    # the queued step fed their token
                    if len(rows) == len(was):
                        cur = ahead
                        continue
                    sampled = engine.decode_fetch(ahead)
                    stats.decode_steps += 1
                    keep = {id(r) for r in rows}
                    rows = settle(rows, [t for r, t in zip(was, sampled) if id(r) in keep])
                stats.decode_ms += (time.perf_counter() - t0) * 1e3
        finally:
            for r in rows:
                if r.slot >= 0:
                    engine.release(r.slot)
    stats.new_tokens = sum(len(t) for t in tokens)
    return GenerationResult(tokens, reasons, stats)
