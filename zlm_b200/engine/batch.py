"""Turning a step's requests into the integer arrays the kernels read, and
carrying them to the GPU.

All arrays of a step live in one int32 buffer with fixed offsets (sized for the
most tokens and sequences a step may bring), so that their device addresses
never change: a captured decode graph keeps pointing at the right places.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import StepContext


@dataclass
class StepEntry:
    """One sequence's share of a step: its slot, its next tokens, and the places
    among these tokens whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepError(ValueError):
    """A step that cannot run: bad token id, bad position, slot named twice."""


class MetaLayout:
    """Where the per-step arrays sit inside the int32 buffer.  The arrays of a step
    with T tokens and R sequences are packed at the front, so one small copy carries
    them; their addresses depend only on (T, R), which is what a captured decode
    graph is keyed by."""
    ORDER = ("token_ids", "token_pos", "token_slot", "token_seq", "seq_slot", "seq_start", "seq_new",
             "cu_seqlens", "want_rows", "sample_request", "sample_position")

    def __init__(self, max_tokens: int, max_seqs: int):
        self.max_tokens, self.max_seqs = int(max_tokens), int(max_seqs)
        self.size = self.used(self.max_tokens, self.max_seqs)

    @staticmethod
    def offsets(T: int, R: int):
        return {"token_ids": 0, "token_pos": T, "token_slot": 2 * T, "token_seq": 3 * T,
                "seq_slot": 4 * T, "seq_start": 4 * T + R, "seq_new": 4 * T + 2 * R,
                "cu_seqlens": 4 * T + 3 * R, "want_rows": 4 * T + 4 * R + 1,
                # per row of a sampling decode step: the request's number and the position of the
                # token being chosen (what the sampler's random numbers are counted by)
                "sample_request": 5 * T + 4 * R + 1, "sample_position": 5 * T + 5 * R + 1}

    @staticmethod
    def used(T: int, R: int) -> int:
        return 5 * T + 6 * R + 1


class MetaStager:
    """A device int32 buffer and a small ring of pinned host buffers that feed it.
    A host buffer is reused only after the copy that read it has run."""

    RING = 4

    def __init__(self, layout: MetaLayout, device):
        self.layout = layout
        self.device = torch.device(device)
        self.dev = torch.zeros(layout.size, dtype=torch.int32, device=self.device)
        self.cuda = self.device.type == "cuda"
        self.host = [torch.zeros(layout.size, dtype=torch.int32, pin_memory=self.cuda)
                     for _ in range(self.RING)]
        self.events: List[Optional[torch.cuda.Event]] = [None] * self.RING
        self.turn = 0
        self.h2d_bytes = 0
        self.off = MetaLayout.offsets(0, 0)

    def view(self, name: str, n: int) -> torch.Tensor:
        o = self.off[name]
        return self.dev[o:o + n]

    def upload(self, arrays, T: int, R: int) -> None:
        """arrays: name -> numpy int32 array of a step with T tokens and R sequences.
        One copy covers all of them; an array that is absent keeps the device's content
        (token ids that a previous step left there)."""
        i = self.turn
        self.turn = (self.turn + 1) % self.RING
        if self.events[i] is not None:
            self.events[i].synchronize()
        self.off = MetaLayout.offsets(T, R)
        h = self.host[i]
        hn = h.numpy()
        lo, hi = self.layout.size, 0
        for name, a in arrays.items():
            o = self.off[name]
            hn[o:o + len(a)] = a
            lo, hi = min(lo, o), max(hi, o + len(a))
        if hi <= lo:
            return
        self.dev[lo:hi].copy_(h[lo:hi], non_blocking=True)
        self.h2d_bytes = (hi - lo) * 4
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record()
            self.events[i] = ev


def plan_step(entries: Sequence[StepEntry], lengths, vocab_size: int, layout: MetaLayout):
    """Checks the entries and lays their arrays out.  ``lengths`` maps a slot to the
    tokens it already holds.  Returns (arrays, host lists, number of wanted rows)."""
    if not entries:
        raise StepError("a step needs at least one sequence")
    seen = set()
    T = sum(len(e.tokens) for e in entries)
    R = len(entries)
    if T > layout.max_tokens:
        raise StepError(f"the step brings {T} tokens; the engine was built for {layout.max_tokens} per step")
    if R > layout.max_seqs:
        raise StepError(f"the step brings {R} sequences; the engine was built for {layout.max_seqs}")
    ids = np.empty(T, np.int32)
    pos = np.empty(T, np.int32)
    slot = np.empty(T, np.int32)
    seq = np.empty(T, np.int32)
    s_slot = np.empty(R, np.int32)
    s_start = np.empty(R, np.int32)
    s_new = np.empty(R, np.int32)
    cu = np.zeros(R + 1, np.int32)
    want: List[int] = []
    t = 0
    for r, e in enumerate(entries):
        n = len(e.tokens)
        if n == 0:
            raise StepError(f"sequence in slot {e.slot} brings no token")
        if e.slot in seen:
            raise StepError(f"slot {e.slot} appears twice in one step")
        seen.add(e.slot)
        if e.slot not in lengths:
            raise StepError(f"slot {e.slot} is not held by any sequence")
        start = lengths[e.slot]
        tok = np.asarray(e.tokens, dtype=np.int64)
        if tok.min() < 0 or tok.max() >= vocab_size:
            bad = int(tok[(tok < 0) | (tok >= vocab_size)][0])
            raise StepError(f"token id {bad} is outside the vocabulary [0, {vocab_size})")
        ids[t:t + n] = tok
        pos[t:t + n] = np.arange(start, start + n)
        slot[t:t + n] = e.slot
        seq[t:t + n] = r
        s_slot[r], s_start[r], s_new[r] = e.slot, start, n
        cu[r + 1] = t + n
        for w in e.want:
            if not 0 <= w < n:
                raise StepError(f"wanted place {w} is outside the {n} tokens of slot {e.slot}")
            want.append(t + w)
        t += n
    if len(want) > T:
        # a place named twice: the wanted rows have room for one row per token
        raise StepError(f"{len(want)} places are wanted among {T} tokens; a place may be named once")
    arrays = {"token_ids": ids, "token_pos": pos, "token_slot": slot, "token_seq": seq,
              "seq_slot": s_slot, "seq_start": s_start, "seq_new": s_new, "cu_seqlens": cu,
              "want_rows": np.asarray(want, np.int32)}
    return arrays, T, R, len(want)


def make_context(stager: MetaStager, arrays, T: int, R: int, workspace=None) -> StepContext:
    s_new = arrays["seq_new"]
    s_start = arrays["seq_start"]
    max_len = int((s_start + s_new).max())
    return StepContext(
        workspace=workspace,
        T=T, R=R,
        token_ids=stager.view("token_ids", T), token_pos=stager.view("token_pos", T),
        token_slot=stager.view("token_slot", T), token_seq=stager.view("token_seq", T),
        seq_slot=stager.view("seq_slot", R), seq_start=stager.view("seq_start", R),
        seq_new=stager.view("seq_new", R), cu_seqlens=stager.view("cu_seqlens", R + 1),
        h_seq_slot=arrays["seq_slot"].tolist(), h_seq_start=s_start.tolist(), h_seq_new=s_new.tolist(),
        is_decode=bool((s_new == 1).all()), max_new=int(s_new.max()),
        max_len=max_len)
