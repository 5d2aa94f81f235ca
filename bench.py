#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes, random
bf16 weights, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout.  ``value`` is decoded tokens per second at batch 8
(device-timed, sampled tokens fed back on the device), timed at contexts of 2,048,
3,072 and 4,095 tokens and averaged: the run from 2,048-token prompts to the 4,096
context; ``e2e`` is decode through ``Engine.generate`` with host tokens in and out
every step; ``prefill`` is one 2,048-token prompt; ``roofline`` relates the decode
step's mandatory HBM reads to the measured copy bandwidth; ``points`` holds, as flat
numbers, each context of the headline, decode at batch 1 and 64, and the baseline's
other configurations (Qwen3-0.6B sizes incl. the 64 unequal prompts through
``generate``, Qwen3-32B sizes with a cache for 64 x 4,096 tokens); ``kernels`` gives
every operation of a prefill and of a decode step by CUDA events with its fraction of
the measured peak; ``cpu_baseline`` times the plain implementation on the two tiny
configurations.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 36, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 40960, "hidden_act": "silu",
}
# the other layer sizes that the baseline's configurations name (--sizes); the default run stays Qwen3-8B
OTHER_SIZES = {
    "0.6b": dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
                 intermediate_size=3072, tie_word_embeddings=True),
    "32b": dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8,
                intermediate_size=25600),
}
PROMPT_LEN = 2048
CONTEXT = 4096
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(d.get(k), (int, float)):
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[2:]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def model_numbers(cfg, layers: int):
    """Bytes of weights a decode step reads once and FLOPs per token of the linears."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    Q, KV = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_layer = (Q + 2 * KV) * H + H * Q + 2 * I * H + H * I
    norms = layers * (2 * H + 2 * cfg.head_dim) + H
    weight_bytes = 2 * (layers * per_layer + V * H) + 4 * norms
    kv_bytes_per_token = layers * 2 * KV * 2
    return per_layer, weight_bytes, kv_bytes_per_token


CONTEXTS = (2048, 3072, 4095)      # where decode is timed: the start, the middle and the end of the run


class Runner:
    """One set of layer sizes: builds engines as the cases need them and times decode
    (device-timed, tokens fed back on the device), the same through ``Engine.generate``,
    prefill, and every operation of a step by CUDA events."""

    def __init__(self, sizes: str, layers, args, pk):
        import torch
        from zlm_b200.registry import config_from_dict
        from zlm_b200.sampling import SamplingParams
        self.torch = torch
        self.args, self.pk, self.sizes = args, pk, sizes
        d = dict(OTHER_SIZES.get(sizes, QWEN3_8B))
        self.full_layers = d["num_hidden_layers"]
        self.layers = self.full_layers if layers is None else layers
        d["num_hidden_layers"] = self.layers
        self.cfg = config_from_dict(d)
        self.per_layer, self.weight_bytes, self.kv_per_tok = model_numbers(self.cfg, self.layers)
        self.greedy = SamplingParams()
        self.g = torch.Generator().manual_seed(0)
        self.eng = None
        self.shape = None

    # ---- engines ------------------------------------------------------------------
    def engine(self, batch: int, tokens_per_seq: int):
        """An engine whose cache holds ``batch`` sequences of ``tokens_per_seq`` tokens (kept
        while it is large enough)."""
        torch = self.torch
        from zlm_b200 import Engine
        need = (batch, batch * tokens_per_seq)
        if self.eng is not None and self.shape[0] >= need[0] and self.shape[1] >= need[1]:
            return self.eng
        self.drop()
        e = Engine.from_random(self.cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=need[1],
                               max_batch=batch, max_seq_len=CONTEXT,
                               max_step_tokens=max(8 * CONTEXT, batch * PROMPT_LEN))      # `generate` takes all prompts in one step
        if self.args.pdl or self.args.no_pdl:
            e.decoder.use_pdl = bool(self.args.pdl)
        self.eng, self.shape = e, need
        return e

    def drop(self):
        if self.eng is not None:
            self.eng = None
            gc.collect()
            self.torch.cuda.empty_cache()

    def prompts(self, n: int, length: int):
        return [self.torch.randint(0, self.cfg.vocab_size, (length,), generator=self.g).tolist() for _ in range(n)]

    def prefill(self, eng, ps, chunk_tokens=8 * 2048):
        """Prompts into fresh slots, a few at a time; returns (slots, first sampled tokens)."""
        slots = [eng.new_sequence() for _ in ps]
        per = max(1, chunk_tokens // max(len(p) for p in ps))
        first = []
        for i in range(0, len(ps), per):
            first += eng.prefill_sample(slots[i:i + per], ps[i:i + per], self.greedy,
                                        list(range(i, i + len(ps[i:i + per]))))
        return slots, first

    # ---- decode ---------------------------------------------------------------------
    def decode_at(self, batch: int, context: int, steps: int, warmup: int, clocks=None) -> dict:
        """``steps`` decode steps of ``batch`` sequences that hold about ``context`` tokens,
        timed on the device around the whole run of steps."""
        torch = self.torch
        start = max(1, min(context, CONTEXT - warmup - steps))    # the timed steps end inside the context
        eng = self.engine(batch, CONTEXT)
        slots, first = self.prefill(eng, self.prompts(batch, start))
        dec, k = eng.decoder, eng.rt.k
        dec.step(slots, first, self.greedy)
        for _ in range(max(0, warmup - 1)):
            dec.step(slots, None, self.greedy)
        torch.cuda.synchronize()
        if clocks:
            clocks.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx0 = eng.length(slots[0])
        ev0.record()
        for _ in range(steps):
            dec.step(slots, None, self.greedy)
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1) / steps
        for sl in slots:
            eng.release(sl)
        eng.check(sync=True)
        mean_ctx = ctx0 + (steps - 1) / 2.0
        nbytes = self.weight_bytes + batch * self.cfg.hidden_size * 2 + batch * mean_ctx * self.kv_per_tok
        gbs = nbytes / (ms * 1e-3) / 1e9
        return {"ms": ms, "tok_s": batch / ms * 1e3, "context": mean_ctx, "nominal": context, "gbs": gbs,
                "frac": gbs / self.pk["hbm_gbs"], "launches": dec.launches_per_step, "steps": steps}

    def decode_over_contexts(self, batch: int, steps: int, warmup: int, clocks=None) -> dict:
        """Decode timed at three contexts of the run from 2,048 to 4,096 tokens; a step's time
        grows linearly with the context, so the mean of the three is the run's time per step."""
        runs = [self.decode_at(batch, c, steps, warmup, clocks if i == 0 else None) for i, c in enumerate(CONTEXTS)]
        ms = sum(r["ms"] for r in runs) / len(runs)
        ctx = sum(r["context"] for r in runs) / len(runs)
        nbytes = self.weight_bytes + batch * self.cfg.hidden_size * 2 + batch * ctx * self.kv_per_tok
        gbs = nbytes / (ms * 1e-3) / 1e9
        return {"ms": ms, "tok_s": batch / ms * 1e3, "context": ctx, "gbs": gbs, "frac": gbs / self.pk["hbm_gbs"],
                "runs": runs, "launches": runs[0]["launches"], "steps": runs[0]["steps"]}

    def e2e(self, batch: int, steps: int) -> dict:
        """The same decode through the Python entry point: host tokens in, host tokens out."""
        eng = self.engine(batch, CONTEXT)
        ps = self.prompts(batch, PROMPT_LEN)
        # at least 128 steps: the first dozen steps after a prefill run at the clocks that the
        # prefill's power draw left (measured: 5.0 instead of 3.8 ms a step for about 15 steps),
        # which says nothing about the loop and would weigh a fifth in a run of 20 steps
        n = max(steps, 128)
        # once before, so that the decode graphs of every context length the run passes through
        # exist before the timed call (a capture costs as much as several steps)
        eng.generate(ps, max_tokens=n + 1, stop_token_ids=())
        st = eng.generate(ps, max_tokens=n + 1, stop_token_ids=()).stats
        return {"value": round(batch * st.decode_steps / st.decode_ms * 1e3, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": int(eng.stager.h2d_bytes), "d2h_bytes_per_step": 4 * batch,
                "steps": st.decode_steps}

    # ---- prefill ----------------------------------------------------------------------
    def prefill_2048(self) -> dict:
        torch = self.torch
        from zlm_b200 import StepEntry
        eng = self.engine(1, CONTEXT)
        (p,) = self.prompts(1, PROMPT_LEN)
        times = []
        for i in range(4):
            s = eng.new_sequence()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            # a prefill step timed alone: a step of 25 ms at full tensor load leaves the clocks
            # lower for the step after it (measured: 27.5 ms back to back, 24.9 after a pause)
            time.sleep(0.3)
            e0.record()
            eng.step([StepEntry(s, p, [PROMPT_LEN - 1])])
            e1.record()
            torch.cuda.synchronize()
            if i:
                times.append(e0.elapsed_time(e1))
            eng.release(s)
        ms = min(times)
        T, cfg = PROMPT_LEN, self.cfg
        attn = self.layers * 4 * cfg.num_attention_heads * cfg.head_dim * (T * (T + 1) // 2)
        flops = 2 * T * self.layers * self.per_layer + 2 * cfg.vocab_size * cfg.hidden_size + attn
        return {"value": round(T / ms * 1e3, 1), "tokens": T, "ms": round(ms, 3),
                "frac": round(flops / (ms * 1e-3) / (self.pk["bf16_tflops"] * 1e12), 4)}

    # ---- every operation of a step -------------------------------------------------------
    def kernels(self, batch: int, phase: str) -> dict:
        """Per-operation CUDA-event times inside a real step (weights stream from HBM: the whole
        model is larger than L2): microseconds per call, GB/s and TFLOP/s, and the larger of
        their fractions of the measured peaks."""
        from zlm_b200.profiling import profile_engine
        eng = self.engine(batch, CONTEXT)
        n = 1 if phase == "prefill" else batch
        rows = profile_engine(eng, self.prompts(n, PROMPT_LEN), decode_steps=0 if phase == "prefill" else 6)
        out = {}
        for r in rows:
            if r["phase"] != phase or r["op"] in ("argmax", "sample", "embed"):
                continue
            f_b = r["gb_s"] / self.pk["hbm_gbs"]
            f_f = r["tflop_s"] / self.pk["bf16_tflops"]
            out[r["op"]] = {"us": r["us_per_call"], "calls": r["calls"], "gb_s": r["gb_s"], "tflop_s": r["tflop_s"],
                            "frac": round(max(f_b, f_f), 3), "bound": "hbm" if f_b >= f_f else "tensor"}
        return out


def cpu_baseline() -> dict:
    """The two tiny configurations on the CPU with the plain implementation (no cache: every
    token recomputes its whole sequence), the baseline's workloads: tokens a second."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_qwen3 as P
    from tiny_configs import TINY, plain_sizes
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    from zlm_b200.weights import random_tensors
    out = {}
    for name, lens, steps in (("A", [5, 9, 13], 8), ("B", [1, 7, 16, 31], 12)):
        cfg = config_from_dict(TINY[name])
        t = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 0, "cpu", torch.float32)
        g = torch.Generator().manual_seed(1)
        ps = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
        t0 = time.perf_counter()
        n = sum(len(P.greedy_generate(t, plain_sizes(cfg), p, steps)) for p in ps)
        dt = time.perf_counter() - t0
        out[f"tiny_{name.lower()}_tok_s"] = round(n / dt, 1)
    out["what"] = "tests/plain_qwen3.py, greedy, float32, torch on the host's cores"
    return out


def run(args) -> dict:
    import torch
    torch.cuda.set_device(0)
    pk = peaks()
    B, steps, warmup = args.batch, args.steps, args.warmup
    R = Runner(args.sizes, args.layers, args, pk)
    cfg = R.cfg
    clocks = ClockSampler()

    prefill_rec = R.prefill_2048()
    kern = {}
    if not args.no_kernels:
        kern["prefill_2048"] = R.kernels(1, "prefill")
    head = R.decode_over_contexts(B, steps, warmup, clocks)
    clock_rec = clocks.stop()
    e2e = R.e2e(B, steps)
    if not args.no_kernels:
        kern[f"decode_b{B}"] = R.kernels(B, "decode")
    points = {}
    for r in head["runs"]:
        points[f"decode_b{B}_ctx{r['nominal']}"] = round(r["tok_s"], 1)
    if not args.no_points:
        for b in (1, 64):
            if b == B:
                continue
            r = R.decode_over_contexts(b, args.point_steps, warmup)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_frac"] = round(r["frac"], 4)
            points[f"decode_b{b}_ctx2048"] = round(r["runs"][0]["tok_s"], 1)
            if not args.no_kernels and b == 64:
                kern["decode_b64"] = {k: v for k, v in R.kernels(64, "decode").items() if k.startswith("attention")}
    R.drop()
    others = {}
    if not (args.no_points or args.no_other_sizes) and args.sizes == "8b":
        others = other_sizes(args, pk, warmup)
        for name, rec in others.items():
            for k, v in rec.items():
                points[f"{name}_{k}"] = v

    return {
        "metric": f"decode tokens/s (Qwen3-{args.sizes.upper()} sizes, bf16, batch {B}, 2048-token prompts, context 4096)",
        "value": round(head["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": head["steps"], "warmup": warmup,
        "ms_per_step": round(head["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
        "impl": "zlm_b200",
        "config": {"model": f"qwen3-{args.sizes}-sizes", "layers": R.layers, "layers_full": R.full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": B,
                   "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "context_at_timing": int(head["context"]),
                   "timed": f"{head['steps']} steps at each of contexts 2048, 3072 and 4095; their mean",
                   "parallelism": "single-gpu", "l2": "inputs larger than L2 (weights read every step)",
                   "peaks": pk["source"]},
        "e2e": e2e, "gpu_launches": int(head["launches"] * head["steps"] * len(CONTEXTS)),
        "launches_per_step": int(head["launches"]), "clocks": clock_rec,
        "prefill": prefill_rec,
        "roofline": {"bound": "hbm", "achieved": round(head["gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(head["frac"], 4)},
        "points": points, "kernels": kern, "cpu_baseline": cpu_baseline(),
    }


def other_sizes(args, pk, warmup: int) -> dict:
    """The baseline's other configurations, each as flat numbers: Qwen3-0.6B sizes (decode at
    batch 1 / 8 / 64 at a 2,048-token context, and 64 prompts of unequal lengths with 256
    decode steps through ``generate``) and Qwen3-32B sizes (prefill of 2,048 tokens, decode at
    batch 1 / 8 / 64, the cache sized for 64 x 4,096 tokens)."""
    out = {}
    R = Runner("0.6b", None, args, pk)
    rec = {}
    for b in (1, 8, 64):
        r = R.decode_at(b, PROMPT_LEN, args.point_steps, warmup)
        rec[f"decode_b{b}"] = round(r["tok_s"], 1)
        rec[f"decode_b{b}_frac"] = round(r["frac"], 4)
        if b == 8:
            rec["launches_per_step"] = int(r["launches"])
        if b in (1, 8):
            rec[f"e2e_b{b}"] = R.e2e(b, 64)["value"]
    rec["prefill_2048_tok_s"] = R.prefill_2048()["value"]
    R.drop()
    rec.update(unequal_numbers(args, "0.6b"))
    out["q06b"] = rec
    R = Runner("32b", None, args, pk)
    rec = {}
    R.engine(64, CONTEXT)                     # the cache the configuration names: 64 x 4,096 tokens
    p = R.prefill_2048()
    rec["prefill_2048_tok_s"], rec["prefill_frac"] = p["value"], p["frac"]
    for b in (1, 8, 64):
        r = R.decode_at(b, PROMPT_LEN, max(8, args.point_steps // 2), warmup)
        rec[f"decode_b{b}"] = round(r["tok_s"], 1)
        rec[f"decode_b{b}_frac"] = round(r["frac"], 4)
    rec["cache_tokens"] = 64 * CONTEXT
    R.drop()
    out["q32b"] = rec
    return out


def unequal_numbers(args, sizes: str, layers=None) -> dict:
    """64 prompts of unequal lengths (uniform in [16, 2048]) prefilled as one batch, then 256
    decode steps, through ``Engine.generate`` (host tokens in and out).  The call is made
    twice; the second is reported."""
    import torch
    from zlm_b200 import Engine
    from zlm_b200.registry import config_from_dict
    d = dict(OTHER_SIZES.get(sizes, QWEN3_8B))
    if layers is not None:
        d["num_hidden_layers"] = layers
    cfg = config_from_dict(d)
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(16, 2049, (64,), generator=g).tolist()
    ps = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    eng = Engine.from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=64 * 2368, max_batch=64,
                             max_seq_len=CONTEXT)
    for _ in range(2):
        st = eng.generate(ps, max_tokens=256, stop_token_ids=()).stats
    eng.check(sync=True)
    del eng
    gc.collect()
    torch.cuda.empty_cache()
    return {"unequal64_prompt_tokens": st.prompt_tokens,
            "unequal64_prefill_tok_s": round(st.prompt_tokens / st.prefill_ms * 1e3, 1),
            "unequal64_decode_tok_s": round(64 * st.decode_steps / st.decode_ms * 1e3, 1),
            "unequal64_decode_ms_per_step": round(st.decode_ms / st.decode_steps, 4)}


def unequal(args) -> int:
    d = dict(OTHER_SIZES.get(args.sizes, QWEN3_8B))
    rec = unequal_numbers(args, args.sizes, args.layers)
    print(json.dumps({"scenario": f"64 unequal prompts (16..2048 tokens) and 256 decode steps through generate, "
                                  f"Qwen3-{args.sizes.upper()} sizes, bf16",
                      "layers": args.layers if args.layers is not None else d["num_hidden_layers"],
                      "layers_full": d["num_hidden_layers"], **rec}))
    return 0


def profile(args) -> int:
    """A small case for ncu: the engine at the bench's layer sizes with ``--layers``
    layers; the wanted phase runs eagerly (no graph) between cudaProfilerStart and
    cudaProfilerStop, so that ``ncu --profile-from-start off`` sees only it."""
    import torch
    from zlm_b200 import Engine, StepEntry
    from zlm_b200.registry import config_from_dict
    from zlm_b200.sampling import SamplingParams
    d = dict(OTHER_SIZES.get(args.sizes, QWEN3_8B))
    d["num_hidden_layers"] = args.layers if args.layers is not None else d["num_hidden_layers"]
    cfg = config_from_dict(d)
    B, L = args.batch, args.prompt_len
    eng = Engine.from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=B * (L + 256),
                             max_batch=B, max_seq_len=L + 256, max_step_tokens=min(B, 8) * L)
    eng.decoder.use_graphs = False
    g = torch.Generator().manual_seed(0)
    ps = [torch.randint(0, cfg.vocab_size, (L,), generator=g).tolist() for _ in range(B)]
    slots = [eng.new_sequence() for _ in ps]
    rt = torch.cuda.cudart()
    greedy = SamplingParams(0.8, 40, 0.9, 1) if args.sample else SamplingParams()
    if args.profile == "prefill":
        eng.step([StepEntry(slots[0], ps[0], [L - 1])])          # warm
        eng.release(slots[0])
        slots[0] = eng.new_sequence()
        torch.cuda.synchronize()
        rt.cudaProfilerStart()
        eng.step([StepEntry(slots[0], ps[0], [L - 1])])
        torch.cuda.synchronize()
        rt.cudaProfilerStop()
    else:
        first = []
        for i in range(0, B, 8):
            first += eng.prefill_sample(slots[i:i + 8], ps[i:i + 8], greedy, list(range(i, min(B, i + 8))))
        eng.decoder.step(slots, first, greedy)
        eng.decoder.step(slots, None, greedy)
        torch.cuda.synchronize()
        rt.cudaProfilerStart()
        for _ in range(args.steps):
            eng.decoder.step(slots, None, greedy)
        torch.cuda.synchronize()
        rt.cudaProfilerStop()
    print(f"profiled {args.profile}: layers={args.layers} batch={B} prompt_len={L} steps={args.steps}")
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="zlm_b200")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the sizes' own (both numbers go into config)")
    ap.add_argument("--sizes", choices=["8b", "0.6b", "32b"], default="8b",
                    help="layer sizes: Qwen3-8B (the headline configuration), Qwen3-0.6B or Qwen3-32B")
    ap.add_argument("--point-steps", type=int, default=64)
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--profile", choices=["decode", "prefill"], help="run a small case for ncu and exit")
    ap.add_argument("--unequal", action="store_true",
                    help="instead of the headline run: 64 prompts of unequal lengths and 256 decode steps through generate")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN)
    ap.add_argument("--pdl", action="store_true",
                    help="decode kernels with programmatic dependent launch at every batch size (default: up to 16 rows)")
    ap.add_argument("--no-pdl", action="store_true", help="decode kernels in plain stream order")
    ap.add_argument("--sample", action="store_true",
                    help="with --profile decode: temperature 0.8, top-k 40, top-p 0.9 instead of greedy")
    ap.add_argument("--no-kernels", action="store_true", help="leave out the per-operation times")
    ap.add_argument("--no-other-sizes", action="store_true",
                    help="leave out the Qwen3-0.6B and Qwen3-32B sizes that the default run adds under points")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "Lucas-Palomo/zlm is a Zig 0.16 program with a Vulkan GPU path: no Python package to "
                          "install offline, no zig toolchain and no graphics stack on this box"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.profile:
        return profile(args)
    if args.unequal:
        return unequal(args)
    args.warmup = max(3, args.warmup)
    print(json.dumps(run(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
