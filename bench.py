#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes, random
bf16 weights, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout.  ``value`` is decoded tokens per second at batch 8
(device-timed, sampled tokens fed back on the device); ``e2e`` is the same
through ``Engine.generate`` with host tokens in and out every step; ``prefill``
is one 2,048-token prompt; ``roofline`` relates the decode step's mandatory HBM
reads to the measured copy bandwidth; ``points`` holds decode at batch 1 and 64.
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


def run(args) -> dict:
    import torch
    from zlm_b200 import Engine
    from zlm_b200.registry import config_from_dict
    from zlm_b200.sampling import SamplingParams

    pk = peaks()
    d = dict(OTHER_SIZES.get(args.sizes, QWEN3_8B))
    full_layers = d["num_hidden_layers"]
    if args.layers is None:
        args.layers = full_layers
    d["num_hidden_layers"] = args.layers
    cfg = config_from_dict(d)
    B = args.batch
    steps, warmup = args.steps, args.warmup
    torch.cuda.set_device(0)
    greedy = SamplingParams()

    def make_engine(batch, tokens):
        # the headline numbers come from an engine whose cache is sized for the headline
        # configuration (batch x context); the batch-64 point gets an engine of its own
        e = Engine.from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=tokens,
                               max_batch=batch, max_seq_len=CONTEXT, max_step_tokens=max(B, 8) * PROMPT_LEN)
        if args.pdl or args.no_pdl:
            e.decoder.use_pdl = bool(args.pdl)
        if args.decode == "stream":
            e.decoder.use_stream = e.decoder.can_stream
        return e

    eng = make_engine(max(B, 1), B * CONTEXT)
    g = torch.Generator().manual_seed(0)
    per_layer, weight_bytes, kv_per_tok = model_numbers(cfg, args.layers)
    k = eng.rt.k

    def prompts(n):
        return [torch.randint(0, cfg.vocab_size, (PROMPT_LEN,), generator=g).tolist() for _ in range(n)]

    def prefill(ps, chunk=8):
        slots = [eng.new_sequence() for _ in ps]
        first = []
        for i in range(0, len(ps), chunk):
            first += eng.prefill_sample(slots[i:i + chunk], ps[i:i + chunk], greedy, list(range(i, i + len(ps[i:i + chunk]))))
        return slots, first

    def timed_decode(slots, first, n_warm, n_steps, clocks=None):
        dec = eng.decoder
        dec.step(slots, first, greedy)
        for _ in range(max(0, n_warm - 1)):
            dec.step(slots, None, greedy)
        torch.cuda.synchronize()
        l0 = k.launches()
        if clocks:
            clocks.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx0 = eng.length(slots[0])
        ev0.record()
        for _ in range(n_steps):
            dec.step(slots, None, greedy)
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
        launches = dec.launches_per_step * n_steps if (dec.use_graphs or dec.use_stream) else k.launches() - l0
        return ms, ctx0, launches

    # ---- prefill of 2,048 tokens at batch 1 ------------------------------------------
    p1 = prompts(1)
    s, _ = prefill(p1)
    eng.release(s[0])
    torch.cuda.synchronize()
    pre_ms = []
    for _ in range(3):
        s = [eng.new_sequence()]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        from zlm_b200 import StepEntry
        eng.step([StepEntry(s[0], p1[0], [PROMPT_LEN - 1])])
        e1.record()
        torch.cuda.synchronize()
        pre_ms.append(e0.elapsed_time(e1))
        eng.release(s[0])
    pms = min(pre_ms)
    T = PROMPT_LEN
    attn_flops = args.layers * 4 * cfg.num_attention_heads * cfg.head_dim * (T * (T + 1) // 2)
    pre_flops = 2 * T * args.layers * per_layer + 2 * cfg.vocab_size * cfg.hidden_size + attn_flops
    prefill_rec = {"value": round(T / pms * 1e3, 1), "tokens": T, "ms": round(pms, 3),
                   "frac": round(pre_flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- decode at the headline batch ------------------------------------------------
    clocks = ClockSampler()
    slots, first = prefill(prompts(B))
    ms, ctx0, launches = timed_decode(slots, first, warmup, steps, clocks)
    clock_rec = clocks.stop()
    value = B * steps / ms * 1e3
    mean_ctx = ctx0 + (steps - 1) / 2.0
    step_bytes = weight_bytes + B * cfg.hidden_size * 2 + B * mean_ctx * kv_per_tok
    achieved = step_bytes / (ms / steps * 1e-3) / 1e9
    for sl in slots:
        eng.release(sl)

    # ---- the same through the Python entry point ------------------------------------
    ps = prompts(B)
    n_e2e = min(steps, 128)
    # warm-up: the same call once, so that the decode graphs of every context length the run
    # passes through exist before the timed call (a capture costs as much as several steps)
    eng.generate(ps, max_tokens=n_e2e + 1, stop_token_ids=())
    res = eng.generate(ps, max_tokens=n_e2e + 1, stop_token_ids=())
    st = res.stats
    e2e = {"value": round(st.new_tokens and (B * st.decode_steps) / st.decode_ms * 1e3, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": int(eng.stager.h2d_bytes), "d2h_bytes_per_step": 4 * B,
           "steps": st.decode_steps}

    # ---- decode at batch 1 and 64 ------------------------------------------------------
    points = {}
    if not args.no_points:
        for b in (1, 64):
            if b > eng.max_batch or b * (PROMPT_LEN + args.point_steps + warmup + 64) > eng.max_tokens:
                del eng, k
                gc.collect()                 # the engine and its decode runner refer to each other
                torch.cuda.empty_cache()
                eng = make_engine(b, b * (PROMPT_LEN + args.point_steps + warmup + 64))
                k = eng.rt.k
            slots, first = prefill(prompts(b))
            pm, _, _ = timed_decode(slots, first, warmup, args.point_steps)
            points[f"decode_b{b}"] = round(b * args.point_steps / pm * 1e3, 1)
            for sl in slots:
                eng.release(sl)

    return {
        "metric": f"decode tokens/s (Qwen3-{args.sizes.upper()} sizes, bf16, batch {B}, 2048-token prompts, context 4096)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms / steps, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
        "impl": "zlm_b200",
        "config": {"model": f"qwen3-{args.sizes}-sizes", "layers": args.layers, "layers_full": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": B,
                   "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "context_at_timing": int(mean_ctx),
                   "parallelism": "single-gpu", "l2": "inputs larger than L2 (weights read every step)",
                   "peaks": pk["source"]},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clock_rec,
        "prefill": prefill_rec,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }


def unequal(args) -> int:
    """The baseline's small-model scenario: 64 prompts of unequal lengths (uniform in
    [16, 2048]) prefilled as one batch, then 256 decode steps, through ``Engine.generate``
    (host tokens in and out).  The call is made twice; the second is reported."""
    import torch
    from zlm_b200 import Engine
    from zlm_b200.registry import config_from_dict
    d = dict(OTHER_SIZES.get(args.sizes, QWEN3_8B))
    full_layers = d["num_hidden_layers"]
    d["num_hidden_layers"] = args.layers if args.layers is not None else full_layers
    cfg = config_from_dict(d)
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(16, 2049, (64,), generator=g).tolist()
    ps = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    eng = Engine.from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=64 * 2368, max_batch=64,
                             max_seq_len=CONTEXT)
    for _ in range(2):
        res = eng.generate(ps, max_tokens=256, stop_token_ids=())
    st = res.stats
    print(json.dumps({
        "scenario": f"64 unequal prompts (16..2048 tokens) and 256 decode steps, Qwen3-{args.sizes.upper()} sizes, bf16",
        "layers": d["num_hidden_layers"], "layers_full": full_layers, "prompt_tokens": st.prompt_tokens,
        "prefill_ms": round(st.prefill_ms, 2), "prefill_tokens_per_s": round(st.prompt_tokens / st.prefill_ms * 1e3, 1),
        "decode_steps": st.decode_steps, "decode_ms_per_step": round(st.decode_ms / st.decode_steps, 4),
        "decode_tokens_per_s": round(64 * st.decode_steps / st.decode_ms * 1e3, 1), "batches": st.batches,
        "bounded_waits_given_up": eng.rt.k.gemm_tc_status()}))
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
    if args.decode == "stream":
        eng.decoder.use_stream = eng.decoder.can_stream
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
    ap.add_argument("--decode", choices=["graph", "stream"], default="graph",
                    help="graph: a CUDA graph of one kernel per operation; stream: the persistent decode kernel where it applies")
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
