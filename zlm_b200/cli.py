"""Command line in the manner of the reference's ``zlm run``
(src/cli/commands/run.zig:62-133): the same option names with the same meanings
and defaults where the reference has them (--prompt/-p, --max-tokens 256,
--temperature 0, --top-k 0, --top-p 1, --stream/--no-stream, --metrics[=full],
--profile, --verbose); the positional argument is a model folder instead of a tuned plan's
alias, and prompts are token ids because tokenizing happens before this library.

    python -m zlm_b200 run MODEL_DIR -p "1 2 3" --max-tokens 32
    python -m zlm_b200 run MODEL_DIR --random-prompts 8 --min-len 5 --max-len 40 --temperature 0.8 --seed 1
    python -m zlm_b200 run MODEL_DIR -p "1 2 3" --profile --dump-logits logits.f32
    python -m zlm_b200 random-model --config config.json --seed 0 --out DIR

``--profile`` prints, for one prefill step and one decode step of the given prompts,
every operation's time by CUDA events with the bytes it moves and GB/s (the reference's
per-op profile with weight bytes per token and matvec GB/s: src/cli/commands/run.zig:233-299).
``--dump-logits FILE`` writes the fp32 logits every generated token was chosen from, one
row [vocab] per token in the order of emission, and FILE.json with each row's request,
position, chosen token and its logit (the reference's ``--verbose=all`` trace of
{id, logit} per token: src/runtime/session.zig:89-104,1556-1576).
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List


def _ids(text: str) -> List[int]:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise SystemExit(f"run: --prompt takes token ids separated by spaces or commas, got {text!r}")


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="zlm_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    run = sub.add_parser("run", help="generate from token-id prompts")
    run.add_argument("model", help="folder with config.json and model.safetensors")
    run.add_argument("--prompt", "-p", action="append", default=[], help="token ids of one prompt (repeatable)")
    run.add_argument("--prompt-file", help="JSON file with a list of token-id lists")
    run.add_argument("--random-prompts", type=int, default=0, help="make this many random prompts")
    run.add_argument("--min-len", type=int, default=8)
    run.add_argument("--max-len", type=int, default=64)
    run.add_argument("--max-tokens", type=int, default=256, help="new tokens per request (default 256)")
    run.add_argument("--temperature", type=float, default=0.0, help="0 = greedy (default)")
    run.add_argument("--top-k", type=int, default=0, help="0 disables (default)")
    run.add_argument("--top-p", type=float, default=1.0, help="1 disables (default)")
    run.add_argument("--seed", type=int, default=0)
    run.add_argument("--stop", action="append", type=int, default=None,
                     help="stop token id (repeatable; default: the configuration's eos_token_id)")
    run.add_argument("--stream", dest="stream", action="store_true", default=True)
    run.add_argument("--no-stream", dest="stream", action="store_false")
    run.add_argument("--metrics", nargs="?", const="", default=None, help="print timings (=full for phases)")
    run.add_argument("--verbose", nargs="?", const="min", default=None)
    run.add_argument("--profile", action="store_true",
                     help="time every operation of one prefill step and of one decode step, then generate")
    run.add_argument("--dump-logits", metavar="FILE",
                     help="write the logits every generated token was chosen from (float32 rows) and FILE.json")
    run.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    run.add_argument("--cache-tokens", type=int, default=0, help="tokens the cache holds (default: what the requests need)")
    run.add_argument("--max-batch", type=int, default=0)
    run.add_argument("--device", default="cuda:0")

    rnd = sub.add_parser("random-model", help="write a model folder with random weights")
    rnd.add_argument("--config", required=True, help="a config.json of the architecture")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--out", required=True)
    rnd.add_argument("--dtype", default="float32", choices=["bfloat16", "float32"])
    return ap


def _run(a) -> int:
    import time
    import torch
    from . import Engine
    from .registry import config_from_folder

    prompts = [_ids(p) for p in a.prompt]
    if a.prompt_file:
        with open(a.prompt_file) as f:
            prompts += [list(map(int, p)) for p in json.load(f)]
    cfg = config_from_folder(a.model)
    if a.random_prompts:
        g = torch.Generator().manual_seed(a.seed)
        for _ in range(a.random_prompts):
            n = int(torch.randint(a.min_len, a.max_len + 1, (1,), generator=g))
            prompts.append(torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist())
    if not prompts:
        raise SystemExit("run: give --prompt, --prompt-file or --random-prompts")
    need = sum(-(-(len(p) + a.max_tokens) // 64) * 64 for p in prompts)
    t0 = time.perf_counter()
    eng = Engine.from_pretrained(a.model, dtype=a.dtype, device=a.device, max_tokens=a.cache_tokens or need,
                                 max_batch=a.max_batch or len(prompts))
    load_ms = (time.perf_counter() - t0) * 1e3

    def on_token(req: int, tok: int) -> None:
        print(f"{req}\t{tok}", flush=True)

    if a.profile:
        from .profiling import format_table, profile_engine
        batch = prompts[: eng.max_batch]
        print(format_table(profile_engine(eng, batch, 1)), file=sys.stderr)

    dump, index = None, []
    on_logits = None
    if a.dump_logits:
        dump = open(a.dump_logits, "wb")

        def on_logits(requests, positions, logits) -> None:
            rows = logits[: len(requests)].detach().to("cpu", torch.float32).contiguous()
            rows.numpy().astype("<f4", copy=False).tofile(dump)
            for r, p in zip(requests, positions):
                index.append({"request": int(r), "position": int(p)})

    res = eng.generate(prompts, max_tokens=a.max_tokens, temperature=a.temperature, top_k=a.top_k,
                       top_p=a.top_p, seed=a.seed, stop_token_ids=a.stop,
                       on_token=on_token if a.stream else None, on_logits=on_logits)
    if dump is not None:
        dump.close()
        import numpy as np
        rows = np.fromfile(a.dump_logits, dtype="<f4").reshape(len(index), -1) if index else None
        # the token chosen at (request, position): the request's output at position - len(prompt);
        # a stop token that was chosen but not emitted has no entry in the output
        for i, rec in enumerate(index):
            out = res.tokens[rec["request"]]
            j = rec["position"] - len(prompts[rec["request"]])
            if 0 <= j < len(out):
                rec["token"] = int(out[j])
                rec["logit"] = float(rows[i, out[j]])
        with open(a.dump_logits + ".json", "w") as f:
            json.dump({"vocab": int(cfg.vocab_size), "rows": index}, f)
    if not a.stream:
        for i, t in enumerate(res.tokens):
            print(f"{i}\t{' '.join(map(str, t))}")
    if a.verbose:
        for i, (p, t, r) in enumerate(zip(prompts, res.tokens, res.finish_reasons)):
            print(f"request {i}: {len(p)} prompt tokens, {len(t)} new tokens, ended by {r}", file=sys.stderr)
    if a.metrics is not None:
        s = res.stats
        rate = lambda n, ms: (n / ms * 1e3) if ms > 0 else 0.0
        print("\nmetrics:")
        print(f"  ttft:       {s.prefill_ms:.1f} ms")
        print(f"  generation: {s.prefill_ms + s.decode_ms:.1f} ms  "
              f"{rate(s.new_tokens, s.prefill_ms + s.decode_ms):.1f} tok/s  ({s.new_tokens} tok)")
        print(f"  prefill:  {s.prefill_ms:.1f} ms  {rate(s.prompt_tokens, s.prefill_ms):.1f} tok/s  ({s.prompt_tokens} tok)")
        print(f"  decode:   {s.decode_ms:.1f} ms  {rate(s.new_tokens, s.decode_ms):.1f} tok/s  ({s.new_tokens} tok)")
        if a.metrics == "full":
            print(f"  phases:   load={load_ms:.1f} ms prefill={s.prefill_ms:.1f} ms decode={s.decode_ms:.1f} ms "
                  f"batches={s.batches} steps={s.prefill_steps}+{s.decode_steps}")
    return 0


def _random_model(a) -> int:
    import torch
    from .registry import config_from_dict
    from .weights import write_random_model
    with open(a.config) as f:
        cfg = config_from_dict(json.load(f))
    write_random_model(a.out, cfg, a.seed, torch.float32 if a.dtype == "float32" else torch.bfloat16)
    print(f"wrote {a.out}/config.json and model.safetensors")
    return 0


def main(argv=None) -> int:
    a = _parser().parse_args(argv)
    if a.command == "run":
        return _run(a)
    return _random_model(a)
