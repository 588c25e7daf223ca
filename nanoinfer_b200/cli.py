"""Command line in the manner of the reference's ``nanoinfer`` binary (crates/cli/src/main.rs:28-83):

    python -m nanoinfer_b200 --weights DIR generate --prompt "Hello" --tokens 40
    python -m nanoinfer_b200 --weights DIR generate --prompt-ids 464,3616 --tokens 40
    python -m nanoinfer_b200 --weights DIR bench --tokens 64 --prompt-len 64 --batch 1,8,64
    python -m nanoinfer_b200 --weights DIR serve-bench --requests 128 --max-batch 32
    python -m nanoinfer_b200 --weights DIR tokenize "Hello world"
    python -m nanoinfer_b200 random-weights --config gpt2-small --seed 1 --out DIR

``--weights`` is the reference's global option (main.rs:30-32): the folder with
``model.safetensors`` (and here ``config.json``).  ``generate`` keeps the reference's options
and defaults (main.rs:48-72): ``--prompt TEXT --tokens 40 --temperature 0.0 --top-k 40 --seed 42
--profile --trace-out FILE``; a text prompt needs the tokenizer's ``vocab.json`` and ``merges.txt``
in the folder (main.rs:85-89), token ids can be given instead with ``--prompt-ids``.  ``bench`` keeps ``--tokens 64 --prompt-len 64
--runs 5 --warmup 1 --bandwidth-gbs`` (crates/cli/src/bench.rs:24-58) and ``--batch``/``--dtype``
of the batch sweep (crates/cli/src/metal_batch.rs:20-58).  The reference chooses a strategy
with ``--stage``; here the one choice left is ``--dtype``.  ``serve-bench`` keeps the options of the
reference's ``metal-serve`` (crates/cli/src/metal_serve.rs:33-79): ``--requests --max-batch
--prompt-min/max --out-min/max --rate --prefill-budget --kv-blocks --seed --gantt --out --summary``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List


def _preset_path(name: str) -> str:
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config", "presets")
    return name if os.path.isfile(name) else os.path.join(here, name + ".json")


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(" ", ",").split(",") if t]


def cmd_random_weights(args) -> int:
    import torch

    from .registry import get_architecture
    from .config.base import architecture_name
    from .models.model import Model
    from .weights.random_init import write_random_model

    with open(_preset_path(args.config)) as fh:
        raw = json.load(fh)
    cfg = get_architecture(architecture_name(raw)).config_cls.from_dict(raw)
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    write_random_model(cfg, args.out, args.seed, dtype)
    if args.tokenizer:
        from .tokenizer import write_byte_tokenizer
        write_byte_tokenizer(args.out, Model(get_architecture(cfg.architecture).build_spec(cfg), cfg).vocab_size)
    from .measure import parameter_count_of_spec
    n_params = parameter_count_of_spec(Model(get_architecture(cfg.architecture).build_spec(cfg), cfg))
    print(f"wrote {args.out} ({n_params / 1e6:.1f}M params, {args.dtype}, seed {args.seed})", file=sys.stderr)
    return 0


def cmd_tokenize(args) -> int:
    """The reference's ``tokenize TEXT`` (crates/cli/src/main.rs:81-82, 121-128): each id with its piece, then
    the count; needs no GPU."""
    from .tokenizer import Tokenizer, TokenizerError
    try:
        tok = Tokenizer.from_folder(args.weights)
    except TokenizerError as e:
        print(str(e), file=sys.stderr)
        return 2
    ids = tok.encode(args.text)
    for i in ids:
        print(f"{i:>6}  {tok.decode([i])!r}")
    print(f"{len(ids)} tokens")
    return 0


def cmd_generate(args) -> int:
    import torch

    from .engine.engine import Engine
    from .sampling.sampler import SamplingParams

    tok = None
    if args.prompt_ids is not None:
        prompt = _ids(args.prompt_ids)
    elif args.prompt is not None:
        from .tokenizer import Tokenizer, TokenizerError
        try:
            tok = Tokenizer.from_folder(args.weights)
        except TokenizerError as e:
            print(str(e), file=sys.stderr)
            return 2
        prompt = tok.encode(args.prompt)
    else:
        print("generate: give the prompt as --prompt TEXT, or as token ids with --prompt-ids a,b,c", file=sys.stderr)
        return 2
    if not prompt:
        print("generate: the prompt is empty", file=sys.stderr)
        return 2
    t0 = time.perf_counter()
    eng = Engine(args.weights, dtype=args.dtype, max_batch=1, max_rows=max(64, len(prompt)),
                 use_graphs=not args.trace_out, run_ahead=not args.trace_out)
    rec = None
    if args.trace_out:
        from . import trace
        rec = trace.start()
    from .measure import parameter_count
    print(f"loaded {args.weights} ({parameter_count(eng.model) / 1e6:.1f}M params) in "
          f"{time.perf_counter() - t0:.2f}s", file=sys.stderr)
    params = SamplingParams(max_new_tokens=args.tokens, temperature=args.temperature, top_k=args.top_k,
                            seed=args.seed)
    req = eng.add_request(prompt, params)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    t_first = None
    printed = 0
    pending = b""       # bytes of tokens that do not yet end a character
    if tok is not None:
        print(args.prompt, end="", flush=True)
    while eng.has_work():
        if rec is not None:   # (one scheduler decision is one step: the whole prompt, then a token at a time)
            n_in = eng.scheduler.running[0].n_pending if eng.scheduler.running else len(prompt)
            rec.begin_step("prefill" if n_in > 1 else "decode", n_in, len(prompt) + len(req.output) + (n_in > 1))
        eng.step()
        # (the engine runs a step ahead of its reads: the newest entry may still be a negative stand-in)
        while printed < len(req.output) and req.output[printed] >= 0:
            if t_first is None:
                t_first = time.perf_counter() - t0
            if tok is None:
                print(req.output[printed], end=" ", flush=True)
            else:      # a token may be part of a multi-byte character: print what is whole
                pending += tok.token_bytes(req.output[printed])
                text = pending.decode("utf-8", errors="ignore")
                if text and text.encode("utf-8") == pending or len(pending) > 8:
                    print(pending.decode("utf-8", errors="replace"), end="", flush=True)
                    pending = b""
            printed += 1
    total = time.perf_counter() - t0
    print()
    n = len(req.output)
    t_first = t_first or total
    print(f"[{args.dtype}] prompt {len(prompt)} tok, prefill {t_first * 1e3:.1f} ms "
          f"({len(prompt) / t_first:.1f} tok/s), decode {(n - 1) / max(total - t_first, 1e-9):.2f} tok/s",
          file=sys.stderr)
    if rec is not None:
        from . import trace
        from .measure import kv_bytes
        trace.stop()
        limit = eng.model.max_positions or (len(prompt) + n)
        trace.write_jsonl(rec, args.trace_out,
                          {"config": {"model": os.path.basename(os.path.normpath(args.weights)), "dtype": args.dtype,
                                      "backend": "sm_100a", "step": "paged-kv", "params": parameter_count(eng.model)},
                           "prompt_tokens": prompt},
                          [{"id": t} for t in req.output],
                          {"len": len(prompt) + n, "capacity": limit, "bytes": int(kv_bytes(eng.cache, [len(prompt) + n]))})
        print(f"wrote {len(rec.events)} launches of {len(rec.steps)} steps to {args.trace_out}", file=sys.stderr)
    if args.profile:
        from .bench_support import print_profile
        print_profile(eng, prompt)
    return 0


def cmd_bench(args) -> int:
    from .bench_support import run_cli_bench

    return run_cli_bench(args)


def cmd_serve_bench(args) -> int:
    from .serve_bench import run_cli

    return run_cli(args)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="nanoinfer_b200", description="A small LLM inference engine for one B200")
    ap.add_argument("--weights", default="weights/gpt2",
                    help="folder with config.json and model.safetensors")
    sub = ap.add_subparsers(dest="cmd", required=True)

    g = sub.add_parser("generate", help="generate tokens from a prompt")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--prompt", default=None, help="the prompt as text (needs vocab.json and merges.txt in the folder)")
    g.add_argument("--prompt-ids", default=None, help="the prompt as comma-separated token ids")
    g.add_argument("--tokens", type=int, default=40, help="number of tokens to generate")
    g.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    g.add_argument("--top-k", type=int, default=40)
    g.add_argument("--seed", type=int, default=42)
    g.add_argument("--profile", action="store_true",
                   help="print afterwards where the time goes, op by op, with GFLOP/s, GB/s and the fraction of the roofline")
    g.add_argument("--trace-out", default=None,
                   help="write every launch of the run (op, layer, time, FLOPs, bytes) as JSON lines to this file; "
                        "the run then launches its kernels one by one instead of replaying graphs")
    g.set_defaults(fn=cmd_generate)

    b = sub.add_parser("bench", help="measure prefill and decode throughput")
    b.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    b.add_argument("--tokens", type=int, default=64, help="decode steps to time per run")
    b.add_argument("--prompt-len", type=int, default=64)
    b.add_argument("--batch", default="1", help="batch sizes, e.g. 1,8,64")
    b.add_argument("--runs", type=int, default=5)
    b.add_argument("--warmup", type=int, default=1)
    b.add_argument("--bandwidth-gbs", type=float, default=None,
                   help="memory bandwidth for the decode ceiling (default: the measured peak)")
    b.add_argument("--out", default=None, help="append the result line (with commit, tools and time) to this file")
    b.add_argument("--note", default="")
    b.add_argument("--profile", action="store_true",
                   help="also print, per batch size, where a prefill and a decode step spend their time, op by op")
    b.set_defaults(fn=cmd_bench)

    s = sub.add_parser("serve-bench", help="many requests of random lengths: continuous against static batching")
    s.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    s.add_argument("--requests", type=int, default=128, help="number of requests")
    s.add_argument("--max-batch", type=int, default=32, help="most requests in flight")
    s.add_argument("--prompt-min", type=int, default=16)
    s.add_argument("--prompt-max", type=int, default=256, help="prompt lengths are uniform in [min, max]")
    s.add_argument("--out-min", type=int, default=16)
    s.add_argument("--out-max", type=int, default=256, help="output lengths are uniform in [min, max] (no end token)")
    s.add_argument("--rate", type=float, default=0.0, help="mean arrivals per second (0: everything at t = 0)")
    s.add_argument("--prefill-budget", type=int, default=256, help="most prompt tokens per step")
    s.add_argument("--kv-blocks", type=int, default=None,
                   help="pages of 16 positions in the pool (default: max_batch full requests and 8 more)")
    s.add_argument("--seed", type=int, default=7)
    s.add_argument("--temperature", type=float, default=0.0, help="0 = greedy; else every request samples, seeded by --seed + its number")
    s.add_argument("--top-k", type=int, default=40)
    s.add_argument("--gantt", type=int, default=32, help="requests in the summary's timeline")
    s.add_argument("--out", default=None, help="append one result line per policy to this file")
    s.add_argument("--summary", default=None, help="write the full summary (JSON) to this file")
    s.add_argument("--note", default="")
    s.set_defaults(fn=cmd_serve_bench)

    t = sub.add_parser("tokenize", help="print the token ids of a text (needs vocab.json and merges.txt in the folder)")
    t.add_argument("text")
    t.set_defaults(fn=cmd_tokenize)

    r = sub.add_parser("random-weights", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True, help="a preset name (gpt2-small, gpt2-medium, gpt2-xl, "
                                                   "gpt2-tiny-a, gpt2-tiny-b) or a config.json file")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--tokenizer", action="store_true",
                   help="also write a byte-level tokenizer (256 byte tokens, no merges), so that text can be given")
    r.set_defaults(fn=cmd_random_weights)

    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
