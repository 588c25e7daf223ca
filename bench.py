#!/usr/bin/env python3
"""Headline benchmark: decoded tokens per second of GPT-2 small (124M layer sizes, seeded random
weights, bfloat16) at batch 8 on one B200, with prefill, roofline and end-to-end figures.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line is printed.  A "step" is one decode step of the whole batch.
  value     decoded tokens per second, device-timed (CUDA events) around each step's kernels,
            L2 flushed between steps.
  e2e       the same through ``Engine.step`` (scheduler, step function, sampler), host token
            lists in, tokens read back to the host every step, wall clock.
  prefill   one step of 2 prompts x 1,024 tokens; frac = FLOPs / time / the bf16 peak.
  roofline  bytes a decode step must read (weights once + the live requests' cache) / time /
            the HBM peak.
  points    decode at batch 1 and 64.
Peaks come from MEASURED_PEAKS.json beside this file when present, else from the fallback
figures (6.65 TB/s, 1.59 PFLOP/s).  More than one GPU is out of scope: --gpus N>1 says so and
exits with 2.  The reference (Rust, Metal, WebGPU) cannot be installed here, so
--impl reference prints its "unavailable" line.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

#: the reference's published batched decode at B = 8 in 16-bit floats on an Apple M4 GPU
#: (docs/LOG.md:1176 of the reference; bench/batching.json series f16), the nearest published figure
REFERENCE_B8_TOK_S = 2205.0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=None, help="context length the decode ends at (default n_positions)")
    ap.add_argument("--preset", default="gpt2-small")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the preset (recorded in config)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--preheat", type=float, default=1.5,
                    help="seconds of untimed prefill steps before the timed loops (0: none)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust/Metal/WebGPU project without setup.py or pyproject.toml: "
                          "pip cannot install it, and no Rust toolchain or graphics stack exists here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: --gpus {args.gpus} is out of scope for this engine")
        return 2

    import torch

    from nanoinfer_b200 import bench_support as bs

    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    peaks = bs.measured_peaks()
    dtype = torch.bfloat16
    model_dir, cfg = bs.model_folder(args.preset, seed=1234, dtype=dtype, n_layer=args.layers)
    from nanoinfer_b200.cli import _preset_path
    with open(_preset_path(args.preset)) as fh:
        full_layers = json.load(fh)["n_layer"]
    context = args.context or cfg.n_positions
    prompt_len = context - steps - warmup
    if prompt_len < 1:
        print(json.dumps({"error": f"steps + warmup must be < the context length {context}"}))
        return 2

    def decode_point(batch: int):
        eng = bs.build_engine(model_dir, "bfloat16", batch, context, max_rows=2048)
        bs.preheat(eng, args.preheat)
        d = bs.time_decode(eng, batch, prompt_len, steps, warmup)
        del eng
        torch.cuda.empty_cache()
        return d

    eng = bs.build_engine(model_dir, "bfloat16", args.batch, context, max_rows=2048)
    bs.preheat(eng, args.preheat)   # untimed: the device leaves its idle state before anything is timed
    dec = bs.time_decode(eng, args.batch, prompt_len, steps, warmup, clocks=bs.ClockSampler())
    launches = dec["launches_per_step"]
    clock_record = dec["clocks"]
    e2e = bs.time_e2e_decode(eng, args.batch, prompt_len, steps, warmup)
    pre = bs.time_prefill(eng, 2, 1024, runs=5, warmup=3)
    weight_bytes, n_params, kv_groups = bs.weight_bytes_per_step(eng.model), bs.parameter_count(eng.model), eng.cache
    del eng
    torch.cuda.empty_cache()

    step_bytes = weight_bytes + bs.kv_bytes(kv_groups, [dec["mean_context"]] * args.batch)
    achieved_gbs = step_bytes / (dec["ms_per_step"] / 1e3) / 1e9
    prefill_frac = pre["flops"] / (pre["ms"] / 1e3) / (peaks["bf16_tflops"] * 1e12)
    points = {}
    if not args.skip_points:
        points = {"decode_b1": decode_point(1)["tokens_per_s"], "decode_b64": decode_point(64)["tokens_per_s"]}

    out = {
        "metric": "decode tok/s", "value": dec["tokens_per_s"], "unit": "tok/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": dec["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": dec["tokens_per_s"] / REFERENCE_B8_TOK_S, "dtype": "bf16", "data": "synthetic",
        "config": {
            "model": f"{args.preset}-{n_params / 1e6:.0f}M random weights", "n_layer": cfg.n_layer, "n_layer_full": full_layers,
            "n_embd": cfg.n_embd, "n_head": cfg.n_head, "head_dim": cfg.head_dim, "n_inner": cfg.inner_dim,
            "vocab_size": cfg.vocab_size, "n_positions": cfg.n_positions, "global_batch": args.batch,
            "seq_len": context, "prompt_len": prompt_len, "mean_context": round(dec["mean_context"], 1),
            "page_size": 16, "kv_dtype": "bf16", "parallelism": "single GPU", "sampling": "greedy",
            "l2": "flushed between timed steps", "peaks": peaks["source"],
        },
        "clocks": clock_record,
        "e2e": {"value": e2e["tokens_per_s"], "unit": "tok/s", "ms_per_step": e2e["ms_per_step"],
                "h2d_bytes_per_step": e2e["h2d_bytes_per_step"], "d2h_bytes_per_step": e2e["d2h_bytes_per_step"]},
        "gpu_launches": (launches or 0) * steps,
        "prefill": {"value": pre["tokens_per_s"], "tokens": pre["tokens"], "ms": pre["ms"], "frac": prefill_frac},
        "roofline": {"bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved_gbs / peaks["hbm_gbs"]},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
