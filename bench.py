#!/usr/bin/env python3
"""Headline benchmark: decoded tokens per second of GPT-2 small (124M layer sizes, seeded random
weights, bfloat16) at batch 8 on one B200, with prefill, roofline and end-to-end figures.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--preset NAME]

One JSON line is printed.  A "step" is one decode step of the whole batch.
  value      decoded tokens per second, device-timed (CUDA events) around each step's kernels,
             L2 flushed between steps; exactly K steps after W warm-up steps.
  e2e        the same through ``Engine.step`` (scheduler, step function, sampler), host token
             lists in, tokens read back to the host every step, wall clock; ``host_ms_per_step`` is
             what the host spends on a step without its waits for the device.
  prefill    one step of 2 prompts x 1,024 tokens; frac = FLOPs / time / the bf16 peak.
  roofline   bytes a decode step must read (weights once + the live requests' cache) / time /
             the HBM peak.
  points     decode at batch 1 and 64, same context.
  workloads  the reference's own small workload (prompts of 64 tokens, 64 greedy tokens, batch 1, 8
             and 64: tokens a second and the fraction of the HBM ceiling); with ``--preset
             gpt2-medium`` the mixed continuous batch (64 requests, prompts of 16 to 1023 tokens, outputs
             of 16 to 255, at most 2,048 prompt tokens a step, temperature 0.8: generated tokens a second, time to first token,
             time per output token, pages, bytes the steps had to read over the memory's rate); with
             ``--preset gpt2-xl`` decode at batch 1, 8 and 64 with prompts of 512 tokens and 256 new
             ones, and the pages they fill of the pool; with the default preset the same layers
             with 8,192 positions, decoding at batch 1, 8 and 32 behind prompts of 8,144 tokens, and 512
             requests arriving at 400 a second (prompts and outputs of 16 to 256 tokens, temperature 0.8)
             through static and continuous batching.
  provenance the commit, whether the tree was clean, the tools, the device, the time.
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
    ap.add_argument("--context", type=int, default=None, help="context length the decode ends at (default: the model's)")
    ap.add_argument("--preset", default="gpt2-small")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the preset (recorded in config)")
    ap.add_argument("--skip-points", action="store_true", help="leave out the points at batch 1 and 64")
    ap.add_argument("--skip-workloads", action="store_true", help="leave out the workloads object")
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

    from nanoinfer_b200.registry import get_architecture
    context = args.context or get_architecture(cfg.architecture).build_spec(cfg).max_positions or 1024
    eng = bs.build_engine(model_dir, "bfloat16", args.batch, context, max_rows=2048)
    prompt_len = context - steps - warmup
    if prompt_len < 1:
        print(json.dumps({"error": f"steps + warmup must be < the context length {context}"}))
        return 2

    def decode_point(batch: int):
        e = bs.build_engine(model_dir, "bfloat16", batch, context, max_rows=2048)
        bs.preheat(e, args.preheat)
        d = bs.time_decode(e, batch, prompt_len, steps, warmup)
        del e
        torch.cuda.empty_cache()
        return d

    clocks = bs.ClockSampler()
    clocks.start()                  # (it takes a moment to start: the untimed load below gives it that)
    bs.preheat(eng, args.preheat)   # untimed: the device leaves its idle state before anything is timed
    dec = bs.time_decode(eng, args.batch, prompt_len, steps, warmup)
    clock_record = clocks.stop()
    launches = dec["launches_per_step"]
    e2e = bs.time_e2e_decode(eng, args.batch, prompt_len, steps, warmup)
    pre = bs.time_prefill(eng, 2, 1024, runs=5, warmup=3)
    weight_bytes, n_params = bs.weight_bytes_per_step(eng.model), bs.parameter_count(eng.model)
    step_bytes = weight_bytes + bs.kv_bytes(eng.cache, [dec["mean_context"]] * args.batch)
    del eng
    torch.cuda.empty_cache()

    achieved_gbs = step_bytes / (dec["ms_per_step"] / 1e3) / 1e9
    prefill_frac = pre["flops"] / (pre["ms"] / 1e3) / (peaks["bf16_tflops"] * 1e12)
    points = {}
    if not args.skip_points:
        points = {"decode_b1": decode_point(1)["tokens_per_s"], "decode_b64": decode_point(64)["tokens_per_s"]}

    workloads = {}
    if not args.skip_workloads:
        # the reference's own workload: prompts of 64 tokens, 64 greedy tokens (crates/cli/src/bench.rs:24-58)
        short = bs.decode_points(model_dir, "bfloat16", [1, 8, 64], 64, 64, warmup=3, runs=2)
        workloads["prompt64_gen64"] = {f"b{p['batch']}": {"decode_tok_s": p["decode_tok_s"], "frac_of_hbm": p["frac_of_hbm"],
                                                          "prefill_tok_s": p["prefill_tok_s"]} for p in short}
        # prefill where one tile per SM is no longer the limit: 8 prompts of 1,024 tokens in one step
        big = bs.build_engine(model_dir, "bfloat16", 8, context, max_rows=8192)
        p8 = bs.time_prefill(big, 8, min(1024, context), runs=3, warmup=3)
        workloads["prefill_8x1024"] = {"tok_s": p8["tokens_per_s"], "ms": p8["ms"],
                                       "frac": p8["flops"] / (p8["ms"] / 1e3) / (peaks["bf16_tflops"] * 1e12)}
        del big
        torch.cuda.empty_cache()
        if args.preset == "gpt2-small":
            # the same layers with a context of 8,192 positions: a decode step is then mostly keys and values
            far_dir, _ = bs.model_folder(args.preset, seed=1234, dtype=dtype, n_layer=args.layers,
                                         overrides={"n_positions": 8192})
            far = bs.decode_points(far_dir, "bfloat16", [1, 8, 32], 8192 - 48, 32, warmup=6, runs=2)
            workloads["context_8192"] = {f"b{p['batch']}": {k: p[k] for k in (
                "decode_tok_s", "decode_ms_per_step", "frac_of_hbm", "prefill_tok_s", "prefill_ms")} for p in far}
            # requests arriving at a steady rate (the reference's serving workload, crates/cli/src/metal_serve.rs:97-131:
            # prompts and outputs of 16 to 256 tokens), continuous against static batching
            from nanoinfer_b200.serve_bench import run_serving
            s = run_serving(model_dir, "bfloat16", requests=512, max_batch=64, prompt_min=16, prompt_max=256, out_min=16,
                            out_max=256, rate=400.0, prefill_budget=2048, temperature=0.8, top_k=40, seed=7, quiet=True)
            workloads["arrivals_400_a_second_t0.8"] = {
                p["policy"]: {k: p[k] for k in ("throughput_tok_s", "generated_tokens", "makespan_s", "iterations",
                                                "ttft_ms", "tpot_ms", "kv_pages_peak", "preemptions")} for p in s["policies"]}
        if args.preset == "gpt2-medium":
            from nanoinfer_b200.serve_bench import run_serving
            # (at most 2,048 prompt tokens a step, the engine's own default: with 512 the same requests take 0.57 s
            # instead of 0.48 s and the first token comes after 98 ms instead of 34 ms at the median)
            s = run_serving(model_dir, "bfloat16", requests=64, max_batch=64, prompt_min=16, prompt_max=1023, out_min=16,
                            out_max=255, prefill_budget=2048, temperature=0.8, top_k=40, seed=7, quiet=True)
            workloads["mixed_64_requests_t0.8"] = {
                p["policy"]: {k: p[k] for k in ("throughput_tok_s", "generated_tokens", "makespan_s", "iterations",
                                                "ttft_ms", "tpot_ms", "kv_pages_peak", "kv_pages_total", "hbm_gbs",
                                                "hbm_frac", "preemptions")} for p in s["policies"]}
            workloads["mixed_64_requests_t0.8"]["prefill_budget"] = s["prefill_budget"]
        if args.preset == "gpt2-xl":
            long = bs.decode_points(model_dir, "bfloat16", [1, 8, 64], 512, 256, warmup=3, runs=2)
            workloads["prompt512_gen256"] = {f"b{p['batch']}": {k: p[k] for k in (
                "decode_tok_s", "decode_ms_per_step", "frac_of_hbm", "prefill_tok_s", "pages_used", "pages_total")}
                for p in long}

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
                "host_ms_per_step": e2e["host_ms_per_step"], "all_rows_in_every_step": e2e["all_rows_in_every_step"],
                "h2d_bytes_per_step": e2e["h2d_bytes_per_step"], "d2h_bytes_per_step": e2e["d2h_bytes_per_step"]},
        "gpu_launches": (launches or 0) * steps,
        "prefill": {"value": pre["tokens_per_s"], "tokens": pre["tokens"], "ms": pre["ms"], "frac": prefill_frac},
        "roofline": {"bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved_gbs / peaks["hbm_gbs"]},
        "points": points,
        "workloads": workloads,
        "provenance": bs.provenance(),
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
