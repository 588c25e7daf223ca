"""Times the matrix products of one layer alone, as a decode step runs them.

    python -m nanoinfer_b200.kernels.microbench --rows 8,16,32,64 [--width 768 --inner 3072 --vocab 50257]

For each product of a GPT-2 layer (q/k/v, attention output, MLP up, MLP down) and the LM head it
captures 60 back-to-back launches into one CUDA graph (programmatic dependent launch on, as in a
step), cycling through enough copies of the weights that each launch reads them from DRAM, and
prints the time per launch of the few-row kernel (warp-level MMAs; the split of K chosen by the
library, then forced to 1, 2, 4 and 8 blocks of a cluster) beside the tcgen05 kernel.  Times are CUDA
events around a graph replay, in microseconds.
"""
from __future__ import annotations

import argparse

import torch

from . import ops

LAUNCHES = 60


def _time_graph(fn, copies: int) -> float:
    for i in range(3):
        fn(i % copies)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(LAUNCHES):
            fn(i % copies)
    graph.replay()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    graph.replay()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / LAUNCHES * 1e3


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--rows", default="8,16,32,64", help="rows of the step, comma separated")
    ap.add_argument("--width", type=int, default=768)
    ap.add_argument("--inner", type=int, default=3072)
    ap.add_argument("--vocab", type=int, default=50257)
    args = ap.parse_args(argv)
    dev = torch.device("cuda")
    torch.manual_seed(0)
    C, I, V = args.width, args.inner, args.vocab
    shapes = [("q/k/v", 3 * C, C), ("out", C, C), ("MLP up", I, C), ("MLP down", C, I), ("head", V, C)]
    for name, N, K in shapes:
        copies = max(2, int(300e6 / (N * K * 2)))          # more than the L2 holds
        ws = [(torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16) for _ in range(copies)]
        bias = torch.randn(N, device=dev)
        for M in (int(v) for v in args.rows.split(",")):
            a = torch.randn(M, K, device=dev).to(torch.bfloat16)
            out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
            cols = []
            for split in (0, 1, 2, 4, 8):
                try:
                    taken = M <= ops.SKINNY_MAX_ROWS and ops.linear_skinny(a, None, ws[0], bias, out, M, split=split)
                except ops.KernelError:
                    taken = False
                if taken:
                    t = _time_graph(lambda i: ops.linear_skinny(a, None, ws[i], bias, out, M, split=split), copies)
                    cols.append(f"{'auto' if split == 0 else 'x%d' % split} {t:.1f}")
            t = _time_graph(lambda i: ops.linear_tc(a, ws[i], bias, out, M), copies)
            print(f"{name:<9} {N:>6} x {K:<5} rows {M:<4} few-row: {'  '.join(cols) or '-':<48} tcgen05: {t:.1f}", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
