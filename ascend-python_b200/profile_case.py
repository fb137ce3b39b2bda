"""Runs one kernel of the library a few times on synthetic data: the target of `ncu` captures.

    python ascend-python_b200/profile_case.py quant_matmul --M 8192 --K 4096 --N 6144 [--algo 1] [--iters 3]
    python ascend-python_b200/profile_case.py dynamic_quant --M 8192 --K 14336
    python ascend-python_b200/profile_case.py w4a16 --M 16 --K 8192 --N 28672

Prints the CUDA-event time per launch (not meaningful under a profiler).
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from __graft_entry__ import load_package  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["quant_matmul", "dynamic_quant", "w4a16"])
    ap.add_argument("--M", type=int, default=8192)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--N", type=int, default=6144)
    ap.add_argument("--algo", type=int, default=0)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--buffers", type=int, default=1, help="rotate over this many weight/input buffers")
    ap.add_argument("--graph", action="store_true", help="also time the launches replayed from a CUDA graph")
    args = ap.parse_args()
    capi = load_package().capi
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    M, K, N = args.M, args.K, args.N
    if args.op == "quant_matmul":
        a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev)
        ws = [torch.randint(-127, 128, (K, N), dtype=torch.int8, device=dev) for _ in range(args.buffers)]
        scale = torch.empty(N, device=dev).uniform_(1e-3, 1e-2)
        pt = torch.empty(M, device=dev).uniform_(1e-2, 5e-2)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        fn = lambda i: capi.quant_matmul(a, ws[i % len(ws)], scale, pertoken_scale=pt,  # noqa: E731
                                         output_dtype=torch.bfloat16, algo=args.algo, out=out)
    elif args.op == "dynamic_quant":
        xs = [torch.randn((M, K), device=dev, dtype=torch.bfloat16) for _ in range(args.buffers)]
        fn = lambda i: capi.dynamic_quant(xs[i % len(xs)])  # noqa: E731
    else:
        x = torch.randn((M, K), device=dev, dtype=torch.bfloat16)
        packs = [torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), device=dev, dtype=torch.int64).to(torch.int32)
                 for _ in range(args.buffers)]
        sc = torch.empty((K // 128, N), device=dev).uniform_(5e-3, 2e-2).to(torch.bfloat16)
        of = torch.empty((K // 128, N), device=dev).uniform_(-1, 1).to(torch.bfloat16)
        fn = lambda i: capi.weight_quant_batchmatmul(x, packs[i % len(packs)], sc, of, group_size=128)  # noqa: E731
    fn(0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.iters):
        fn(i + 1)
    e1.record()
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    eager_us = e0.elapsed_time(e1) / args.iters * 1e3
    graph_us = float("nan")
    if args.graph:
        # the same launches replayed from a CUDA graph: device time without the host's per-call cost
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for i in range(3):
                fn(i)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(args.iters):
                fn(i)
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(5):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        graph_us = e0.elapsed_time(e1) / (5 * args.iters) * 1e3
        assert capi.device_status() == 0
    print(f"{args.op} M={M} K={K} N={N}: {eager_us:.1f} us per eager launch, {graph_us:.1f} us per launch in a graph")


if __name__ == "__main__":
    main()
