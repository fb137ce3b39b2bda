#!/usr/bin/env python
"""Benchmark of the quantized-matmul path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

N = 1  workload "w8a8_prefill_8b": one step = the four W8A8 prefill GEMMs of an 8B-class decoder
       layer at M = 8192 tokens (K x N = 4096x6144, 4096x28672, 4096x4096, 14336x4096), each
       preceded by the per-token dynamic quantization of its bf16 activations; bf16 outputs.
N > 1  workload "w8a8_row_parallel_allreduce": M = 4096, K = 28672 sharded evenly over the ranks,
       N = 8192; one step = dynamic quantization of the rank's activation shard + matmul +
       allreduce of the bf16 partials (strong scaling: the total work is fixed).

`value` counts GEMM operations only (2*M*N*K) over the device time of whole steps with inputs
resident in HBM; `e2e` is the same metric through the torch operators with pinned host buffers,
host<->device copies inside the timed region.  `roofline` describes the dominant kernel (the
tcgen05 CTA-pair GEMM; its four launches are timed with CUDA events around CUDA-graph replays, so
the host's launch cost is not in the figure), `cpu_baseline` the CPU restatement of the path timed
on this host's cores; `extras` holds the other configurations at one GPU (dynamic quant, W8A8
decode, W4A16 decode) as GB/s of algorithmic bytes against the measured copy bandwidth.
With `--impl reference` the CPU path itself is the thing measured.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PREFILL_M = 8192
PREFILL_GEMMS = [("qkv", 4096, 6144), ("gate_up", 4096, 28672), ("o_proj", 4096, 4096), ("down", 14336, 4096)]
ROWPAR = dict(M=4096, K=28672, N=8192)
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of w8a8_pair_kernel per prefill shape (K, N), from ncu
PAIR_DRAM_BYTES = {(4096, 6144): 65926656 + 69236736, (4096, 28672): 203958272 + 439107328,
                   (4096, 4096): 53308928 + 34690816, (14336, 4096): 510722048 + 59542528}
NOMINAL_INT8_TOPS = 4500.0  # NVIDIA's B200 dense int8 figure (9 POPS with 2:4 sparsity / 2)
NOMINAL_HBM_GBS = 8000.0


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


# ----------------------------------------------------------------------------------------------
# clocks sampler (reads only)
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.01)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


# ----------------------------------------------------------------------------------------------
# distributed plumbing
# ----------------------------------------------------------------------------------------------
def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def max_over_ranks(ms: float, world: int, dev) -> float:
    if world == 1:
        return ms
    import torch.distributed as dist

    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def timed_region(step_fn, steps: int, world: int, dev) -> float:
    """barrier+sync, `steps` steps between two CUDA events on the launching stream, sync; max over ranks (ms)."""
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step_fn()
    e1.record()
    torch.cuda.synchronize()
    barrier(world)
    return max_over_ranks(e0.elapsed_time(e1), world, dev)


# ----------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the CPU restatement on the host cores
# ----------------------------------------------------------------------------------------------
def cpu_prefill_sample(rows: int, seed: int = 0):
    """The 4-GEMM prefill step on `rows` of the 8192 tokens, reference-style CPU path."""
    from oracle import qmm_oracle as O

    g = torch.Generator().manual_seed(seed)
    work = []
    ops = 0
    for _, K, N in PREFILL_GEMMS:
        x = torch.randn((rows, K), generator=g).to(torch.bfloat16)
        w = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8).float()
        scale = torch.empty(N).uniform_(1e-3, 1e-2, generator=g)
        work.append((x, w, scale))
        ops += 2 * rows * K * N

    def step():
        for x, w, scale in work:
            O.cpu_path_w8a8(x, w, scale, None)

    return step, ops


def cpu_rowpar_sample(rows: int, seed: int = 0):
    from oracle import qmm_oracle as O

    g = torch.Generator().manual_seed(seed)
    K, N = ROWPAR["K"], ROWPAR["N"]
    x = torch.randn((rows, K), generator=g).to(torch.bfloat16)
    w = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8).float()
    scale = torch.empty(N).uniform_(1e-3, 1e-2, generator=g)

    def step():
        O.cpu_path_w8a8(x, w, scale, None)

    return step, 2 * rows * K * N


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    rows = 256
    if args.gpus == 1:
        step, ops = cpu_prefill_sample(rows)
        workload = "w8a8_prefill_8b"
        sample = f"{rows} of 8192 token rows through all four GEMMs per step"
    else:
        step, ops = cpu_rowpar_sample(rows)
        workload = "w8a8_row_parallel_allreduce"
        sample = f"{rows} of 4096 token rows, full K=28672 on one host (no sharding: one CPU)"
    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    tops = ops * args.steps / dt / 1e12
    line = {
        "impl": "reference", "metric": "W8A8 GEMM TOPS", "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": workload, "sample": sample},
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference = CPU restatement of the path (oracle port, torch fp32 BLAS in exact K chunks); the "
                "reference snapshot has no implementation of these operators and cannot be built here",
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------------
def time_kernel(fn, iters: int) -> float:
    """Average device time of one call (ms), CUDA events on the launching stream."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def time_kernel_graph(fn, launches: int = 6, replays: int = 5) -> float:
    """Average device time of one call (ms) with the host taken out: `launches` calls are captured into a
    CUDA graph on a side stream (after a warm-up there) and the graph is replayed.  For kernels of a few
    tens of microseconds the Python + tensor-map + launch cost of a call exceeds the kernel itself, and
    back-to-back eager launches would time the host.  Falls back to eager timing if capture fails."""
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(launches):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (replays * launches)
    except Exception:
        torch.cuda.synchronize()
        return time_kernel(fn, launches * replays)


def run_prefill(args, pkg, dev):
    capi = pkg.capi
    ops_mod = pkg.load_ops()
    peaks = measured_peaks()
    M = PREFILL_M
    g = torch.Generator(device=dev).manual_seed(2024)
    layers = []
    for name, K, N in PREFILL_GEMMS:
        x = torch.randn((M, K), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        w = torch.randint(-127, 128, (K, N), generator=g, device=dev, dtype=torch.int8)
        scale = torch.empty(N, device=dev).uniform_(1e-3, 1e-2, generator=g)
        out = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
        layers.append(dict(name=name, K=K, N=N, x=x, w=w, scale=scale, out=out))
    total_ops = sum(2 * M * L["K"] * L["N"] for L in layers)
    resident_bytes = sum(L["x"].numel() * 2 + L["w"].numel() + L["out"].numel() * 2 for L in layers)

    def step():
        for L in layers:
            q, s = capi.dynamic_quant(L["x"])
            capi.quant_matmul(q, L["w"], L["scale"], pertoken_scale=s, output_dtype=torch.bfloat16, out=L["out"])

    for _ in range(max(args.warmup, 3)):
        step()
    with ClockSampler(dev.index) as clocks:
        ms = timed_region(step, args.steps, 1, dev)
    value = total_ops * args.steps / (ms * 1e-3) / 1e12

    # ---- roofline of the dominant kernel: the tile GEMM alone, event-timed per shape
    gemm_ms = 0.0
    per_shape = {}
    for L in layers:
        q, s = capi.dynamic_quant(L["x"])
        fn = lambda L=L, q=q, s=s: capi.quant_matmul(q, L["w"], L["scale"], pertoken_scale=s,  # noqa: E731
                                                      output_dtype=torch.bfloat16, out=L["out"])
        for _ in range(3):
            fn()
        # replayed from a CUDA graph: an eager launch through ctypes costs more host time than the
        # shorter GEMMs run, and the events would then time the host
        t = time_kernel_graph(fn)
        gemm_ms += t
        per_shape[L["name"]] = {"ms": t, "tops": 2 * M * L["K"] * L["N"] / (t * 1e-3) / 1e12}
    achieved = total_ops / (gemm_ms * 1e-3) / 1e12
    int8_peak = 2.0 * peaks["bf16_sustained"]
    roofline = {"bound": "tensor", "kernel": "w8a8_pair_kernel", "achieved": achieved, "peak": int8_peak,
                "unit": "TFLOP/s", "frac": achieved / int8_peak, "traffic": sum(PAIR_DRAM_BYTES.values()),
                "traffic_note": "dram read+write bytes of one ncu-captured launch per shape, summed over the four "
                                "launches of a step (profiles/w8a8_pair_kernel_prefill_8b.md)",
                "algorithmic_bytes": sum(M * L["K"] + L["K"] * L["N"] + 2 * M * L["N"] for L in layers),
                "peak_note": f"2 x {peaks['source']} sustained bf16 cuBLAS throughput (int8 MMA issues at twice the "
                             "bf16 rate); no int8 figure is in MEASURED_PEAKS.json",
                "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS, "per_shape": per_shape}

    # ---- end to end through the torch operators, host buffers pinned
    host_x = [torch.empty((M, L["K"]), dtype=torch.bfloat16).pin_memory() for L in layers]
    host_y = [torch.empty((M, L["N"]), dtype=torch.bfloat16).pin_memory() for L in layers]
    for hx, L in zip(host_x, layers):
        hx.copy_(L["x"])
    h2d = sum(hx.numel() * 2 for hx in host_x)
    d2h = sum(hy.numel() * 2 for hy in host_y)
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    dx = [torch.empty_like(L["x"]) for L in layers]

    def e2e_step():
        evs = []
        with torch.cuda.stream(copy_in):
            for hx, d in zip(host_x, dx):
                d.copy_(hx, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_in)
                evs.append(ev)
        for i, L in enumerate(layers):
            main.wait_event(evs[i])
            q, s = ops_mod.npu_dynamic_quant(dx[i])
            y = ops_mod.npu_quant_matmul(q, L["w"], L["scale"], pertoken_scale=s, output_dtype=torch.bfloat16)
            done = torch.cuda.Event()
            done.record(main)
            copy_out.wait_event(done)
            with torch.cuda.stream(copy_out):
                host_y[i].copy_(y, non_blocking=True)
                y.record_stream(copy_out)
        main.wait_stream(copy_out)
        main.wait_stream(copy_in)

    e2e_steps = max(2, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    e2e_ms = timed_region(e2e_step, e2e_steps, 1, dev)
    e2e_value = total_ops * e2e_steps / (e2e_ms * 1e-3) / 1e12

    extras = secondary_workloads(capi, dev, peaks)
    cpu = cpu_baseline()
    line = {
        "metric": "W8A8 GEMM TOPS", "value": value, "unit": "TOPS", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "w8a8_prefill_8b", "M": M, "gemms_KxN": [[L["K"], L["N"]] for L in layers],
                   "step": "per GEMM: dynamic quant of bf16 activations + W8A8 matmul with fused dequant to bf16",
                   "l2": f"inputs larger than L2: {resident_bytes / 1e6:.0f} MB touched per step"},
        "clocks": clocks.summary(),
        "e2e": {"value": e2e_value, "unit": "TOPS", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                "path": "torch.ops.npu.npu_dynamic_quant + npu_quant_matmul, pinned host buffers, weights resident"},
        "gpu_launches": 8 * args.steps,
        "roofline": roofline, "cpu_baseline": cpu, "extras": extras,
    }
    print(json.dumps(line), flush=True)


def secondary_workloads(capi, dev, peaks):
    """Other configurations at 1 GPU: HBM-bound kernels in GB/s of algorithmic bytes (weights rotate over
    buffers larger than L2 in total, so they are never L2-resident)."""
    out = {}
    hbm = peaks["hbm_gbs"]
    try:
        # dynamic quant: 2*M*K read + M*K written + 4*M
        for (M, K) in [(8192, 4096), (8192, 14336)]:
            xs = [torch.randn((M, K), device=dev, dtype=torch.bfloat16) for _ in range(3)]
            i = [0]

            def f():
                i[0] += 1
                capi.dynamic_quant(xs[i[0] % 3])

            for _ in range(3):
                f()
            t = time_kernel_graph(f)
            gbs = (3 * M * K + 4 * M) / (t * 1e-3) / 1e9
            out[f"dynamic_quant_{M}x{K}"] = {"us": t * 1e3, "GB/s": gbs, "frac_of_measured_hbm": gbs / hbm,
                                             "frac_of_8TB/s": gbs / NOMINAL_HBM_GBS}
            del xs
        # W8A8 decode
        for (K, N) in [(8192, 28672), (28672, 8192)]:
            ws = [torch.randint(-127, 128, (K, N), dtype=torch.int8, device=dev) for _ in range(3)]
            scale = torch.empty(N, device=dev).uniform_(1e-3, 1e-2)
            for M in (1, 8, 32, 128):
                a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev)
                pt = torch.empty(M, device=dev).uniform_(1e-2, 5e-2)
                y = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
                i = [0]

                def f():
                    i[0] += 1
                    capi.quant_matmul(a, ws[i[0] % 3], scale, pertoken_scale=pt, output_dtype=torch.bfloat16, out=y)

                for _ in range(3):
                    f()
                t = time_kernel_graph(f)
                nbytes = K * N + M * K + 2 * M * N + 4 * N + 4 * M
                gbs = nbytes / (t * 1e-3) / 1e9
                out[f"w8a8_decode_M{M}_K{K}_N{N}"] = {"us": t * 1e3, "GB/s": gbs, "frac_of_measured_hbm": gbs / hbm,
                                                      "frac_of_8TB/s": gbs / NOMINAL_HBM_GBS}
            del ws
        # W4A16 decode
        K, N, group = 8192, 28672, 128
        packs = [torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), device=dev, dtype=torch.int64).to(torch.int32)
                 for _ in range(3)]
        sc = torch.empty((K // group, N), device=dev).uniform_(5e-3, 2e-2).to(torch.bfloat16)
        of = torch.empty((K // group, N), device=dev).uniform_(-1, 1).to(torch.bfloat16)
        for M in (1, 16, 64):
            x = torch.randn((M, K), device=dev, dtype=torch.bfloat16)
            i = [0]

            def f():
                i[0] += 1
                capi.weight_quant_batchmatmul(x, packs[i[0] % 3], sc, of, group_size=group)

            t = time_kernel_graph(f)
            nbytes = K * N // 2 + 2 * 2 * (K // group) * N + 2 * M * K + 2 * M * N
            gbs = nbytes / (t * 1e-3) / 1e9
            out[f"w4a16_decode_M{M}_K{K}_N{N}"] = {"us": t * 1e3, "GB/s": gbs, "frac_of_measured_hbm": gbs / hbm,
                                                   "frac_of_8TB/s": gbs / NOMINAL_HBM_GBS}
    except Exception as e:  # secondary numbers must not take the headline line down
        out["error"] = repr(e)
    return out


def cpu_baseline():
    """The CPU restatement of the prefill step on a bounded sample, all host threads."""
    torch.set_num_threads(os.cpu_count() or 1)
    rows = 256
    step, ops = cpu_prefill_sample(rows)
    step()
    t0 = time.perf_counter()
    n = 0
    while True:
        step()
        n += 1
        dt = time.perf_counter() - t0
        if dt >= 10.0 or n >= 50:
            break
    return {"value": ops * n / dt / 1e12, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{rows} of 8192 token rows through all four GEMMs, {n} repetitions in {dt:.1f} s"}


def run_rowpar(args, pkg, dev, rank, world):
    import torch.distributed as dist

    sys.path.insert(0, str(ROOT / "ascend-python_b200"))
    import torch_npu
    from ascend_python_b200.sharding import k_shard_bounds

    capi = pkg.capi
    M, K, N = ROWPAR["M"], ROWPAR["K"], ROWPAR["N"]
    b = k_shard_bounds(K, world)
    Kr = b[rank + 1] - b[rank]
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn((M, Kr), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    w = torch.randint(-127, 128, (Kr, N), generator=g, device=dev, dtype=torch.int8)
    scale = torch.empty(N, device=dev).uniform_(1e-3, 1e-2, generator=torch.Generator(device=dev).manual_seed(7))
    hcom = torch_npu.get_comm_name()
    total_ops = 2 * M * N * K

    def step():
        q, s = torch_npu.npu_dynamic_quant(x)
        return torch_npu.npu_mm_all_reduce_base(q, w, hcom, reduce_op="sum", dequant_scale=scale, pertoken_scale=s)

    for _ in range(max(args.warmup, 3)):
        step()
    with ClockSampler(dev.index) as clocks:
        ms = timed_region(step, args.steps, world, dev)
    value = total_ops * args.steps / (ms * 1e-3) / 1e12

    # matmul alone and allreduce alone (for the overlap figure), max over ranks
    q, s = torch_npu.npu_dynamic_quant(x)
    y = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
    gemm = lambda: capi.quant_matmul(q, w, scale, pertoken_scale=s, output_dtype=torch.bfloat16, out=y)  # noqa: E731
    for _ in range(3):
        gemm()
    gemm_ms = max_over_ranks(time_kernel(gemm, 10), world, dev)
    ar = lambda: dist.all_reduce(y)  # noqa: E731
    for _ in range(3):
        ar()
    barrier(world)
    ar_ms = max_over_ranks(time_kernel(ar, 10), world, dev)

    host_x = torch.empty((M, Kr), dtype=torch.bfloat16).pin_memory()
    host_x.copy_(x)
    host_y = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    dx = torch.empty_like(x)

    def e2e_step():
        dx.copy_(host_x, non_blocking=True)
        q, s = torch_npu.npu_dynamic_quant(dx)
        out = torch_npu.npu_mm_all_reduce_base(q, w, hcom, reduce_op="sum", dequant_scale=scale, pertoken_scale=s)
        host_y.copy_(out, non_blocking=True)

    e2e_steps = max(2, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    e2e_ms = timed_region(e2e_step, e2e_steps, world, dev)
    peaks = measured_peaks()
    int8_peak = 2.0 * peaks["bf16_sustained"]
    if rank == 0:
        step_ms = ms / args.steps
        achieved = (total_ops / world) / (gemm_ms * 1e-3) / 1e12
        line = {
            "metric": "W8A8 GEMM TOPS", "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": "w8a8_row_parallel_allreduce", "M": M, "K": K, "N": N, "k_per_rank": Kr,
                       "step": "dynamic quant of the rank's shard + W8A8 matmul + allreduce of bf16 partials "
                               + ("(NCCL)" if os.environ.get("QMM_ALLREDUCE", "") == "nccl"
                                  else "(one reduce+gather kernel per rank over peer memory; NCCL if unavailable)"),
                       "l2": f"inputs larger than L2: {(x.numel() * 2 + w.numel() + M * N * 2) / 1e6:.0f} MB per rank"},
            "clocks": clocks.summary(),
            "e2e": {"value": total_ops * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS",
                    "h2d_bytes_per_step": host_x.numel() * 2, "d2h_bytes_per_step": host_y.numel() * 2,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": args.steps * 3,
            "roofline": {"bound": "tensor", "kernel": "w8a8_pair_kernel", "achieved": achieved, "peak": int8_peak,
                         "unit": "TFLOP/s", "frac": achieved / int8_peak, "traffic": None,
                         "peak_note": f"2 x {peaks['source']} sustained bf16 cuBLAS throughput"},
            "overlap": {"gemm_ms": gemm_ms, "nccl_allreduce_ms": ar_ms, "step_ms": step_ms,
                        "allreduce_busbw_GB/s": 2 * (world - 1) / world * M * N * 2 / (ar_ms * 1e-3) / 1e9,
                        "roofline_ms": max(gemm_ms, ar_ms)},
            "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    barrier(world)
    torch_npu.destroy_comm(hcom)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()

    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        # launched by hand without torchrun: start one rank per GPU ourselves
        os.execvp(sys.executable, [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                                   f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port",
                                   str(29400 + os.getpid() % 500), str(Path(__file__).resolve()), *sys.argv[1:]])

    if args.impl == "reference":
        run_reference(args)
        return

    from __graft_entry__ import load_package

    rank, local_rank, world = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    pkg = load_package()
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        try:
            run_rowpar(args, pkg, dev, rank, world)
        finally:
            dist.destroy_process_group()
    else:
        run_prefill(args, pkg, dev)


if __name__ == "__main__":
    main()
