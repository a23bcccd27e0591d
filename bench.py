#!/usr/bin/env python3
"""Benchmark of the speculative-verify quantized matmul.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: GGUF Q4_K projections with the MLP shapes of a 27B model,
gate / up (K = 5120, N = 17408) and down (K = 17408, N = 5120), against M = 8 drafted rows
(fp16 activations, fp32 accumulate, fp16 outputs). One step is one pass over `layers` such MLP
blocks, every projection with its own weight buffer, so a step streams layers * 150 MB of
distinct compressed weights (far more than L2). Inputs are synthetic with the configured value
distributions: real GGUF files are not available where this runs.

The metric is weight GB/s: compressed weight bytes streamed per second (GB = 1e9), the
reference's own convention (block bytes only). With N > 1 every projection is sharded along its
output rows across the ranks, each rank computes its rows transposed ([N/G, M]) and one NCCL
all-gather per projection assembles [N, M]; the workload is the same at every N (strong scaling).

Prints one JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MLP_SHAPES = [("gate", 17408, 5120), ("up", 17408, 5120), ("down", 5120, 17408)]  # (name, N, K)
# --workload stack: all seven projections of a 27B layer (the full verify stack is 64 such layers)
STACK_SHAPES = [("q", 6144, 5120), ("k", 1024, 5120), ("v", 1024, 5120), ("o", 5120, 6144)] + MLP_SHAPES
# which projections wait for the other ranks' previous exchange (N > 1): those whose input is made
# from exchanged outputs. q and gate read the block input (the previous down / o output); k, v and
# up read what q / gate already waited for; o reads the attention output, down reads gate and up.
STACK_WAITS = "1001101"
SHAPES = MLP_SHAPES
WORKLOAD_NAME = {
    "mlp": "GGUF Q4_K MLP projections of a 27B model (K=5120/N=17408, K=17408/N=5120), M=8",
    "stack": "GGUF Q4_K q/k/v/o/gate/up/down projections of a 27B layer (the verify stack is 64 such layers), M=8",
}
Q4_K = 12
ROWS = 8
METRIC = "quantized-matmul weight GB/s (% of HBM peak) at M=1/8 draft rows; µs/layer"


# dram__bytes read + written per launch of the product kernel, from the ncu capture summarised
# under profiles/ (mean of gate, up, down: 50.28, 50.28, 50.49 MB)
NCU_DRAM_BYTES_PER_LAUNCH = 50.35e6


def weight_bytes(n: int, k: int) -> int:
    return n * (k // 256) * 144


def algorithmic_bytes(n: int, k: int, m: int) -> int:
    return weight_bytes(n, k) + m * k * 2 + m * n * 2


def measured_peak() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.02)

    def stop(self) -> dict:
        self._halt.set()
        if self.is_alive():
            self.join(timeout=1.0)
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def physical_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


# --------------------------------------------------------------------------------------------------
# reference arm: the CPU restatement of the reference's algorithm, all host threads


def cpu_sample(seed: int = 0):
    from ishizuki_b200 import synth

    rng = np.random.default_rng(seed)
    layer = []
    for _, n, k in SHAPES:
        layer.append((n, k, synth.q4k_blocks(rng, n, k), synth.activations(rng, ROWS, k)))
    return layer


def cpu_pass(layer) -> float:
    from oracle import oracle

    t0 = time.perf_counter()
    for n, k, blocks, x in layer:
        oracle.ggml_matmul(Q4_K, blocks, x, n)
    return time.perf_counter() - t0


def run_reference(args) -> dict:
    from oracle import oracle

    layer = cpu_sample()
    bytes_per_pass = sum(weight_bytes(n, k) for n, k, _, _ in layer)
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_pass(layer)
    steps = max(1, args.steps)
    t = sum(cpu_pass(layer) for _ in range(steps))
    value = bytes_per_pass * steps / t / 1e9
    cores = oracle.threads()
    sample = "one block of the workload at M=8 per step, dequantize-on-the-fly + fp32-exact products"
    return {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": t / steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "u8/f16 in, f32 accumulate", "data": "synthetic", "impl": "reference",
        "config": {"workload": WORKLOAD_NAME[args.workload], "layers": 1, "rows": ROWS},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# --------------------------------------------------------------------------------------------------
# every format on the gate shape (a side table beside the headline, one GPU only)


def format_table(peak: float) -> dict:
    """us per projection and weight GB/s of each weight format on the gate / up shape
    (N = 17408, K = 5120) at M = 1 and M = 8: four projections with their own weights per format,
    replayed as one CUDA graph, timed with CUDA events."""
    import torch

    from ishizuki_b200 import synth
    from ishizuki_b200.interface import GGMLType, GGUFBlocks, PackedLinear

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()

    n, k, copies = 17408, 5120, 4
    rng = np.random.default_rng(99)

    def make(fmt):
        if fmt == "q4_k":
            return PackedLinear(ggml=GGUFBlocks(dev(synth.q4k_blocks(rng, n, k)), GGMLType.q4K, (n, k)))
        if fmt == "q6_k":
            return PackedLinear(ggml=GGUFBlocks(dev(synth.q6k_blocks(rng, n, k)), GGMLType.q6K, (n, k)))
        if fmt == "iq2_xs":
            return PackedLinear(ggml=GGUFBlocks(dev(synth.iq2xs_blocks(rng, n, k)), GGMLType.iq2Xs, (n, k)))
        if fmt == "affine4_g64":
            w, s, b = synth.affine_pack(rng, n, k, 4, 64, np.float16)
            return PackedLinear(dev(w), dev(s), dev(b), None, 0, groupSize=64, bits=4)
        w, sb, bb = synth.ternary_pack(rng, n, k, 128)  # "ternary2_g128_h128": rotation inside the kernel
        return PackedLinear(dev(w), dev(sb).view(torch.bfloat16), dev(bb).view(torch.bfloat16), None, 128,
                            groupSize=128, bits=2)

    table = {}
    stream = torch.cuda.Stream()
    for fmt in ("q4_k", "affine4_g64", "ternary2_g128_h128", "iq2_xs", "q6_k"):
        lins = [make(fmt) for _ in range(copies)]
        row = {"weight_mb": lins[0].weightBytes / 1e6}
        for m in (1, 8):
            x = dev(synth.activations(rng, m, k))
            outs = [torch.empty((m, n), dtype=torch.float16, device="cuda") for _ in lins]
            with torch.cuda.stream(stream):
                for lin, o in zip(lins, outs):
                    lin(x, out=o)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    for lin, o in zip(lins, outs):
                        lin(x, out=o)
                for _ in range(3):
                    g.replay()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                reps = 20
                e0.record(stream)
                for _ in range(reps):
                    g.replay()
                e1.record(stream)
                torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
            gbs = lins[0].weightBytes / us / 1e3
            row["m%d" % m] = {"us": round(us, 2), "gbs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 3)}
        table[fmt] = row
        del lins
        torch.cuda.empty_cache()
    return table


# --------------------------------------------------------------------------------------------------
# our arm


def run_ours(args) -> dict | None:
    import torch
    import torch.distributed as dist

    from ishizuki_b200 import synth
    from ishizuki_b200.interface import Context, GGMLType, GGUFBlocks, PackedLinear

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = Context.get(local)

    layers = args.layers
    rng = np.random.default_rng(1234)
    use_nccl = os.environ.get("ISHI_BENCH_NCCL") == "1"  # N > 1: all-gather per projection instead of the exchange
    exchange = None
    exchange_note = None
    if world > 1 and not use_nccl:
        from ishizuki_b200.sharding import OutputExchange

        # all ranks take the same path: if one cannot map its peers, every rank falls back to NCCL
        try:
            exchange = OutputExchange(sum(((n * 16 + 255) & ~255) for _, n, _ in SHAPES) * layers + 4096)
            ok = 1
        except Exception as exc:  # noqa: BLE001
            exchange_note = "output exchange unavailable (%s): NCCL all-gather instead" % str(exc)[:120]
            ok = 0
        flag = torch.tensor([ok], dtype=torch.int32, device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            if exchange is not None:
                exchange.close()
            exchange = None
            exchange_note = exchange_note or "output exchange unavailable on another rank: NCCL all-gather instead"
    projections = []  # (lin, x, y_local, y_full, n_full, k)
    total_weight = 0
    total_alg = 0
    for layer in range(layers):
        for _, n, k in SHAPES:
            n_lo, n_hi = rank * n // world, (rank + 1) * n // world
            blocks_full_rows = n_hi - n_lo
            blocks = synth.q4k_blocks(rng, blocks_full_rows, k)
            dev = torch.from_numpy(blocks).cuda()
            lin = PackedLinear(ggml=GGUFBlocks(dev, GGMLType.q4K, (blocks_full_rows, k)))
            del dev  # the projection keeps its own tiled copy
            x = torch.from_numpy(synth.activations(rng, ROWS, k)).cuda()
            if exchange is not None:
                y_local, y_full = exchange.reserve(n)  # (byte offset, [n, 8] view of this rank's copy)
            elif world > 1:
                y_local = torch.empty((blocks_full_rows, ROWS), dtype=torch.float16, device="cuda")
                y_full = torch.empty((n, ROWS), dtype=torch.float16, device="cuda")
            else:
                y_local = torch.empty((ROWS, n), dtype=torch.float16, device="cuda")
                y_full = y_local
            projections.append((lin, x, y_local, y_full, n, k, n_lo))
            total_weight += weight_bytes(n, k)
            total_alg += algorithmic_bytes(n, k, ROWS)
    torch.cuda.empty_cache()

    # Which projections wait for the other ranks' previous exchange, in the order gate, up, down:
    # gate reads the previous block's down output and down reads gate and up, so both wait; up reads
    # what gate already waited for. ISHI_BENCH_WAITS=111 makes every projection wait, 000 none.
    WAITS = [c == "1" for c in os.environ.get("ISHI_BENCH_WAITS", STACK_WAITS if args.workload == "stack" else "101")]
    waits_seen = []

    def one_pass():
        for lin, x, y_local, y_full, _, _, n_lo in projections:
            if exchange is not None:
                # every kernel stores its rows into all ranks' copies and waits for the other
                # ranks' previous projection first, as a layer stack's data flow would make it
                exchange.apply(lin, x, y_local, n_lo, wait_previous=WAITS[len(waits_seen) % len(WAITS)])
                waits_seen.append(0)
            elif world > 1:
                lin(x, transposed=True, out=y_local)
                dist.all_gather_into_tensor(y_full, y_local)
            else:
                lin(x, out=y_local)
        if exchange is not None:
            exchange.wait()

    stream = torch.cuda.Stream()
    graph = None
    with torch.cuda.stream(stream):
        one_pass()
        torch.cuda.synchronize()
        # One CUDA graph per step. With NCCL all-gathers in the step the launches stay eager:
        # capturing them in the graph did not finish when tried at two ranks (with and without
        # early launch of the product kernels), cause not established.
        if world == 1 or exchange is not None:
            if world > 1:
                dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                one_pass()

        def step():
            if graph is not None:
                graph.replay()
            else:
                one_pass()

        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        sampler = ClockSampler(physical_index(local))
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            dist.barrier()
        ctx.poll()

        # end to end through the host-buffer entry point: every projection's x comes from page-locked
        # host memory and its y goes back to page-locked host memory inside the timed region; one
        # stream synchronisation per step, after which the step's last output is read on the host
        e2e = None
        if world == 1:
            host = [(lin, x.cpu().pin_memory(), torch.empty((ROWS, n), dtype=torch.float16).pin_memory())
                    for lin, x, _, _, n, _, _ in projections]
            for lin, xh, yh in host:
                lin.apply_host_async(xh, yh)
            torch.cuda.synchronize()
            e2e_steps = max(1, min(args.steps, 10))
            checksum = 0.0
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                for lin, xh, yh in host:
                    lin.apply_host_async(xh, yh)
                torch.cuda.current_stream().synchronize()
                checksum += float(host[-1][2][0, 0])
            dt = time.perf_counter() - t0
            ctx.poll()
            e2e = {
                "value": total_weight * e2e_steps / dt / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": int(sum(xh.numel() * 2 for _, xh, _ in host)),
                "d2h_bytes_per_step": int(sum(yh.numel() * 2 for _, _, yh in host)),
                "api": "ishi_projection_apply_host_async per projection, one stream synchronisation per step",
                "checksum": checksum,
            }

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return None

    launches_per_step = len(projections)
    ms_per_step = ms / args.steps
    value = total_weight / (ms_per_step * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    avg_launch_s = ms_per_step * 1e-3 / launches_per_step
    achieved = (total_alg / world / launches_per_step) / avg_launch_s / 1e9  # this rank's bytes per launch
    out = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "u8/f16 in, f32 accumulate", "data": "synthetic",
        "config": {
            "workload": WORKLOAD_NAME[args.workload],
            "layers": layers, "rows": ROWS, "l2": "every projection has its own weights: %.2f GB per step" %
            (total_weight / 1e9),
            "parallelism": ("N-sharded x%d, outputs exchanged by the product kernels over NVLink" % world if exchange is not None
                            else "N-sharded x%d + NCCL all-gather" % world) if world > 1 else "single GPU",
            "launch": "CUDA graph" if graph is not None else "eager",
        },
        **({"note": exchange_note} if exchange_note else {}),
        "us_per_layer": ms_per_step * 1e3 / layers,
        **({"us_per_64_layer_stack": ms_per_step * 1e3 / layers * 64} if args.workload == "stack" else {}),
        "pct_of_hbm_peak": {"measured_%d" % int(peak): 100.0 * value / world / peak, "nominal_8000": 100.0 * value / world / 8000.0},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH if world == 1 and args.workload == "mlp" else None,
                     "kernel": "frag_kernel<FragQ4K, 0>", "peak_kind": peak_kind},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    if e2e is not None:
        out["e2e"] = e2e
    if world == 1 and args.workload == "mlp" and os.environ.get("ISHI_BENCH_NO_FORMATS") != "1":
        out["formats"] = format_table(peak)
    if world == 1:
        layer = cpu_sample()
        cpu_pass(layer)
        reps, t = 0, 0.0
        while t < 8.0 and reps < 20:
            t += cpu_pass(layer)
            reps += 1
        from oracle import oracle

        out["cpu_baseline"] = {
            "value": sum(weight_bytes(n, k) for n, k, _, _ in layer) * reps / t / 1e9, "unit": "GB/s",
            "cores": oracle.threads(), "kind": "port",
            "sample": "%d passes over one MLP block (gate, up, down) at M=8" % reps,
        }
    if world > 1:
        dist.destroy_process_group()
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--workload", default="mlp", choices=["mlp", "stack"],
                    help="mlp: gate/up/down (the headline); stack: all seven projections of a layer")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.workload == "stack":
        global SHAPES
        SHAPES = STACK_SHAPES
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        print(json.dumps(run_reference(args)), flush=True)
        return
    out = run_ours(args)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
