#!/usr/bin/env python3
"""Benchmark of the speculative-verify quantized matmul.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload stack|mlp|formats] [--layers L] [--impl ours|reference]

Workload (default, at every N): the verify stack of a 27B model in GGUF Q4_K, 64 layers of
q / k / v / o / gate / up / down projections (q 6144x5120, k and v 1024x5120, o 5120x6144, gate and
up 17408x5120, down 5120x17408) against M = 8 drafted rows of fp16 activations, fp32 accumulate,
fp16 outputs. Projections that read the same input are stacked into one launch (q+k+v, gate+up), so
a layer is four launches; every projection has its own weights (12.27 GB per pass, far more than
L2) and its own fresh N(0,1) activations. `--workload mlp` runs gate/up/down only (the 1-GPU MLP
configuration), `--workload formats` only the per-format side table (every weight format on the
gate shape at M = 1 and M = 8, the 4096 x 4096 affine projection, a ternary layer, an MLP block with
its stages, EXL3; ISHI_BENCH_FORMATS and ISHI_BENCH_ROWS narrow it for profiler captures). Inputs are synthetic with the configured value distributions, drawn on the GPU
from seeded generators: real GGUF files are not available where this runs.

The metric is weight GB/s: compressed weight bytes streamed per second (GB = 1e9), the
reference's own convention (block bytes only). With N > 1 every matrix is sharded along its
output rows across the ranks (strong scaling: the same pass at every N); by default the product
kernels store their rows into every rank's copy of the output over NVLink (no collective), with
ISHI_BENCH_NCCL=1 one NCCL all-gather per launch assembles them instead (ISHI_BENCH_NO_PEER_WAIT=1,
a diagnostic: the launches do not wait for the other ranks' previous launch). After the timed region
every rank checks exchanged outputs against the ranks' shards recomputed locally.

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

# (launch name, K, [(matrix, N), ...]): matrices that read the same input are one stacked projection
STACK_GROUPS = [
    ("qkv", 5120, [("q", 6144), ("k", 1024), ("v", 1024)]),
    ("o", 6144, [("o", 5120)]),
    ("gate_up", 5120, [("gate", 17408), ("up", 17408)]),
    ("down", 17408, [("down", 5120)]),
]
MLP_GROUPS = [STACK_GROUPS[2], STACK_GROUPS[3]]
WORKLOAD_NAME = {
    "stack": "GGUF Q4_K verify stack of a 27B model: q/k/v/o/gate/up/down per layer, M=8",
    "mlp": "GGUF Q4_K MLP projections of a 27B model (K=5120/N=17408, K=17408/N=5120), M=8",
}
Q4_K = 12
ROWS = 8
SEED = 1234
METRIC = "quantized-matmul weight GB/s (% of HBM peak) at M=1/8 draft rows; µs/layer"


def log(msg: str) -> None:
    """Progress lines on stderr (ISHI_BENCH_VERBOSE=1); stdout carries the one JSON line only."""
    if os.environ.get("ISHI_BENCH_VERBOSE") == "1":
        print("[bench rank %s] %s" % (os.environ.get("RANK", "0"), msg), file=sys.stderr, flush=True)


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


def profiled_traffic() -> dict | None:
    """DRAM bytes per launch of the dominant kernel from the tracked ncu summary (with the commit
    and command it was captured at), or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "frag_kernel_q4k_traffic.json")) as f:
            return json.load(f)
    except Exception:
        return None


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
# reference arm: the CPU restatement of the reference's algorithm, all host cores


def cpu_sample(seed: int = 0):
    """One MLP block of the workload (gate, up, down) with its activations."""
    from ishizuki_b200 import synth

    rng = np.random.default_rng(seed)
    layer = []
    for n, k in ((17408, 5120), (17408, 5120), (5120, 17408)):
        layer.append((n, k, synth.q4k_blocks(rng, n, k), synth.activations(rng, ROWS, k)))
    return layer


def cpu_pass(layer) -> float:
    from oracle import oracle

    t0 = time.perf_counter()
    for n, k, blocks, x in layer:
        oracle.ggml_matmul(Q4_K, blocks, x, n)
    return time.perf_counter() - t0


def gguf_py_pass(layer) -> float | None:
    """The same products through ggml's own Python reference: gguf.quants.dequantize, then a numpy
    fp32 matmul (the 'ggml reference' stand-in; libggml itself is not installed here)."""
    try:
        import gguf
    except Exception:
        return None
    n, k, blocks, x = layer[0]
    rows = 2048  # a bounded slice of the gate projection: the decoder is pure numpy
    part = blocks.reshape(n, -1)[:rows].reshape(-1, 144)
    xf = x.astype(np.float32)
    t0 = time.perf_counter()
    w = gguf.quants.dequantize(part, gguf.GGMLQuantizationType(Q4_K)).reshape(rows, k)
    _ = xf @ w.T
    dt = time.perf_counter() - t0
    return weight_bytes(rows, k) / dt / 1e9


def cpu_baseline(max_seconds: float, max_reps: int) -> dict:
    from oracle import oracle

    cores = oracle.use_all_cores()  # a launcher's OMP_NUM_THREADS=1 must not make this single-threaded
    layer = cpu_sample()
    cpu_pass(layer)
    reps, t = 0, 0.0
    while t < max_seconds and reps < max_reps:
        t += cpu_pass(layer)
        reps += 1
    out = {
        "value": sum(weight_bytes(n, k) for n, k, _, _ in layer) * reps / t / 1e9, "unit": "GB/s", "cores": cores,
        "kind": "port", "sample": "%d passes over one MLP block (gate, up, down) at M=8, dequantize-on-the-fly" % reps,
    }
    g = gguf_py_pass(layer)
    if g is not None:
        out["gguf_py"] = {"value": g, "unit": "GB/s", "sample": "gguf.quants.dequantize + numpy fp32 matmul on 2048 rows of gate"}
    return out


def run_reference(args) -> dict:
    from oracle import oracle

    cores = oracle.use_all_cores()
    layer = cpu_sample()
    bytes_per_pass = sum(weight_bytes(n, k) for n, k, _, _ in layer)
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_pass(layer)
    steps = max(1, min(args.steps, 20))
    t = sum(cpu_pass(layer) for _ in range(steps))
    value = bytes_per_pass * steps / t / 1e9
    sample = "one MLP block (gate, up, down) of the workload at M=8 per step, dequantize-on-the-fly + fp32-exact products"
    return {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": t / steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "u8/f16 in, f32 accumulate", "data": "synthetic", "impl": "reference",
        "config": {"workload": WORKLOAD_NAME[args.workload], "layers": args.layers, "rows": ROWS},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# --------------------------------------------------------------------------------------------------
# synthetic weights, drawn on the GPU


def q4k_blocks_device(seed: int, n: int, k: int):
    """[n][k/256][144] bytes with the benchmark's distributions: d, dmin = fp16 |N(0,1)| * 2e-3,
    uniform scale bytes (each 6-bit field uniform in 0..63), uniform 4-bit codes. The same seed
    gives the same bytes on every rank."""
    import torch

    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    nb = n * (k // 256)
    blocks = torch.randint(0, 256, (nb, 144), dtype=torch.uint8, device="cuda", generator=gen)
    d = (torch.randn((nb, 2), device="cuda", generator=gen).abs() * 2e-3).to(torch.float16)
    blocks[:, 0:4] = d.view(torch.uint8).view(nb, 4)
    return blocks.view(-1)


def activations_device(seed: int, m: int, k: int):
    import torch

    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    return torch.randn((m, k), device="cuda", generator=gen).to(torch.float16)


def matrix_seed(layer: int, group: int, part: int) -> int:
    return SEED + 1000 * layer + 10 * group + part


def shard_parts(layer: int, gi: int, group, rank: int, world: int):
    """The stacked projection of `rank` for launch `gi` of `layer`: that rank's rows of every matrix."""
    from ishizuki_b200.interface import GGMLType, GGUFBlocks

    _, k, mats = group
    row_bytes = (k // 256) * 144
    parts = []
    for pi, (_, n) in enumerate(mats):
        full = q4k_blocks_device(matrix_seed(layer, gi, pi), n, k)
        lo, hi = rank * n // world, (rank + 1) * n // world
        parts.append(GGUFBlocks(full[lo * row_bytes: hi * row_bytes].clone(), GGMLType.q4K, (hi - lo, k)))
        del full
    return parts


def make_projection(parts, fused: bool):
    from ishizuki_b200.interface import FusedLinear, PackedLinear

    if fused and len(parts) > 1:
        return [FusedLinear(parts)]
    return [PackedLinear(ggml=p) for p in parts]


# --------------------------------------------------------------------------------------------------
# every format on the gate shape (a side table beside the headline, one GPU only)


def timed_graph(run, reps: int = 20) -> float:
    """Microseconds per replay of `run` captured as one CUDA graph."""
    import torch

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        run()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            run()
        for _ in range(3):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(reps):
            g.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def format_table(peak: float) -> dict:
    """us per projection and weight GB/s of each weight format on the gate / up shape
    (N = 17408, K = 5120) at M = 1 and M = 8, plus the other configurations of the benchmark: the
    4096 x 4096 affine projection, the seven ternary projections of a layer, and a single row on
    CUDA cores beside the tensor-core kernel. Distinct weights per launch, one CUDA graph, CUDA
    events."""
    import torch

    from ishizuki_b200 import _lib, synth
    from ishizuki_b200.interface import BonsaiRuntime, FusedLinear, GGMLType, GGUFBlocks, PackedLinear

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()

    rng = np.random.default_rng(99)

    def make(fmt, n, k):
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

    def measure(lins, m, k):
        x = dev(synth.activations(rng, m, k))
        outs = [torch.empty((m, lin.outputDim), dtype=torch.float16, device="cuda") for lin in lins]

        def run():
            for lin, o in zip(lins, outs):
                lin(x, out=o)

        us = timed_graph(run) / len(lins)
        gbs = sum(lin.weightBytes for lin in lins) / len(lins) / us / 1e3
        return {"us": round(us, 2), "gbs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 3)}

    table = {}
    n, k, copies = 17408, 5120, 4
    # ISHI_BENCH_FORMATS=name[,name]: only these rows of the first group (profiler captures of one format)
    only = [f for f in os.environ.get("ISHI_BENCH_FORMATS", "").split(",") if f]
    row_counts = [int(r) for r in os.environ.get("ISHI_BENCH_ROWS", "1,8").split(",")]  # activation rows M
    def other_rows():
        # four of the eight other GGML block types on their own fragment decoders, and one of them
        # through the dense decoder (ISHI_DENSE_DECODER at projection create), the path they ran on before
        for name, type_id in (("iq4_xs", GGMLType.iq4Xs), ("iq3_s", GGMLType.iq3S), ("q2_k", GGMLType.q2K), ("iq1_s", GGMLType.iq1S),
                              ("iq3_s_dense_decoder", GGMLType.iq3S)):
            if only and name not in only:
                continue
            if name.endswith("_dense_decoder"):
                os.environ["ISHI_DENSE_DECODER"] = "1"
            try:
                lins = [PackedLinear(ggml=GGUFBlocks(dev(synth.ggml_blocks(rng, int(type_id), n, k)), type_id, (n, k)))
                        for _ in range(2)]
            finally:
                os.environ.pop("ISHI_DENSE_DECODER", None)
            table[name] = {"weight_mb": lins[0].weightBytes / 1e6}
            for m in row_counts:
                table[name]["m%d" % m] = measure(lins, m, k)
            del lins
        torch.cuda.empty_cache()

    def exl3_rows():
        # EXL3 trellis-coded weights on the gate shape, 4 bits, the product kernel alone (no rotations)
        from ishizuki_b200.interface import EXL3Kernels, EXL3Tensor

        for name, codebook in (("exl3_4bit_3inst", EXL3Tensor.threeInst), ("exl3_4bit_mul1", EXL3Tensor.mul1)):
            if only and name not in only:
                continue
            tensors = [EXL3Tensor(torch.randint(-32768, 32768, (k // 16, n // 16, 64), dtype=torch.int16, device="cuda"), None,
                                  None, codebook) for _ in range(copies)]
            row = {"weight_mb": tensors[0].trellis.numel() * 2 / 1e6}
            for m in row_counts:
                x = dev(synth.activations(rng, m, k))

                def run():
                    for t in tensors:
                        EXL3Kernels.matvec(x, t)

                us = timed_graph(run) / copies
                gbs = row["weight_mb"] * 1e3 / us
                row["m%d" % m] = {"us": round(us, 2), "gbs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 3)}
            table[name] = row
            del tensors

    for fmt in ("q4_k", "affine4_g64", "ternary2_g128_h128", "iq2_xs", "q6_k"):
        if only and fmt not in only:
            continue
        lins = [make(fmt, n, k) for _ in range(copies)]
        row = {"weight_mb": lins[0].weightBytes / 1e6}
        for m in row_counts:
            row["m%d" % m] = measure(lins, m, k)
        if fmt in ("q4_k", "q6_k", "iq2_xs") and not only:
            # the same format on the tcgen05 kernel (ISHI_KERNEL=tcgen05 at projection create)
            os.environ["ISHI_KERNEL"] = "tcgen05"
            try:
                slow = [make(fmt, n, k) for _ in range(copies)]
            finally:
                del os.environ["ISHI_KERNEL"]
            row["m8_tcgen05_kernel"] = measure(slow, 8, k)
            del slow
        if fmt in ("q4_k", "affine4_g64") and not only:
            # the single-row CUDA-core variant beside the tensor-core kernel (ISHI_ROUTE_GEMV)
            BonsaiRuntime.route = _lib.ROUTE_GEMV
            try:
                row["m1_cuda_cores"] = measure(lins, 1, k)
            finally:
                BonsaiRuntime.route = _lib.ROUTE_AUTO
        table[fmt] = row
        del lins
        torch.cuda.empty_cache()
    if only:
        other_rows()
        exl3_rows()
        return table
    # one row on CUDA cores beside the tensor-core kernel on the smallest and the tallest projection
    for name, n_, k_ in (("q4_k_kv_1024x5120", 1024, 5120), ("q4_k_down_5120x17408", 5120, 17408)):
        lins = [make("q4_k", n_, k_) for _ in range(8 if n_ < 2048 else 4)]
        row = {"weight_mb": lins[0].weightBytes / 1e6, "m1": measure(lins, 1, k_)}
        BonsaiRuntime.route = _lib.ROUTE_GEMV
        try:
            row["m1_cuda_cores"] = measure(lins, 1, k_)
        finally:
            BonsaiRuntime.route = _lib.ROUTE_AUTO
        table[name] = row
        del lins
    other_rows()
    # configuration 1: a single 4096 x 4096 affine 4-bit group-64 projection (32 distinct weights)
    lins = [make("affine4_g64", 4096, 4096) for _ in range(32)]
    table["affine4_g64_4096x4096"] = {"weight_mb": lins[0].weightBytes / 1e6, "m1": measure(lins, 1, 4096),
                                      "m8": measure(lins, 8, 4096)}
    del lins
    # configuration 4: the seven ternary projections of a layer, per layer; as in the headline
    # stack, projections that read the same input are one stacked launch (q+k+v, gate+up)
    def ternary_group(k_, sizes):
        packs = [synth.ternary_pack(rng, n_, k_, 128) for n_ in sizes]
        parts = [(dev(w), dev(sb).view(torch.bfloat16), dev(bb).view(torch.bfloat16)) for w, sb, bb in packs]
        if len(parts) == 1:
            return PackedLinear(parts[0][0], parts[0][1], parts[0][2], None, 128, groupSize=128, bits=2)
        return FusedLinear(parts, None, 128, groupSize=128, bits=2)

    groups4 = [(5120, (6144, 1024, 1024)), (6144, (5120,)), (5120, (17408, 17408)), (17408, (5120,))]
    layers = [[ternary_group(k_, sizes) for k_, sizes in groups4] for _ in range(3)]
    row = {"weight_mb": sum(lin.weightBytes for lin in layers[0]) / 1e6, "launches_per_layer": len(groups4)}
    for m in (1, 8):
        xs = {k_: dev(synth.activations(rng, m, k_)) for k_ in (5120, 6144, 17408)}
        outs = [[torch.empty((m, lin.outputDim), dtype=torch.float16, device="cuda") for lin in layer] for layer in layers]

        def run():
            for layer, os_ in zip(layers, outs):
                for lin, o in zip(layer, os_):
                    lin(xs[lin.inputDim], out=o)

        us = timed_graph(run) / len(layers)
        gbs = row["weight_mb"] * 1e6 / us / 1e3
        row["m%d" % m] = {"us_per_layer": round(us, 2), "gbs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 3)}
    table["ternary2_g128_h128_layer"] = row
    del layers
    torch.cuda.empty_cache()
    # An MLP block (Q4_K, M = 8): down(silu(gate(x)) * up(x)). "gated": gate and up as one launch
    # whose epilogue writes silu(gate) * up, then down: two launches. "stacked_and_elementwise":
    # the stacked gate+up launch, silu(gate) * up as element-wise kernels of the host framework
    # (what the reference does through MLX), then down.
    blocks = 4
    mlps = []
    for _ in range(blocks):
        parts = [GGUFBlocks(dev(synth.q4k_blocks(rng, 17408, 5120)), GGMLType.q4K, (17408, 5120)) for _ in range(2)]
        mlps.append((FusedLinear(parts, gated=True), FusedLinear(parts), make("q4_k", 5120, 17408)))
        del parts
    x = dev(synth.activations(rng, 8, 5120))
    h = torch.empty((8, 17408), dtype=torch.float16, device="cuda")
    gu = torch.empty((8, 2 * 17408), dtype=torch.float16, device="cuda")
    ys = [torch.empty((8, 5120), dtype=torch.float16, device="cuda") for _ in range(blocks)]

    def run_gated():
        for (gated, _, down), y in zip(mlps, ys):
            gated(x, out=h)
            down(h, out=y)

    def run_stacked():
        for (_, stacked, down), y in zip(mlps, ys):
            stacked(x, out=gu)
            torch.mul(torch.nn.functional.silu(gu[:, :17408]), gu[:, 17408:], out=h)
            down(h, out=y)

    # the same with the RMS norm of the fp32 residual ahead of gate / up: this library's norm launch
    # and the gated pair, against the host framework's norm and element-wise kernels
    from ishizuki_b200.interface import rmsNorm

    res = dev(synth.activations(rng, 8, 5120).astype(np.float32))
    nw = dev(np.ones(5120, dtype=np.float16))

    def run_normed_gated():
        for (gated, _, down), y in zip(mlps, ys):
            gated(rmsNorm(res, nw, 1e-6), out=h)
            down(h, out=y)

    def run_normed_stacked():
        for (_, stacked, down), y in zip(mlps, ys):
            xn = torch.nn.functional.rms_norm(res, (5120,), nw.float(), 1e-6).half()
            stacked(xn, out=gu)
            torch.mul(torch.nn.functional.silu(gu[:, :17408]), gu[:, 17408:], out=h)
            down(h, out=y)

    mb = sum(lin.weightBytes for lin in mlps[0][1:]) / 1e6
    row = {"weight_mb": mb}
    for name, run in (("gated", run_gated), ("stacked_and_elementwise", run_stacked), ("norm_gated", run_normed_gated),
                      ("norm_stacked_and_elementwise", run_normed_stacked)):
        us = timed_graph(run) / blocks
        row[name] = {"us_per_block": round(us, 2), "gbs": round(mb * 1e3 / us, 1), "frac_of_peak": round(mb * 1e3 / us / peak, 3)}
    table["q4_k_mlp_block_m8"] = row
    del mlps
    torch.cuda.empty_cache()
    exl3_rows()
    torch.cuda.empty_cache()
    # the LM head of the verify step (248320 x 5120, Q4_K) with the arg-max of every drafted row:
    # ishi_projection_apply_argmax = the product into the projection's own logits buffer and the
    # arg-max kernel; two heads alternate so that the weights come from HBM
    heads = [PackedLinear(ggml=GGUFBlocks(q4k_blocks_device(4242 + i, 248320, 5120), GGMLType.q4K, (248320, 5120)))
             for i in range(2)]
    row = {"weight_mb": heads[0].weightBytes / 1e6}
    for m in (1, 8):
        x = dev(synth.activations(rng, m, 5120))
        heads[0].argmax(x)  # the first call allocates the logits buffer, outside the capture
        heads[1].argmax(x)

        def run():
            for head in heads:
                head.argmax(x)

        us = timed_graph(run, reps=10) / len(heads)
        gbs = row["weight_mb"] * 1e3 / us
        row["m%d" % m] = {"us": round(us, 2), "gbs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 3)}
    table["lm_head_q4_k_248320x5120_argmax"] = row
    del heads
    torch.cuda.empty_cache()
    return table


# --------------------------------------------------------------------------------------------------
# our arm


def run_ours(args) -> dict | None:
    import torch
    import torch.distributed as dist

    from ishizuki_b200.interface import Context, HostBatch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = Context.get(local)

    groups = STACK_GROUPS if args.workload == "stack" else MLP_GROUPS
    layers = args.layers
    fused = not args.unfused
    use_nccl = os.environ.get("ISHI_BENCH_NCCL") == "1"  # N > 1: all-gather per launch instead of the exchange
    exchange = None
    exchange_note = None
    nccl_group = None
    out_rows_per_layer = sum(sum(n for _, n in mats) for _, _, mats in groups)
    if world > 1 and not use_nccl:
        from ishizuki_b200.sharding import OutputExchange

        # all ranks take the same path: if one cannot map its peers, every rank falls back to NCCL
        try:
            exchange = OutputExchange((out_rows_per_layer * 16 + 256 * 8) * layers + 4096)
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

    if world > 1 and exchange is None:
        from ishizuki_b200.sharding import NcclGroup

        nccl_group = NcclGroup()  # ishi_group_*: the library's own communicator, NCCL's non-blocking mode

    # (projection, x, y_local or exchange offset, y_full view, rows of all ranks, k, row offset, (layer, group, first part, parts))
    launches = []
    total_weight = 0
    total_alg = 0
    for layer in range(layers):
        for gi, group in enumerate(groups):
            name, k, mats = group
            parts = shard_parts(layer, gi, group, rank, world)
            lins = make_projection(parts, fused)
            del parts
            x = activations_device(SEED + 7 + 1000 * layer + 10 * gi, ROWS, k)
            first = 0
            for lin in lins:
                n_local = lin.outputDim
                n_all = n_local * world if all(n % world == 0 for _, n in mats) else None
                if n_all is None:
                    raise SystemExit("the benchmark's shapes divide evenly over 1, 2, 4 and 8 ranks only")
                if exchange is not None:
                    y_local, y_full = exchange.reserve(n_all)  # (byte offset, [n_all, 8] view of this rank's copy)
                elif world > 1:
                    y_full = torch.empty((n_all, ROWS), dtype=torch.float16, device="cuda")
                    y_local = y_full[rank * n_local: (rank + 1) * n_local]  # the product writes its slab in place
                else:
                    y_local = torch.empty((ROWS, n_local), dtype=torch.float16, device="cuda")
                    y_full = y_local
                nparts = len(mats) if (fused and len(mats) > 1) else 1
                launches.append((lin, x, y_local, y_full, n_all, k, rank * n_local, (layer, gi, first, nparts)))
                first += nparts
                total_weight += weight_bytes(n_all, k)
                total_alg += algorithmic_bytes(n_all, k, ROWS)
    torch.cuda.empty_cache()
    log("%d launches per step, %.2f GB of weights" % (len(launches), total_weight / 1e9))

    def one_pass():
        for lin, x, y_local, y_full, _, _, row0, _ in launches:
            if exchange is not None:
                # every kernel stores its rows into all ranks' copies; it first waits for the other
                # ranks' previous launch, whose outputs a layer stack's data flow makes it depend on
                exchange.apply(lin, x, y_local, row0, wait_previous=os.environ.get("ISHI_BENCH_NO_PEER_WAIT") != "1")
            elif world > 1:
                nccl_group.apply(lin, x, y_full)  # ishi_projection_apply_sharded: product + ncclAllGather
            else:
                lin(x, out=y_local)
        if exchange is not None:
            exchange.wait()

    stream = torch.cuda.Stream()
    graph = None
    with torch.cuda.stream(stream):
        one_pass()
        torch.cuda.synchronize()
        # One CUDA graph per step. With NCCL all-gathers in the step the launches stay eager.
        if world == 1 or exchange is not None:
            if world > 1:
                dist.barrier()
                torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                one_pass()

        def step():
            if graph is not None:
                graph.replay()
            else:
                one_pass()

        log("first pass done, graph %s" % ("captured" if graph is not None else "not used"))
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
        log("timed region done: %.3f ms per step" % (ms / args.steps))

        # N > 1, outside the timed region: are the assembled outputs what the ranks computed? Every
        # rank rebuilds every rank's shard of a sample of launches from the seeds, multiplies it
        # locally and compares with the rows the timed pass left in its copy of the output.
        check = None
        if world > 1:
            sample = sorted({0, 1, 2, 3, len(launches) // 2, len(launches) - 2, len(launches) - 1} & set(range(len(launches))))
            worst, bitwise = 0.0, True
            sums = []
            for li in sample:
                lin, x, _, y_full, n_all, k, _, (layer, gi, first, nparts) = launches[li]
                group = groups[gi]
                n_local = n_all // world
                want = torch.empty((n_all, ROWS), dtype=torch.float16, device="cuda")
                # the launch plan fixes the order of the partial sums: recompute under the owner's
                plans = [None] * world
                dist.all_gather_object(plans, lin.plan)
                for q in range(world):
                    parts = shard_parts(layer, gi, group, q, world)[first: first + nparts]
                    ref = make_projection(parts, fused)[0]
                    ref.set_plan(plans[q])
                    want[q * n_local: (q + 1) * n_local] = ref(x, transposed=True)
                    del ref, parts
                torch.cuda.synchronize()
                got = y_full[:, :ROWS] if y_full.shape[1] == ROWS else y_full
                diff = float((got.float() - want.float()).abs().max() / want.float().abs().max())
                worst = max(worst, diff)
                bitwise = bitwise and bool(torch.equal(got, want))
                sums.append(int(got.contiguous().view(torch.int16).to(torch.int64).sum().item()))
            mine = torch.tensor(sums, dtype=torch.int64, device="cuda")
            everyone = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(everyone, mine)
            same = all(bool(torch.equal(e, mine)) for e in everyone)
            flags = torch.tensor([worst, 0.0 if (bitwise and same) else 1.0], dtype=torch.float64, device="cuda")
            dist.all_reduce(flags, op=dist.ReduceOp.MAX)
            both = torch.tensor([0.0 if bitwise else 1.0, 0.0 if same else 1.0], dtype=torch.float64, device="cuda")
            dist.all_reduce(both, op=dist.ReduceOp.MAX)
            check = {"launches_checked": len(sample), "max_rel_err": float(flags[0].item()),
                     "bitwise_equal_to_local_recompute": bool(both[0].item() == 0.0),
                     "bitwise_equal_across_ranks": bool(both[1].item() == 0.0),
                     "ok": bool(flags[0].item() < 2e-3)}
            ctx.poll()

        log("exchange check: %s" % (check,))
        # End to end through the host-buffer entry point: every launch's x comes from page-locked
        # host memory and its y (this rank's rows) goes back to page-locked host memory inside the
        # timed region, one C call and one stream synchronisation per step, after which a value of
        # the step's last output is read on the host.
        host_x = [x.cpu().pin_memory() for _, x, _, _, _, _, _, _ in launches]
        host_y = [torch.empty((ROWS, lin.outputDim), dtype=torch.float16).pin_memory() for lin, *_ in launches]
        batch = HostBatch([lin for lin, *_ in launches], host_x, host_y)
        batch.run()
        torch.cuda.synchronize()
        e2e_steps = max(1, min(args.steps, 10))
        checksum = 0.0
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            batch.run()
            torch.cuda.current_stream().synchronize()
            checksum += float(host_y[-1][0, 0])
        dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        ctx.poll()
        e2e = {
            "value": total_weight * e2e_steps / dt / 1e9, "unit": "GB/s",
            "h2d_bytes_per_step": int(sum(xh.numel() * 2 for xh in host_x)) * world,
            "d2h_bytes_per_step": int(sum(yh.numel() * 2 for yh in host_y)) * world,
            "api": "ishi_projection_apply_host_batch: one call and one stream synchronisation per step"
                   + ("; every rank returns its own rows to its host" if world > 1 else ""),
            "checksum": checksum,
        }

    log("end to end done")
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        if check is not None and not check["ok"]:
            sys.exit(3)
        return None

    launches_per_step = len(launches)
    ms_per_step = ms / args.steps
    value = total_weight / (ms_per_step * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    avg_launch_s = ms_per_step * 1e-3 / launches_per_step
    achieved = (total_alg / world / launches_per_step) / avg_launch_s / 1e9  # this rank's bytes per launch
    traffic = profiled_traffic()
    out = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "u8/f16 in, f32 accumulate", "data": "synthetic",
        "config": {
            "workload": WORKLOAD_NAME[args.workload],
            "layers": layers, "rows": ROWS,
            "launches_per_layer": len(launches) // layers,
            "stacked": "q+k+v and gate+up are one launch each" if fused else "one launch per matrix",
            "l2": "every projection has its own weights: %.2f GB per step" % (total_weight / 1e9),
            "parallelism": ("N-sharded x%d, outputs exchanged by the product kernels over NVLink" % world if exchange is not None
                            else "N-sharded x%d + one NCCL all-gather per launch (ishi_projection_apply_sharded)" % world)
            if world > 1 else "single GPU",
            "launch": "CUDA graph" if graph is not None else "eager",
        },
        **({"note": exchange_note} if exchange_note else {}),
        "us_per_layer": ms_per_step * 1e3 / layers,
        **({"us_per_64_layer_stack": ms_per_step * 1e3 / layers * 64} if args.workload == "stack" else {}),
        "pct_of_hbm_peak": {"measured_%d" % int(peak): 100.0 * value / world / peak, "nominal_8000": 100.0 * value / world / 8000.0},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic["dram_bytes_per_launch"] if traffic and world == 1 else None,
                     **({"traffic_from": traffic["captured"]} if traffic and world == 1 else {}),
                     "kernel": "frag_kernel<FragQ4K, 0>", "peak_kind": peak_kind,
                     "algorithmic_bytes_per_launch": total_alg / world / launches_per_step},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
        "e2e": e2e,
    }
    if check is not None:
        out["exchange_check"] = check
    if world == 1 and os.environ.get("ISHI_BENCH_NO_FORMATS") != "1":
        del launches, batch
        torch.cuda.empty_cache()
        out["formats"] = format_table(peak)
    if world == 1:
        out["cpu_baseline"] = cpu_baseline(8.0, 20)
    if world > 1:
        dist.destroy_process_group()
    if check is not None and not check["ok"]:
        print(json.dumps(out), flush=True)
        sys.exit(3)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0, help="default: 64 (stack), 8 (mlp)")
    ap.add_argument("--workload", default="stack", choices=["stack", "mlp", "formats"],
                    help="stack: all seven projections of every layer (the headline); mlp: gate/up/down only; "
                         "formats: only the per-format side table (one GPU)")
    ap.add_argument("--unfused", action="store_true", help="one launch per matrix instead of stacked q+k+v and gate+up")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.layers <= 0:
        args.layers = 64 if args.workload == "stack" else 8
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        print(json.dumps(run_reference(args)), flush=True)
        return
    if args.workload == "formats":
        peak, kind = measured_peak()
        print(json.dumps({"formats": format_table(peak), "peak": peak, "peak_kind": kind}), flush=True)
        return
    out = run_ours(args)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
