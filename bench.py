#!/usr/bin/env python
"""Benchmark of the RNS linear hot path on B200.

Workload (``config.workload``): configuration 4 of BASELINE.json, the
OPT-6.7B-shaped layer stack - 32 layers x {QKV 4096->12288, out_proj 4096->4096,
fc1 4096->16384, fc2 16384->4096}, every linear an RNS linear, M = 4096 tokens,
moduli (127,126,125,121) for K = 4096 and (127,126,125,121,113) for K = 16384,
random-init weights and seeded synthetic activations.  It is the largest
configuration that fits one GPU and the one the headline metric (RNS-GEMM int8
channel-TOPS at M >= 1024) is defined on.  One *step* is one pass of the 128
linears over one 4096-token batch: quantise activations -> fused RNS GEMM
(residue encode, one int8 tensor-core GEMM per channel, Garner, dequantise).

``python bench.py --gpus N --steps K --warmup W`` prints ONE JSON line on rank 0.
With N > 1 (launched by torchrun, one rank per GPU) every linear is column
sharded along its output features and the fp16 shards are all-gathered with
NCCL; the total work is fixed, so scaling is "strong".

``--impl reference`` times the CPU restatement of the reference's own path
(oracle/) on the host cores instead; that is the only place this file executes
anything from oracle/, besides the ``cpu_baseline`` block of the normal run.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

MODULI_4 = (127, 126, 125, 121)
MODULI_5 = (127, 126, 125, 121, 113)
HIDDEN, FFN = 4096, 16384
# (name, K, N, moduli, groups)   groups=3: q|k|v concatenated along N
LINEARS = (
    ("qkv", HIDDEN, 3 * HIDDEN, MODULI_4, 3),
    ("out_proj", HIDDEN, HIDDEN, MODULI_4, 1),
    ("fc1", HIDDEN, FFN, MODULI_4, 1),
    ("fc2", FFN, HIDDEN, MODULI_5, 1),
)
METRIC = "rns_gemm_int8_channel_tops"
UNIT = "TOPS"


def channel_ops_per_step(tokens: int, layers: int) -> float:
    """2 * R * M * K * N summed over the stack (benchmarks/benchmark_cuda.py:256-261
    of the reference defines rns_channel_tops this way)."""
    return float(sum(2.0 * len(mods) * tokens * k * n for _, k, n, mods, _ in LINEARS) * layers)


# Mean DRAM traffic of one rns_gemm_kernel launch of this workload on one GPU
# (dram__bytes_read.sum + dram__bytes_write.sum over the four linears of a layer:
# 286 + 99 + 362 + 1153 MB), from an ncu capture of `bench.py --layers 2`.
NCU_DRAM_BYTES_PER_LAUNCH = 476.3e6


def algorithmic_bytes_per_launch(tokens: int) -> float:
    """M*K (int8 activations) + K*N (1 B/value weights) + 4*(1+N) scales + 4*N
    bias + 2*M*N (fp16 out), mean over the four linears of a layer."""
    total = sum(tokens * k + k * n + 4 * (1 + n) + 4 * n + 2 * tokens * n for _, k, n, _, _ in LINEARS)
    return total / len(LINEARS)


def useful_ops_per_step(tokens: int, layers: int) -> float:
    return float(sum(2.0 * tokens * k * n for _, k, n, _, _ in LINEARS) * layers)


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        data["source"] = "measured"
        return data
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def measure_int8_peak(device, sustained_seconds: float = 3.0) -> dict:
    """Dense int8 tensor throughput of this GPU through the library GEMM (torch._int_mm,
    cuBLASLt int8 -> int32) at 8192^3: best of 10 single launches (burst) and the mean over
    back-to-back launches for `sustained_seconds` (sustained, under the power cap).  It is
    the denominator of roofline.frac: MEASURED_PEAKS.json records no int8 figure."""
    import torch

    n = 8192
    a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device)
    b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device).t()
    ops = 2.0 * n * n * n
    for _ in range(3):
        torch._int_mm(a, b)
    torch.cuda.synchronize(device)
    best = float("inf")
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); torch._int_mm(a, b); e1.record()
        e1.synchronize()
        best = min(best, e0.elapsed_time(e1))
    per_launch_s = best * 1e-3
    launches = max(20, int(sustained_seconds / per_launch_s))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        torch._int_mm(a, b)
    e1.record()
    e1.synchronize()
    sustained = ops * launches / (e0.elapsed_time(e1) * 1e-3) / 1e12
    del a, b
    return {"burst": ops / per_launch_s / 1e12, "sustained": sustained, "unit": "TOPS",
            "how": f"torch._int_mm {n}^3: best of 10 launches; mean of {launches} back-to-back launches"}


# --------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.file = None

    def start(self) -> None:
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", "100"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, sm_max, power, reasons = [], [], [], set()
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); sm_max.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                   parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        name = self.file.name
        self.file.close()
        os.unlink(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(sm_max), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------
# CPU arm (oracle port)
# --------------------------------------------------------------------------
def cpu_port_sample(target_seconds: float = 12.0) -> dict:
    """Times the C restatement of the reference path (oracle/rns_oracle.c, all
    host threads) on rows of the workload's QKV linear; the sample grows until
    it takes about ``target_seconds``."""
    import numpy as np
    from oracle import c_oracle

    c_oracle.build()
    threads = c_oracle.threads()
    name, k, n, mods, _ = LINEARS[0]
    rng = np.random.default_rng(1004)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int64).astype(np.int8)
    rows = max(threads, 8)
    elapsed = 0.0
    while True:
        a = rng.integers(-127, 128, size=(rows, k), dtype=np.int64).astype(np.int8)
        scale = np.ones(1, dtype=np.float32)
        col = np.ones(n, dtype=np.float32)
        t0 = time.perf_counter()
        c_oracle.linear(a, w, mods, scale, col, None, want_float=True)
        elapsed = time.perf_counter() - t0
        if elapsed >= target_seconds / 3 or rows >= 4096:
            break
        rows = min(4096, int(rows * max(2.0, target_seconds / max(elapsed, 1e-3) / 1.5)))
    ops = 2.0 * len(mods) * rows * k * n
    return {"value": ops / elapsed / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{rows} rows of the {name} linear (K={k}, N={n}, R={len(mods)}), "
                      f"C restatement of the reference path incl. weight encode, {elapsed:.1f} s",
            "seconds": elapsed}


def numpy_reference_sample() -> dict:
    """The reference's own NumPy algorithm (rns_matmul_numpy) restated in
    oracle/rns_oracle.py, on configuration 0 (M=128, K=N=768)."""
    import numpy as np
    from oracle import rns_oracle as O

    rng = np.random.default_rng(1000)
    a = rng.integers(-127, 128, size=(128, 768), dtype=np.int64).astype(np.int8)
    b = rng.integers(-127, 128, size=(768, 768), dtype=np.int64).astype(np.int8)
    best = min(_timed(lambda: O.rns_matmul(a, b, MODULI_4)) for _ in range(3))
    return {"seconds": best, "channel_tops": 2.0 * 4 * 128 * 768 * 768 / best / 1e12,
            "what": "NumPy restatement of rns_matmul_numpy on configuration 0, 1 effective core"}


def _timed(fn) -> float:
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    samples = []
    for _ in range(max(1, args.warmup // 3)):
        cpu_port_sample(target_seconds=3.0)
    for _ in range(args.steps):
        samples.append(cpu_port_sample(target_seconds=10.0))
    value = statistics.median(s["value"] for s in samples)
    seconds = statistics.median(s["seconds"] for s in samples)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3,
        "ms_per_step_is": "one bounded sample of the workload (rows of the QKV linear), not a full pass over "
                          "the 128 linears; a full pass at this rate would take "
                          f"{channel_ops_per_step(args.tokens, args.layers) / (value * 1e12):.0f} s",
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": workload_config(args, sharded=False),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": samples[0]["cores"], "kind": "port",
                         "sample": samples[0]["sample"]},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, sharded: bool) -> dict:
    return {
        "workload": "opt6.7b_layer_stack_prefill (BASELINE.json configs[4])",
        "layers": args.layers, "tokens": args.tokens, "hidden": HIDDEN, "ffn": FFN,
        "linears_per_layer": [f"{name}:{k}->{n}:R{len(mods)}" for name, k, n, mods, _ in LINEARS],
        "moduli_k4096": list(MODULI_4), "moduli_k16384": list(MODULI_5),
        "activation_scale": "per-tensor", "out_dtype": "float16",
        "parallelism": f"column-sharded N x{args.gpus}" if sharded else "single GPU",
        "l2_policy": "inputs larger than L2 (about 6.4 GB of int8 weights streamed per step)",
    }


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
def make_peer_arena(args, world: int, device):
    """Symmetric memory for the sharded stack's outputs (the exchange then runs inside the
    GEMM epilogues as peer stores); None, with the reason, when the platform does not offer
    it or `--exchange nccl` asks for the all-gather.  All ranks take the same decision."""
    import torch
    import torch.distributed as dist
    from rns_llm_b200.parallel import ABSMAX_PAD, PeerArena

    if world == 1:
        return None, "single GPU"
    if args.exchange == "nccl":
        return None, "--exchange nccl"
    nbytes = args.layers * sum(world * ((args.tokens * (n // world) + ABSMAX_PAD) * 2 + 256) for _, _, n, _, _ in LINEARS)
    arena, why = None, ""
    try:
        arena = PeerArena(nbytes, device)
    except Exception as exc:            # not available here: every rank must fall back together
        why = f"{type(exc).__name__}: {exc}"
    # [arena exists, it has an NVLink multicast mapping]: the minimum over ranks decides for all
    flag = torch.tensor([1 if arena is not None else 0,
                         1 if arena is not None and arena.multicast_base != 0 else 0],
                        dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag[0].item()) == 0:
        return None, why or "symmetric memory failed on another rank"
    arena.multicast_everywhere = bool(int(flag[1].item()))
    return arena, ""


def build_stack(backend, args, rank: int, world: int, device, peer_arena=None):
    """Random-init weights, quantised and prepared layer by layer (the fp16
    weights are not kept).  Returns a list of layers, each a list of sharded
    linears in LINEARS order."""
    import torch
    from rns_llm_b200.parallel import ColumnShardedRNSLinear, shard_tensor

    gen = torch.Generator(device=device)
    gen.manual_seed(1004)
    stack = []
    for _ in range(args.layers):
        layer = []
        for name, k, n, mods, groups in LINEARS:
            weight = torch.randn((n, k), generator=gen, device=device, dtype=torch.float16) * (1.0 / k ** 0.5)
            bias = torch.randn((n,), generator=gen, device=device, dtype=torch.float16) * 0.01
            shard_w = shard_tensor(weight, world, rank, groups)
            shard_b = shard_tensor(bias, world, rank, groups)
            layer.append(ColumnShardedRNSLinear(shard_w, shard_b, backend=backend, moduli=mods, rank=rank,
                                                world=world, groups=groups, reuse_buffer=True,
                                                peer_arena=peer_arena,
                                                multicast=(args.exchange in ("auto", "multicast") and
                                                           getattr(peer_arena, "multicast_everywhere", False))))
            del weight, bias, shard_w, shard_b
        stack.append(layer)
    return stack


def run_stack(stack, x):
    """One step: the 4*layers linears in data-flow order.  The q block of the
    fused QKV output stands in for the attention output that feeds out_proj."""
    from rns_llm_b200.parallel import group_view

    h = x
    for qkv, out_proj, fc1, fc2 in stack:
        t = qkv(h)                                   # [G, M, 3*H/G]
        t = out_proj(group_view(t, 3, 0))            # q block, gathered layout
        t = fc1(t)
        h = fc2(t)
    return h


def gpu_library_baselines(tokens: int, layers: int, device) -> dict:
    """The same four linears per layer through library kernels on this GPU, for scale (not
    optimisation targets): fp16 F.linear, and native int8 (torch._int_mm on the same int8
    tensors, int32 -> fp32 dequantisation and bias in eager torch).  One layer's weights,
    CUDA events over 20 passes; returns ms per layer-pass and the tokens/s of a stack of
    `layers` such layers."""
    import torch
    import torch.nn.functional as F

    gen = torch.Generator(device=device)
    gen.manual_seed(1004)
    ws, bs, wq, ws_scale = [], [], [], []
    for _, k, n, _, _ in LINEARS:
        w = torch.randn((n, k), generator=gen, device=device, dtype=torch.float16) * (1.0 / k ** 0.5)
        ws.append(w)
        bs.append(torch.randn((n,), generator=gen, device=device, dtype=torch.float16) * 0.01)
        scale = w.float().abs().amax(dim=1).clamp_min(1e-8) / 127.0
        wq.append(torch.clamp(torch.round(w.float() / scale[:, None]), -127, 127).to(torch.int8).t().contiguous())
        ws_scale.append(scale)
    xs = [torch.randn((tokens, k), generator=gen, device=device, dtype=torch.float16) for _, k, _, _, _ in LINEARS]

    def fp16_pass():
        for x, w, b in zip(xs, ws, bs):
            F.linear(x, w, b)

    def int8_pass():
        for x, w, s_w, b in zip(xs, wq, ws_scale, bs):
            s_a = x.float().abs().amax().clamp_min(1e-8) / 127.0
            xq = torch.clamp(torch.round(x.float() / s_a), -127, 127).to(torch.int8)
            acc = torch._int_mm(xq, w)
            (acc.float() * s_a * s_w + b.float()).half()

    def time_ms(fn) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(20):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / 20

    useful = sum(2.0 * tokens * k * n for _, k, n, _, _ in LINEARS)
    out = {}
    for name, fn in (("fp16_f_linear", fp16_pass), ("int8_int_mm_eager_dequant", int8_pass)):
        ms = time_ms(fn)
        out[name] = {"ms_per_layer": ms, "useful_tops": useful / (ms * 1e-3) / 1e12,
                     "tokens_per_s": tokens / (ms * layers * 1e-3)}
    return out


def _reference_package():
    """The unmodified reference (its Python package and its CUDA extension built for this
    GPU) when it is installed under baseline/_ref, else None with the reason."""
    root = ROOT / "baseline" / "_ref"
    if not (root / "rns_llm").is_dir():
        return None, "the reference is not installed under baseline/_ref"
    if str(root) not in sys.path:
        sys.path.insert(0, str(root))
    try:
        import rns_llm  # noqa: F401
        from rns_llm.backends import cuda_backend as module
        if not module.cuda_extension_available():
            return None, "the reference's CUDA extension is not built"
        return module, ""
    except Exception as exc:       # an import problem must not lose the other columns
        return None, f"{type(exc).__name__}: {exc}"


def _median_us(fn, iters: int, warm: int) -> float:
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record()
        b.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    return statistics.median(times)


def _graph_us(fn, iters: int, warm: int):
    """The same call replayed from a CUDA graph (device time without the host's share)."""
    import torch
    try:
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            fn()
        return _median_us(graph.replay, iters, warm)
    except Exception as exc:   # graph capture is an extra, not the measurement
        return f"capture failed: {type(exc).__name__}"


def _int8_library_linear(weights, biases):
    """Native int8 baseline on the same tensors: per-tensor activation quantisation in eager
    torch, torch._int_mm on the concatenated int8 weight (rows padded to 32: the library GEMM
    refuses fewer than 17), fp32 dequantisation with the same scales, bias, cast."""
    import torch
    w = torch.cat(weights, dim=0).float()
    scale = w.abs().amax(dim=1).clamp_min(1e-8) / 127.0
    wq = torch.clamp(torch.round(w / scale[:, None]), -127, 127).to(torch.int8).t().contiguous()
    bias = torch.cat(biases).float()

    def run(x):
        flat = x.reshape(-1, x.shape[-1]).float()
        s_a = flat.abs().amax().clamp_min(1e-8) / 127.0
        xq = torch.clamp(torch.round(flat / s_a), -127, 127).to(torch.int8)
        rows = xq.shape[0]
        if rows < 32:
            xq = torch.nn.functional.pad(xq, (0, 0, 0, 32 - rows))
        acc = torch._int_mm(xq, wq)[:rows]
        return (acc.float() * s_a * scale + bias).to(x.dtype)
    return run


def run_fused_qkv_latency(args) -> None:
    """Configuration 1 of BASELINE.json: hidden 768, three nn.Linear(768, 768) fused into
    one RNS QKV projection, M in {1, 16, 128, 256} tokens (the shapes and the protocol of the
    reference's benchmarks/benchmark_qkv_fusion.py:60-90).  One JSON line with, per M, the
    median latency (CUDA events) of: the fused module call, three separate RNSLinear calls,
    the fused call replayed from a CUDA graph, and as baselines on the same GPU and tensors:
    fp16 F.linear on the concatenated weight, native int8 (torch._int_mm + eager quantise /
    dequantise) and the unmodified reference's fused-QKV module on its own CUDA path."""
    import torch
    import torch.nn.functional as F
    from torch import nn
    from rns_llm_b200.backends import CudaRNSBackend
    from rns_llm_b200.layers import RNSLinear, RNSQKVProjection

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the RNS path has no CPU implementation")
    backend = CudaRNSBackend()
    torch.manual_seed(1001)
    hidden = 768
    linears = []
    for _ in range(3):
        layer = nn.Linear(hidden, hidden, bias=True, device="cuda", dtype=torch.float16).eval()
        with torch.no_grad():
            layer.weight.normal_(0, 0.02)
            layer.bias.normal_(0, 0.02)
        linears.append(layer)
    fused = RNSQKVProjection.from_linears(*linears, backend=backend, mode="rns", moduli=MODULI_4).eval()
    separate = [RNSLinear.from_linear(l, backend=backend, mode="rns", moduli=MODULI_4).eval() for l in linears]
    w_cat = torch.cat([l.weight.detach() for l in linears], dim=0)
    b_cat = torch.cat([l.bias.detach() for l in linears], dim=0)
    int8_linear = _int8_library_linear([l.weight.detach() for l in linears], [l.bias.detach() for l in linears])
    ref_module, ref_why = _reference_package()
    ref_fused = None
    if ref_module is not None:
        from rns_llm.layers import RNSQKVProjection as RefQKV
        ref_backend = ref_module.CudaRNSBackend()
        ref_fused = RefQKV.from_linears(*linears, backend=ref_backend, mode="rns", moduli=MODULI_4).eval()
    iters, warm = max(20, args.steps * 20), max(args.warmup, 3) * 5

    rows = []
    with torch.no_grad():
        for tokens in (1, 16, 128, 256):
            x = torch.randn((1, tokens, hidden), dtype=torch.float16, device="cuda")
            q, k, v = fused(x)
            ref = [layer(x) for layer in separate]
            equal = all(torch.equal(a, b) for a, b in zip((q, k, v), ref))
            row = {"tokens": tokens, "bit_equal_to_three_layers": bool(equal),
                   "fused_us": _median_us(lambda: fused(x), iters, warm),
                   "three_layers_us": _median_us(lambda: [layer(x) for layer in separate], iters, warm),
                   "fused_graph_us": _graph_us(lambda: fused(x), iters, warm),
                   "fp16_us": _median_us(lambda: F.linear(x, w_cat, b_cat), iters, warm),
                   "fp16_graph_us": _graph_us(lambda: F.linear(x, w_cat, b_cat), iters, warm),
                   "int_mm_us": _median_us(lambda: int8_linear(x), iters, warm),
                   "int_mm_graph_us": _graph_us(lambda: int8_linear(x), iters, warm)}
            if ref_fused is not None:
                rq, rk, rv = ref_fused(x)
                row["reference_cuda_us"] = _median_us(lambda: ref_fused(x), iters, warm)
                row["equal_to_reference_cuda"] = bool(torch.equal(rq, q) and torch.equal(rk, k) and torch.equal(rv, v))
            else:
                row["reference_cuda_us"] = None
            ops = 2.0 * len(MODULI_4) * tokens * hidden * 3 * hidden
            row["channel_tops"] = ops / (row["fused_us"] * 1e-6) / 1e12
            row["weight_stream_gbs_graph"] = (3 * hidden * hidden / (row["fused_graph_us"] * 1e-6) / 1e9
                                              if isinstance(row["fused_graph_us"], float) else None)
            rows.append(row)
    backend.check_status()
    print(json.dumps({"metric": "fused_qkv_latency_us", "unit": "us", "n_gpus": 1, "higher_is_better": False,
                      "data": "synthetic", "dtype": "int8",
                      "config": {"workload": "fused_qkv_hidden768 (BASELINE.json configs[1])", "hidden": hidden,
                                 "moduli": list(MODULI_4), "activation_scale": "per-tensor", "iters": iters,
                                 "reference_cuda": "measured" if ref_fused is not None else f"unavailable: {ref_why}"},
                      "rows": rows}), flush=True)


def run_concurrency(args) -> None:
    """Configuration 2 of BASELINE.json, the protocol of the reference's
    benchmarks/benchmark_concurrency.py:94-118 and benchmark_adaptive_channels.py: (i) 1, 2
    and 4 requests of one token each (K = N = 768, int8) merged along M into one RNS GEMM,
    against the same requests as independent calls on their own CUDA streams; (ii) M = 128
    with activations in [-15, 15]: adaptive channel prefix chosen on the device (3 of 4
    channels) against the fixed 4-channel call.  Exactness is asserted before timing."""
    import numpy as np
    import torch
    from rns_llm_b200.backends import CudaRNSBackend

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the RNS path has no CPU implementation")
    backend = CudaRNSBackend()
    ref_module, ref_why = _reference_package()
    ref_backend = ref_module.CudaRNSBackend() if ref_module is not None else None
    torch.manual_seed(1002)
    k = n = 768
    w = torch.randint(-127, 128, (k, n), dtype=torch.int8, device="cuda")
    iters, warm = max(20, args.steps * 20), max(args.warmup, 3) * 5

    def exact(a):
        return torch.from_numpy(a.cpu().numpy().astype(np.int64) @ w.cpu().numpy().astype(np.int64)).cuda()

    def batching_rows(be, label):
        prepared = be.prepare_weight(w, MODULI_4)
        rows = []
        for count in (1, 2, 4):
            requests = [torch.randint(-127, 128, (1, k), dtype=torch.int8, device="cuda") for _ in range(count)]
            workspace = be.create_request_batch_workspace(device=w.device, dtype=torch.int8,
                                                          rows_per_request=[1] * count, k=k,
                                                          channels=len(MODULI_4), n=n)
            merged = be.matmul_prepared_fused_requests(requests, prepared, workspace=workspace, clone_outputs=True)
            assert all(torch.equal(o, exact(r)) for o, r in zip(merged, requests)), "merged batch is not exact"
            streams = [torch.cuda.Stream() for _ in range(count)]
            spaces = [be.create_workspace(device=w.device, channels=len(MODULI_4), m=1, n=n) for _ in range(count)]

            def independent():
                current = torch.cuda.current_stream()
                for stream, req, space in zip(streams, requests, spaces):
                    stream.wait_stream(current)
                    with torch.cuda.stream(stream):
                        be.matmul_prepared_fused(req, prepared, workspace=space)
                for stream in streams:
                    current.wait_stream(stream)
            independent()
            torch.cuda.synchronize()
            merged_us = _median_us(lambda: be.matmul_prepared_fused_requests(requests, prepared, workspace=workspace),
                                   iters, warm)
            streams_us = _median_us(independent, iters, warm)
            rows.append({"impl": label, "requests": count, "merged_us": merged_us, "independent_streams_us": streams_us,
                         "merged_requests_per_s": count / (merged_us * 1e-6)})
        return rows

    def adaptive_rows(be, label):
        prepared_full = be.prepare_weight(w, MODULI_4)
        prepared_adaptive = be.prepare_weight_adaptive(w, MODULI_4, min_channels=3)
        a = torch.randint(-15, 16, (128, k), dtype=torch.int8, device="cuda")
        out, meta = be.matmul_prepared_adaptive_fused(a, prepared_adaptive, return_metadata=True)
        assert torch.equal(out, exact(a)) and int(meta["channels"]) == 3, "adaptive prefix is wrong"
        full = torch.randint(-127, 128, (128, k), dtype=torch.int8, device="cuda")
        out_full, meta_full = be.matmul_prepared_adaptive_fused(full, prepared_adaptive, return_metadata=True)
        assert torch.equal(out_full, exact(full)) and int(meta_full["channels"]) == 4
        return {"impl": label, "tokens": 128, "selected_channels": int(meta["channels"]),
                "adaptive_us": _median_us(lambda: be.matmul_prepared_adaptive_fused(a, prepared_adaptive), iters, warm),
                "fixed_4_channels_us": _median_us(lambda: be.matmul_prepared_fused(a, prepared_full), iters, warm)}

    batching = batching_rows(backend, "rns_b200")
    adaptive = [adaptive_rows(backend, "rns_b200")]
    if ref_backend is not None:
        batching += batching_rows(ref_backend, "reference_cuda")
        adaptive.append(adaptive_rows(ref_backend, "reference_cuda"))
    backend.check_status()
    print(json.dumps({"metric": "continuous_batching_and_adaptive_latency_us", "unit": "us", "n_gpus": 1,
                      "higher_is_better": False, "data": "synthetic", "dtype": "int8",
                      "config": {"workload": "continuous batching + adaptive channels (BASELINE.json configs[2])",
                                 "k": k, "n": n, "moduli": list(MODULI_4), "iters": iters,
                                 "reference_cuda": "measured" if ref_backend is not None else f"unavailable: {ref_why}"},
                      "continuous_batching": batching, "adaptive_channels": adaptive}), flush=True)


def run_opt_decoder(args) -> None:
    """Configuration 3 of BASELINE.json: an OPT-125m-architecture decoder with random weights
    (12 layers, hidden 768, 12 heads, FFN 3072, vocabulary 50272, learned positions, fp16,
    seed 1003); fused q|k|v and out_proj of all 12 attention blocks replaced by RNS linears as
    the reference's scripts/evaluate_ppl.py:53-94 does, softmax and FFN in fp16.  Synthetic
    token ids uniform over the vocabulary, batch 8 x 512 tokens of prefill, then 128 greedy
    decode steps with the key/value cache.  Three variants on the same weights: fp16, native
    int8 (torch._int_mm on the same int8 tensors and scales in the same four linears per
    block) and RNS.  Reports tokens/s of each and the logits error of the RNS model against
    both; refuses to report when the RNS path did not run (stats counters, as
    scripts/evaluate_ppl.py:212-217)."""
    import copy

    import torch
    from torch import nn
    from transformers import OPTConfig, OPTForCausalLM

    from rns_llm_b200.backends import CudaRNSBackend
    from rns_llm_b200.integration import replace_opt_attention_blocks, replace_selected_linears

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the RNS path has no CPU implementation")
    batch, prompt, new_tokens = 8, 512, 128
    config = OPTConfig(vocab_size=50272, hidden_size=768, num_hidden_layers=12, num_attention_heads=12, ffn_dim=3072,
                       max_position_embeddings=2048, word_embed_proj_dim=768, do_layer_norm_before=True)
    torch.manual_seed(1003)
    base = OPTForCausalLM(config).half().cuda().eval()
    parameters = sum(p.numel() for p in base.parameters())

    class Int8Linear(nn.Module):
        """nn.Linear through the library int8 GEMM: per-output-channel int8 weights, per-tensor
        int8 activations, torch._int_mm, fp32 dequantisation in the reference's order."""

        def __init__(self, layer: nn.Linear) -> None:
            super().__init__()
            w = layer.weight.detach().float()
            scale = w.abs().amax(dim=1).clamp_min(torch.finfo(torch.float32).eps) / 127.0
            self.register_buffer("wq_t", torch.clamp(torch.round(w / scale[:, None]), -127, 127).to(torch.int8).t().contiguous())
            self.register_buffer("scale", scale)
            self.register_buffer("bias", None if layer.bias is None else layer.bias.detach().float())

        def forward(self, x):
            flat = x.reshape(-1, x.shape[-1]).float()
            s_a = flat.abs().amax().clamp_min(torch.finfo(torch.float32).eps) / 127.0
            xq = torch.clamp(torch.round(flat / s_a), -127, 127).to(torch.int8)
            rows = xq.shape[0]
            if rows < 32:
                xq = nn.functional.pad(xq, (0, 0, 0, 32 - rows))
            y = torch._int_mm(xq, self.wq_t)[:rows].float() * s_a * self.scale
            if self.bias is not None:
                y = y + self.bias
            return y.reshape(*x.shape[:-1], -1).to(x.dtype)

    def int8_variant():
        model = copy.deepcopy(base)
        for layer in model.model.decoder.layers:
            attn = layer.self_attn
            for name in ("q_proj", "k_proj", "v_proj", "out_proj"):
                setattr(attn, name, Int8Linear(getattr(attn, name)))
        return model.eval()

    backend = CudaRNSBackend()

    def rns_variant(with_ffn: bool):
        model = copy.deepcopy(base)
        replaced, coordinators = replace_opt_attention_blocks(model, backend=backend, blocks=None, moduli=MODULI_4,
                                                              include_out_proj=True)
        if with_ffn:
            replaced += replace_selected_linears(model, backend=backend, patterns=("fc1", "fc2"), moduli=MODULI_4)
        return model.eval(), replaced, coordinators

    torch.manual_seed(2003)
    ids = torch.randint(0, config.vocab_size, (batch, prompt), device="cuda")

    def generate(model):
        """Prefill + greedy decode with the key/value cache; returns (prefill logits of the
        last position as fp32, seconds of prefill, seconds of decode)."""
        with torch.no_grad():
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            e0.record()
            out = model(input_ids=ids, use_cache=True)
            logits = out.logits[:, -1, :].float()
            e1.record()
            cache = out.past_key_values
            token = logits.argmax(dim=-1, keepdim=True)
            for _ in range(new_tokens):
                out = model(input_ids=token, past_key_values=cache, use_cache=True)
                cache = out.past_key_values
                token = out.logits[:, -1, :].argmax(dim=-1, keepdim=True)
            e2.record()
            torch.cuda.synchronize()
        return logits, e0.elapsed_time(e1) * 1e-3, e1.elapsed_time(e2) * 1e-3

    def measure(model):
        generate(model)                       # warm-up: weight preparation, arenas, autotuning
        best = None
        for _ in range(max(1, min(args.steps, 3))):
            logits, prefill_s, decode_s = generate(model)
            if best is None or prefill_s + decode_s < best[1] + best[2]:
                best = (logits, prefill_s, decode_s)
        logits, prefill_s, decode_s = best
        return logits, {"prefill_s": prefill_s, "decode_s": decode_s,
                        "prefill_tokens_per_s": batch * prompt / prefill_s,
                        "decode_tokens_per_s": batch * new_tokens / decode_s,
                        "tokens_per_s": batch * (prompt + new_tokens) / (prefill_s + decode_s)}

    results = {}
    fp16_logits, results["fp16"] = measure(base)
    int8_model = int8_variant()
    int8_logits, results["int8_int_mm"] = measure(int8_model)
    del int8_model
    backend.reset_stats()
    rns_model, replaced, coordinators = rns_variant(with_ffn=False)
    rns_logits, results["rns"] = measure(rns_model)
    stats = backend.stats_snapshot()
    if stats.get("fused_gemm_calls", 0) <= 0 or any(c.projection.compute_count <= 0 for c in coordinators):
        raise SystemExit("the RNS path did not run (fused_gemm_calls / compute_count are zero): nothing to report")
    backend.check_status()
    del rns_model
    ffn_model, replaced_ffn, _ = rns_variant(with_ffn=True)
    ffn_logits, results["rns_attention_and_ffn"] = measure(ffn_model)
    backend.check_status()

    def errors(got, ref):
        diff = (got - ref).abs()
        return {"max_abs": float(diff.max()), "relative_l2": float(diff.norm() / ref.norm().clamp_min(1e-12)),
                "argmax_agreement": float((got.argmax(-1) == ref.argmax(-1)).float().mean())}

    print(json.dumps({
        "metric": "opt125m_shaped_decoder_tokens_per_s", "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True,
        "data": "synthetic", "dtype": "int8 (RNS linears), fp16 elsewhere",
        "value": results["rns"]["tokens_per_s"],
        "config": {"workload": "opt125m_shaped_decoder (BASELINE.json configs[3])", "parameters": parameters,
                   "batch": batch, "prompt_tokens": prompt, "new_tokens": new_tokens, "moduli": list(MODULI_4),
                   "replaced_modules": len(replaced), "replaced_with_ffn": len(replaced_ffn),
                   "decode": "eager module calls with the key/value cache (no CUDA graph)"},
        "variants": results,
        "logits_error_last_prefill_position": {
            "rns_vs_fp16": errors(rns_logits, fp16_logits), "rns_vs_int8": errors(rns_logits, int8_logits),
            "int8_vs_fp16": errors(int8_logits, fp16_logits),
            "rns_attention_and_ffn_vs_fp16": errors(ffn_logits, fp16_logits)},
        "rns_stats": {k: v for k, v in stats.items() if k.startswith("fused_gemm")},
    }), flush=True)


def run_quantiser(args) -> None:
    """The activation quantiser alone on the layer stack's two activation shapes: fp16
    [tokens, K] in, packed residue planes out (both launches: absmax, then quantise +
    planes), CUDA events over `iters` calls.  Bytes: the fp16 matrix read twice plus R
    plane bytes per value written; the fraction is against the measured copy bandwidth."""
    import torch
    from rns_llm_b200 import _native as N

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the RNS path has no CPU implementation")
    lib = N.load()
    peaks = load_peaks()
    stream = torch.cuda.current_stream().cuda_stream
    iters, rows = 50, []
    for k, mods in ((HIDDEN, MODULI_4), (FFN, MODULI_5)):
        m, r = args.tokens, len(mods)
        torch.manual_seed(k)
        x = torch.randn((m, k), dtype=torch.float16, device="cuda")
        planes = torch.empty(int(lib.rns_packed_activation_bytes(m, k, r)), dtype=torch.int8, device="cuda")
        scale = torch.empty(1, dtype=torch.float32, device="cuda")
        scratch = torch.zeros(16, dtype=torch.int8, device="cuda")
        moduli = N.moduli_array(mods)

        def call():
            N.check(lib.rns_quantize_activations(x.data_ptr(), N.F16, m, k, k, 0, 0, 0, 127, moduli, r, None,
                                                 planes.data_ptr(), 1, scale.data_ptr(), None,
                                                 scratch.data_ptr(), stream))
        for _ in range(max(3, args.warmup)):
            call()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(iters):
            call()
        stop.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(stop) / iters * 1e3
        nbytes = m * k * (2 * 2 + r)
        gbs = nbytes / us / 1e3
        rows.append({"rows": m, "k": k, "planes": r, "us": us, "bytes": nbytes, "gbs": gbs,
                     "frac_of_hbm": gbs / float(peaks["hbm_gbs"])})
    print(json.dumps({"metric": "activation_quantiser_us", "unit": "us", "n_gpus": 1, "higher_is_better": False,
                      "data": "synthetic", "dtype": "f32 -> int8", "peak_gbs": float(peaks["hbm_gbs"]),
                      "peak_source": peaks["source"],
                      "config": {"workload": "activation quantiser on the layer stack's shapes", "iters": iters,
                                 "l2_policy": "back-to-back calls: the K = 4096 case (32 MiB in, 64 MiB out) "
                                              "fits L2, the K = 16384 case (576 MB) does not"},
                      "rows": rows}))


def run_wide_sources(args) -> None:
    """quant_bits 12 and 16 (sources wider than int8, where the residue system is not
    degenerate) on the linears of one layer of the stack's shapes: the module on the
    tensor-core path (residue planes on both sides, one int8 MMA per channel) against the
    same module on the plane-level pipeline (exact SIMT GEMM per channel + Garner kernel,
    the stand-in for the reference's cuBLAS route) and fp16 F.linear; CUDA events over
    `iters` calls, outputs compared."""
    import torch
    import torch.nn.functional as F
    from rns_llm_b200.backends import CudaRNSBackend
    from rns_llm_b200.layers import RNSLinear

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the RNS path has no CPU implementation")
    backend = CudaRNSBackend()
    iters, rows = 10, []

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(n):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / n

    m = args.tokens
    for bits in (12, 16):
        for name, k, n in (("qkv", HIDDEN, 3 * HIDDEN), ("fc2", FFN, HIDDEN)):
            torch.manual_seed(bits + k)
            layer = RNSLinear(k, n, backend=backend, mode="rns", quant_bits=bits).half().cuda().eval()
            x = torch.randn((m, k), dtype=torch.float16, device="cuda")
            with torch.no_grad():
                y = layer(x)
                fast_ms = timed(lambda: layer(x), iters)
                backend.check_status()
                prepared = layer._prepared_weight
                planes, prepared.weight_planes_packed = prepared.weight_planes_packed, None   # plane-level pipeline
                try:
                    y_planes = layer(x)
                    plane_ms = timed(lambda: layer(x), 2)
                finally:
                    prepared.weight_planes_packed = planes
                fp16_ms = timed(lambda: F.linear(x, layer.weight, layer.bias), iters)
            r = len(layer.moduli)
            rows.append({"quant_bits": bits, "linear": name, "m": m, "k": k, "n": n, "channels": r,
                         "moduli": list(layer.moduli), "tensor_core_ms": fast_ms,
                         "channel_tops": 2.0 * r * m * k * n / fast_ms / 1e9,
                         "plane_pipeline_ms": plane_ms, "fp16_linear_ms": fp16_ms,
                         "max_abs_diff_vs_plane_pipeline": float((y.float() - y_planes.float()).abs().max()),
                         "max_abs_diff_vs_fp16": float((y.float() - F.linear(x, layer.weight, layer.bias).float()).abs().max())})
    print(json.dumps({"metric": "wide_source_rns_linear_ms", "unit": "ms", "n_gpus": 1, "higher_is_better": False,
                      "data": "synthetic", "dtype": "int16 sources, int8 residues",
                      "config": {"workload": "RNSLinear quant_bits 12 / 16 on the stack's QKV and fc2 shapes",
                                 "tokens": m, "iters": iters},
                      "rows": rows}))


def run_grouped_attention(args) -> None:
    """Grouped multi-head integer products, scores Q K^T and context P V of all heads of a
    batch in one launch each (`matmul_grouped`), against (a) the same products one head at a
    time through the single-problem integer entry (how the reference's attention benchmark
    shapes them: one head, benchmarks/benchmark_attention.py:107-113), (b) fp16 torch.bmm.
    CUDA events over `iters` calls; results compared with the per-head path."""
    import torch
    from rns_llm_b200.backends import CudaRNSBackend

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the RNS path has no CPU implementation")
    backend = CudaRNSBackend()
    iters, rows = 20, []

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(n):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / n

    gen = torch.Generator(device="cuda")
    gen.manual_seed(2024)
    for label, heads_total, tokens, head_dim in (("opt125m batch 8 x 512", 96, 512, 64),
                                                 ("opt6.7b batch 1 x 2048", 32, 2048, 128)):
        q = torch.randint(-127, 128, (heads_total, tokens, head_dim), generator=gen, device="cuda", dtype=torch.int8)
        k = torch.randint(-127, 128, (heads_total, tokens, head_dim), generator=gen, device="cuda", dtype=torch.int8)
        p = torch.randint(0, 128, (heads_total, tokens, tokens), generator=gen, device="cuda", dtype=torch.int8)
        v_t = torch.randint(-127, 128, (heads_total, head_dim, tokens), generator=gen, device="cuda", dtype=torch.int8)
        for name, a, b in (("scores Q K^T", q, k), ("context P V", p, v_t)):
            groups, m, kk = a.shape
            n = b.shape[1]
            grouped = backend.matmul_grouped(a, b, MODULI_4)
            grouped_ms = timed(lambda: backend.matmul_grouped(a, b, MODULI_4), iters)
            backend.check_status()
            prepared = [backend.prepare_weight_nk(b[g], MODULI_4) for g in range(min(groups, 8))]

            def per_head():
                return [backend.matmul_prepared_fused(a[g], prepared[g]) for g in range(len(prepared))]
            same = all(torch.equal(x, grouped[g]) for g, x in enumerate(per_head()))
            per_head_ms = timed(per_head, 5) * groups / len(prepared)        # weights prepared outside the timing
            scaled_ms = timed(lambda: backend.matmul_grouped(a, b, MODULI_4, out_dtype=torch.float16, scale=1e-4),
                              iters)
            a16, b16 = a.half(), b.half()
            fp16_ms = timed(lambda: torch.bmm(a16, b16.transpose(1, 2)), iters)
            r = len(MODULI_4)
            rows.append({"shape": label, "product": name, "groups": groups, "m": m, "k": kk, "n": n, "channels": r,
                         "grouped_ms": grouped_ms, "channel_tops": 2.0 * r * groups * m * kk * n / grouped_ms / 1e9,
                         "grouped_fp16_scaled_ms": scaled_ms,
                         "one_head_at_a_time_ms": per_head_ms, "fp16_bmm_ms": fp16_ms,
                         "equal_to_one_head_at_a_time": bool(same)})
    print(json.dumps({"metric": "grouped_attention_products_ms", "unit": "ms", "n_gpus": 1, "higher_is_better": False,
                      "data": "synthetic", "dtype": "int8",
                      "config": {"workload": "grouped multi-head Q K^T and P V (exact int64 outputs)",
                                 "moduli": list(MODULI_4), "iters": iters,
                                 "note": "grouped = plane encode + weight pack + one GEMM launch for all heads; "
                                         "one head at a time = plane encode + GEMM per head with the packed "
                                         "operand prepared outside the timed region"},
                      "rows": rows}))


# Where the run is, for the failure report: {"phase": ..., "step": ..., "layer": ..., "linear": ...}
PROGRESS: dict = {"phase": "start"}


def report_failure(exc: BaseException, backend=None) -> None:
    """The last thing a failing rank writes: ONE JSON line on stderr with its rank, the
    exception, where the run was, and the device status word with the place of an
    expired wait (under torchrun only the launcher's table survives otherwise)."""
    import traceback

    line = {"rank": int(os.environ.get("RANK", "0")), "error": f"{type(exc).__name__}: {exc}",
            "progress": dict(PROGRESS), "status_word": None,
            "traceback_tail": traceback.format_exception(type(exc), exc, exc.__traceback__)[-3:]}
    if backend is not None:
        try:
            for index, state in backend._device_state.items():
                line["status_word"] = int(state.status.item())
                line["wait_info"] = [int(v) for v in state.wait_info.cpu().tolist()]
        except Exception as inner:      # the context may be gone; say so instead of hiding the first error
            line["status_word"] = f"unreadable: {type(inner).__name__}: {inner}"
    sys.stderr.write("\n" + json.dumps(line) + "\n")
    sys.stderr.flush()


def locate_failing_linear(backend, stack, x):
    """After a non-zero device status: one more pass with a status check behind every
    linear.  Returns {"layer": i, "linear": name, "error": ...} or None when the pass is clean."""
    import torch
    from rns_llm_b200.parallel import group_view

    names = [name for name, *_ in LINEARS]
    h = x
    for index, layer in enumerate(stack):
        for name, linear in zip(names, layer):
            src = h
            if name == "out_proj":
                src = group_view(h, 3, 0)
            h = linear(src)
            torch.cuda.synchronize()
            try:
                backend.check_status()
            except Exception as exc:
                return {"layer": index, "linear": name, "error": str(exc)}
    return None


def run_layer_stack(args) -> None:
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the RNS path has no CPU implementation")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        PROGRESS["phase"] = "init_process_group"
        dist.init_process_group("nccl", device_id=device)

    from rns_llm_b200.backends import CudaRNSBackend

    backend = CudaRNSBackend()
    try:
        _run_layer_stack(args, backend, rank, world, local_rank, device)
    except BaseException as exc:
        if not isinstance(exc, SystemExit) or exc.code not in (0, None):
            report_failure(exc, backend)
            # Leave without running destructors: a failed rank must not wait for its peers.
            os._exit(1)
        raise


def _run_layer_stack(args, backend, rank, world, local_rank, device) -> None:
    import torch
    import torch.distributed as dist

    warmup = max(args.warmup, 3)
    PROGRESS["phase"] = "build_stack"
    free_bytes, total_bytes = torch.cuda.mem_get_info(device)
    PROGRESS["free_gib_at_start"] = round(free_bytes / 2**30, 1)
    PROGRESS["phase"] = "peer_arena"
    peer_arena, arena_why = make_peer_arena(args, world, device)
    PROGRESS["phase"] = "build_stack"
    stack = build_stack(backend, args, rank, world, device, peer_arena)
    exchange = ("peer stores from the GEMM epilogue into symmetric memory + a barrier per layer"
                if peer_arena is not None else f"NCCL all-gather per layer ({arena_why})")
    if peer_arena is not None and args.exchange in ("auto", "multicast"):
        used = sum(1 for layer in stack for lin in layer if lin.multicast)
        exchange = (f"multicast stores (multimem.st through NVSwitch) from the GEMM epilogue in {used} of "
                    f"{sum(len(layer) for layer in stack)} linears + a barrier per layer"
                    if used else exchange + " (no multicast mapping on this platform)")
    torch.manual_seed(4321)
    host_x = torch.randn((args.tokens, HIDDEN), dtype=torch.float16).pin_memory()
    host_y = torch.empty((args.tokens, HIDDEN), dtype=torch.float16).pin_memory()
    dev_x = host_x.to(device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- GEMM-kernel timing hooks (roofline.achieved) ----------------------
    gemm_events: list = []
    original_launch = backend._launch_fused

    def timed_launch(**kw):
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record()
        original_launch(**kw)
        stop.record()
        gemm_events.append((start, stop))

    def step_device():
        return run_stack(stack, dev_x)

    def step_e2e():
        x = host_x.to(device, non_blocking=True)
        y = run_stack(stack, x)
        from rns_llm_b200.parallel import unshard
        host_y.copy_(unshard(y, 1), non_blocking=True)
        return y

    def checked(phase: str):
        """Device status after a phase, on every rank; a failure names the linear."""
        torch.cuda.synchronize()
        try:
            backend.check_status()
        except Exception as exc:
            PROGRESS["first_failing_linear"] = locate_failing_linear(backend, stack, dev_x) or "not reproduced"
            raise RuntimeError(f"{phase}: {exc}") from exc

    PROGRESS["phase"] = "warmup"
    for i in range(warmup):
        PROGRESS["step"] = i
        step_device()
    barrier()
    y_check = step_device()
    if not bool(torch.isfinite(y_check).all()):
        raise RuntimeError("non-finite activations in the layer stack")
    checked("warm-up")
    # Every rank computed the same replicated activations: compare a checksum across ranks.
    if world > 1:
        digest = y_check.float().sum(dtype=torch.float64).reshape(1)
        lo, hi = digest.clone(), digest.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if float(lo) != float(hi):
            raise RuntimeError(f"ranks disagree on the stack's output checksum: {float(lo)} vs {float(hi)}")

    # ---- timed region: device-resident inputs -------------------------------
    PROGRESS["phase"] = "timed_device"
    backend._launch_fused = timed_launch
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        PROGRESS["step"] = i
        step_device()
    stop.record()
    barrier()
    clocks = sampler.stop()
    backend._launch_fused = original_launch
    elapsed_ms = start.elapsed_time(stop)
    gemm_ms = sum(a.elapsed_time(b) for a, b in gemm_events)
    gemm_launches = len(gemm_events)
    checked("timed region")

    # ---- timed region: end to end from host buffers -------------------------
    PROGRESS["phase"] = "timed_e2e"
    for _ in range(2):
        step_e2e()
    barrier()
    e_start = torch.cuda.Event(enable_timing=True)
    e_stop = torch.cuda.Event(enable_timing=True)
    e_start.record()
    for i in range(args.steps):
        PROGRESS["step"] = i
        step_e2e()
    e_stop.record()
    barrier()
    e2e_ms = e_start.elapsed_time(e_stop)
    checked("end-to-end region")

    PROGRESS["phase"] = "reduce_times"
    times = torch.tensor([elapsed_ms, e2e_ms, gemm_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, gemm_ms = (float(v) for v in times.tolist())

    PROGRESS["phase"] = "report"
    if rank == 0:
        ops = channel_ops_per_step(args.tokens, args.layers)
        ms_per_step = elapsed_ms / args.steps
        value = ops / (ms_per_step * 1e-3) / 1e12
        e2e_value = ops / (e2e_ms / args.steps * 1e-3) / 1e12
        peaks = load_peaks()
        # Dominant kernel: the fused RNS GEMM.  Per launch it performs 2*R*M*K*(N/world)
        # int8 tensor-core operations (the algorithmic work of one RNS linear).
        gemm_ops_per_rank = ops / world * args.steps
        achieved = gemm_ops_per_rank / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
        two_bf16 = 2.0 * float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
        int8_measured = None
        if not args.no_peak:
            int8_measured = measure_int8_peak(device)
        int8_peak = int8_measured["sustained"] if int8_measured else two_bf16
        # Kernels of this library per step: per linear one quantise/encode launch and one fused
        # GEMM; an absmax pass only where the input does not carry the previous layer's
        # absmax word (the q view that feeds out_proj, and the step's very first input).
        launches_per_step = args.layers * (2 * len(LINEARS) + 1) + 1
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": dict(workload_config(args, sharded=world > 1), exchange=exchange),
            "useful_tops": useful_ops_per_step(args.tokens, args.layers) / (ms_per_step * 1e-3) / 1e12,
            "tokens_per_s": args.tokens / (ms_per_step * 1e-3),
            "roofline": {
                "bound": "tensor", "kernel": "rns_gemm_pair_raw_kernel", "achieved": achieved, "peak": int8_peak,
                "unit": "TOPS", "frac": None if achieved is None else achieved / int8_peak,
                "peak_source": ("torch._int_mm 8192^3 back to back on this GPU in this run (sustained, under the "
                                "power cap)" if int8_measured else
                                f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']})"),
                "peak_int8_measured": int8_measured,
                "frac_vs_2x_bf16": None if achieved is None else achieved / two_bf16,
                "peak_2x_bf16_sustained": two_bf16,
                "launches": gemm_launches, "avg_launch_ms": gemm_ms / max(gemm_launches, 1),
                "traffic": NCU_DRAM_BYTES_PER_LAUNCH if (world == 1 and args.tokens == 4096) else None,
                "traffic_measured_in_this_run": False,
                "traffic_unit": "bytes per launch (dram read + write, mean over the four linears)",
                "traffic_source": "recorded constant: ncu capture (dram__bytes_read.sum + dram__bytes_write.sum) of "
                                  "this command with --layers 2; see the stack summary under profiles/",
                "algorithmic_bytes": algorithmic_bytes_per_launch(args.tokens),
            },
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": int(host_x.numel() * 2), "d2h_bytes_per_step": int(host_y.numel() * 2)},
            "gpu_launches": int(launches_per_step * args.steps),
        }
        if args.gpu_baselines and world == 1:
            line["gpu_baselines"] = gpu_library_baselines(args.tokens, args.layers, device)
        if not args.no_cpu_baseline and world == 1:
            try:
                line["cpu_baseline"] = {k: v for k, v in cpu_port_sample().items() if k != "seconds"}
                line["cpu_baseline"]["numpy_reference_config0"] = numpy_reference_sample()
            except Exception as exc:  # the CPU baseline must not lose the GPU measurement
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                                        "sample": f"failed: {exc}"}
        print(json.dumps(line), flush=True)
    PROGRESS["phase"] = "teardown"
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="rns_b200", choices=["rns_b200", "reference"])
    parser.add_argument("--layers", type=int, default=32)
    parser.add_argument("--tokens", type=int, default=4096)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--exchange", default="auto", choices=["auto", "peer", "multicast", "nccl"],
                        help="multi-GPU output exchange from the GEMM epilogue over symmetric memory: NVLink "
                             "multicast stores where every rank has the mapping, else a store per peer (auto, "
                             "multicast); a store per peer (peer); or the NCCL all-gather after the GEMM (nccl)")
    parser.add_argument("--no-peak", action="store_true",
                        help="skip the torch._int_mm peak measurement (roofline.frac then uses 2 x bf16 sustained)")
    parser.add_argument("--gpu-baselines", action="store_true",
                        help="also time F.linear fp16 and torch._int_mm + eager dequantisation on the stack's shapes")
    parser.add_argument("--workload", default="c4", choices=["c4", "c1", "c2", "c3", "quant", "peak", "wide", "attn"],
                        help="c4: the layer stack (the bench contract); c1: fused-QKV latency of configuration 1; "
                             "c2: continuous batching and adaptive channels of configuration 2; c3: the "
                             "OPT-125m-shaped decoder of configuration 3; quant: the activation quantiser alone "
                             "on the stack's shapes; peak: the int8 library-GEMM peak of this GPU")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.workload == "c1":
        run_fused_qkv_latency(args)
        return
    if args.workload == "c2":
        run_concurrency(args)
        return
    if args.workload == "c3":
        run_opt_decoder(args)
        return
    if args.workload == "wide":
        run_wide_sources(args)
        return
    if args.workload == "attn":
        run_grouped_attention(args)
        return
    if args.workload == "quant":
        run_quantiser(args)
        return
    if args.workload == "peak":
        import torch
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device")
        print(json.dumps({"metric": "int8_library_gemm_peak", "unit": "TOPS", "n_gpus": 1,
                          "higher_is_better": True, **measure_int8_peak(torch.device("cuda", 0), 4.0)}), flush=True)
        return
    run_layer_stack(args)


if __name__ == "__main__":
    main()
