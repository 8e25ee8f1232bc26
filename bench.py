#!/usr/bin/env python
"""Benchmark of the quantized-Linear hot path (quantize.rs:463-476 on B200).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A "step" is one pass of the hot path over one batch of synthetic input.  The default
workload is the Llama-7B-shaped MLP block of the benchmark configs (4096 -> 11008 gate/up with
SiLU, 11008 -> 4096 down, INT8 per-channel weights ~N(0,0.02), bf16 activations ~N(0,1),
batch 512), output channels sharded over the N GPUs with an all-gather after each of the
two sharded layers.  Metric: tokens/s (rows of the batch per second) for the whole job.
Other workloads (`--workload`): single Linears of config 3, the block at batch 1, and, on one
GPU, the f32-activation configs 1 (`mnist_mlp_m64`) and 2 (`tinygpt_stack_m4096`: the 25 Linears of
the TinyGPT-shaped stack; its vocabulary head is bound by the 823 MB f32 output it writes).
`--workload quantize_RxC` (config 5) times the per-channel quantizer instead and reports GB/s at
5 B/element + 8 B/row, with the single-threaded CPU restatement beside it.

Prints ONE JSON line on rank 0.  Timing: CUDA events on the launching stream, barrier and
synchronize on both sides, max over ranks; the K timed steps are captured as one CUDA graph (as the
layers of a model would be; `--graph-per-step` replays one graph per step instead, `--no-graph`
launches from the host).  L2: every step uses a different copy of the weights out of a ring larger
than twice the 126 MB L2.

`--gpus N --parallel replicas` is the data-parallel alternative (every GPU the whole block on its own
batch, weak scaling, no collective); the default `shard` is the configured output-channel split.

`--impl reference` times the reference's own CPU algorithm for the same step (the oracle
port: single-threaded f64 dequantization on every call, as quantize.rs:214-224,465 does,
then an f32 GEMM on all host cores) — the Rust reference cannot be built on this image.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

L2_BYTES = 126 * 1024 * 1024

# DRAM bytes (read + write) of one launch of the dominant kernel, from the ncu captures summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum; the capture's workload and command are in the file named):
# (workload, kernel family, GPUs) -> bytes
KNOWN_TRAFFIC = {
    ("llama_mlp_m512", "tcgen05-2cta", 1): 151.4e6,   # profiles/tcgen05_pair_llama_mlp_m512.md: gate/up launch, 136.5 MB read + 14.9 MB written
    ("linear4096_m1", "gemv", 1): 16.81e6,            # profiles/gemv_linear4096_m1.md: the codes once; the 8 KB of output stay in L2
    ("linear4096_m16", "mma-ring", 1): 16.95e6,       # profiles/mma_ring_linear4096_m16.md
    ("quantize_8192x8192", "quantize_rows_reg", 1): 306.6e6,   # profiles/quantize_rows_reg_8192x8192.md: 268.5 MB read + 38.1 MB written (the rest of the 67 MB still in L2)
}

WORKLOADS = {
    # name: (kind, M, dims...)
    "llama_mlp_m512": dict(kind="mlp", M=512, d_model=4096, d_ff=11008),
    "llama_mlp_m1": dict(kind="mlp", M=1, d_model=4096, d_ff=11008),
    "linear4096_m1": dict(kind="linear", M=1, N=4096, K=4096),
    "linear4096_m4": dict(kind="linear", M=4, N=4096, K=4096),
    "linear4096_m16": dict(kind="linear", M=16, N=4096, K=4096),
    "linear4096_m64": dict(kind="linear", M=64, N=4096, K=4096),
    "linear4096_m256": dict(kind="linear", M=256, N=4096, K=4096),
    "linear4096_m1024": dict(kind="linear", M=1024, N=4096, K=4096),
    # config 1: MLP 784 -> 256 -> 10 with ReLU, f32 activations ~U(0,1), batch 64 (the layers are chained)
    "mnist_mlp_m64": dict(kind="stack", M=64, chain=True, uniform=True, std=0.05,
                          layers=[(256, 784, True, True), (10, 256, False, True)]),
    # config 2: the Linear layers of a TinyGPT-shaped stack (d_model 256, d_ff 1024, 4 blocks, vocabulary 50257) on
    # batch 8 x seq 512 = 4096 rows of f32 activations; the glue between the layers (attention, norms, residuals)
    # is not part of the path, so every layer reads a resident N(0,1) stand-in of its input width
    "tinygpt_stack_m4096": dict(kind="stack", M=4096, chain=False, uniform=False, std=0.02,
                                layers=([(256, 256, False, False)] * 4 + [(1024, 256, False, True), (256, 1024, False, True)]) * 4
                                + [(50257, 256, False, False)]),
}


# config 5: the quantizer's bandwidth sweep (f32 ~N(0,1) with 1 % of the entries x50, per-channel absmax INT8).  These
# workloads report GB/s at 5 B/element + 8 B/row instead of tokens/s (there are no tokens in a weight matrix).
for _r, _c in ((1024, 1024), (4096, 4096), (8192, 8192), (16384, 8192), (16384, 16384), (32768, 16384)):
    WORKLOADS[f"quantize_{_r}x{_c}"] = dict(kind="quantize", rows=_r, cols=_c)


def outlier_matrix_host(rows, cols, seed=0):
    rng = np.random.default_rng(seed)
    w = rng.standard_normal((rows, cols), dtype=np.float32)
    w[rng.random((rows, cols), dtype=np.float32) < 0.01] *= np.float32(50.0)
    return w


def quantize_cpu_sample(wl, target_elements=32 << 20):
    """(step_fn, bytes per step, description): the oracle's quantize_tensor (quantize.rs:194-205, one thread, the f64
    widening copy included) on the first rows of the matrix, about 32 M elements of them."""
    from oracle import shrew_oracle as oracle
    oracle.build()
    rows = max(1, min(wl["rows"], target_elements // wl["cols"]))
    w = outlier_matrix_host(rows, wl["cols"])
    return (lambda: oracle.quantize_f32(w, oracle.PER_CHANNEL)), 5 * rows * wl["cols"] + 8 * rows, \
        f"first {rows} of {wl['rows']} rows per step, oracle C restatement on 1 thread"


def run_quantize_reference(args, wl, name):
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    step, nbytes, sample = quantize_cpu_sample(wl)
    step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    val = nbytes * args.steps / dt / 1e9
    print(json.dumps({
        "impl": "reference", "metric": "quantize_gb_per_s", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 -> int8 (f64 arithmetic)", "data": "synthetic",
        "config": config_line(args, wl, name),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": 1, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)
    return 0


def run_quantize_gpu(args, wl, name):
    """Config 5 on one GPU: quantize_tensor (per-channel) over a ring of matrices larger than twice L2."""
    import ctypes

    from shrew_b200 import QuantConfig, _lib, quantize_tensor
    from shrew_b200.quantize import Device
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        raise SystemExit("bench.py: the quantize workloads run on one GPU (rows are independent: N GPUs are N replicas)")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device — this path has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    sdev = Device.get(dev)
    R, C = wl["rows"], wl["cols"]
    cfg = QuantConfig.int8_per_channel()
    nbytes = 5 * R * C + 8 * R
    ring = max(1, -(-2 * L2_BYTES // (4 * R * C)))
    g = torch.Generator(device=dev).manual_seed(0)
    ws = []
    for _ in range(ring):
        w = torch.randn(R, C, device=dev, generator=g)
        w[torch.rand(R, C, device=dev, generator=g) < 0.01] *= 50.0
        ws.append(w)
    for i in range(args.warmup):
        quantize_tensor(ws[i % ring], cfg)
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    launches0 = sdev.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        quantize_tensor(ws[i % ring], cfg)
    e1.record()
    torch.cuda.synchronize()
    sdev.synchronize()
    ms = e0.elapsed_time(e1)
    launches = sdev.launch_count() - launches0
    value = nbytes * args.steps / (ms * 1e-3) / 1e9
    # end to end: host matrix in, host codes and scales out, through the host-buffer entry point
    w_host = ws[0].cpu().pin_memory()
    q_host = torch.empty((R, C), dtype=torch.int8).pin_memory()
    s_host = torch.empty(R, dtype=torch.float64).pin_memory()

    def e2e_step():
        sdev.bind_stream()
        _lib.check(_lib.lib().shrewq_quantize_f32_host(sdev.handle, ctypes.c_void_p(w_host.data_ptr()), R, C, 1,
                                                       ctypes.c_void_p(q_host.data_ptr()), ctypes.c_void_p(s_host.data_ptr())),
                   sdev.handle)
    e2e_step()
    n_e2e = max(3, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        e2e_step()
    e2e_value = nbytes * n_e2e / (time.perf_counter() - t0) / 1e9
    clocks = sampler.stop()
    peaks = measured_peaks()
    out = {
        "metric": "quantize_gb_per_s", "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 -> int8 (f32 with an exact f64 path for near-ties)", "data": "synthetic",
        "config": config_line(args, wl, name),
        "notes": {"l2": f"ring of {ring} matrices ({ring * 4 * R * C / 1e6:.0f} MB of f32)"
                        + (" > 2x L2" if ring * 4 * R * C > 2 * L2_BYTES else "")},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 4 * R * C, "d2h_bytes_per_step": R * C + 8 * R,
                "steps": n_e2e},
        "gpu_launches": int(launches), "launch_mode": "host launches", "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": value, "peak": peaks["hbm"], "unit": "GB/s", "frac": value / peaks["hbm"],
                     "traffic": KNOWN_TRAFFIC.get((name, "quantize_rows_reg", 1)),
                     "kernel": "quantize_rows_reg" if C % 4 == 0 and C <= 32768 else "quantize_rows_generic",
                     "kernel_us": ms / args.steps * 1e3, "peaks": peaks["source"],
                     "timing": "CUDA events around the timed steps (one launch per step)"},
    }
    if not args.no_cpu_baseline:
        step, cbytes, sample = quantize_cpu_sample(wl)
        step()
        t0, n = time.perf_counter(), 0
        while n < 2 or (time.perf_counter() - t0 < 10 and n < 20):
            step()
            n += 1
        out["cpu_baseline"] = {"value": cbytes * n / (time.perf_counter() - t0) / 1e9, "unit": "GB/s", "cores": 1,
                               "kind": "port", "sample": f"{n} x " + sample}
    print(json.dumps(out), flush=True)
    return 0


def host_threads():
    """All host cores this process may use.  torchrun exports OMP_NUM_THREADS=1 to its workers, which would make the
    CPU arm of a multi-GPU launch single-threaded: the CPU legs set the thread count themselves."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def config_line(args, wl, name):
    """`config` of the JSON line: the same keys and values in both arms and at every GPU count (what differs between
    runs of one workload is said in `notes`)."""
    c = {"workload": name, **config_of(wl)}
    if wl["kind"] != "quantize":
        c["weights"] = f"INT8 {args.granularity.replace('_', '-')}, N(0,{wl.get('std', 0.02)})"
    else:
        c["granularity"] = "per-channel"
    if getattr(args, "force_kernel", "auto") != "auto":
        c["forced_kernel"] = args.force_kernel
    return c


def config_of(wl):
    """The workload's entries for the JSON line's `config` (a stack's layer list as one string)."""
    c = {k: v for k, v in wl.items() if k not in ("kind", "layers")}
    if wl["kind"] == "stack":
        c["layers"] = f"{len(wl['layers'])} Linears, " + " ".join(sorted({f"{k}->{n}" for n, k, _, _ in wl["layers"]}))
        c["activations"] = "f32"
    return c


def stack_layers(wl):
    """(N, K, relu, bias) per Linear of a "stack" workload."""
    return [tuple(l) for l in wl["layers"]]


def stack_forward(x, linears, spec, bufs, stand_ins, chain, relu_code=1, none_code=0):
    """One pass over the Linears of a stack workload.  `linears[i].forward(src, epilogue=, out=)` writes layer i's
    output into bufs[i].  chain: every layer reads the previous layer's output (config 1).  Otherwise (config 2, where
    the glue between the layers is not part of the path) a layer as wide as x reads x and the others read the resident
    stand-in of their input width.  Returns the last layer's output."""
    y = x
    for lin, (n, k, relu, _), buf in zip(linears, spec, bufs):
        src = y if chain else (x if k == x.shape[1] else stand_ins[k])
        y = lin.forward(src, epilogue=relu_code if relu else none_code, out=buf)
    return y


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], tc_burst=d["bf16_tflops"], tc_sustained=d["bf16_tflops_sustained"], source="measured")
    return dict(hbm=6650.0, tc_burst=1590.0, tc_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap,utilization.gpu")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, busy, smax, reasons = [], [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                mhz = float(r[1])
                smax = float(r[2])
                for nm, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
            except Exception:
                continue
            sm.append(mhz)
            try:
                if float(r[9]) >= 10.0:
                    busy.append(mhz)
            except Exception:
                pass
        # the median is taken over the samples that saw the GPU busy (all samples if none reported a utilisation)
        use = busy or sm
        return {"sm_mhz": statistics.median(use) if use else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(use), "samples_all": len(sm)}


# ---------------------------------------------------------------------------------------------
# synthetic inputs (seeded; stand in for the reference's unseeded randn — nothing is fetched)
# ---------------------------------------------------------------------------------------------
def gpu_weight(n, k, seed, device):
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(n, k, device=device, generator=g) * 0.02


def host_weight(n, k, seed):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))


# ---------------------------------------------------------------------------------------------
# the CPU arm: reference algorithm on host cores
# ---------------------------------------------------------------------------------------------
def cpu_step_factory(wl, per_tensor=False):
    """Returns (step_fn, tokens, description).  Each call performs one forward exactly as the
    reference does: dequantize every weight afresh (single thread, f64 then f32), then f32
    GEMM on all cores (torch CPU as stand-in for the `gemm` crate), then bias / activation."""
    from oracle import shrew_oracle as oracle
    oracle.build()
    torch.set_num_threads(host_threads())
    gran = oracle.PER_TENSOR if per_tensor else oracle.PER_CHANNEL
    M = wl["M"]
    rng = np.random.default_rng(1)
    if wl["kind"] == "mlp":
        dm, dff = wl["d_model"], wl["d_ff"]
        shapes = [(dff, dm), (dff, dm), (dm, dff)]
    elif wl["kind"] == "stack":
        shapes = [(n, k) for n, k, _, _ in stack_layers(wl)]
    else:
        shapes = [(wl["N"], wl["K"])]
    qs = []
    for i, (n, k) in enumerate(shapes):
        w = host_weight(n, k, i)
        if wl["kind"] == "stack":
            w = w * np.float32(wl["std"] / 0.02)
        q, s = oracle.np_quantize_f32(w, gran)
        qs.append((q, s, np.empty((n, k), dtype=np.float32)))
    if wl["kind"] == "stack":  # f32 activations: U(0,1) for config 1, N(0,1) stand-ins per input width for config 2
        draw = (lambda k: rng.random((M, k), dtype=np.float32)) if wl["uniform"] else (lambda k: rng.standard_normal((M, k), dtype=np.float32))
        xs = {k: torch.from_numpy(draw(k)) for k in sorted({k for _, k in shapes})}
        x = xs[shapes[0][1]]
    else:
        x = torch.from_numpy(rng.standard_normal((M, shapes[0][1]), dtype=np.float32)).to(torch.bfloat16).float()

    def lin(i, inp):
        q, s, buf = qs[i]
        oracle.dequantize_like_reference(q, s, gran, buf)  # quantize.rs:465, every call
        return inp @ torch.from_numpy(buf).t()                          # quantize.rs:468-469

    def step():
        if wl["kind"] == "mlp":
            g, u = lin(0, x), lin(1, x)
            h = torch.nn.functional.silu(g) * u
            return lin(2, h)
        if wl["kind"] == "stack":
            y = x
            for i, (n, k, relu, bias) in enumerate(stack_layers(wl)):
                y = lin(i, y if wl["chain"] else xs[k])
                if bias:
                    y = y + torch.zeros(1, n)      # quantize.rs:471-472: the broadcast add of the [1,out] bias
                if relu:
                    y = torch.relu(y)
            return y
        return lin(0, x)

    return step, M, f"full step: batch {M}, every weight dequantized per call (1 thread) + f32 GEMM on {torch.get_num_threads()} threads"


def run_reference_arm(args, wl, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    step, tokens, sample = cpu_step_factory(wl, args.granularity == "per_tensor")
    for _ in range(max(1, min(args.warmup, 2))):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    val = tokens * args.steps / dt
    out = {
        "impl": "reference", "metric": "quantized_linear_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_line(args, wl, name),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "Rust reference (shrew-cpu: gemm 0.18.2 + rayon) cannot be built on this image; this is the CPU port of "
                "quantize.rs:463-476 with torch CPU matmul standing in for the gemm crate",
    }
    print(json.dumps(out), flush=True)
    return 0


# ---------------------------------------------------------------------------------------------
# the GPU arm
# ---------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="llama_mlp_m512", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from the host instead of replaying a CUDA graph")
    ap.add_argument("--graph-per-step", action="store_true", help="time one graph replay per step instead of one graph of all timed steps")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="multi-GPU exchange: 'fused' = peer stores from the kernel epilogue, 'nccl' = all-gather")
    ap.add_argument("--granularity", default="per_channel", choices=["per_channel", "per_tensor"],
                    help="one scale per output channel (all configs) or one per tensor (the other half of config 3); "
                         "on several GPUs only per_channel (shards of a per-tensor weight must first agree on amax)")
    ap.add_argument("--parallel", default="shard", choices=["shard", "replicas"],
                    help="--gpus N: 'shard' = the weights split by output channel (strong scaling, the configured path); "
                         "'replicas' = every GPU runs the whole block on a batch of its own (weak scaling, no collective)")
    ap.add_argument("--force-kernel", default="auto",
                    help="kernel family for every forward of the run (see shrewq_force_kernel); experiments only")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    wl = WORKLOADS[args.workload]
    if wl["kind"] == "quantize":
        return (run_quantize_reference if args.impl == "reference" else run_quantize_gpu)(args, wl, args.workload)
    if args.impl == "reference":
        return run_reference_arm(args, wl, args.workload)

    import torch.distributed as dist
    from shrew_b200 import Linear, QuantConfig, QuantizedLinear, _lib
    from shrew_b200.quantize import Device
    from shrew_b200.sharded import FusedShardedGatedMLP, FusedShardedLinear, ShardedGatedMLP, ShardedLinear, plan_shards

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device — this path has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL carries only barriers and one-float reductions here (the exchange is peer stores from the kernels, or
        # an all-gather of a few MB): in-switch reduction buys nothing, and every multi-GPU run of this benchmark so
        # far was made with it off
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
        # (every device-side wait of the exchange is bounded: a rank whose peer is gone gets SHREWQ_ERR_TIMEOUT from
        # its next synchronize instead of waiting for ever)
    sdev = Device.get(dev)
    if args.force_kernel != "auto":
        _lib.check(_lib.lib().shrewq_force_kernel(args.force_kernel.encode()), None)
    cfg = QuantConfig.int8() if args.granularity == "per_tensor" else QuantConfig.int8_per_channel()
    if args.granularity == "per_tensor" and world > 1 and args.parallel == "shard":
        raise SystemExit("bench.py: --granularity per_tensor with sharded weights is not a benchmark workload "
                         "(use sharded.quantize_row_shard for it); run it on one GPU or with --parallel replicas")
    M = wl["M"]
    # replicas: the model is not split; sw/sr are the world size and rank the sharding sees
    replicas = world > 1 and args.parallel == "replicas"
    sw, sr = (1, 0) if replicas else (world, rank)
    own_group = None
    if replicas:   # every rank's layers live in a group of one (new_group is collective: all ranks create all groups)
        own_group = [dist.new_group([r]) for r in range(world)][rank]
    if wl["kind"] == "stack" and world > 1:
        raise SystemExit("bench.py: the stack workloads (configs 1 and 2) run on one GPU; --gpus N takes the default workload")

    # ---- build the rank's shards; a ring of weight copies defeats L2 between steps ----
    def make_shard(n, k, seed):
        n0, n1 = plan_shards(n, sw).rows(sr)
        w = gpu_weight(n, k, seed, dev)[n0:n1].contiguous()
        return QuantizedLinear.from_linear(Linear(w, None), cfg)

    if wl["kind"] == "mlp":
        dm, dff = wl["d_model"], wl["d_ff"]
        shard_bytes = (2 * dff * dm + dm * dff) // sw
        in_features = dm
        flops_step = 2 * M * (2 * dff * dm + dm * dff)
    elif wl["kind"] == "stack":
        layers = stack_layers(wl)
        shard_bytes = sum(n * k for n, k, _, _ in layers)
        in_features = layers[0][1]
        flops_step = sum(2 * M * n * k for n, k, _, _ in layers)
    else:
        shard_bytes = wl["N"] * wl["K"] // sw
        in_features = wl["K"]
        flops_step = 2 * M * wl["N"] * wl["K"]
    ring = max(2, -(-2 * L2_BYTES // shard_bytes) + 1)
    if wl["kind"] == "stack":
        ring = min(ring, 32)   # config 1 is 0.2 MB of codes: no ring of sensible length exceeds L2, and the line says so
    fused = sw > 1 and args.gather == "fused"
    x_dt = torch.float32 if wl["kind"] == "stack" else torch.bfloat16

    class Stack:
        """The Linears of a stack workload, one after the other.  Output buffers and the stand-in inputs of
        the other widths are shared by all ring entries; only the weights differ between entries."""
        bufs, stand_ins = None, None

        def __init__(self):
            gb = torch.Generator(device=dev).manual_seed(3)
            self.layers = []
            for i, (n, k, relu, bias) in enumerate(layers):
                w = gpu_weight(n, k, i, dev) * (wl["std"] / 0.02)
                b = torch.randn(n, device=dev, generator=gb) * 0.1 if bias else None
                self.layers.append((QuantizedLinear.from_linear(Linear(w, b), cfg), relu))
            if Stack.bufs is None:
                Stack.bufs = [torch.empty((M, n), dtype=x_dt, device=dev) for n, _, _, _ in layers]
                gs = torch.Generator(device=dev).manual_seed(4)
                Stack.stand_ins = {k: torch.randn(M, k, device=dev, generator=gs) for k in sorted({k for _, k, _, _ in layers})}

        def forward(self, x):
            return stack_forward(x, [ql for ql, _ in self.layers], layers, Stack.bufs, Stack.stand_ins, wl["chain"],
                                 _lib.EPILOGUE_RELU, _lib.EPILOGUE_NONE)

    models = []
    for c in range(ring):
        if wl["kind"] == "stack":
            models.append(Stack())
        elif wl["kind"] == "mlp":
            g, u, d = make_shard(dff, dm, 0), make_shard(dff, dm, 1), make_shard(dm, dff, 2)
            if fused:
                models.append(FusedShardedGatedMLP(g, u, d, dff, dm, M, share=models[0] if models else None))
            else:
                models.append(ShardedGatedMLP(g, u, d, dff, dm, group=own_group))
        else:
            q = make_shard(wl["N"], wl["K"], 0)
            if fused:
                models.append(FusedShardedLinear(wl["N"], q, None, M, torch.bfloat16, out=models[0].out if models else None))
            else:
                models.append(ShardedLinear(wl["N"], lambda x, out, _q=q: _q.forward(x, out=out), group=own_group))
            models[-1].shard = q
    torch.cuda.synchronize()

    gx = torch.Generator(device=dev).manual_seed(1)
    if wl["kind"] == "stack" and wl["uniform"]:
        x_dev = torch.rand(M, in_features, device=dev, generator=gx)
    else:
        x_dev = torch.randn(M, in_features, device=dev, generator=gx).to(x_dt)
    x_host = x_dev.cpu().pin_memory()
    out_features = wl["d_model"] if wl["kind"] == "mlp" else layers[-1][0] if wl["kind"] == "stack" else wl["N"]
    y_host = torch.empty((M, out_features), dtype=x_dt).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def eager_step(i, x):
        return models[i % ring].forward(x)

    # ---- several GPUs: is what the ranks compute the layer's output?  (outside every timed region) ----
    # Rank 0 builds the UNSPLIT layers from the same seeds and runs the one-GPU forward (the path the GPU parity tests hold
    # against the oracle); every rank compares its own copy of the exchanged result with it.
    parity = None
    if world > 1 and not replicas and wl["kind"] in ("mlp", "linear"):
        y_mine = eager_step(0, x_dev).float()
        torch.cuda.synchronize()
        y_ref = torch.empty_like(y_mine)
        if rank == 0:
            def full(n, k, seed):
                return QuantizedLinear.from_linear(Linear(gpu_weight(n, k, seed, dev), None), cfg)
            if wl["kind"] == "mlp":
                g_f, u_f, d_f = full(dff, dm, 0), full(dff, dm, 1), full(dm, dff, 2)
                y_ref.copy_(d_f.forward(g_f.forward_gate_up_silu(u_f, x_dev)).float())
                del g_f, u_f, d_f
            else:
                q_f = full(wl["N"], wl["K"], 0)
                y_ref.copy_(q_f.forward(x_dev).float())
                del q_f
            sdev.synchronize()
        dist.broadcast(y_ref, src=0)
        err = ((y_mine - y_ref).abs().max() / y_ref.abs().max().clamp_min(1e-30)).reshape(1)
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        parity = {"max_rel_err_vs_one_gpu_forward": float(err.item()), "tolerance": 1e-2, "ok": bool(err.item() <= 1e-2),
                  "checked": "every rank's copy of the exchanged output against rank 0's unsplit forward of the same weights"}
        del y_ref, y_mine
        torch.cuda.empty_cache()

    # One CUDA graph per ring entry: a step is a handful of short kernels (and, on several
    # GPUs, device-side barriers), so replaying a captured graph removes the host launch
    # path from the measurement.  x_static is the graph's input buffer, outs[i] its result.
    x_static = x_dev.clone()
    graphs, outs = [], []
    # NCCL collectives captured in a graph left the processes hanging at exit on this software
    # stack (results were printed, the ranks never ended): the NCCL variant is launched eagerly
    use_graphs = not args.no_graph and not (sw > 1 and not fused)
    if use_graphs:
        try:
            for i in range(ring):
                eager_step(i, x_static)  # first use of a kernel sets its attributes: outside capture
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for i in range(ring):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        outs.append(eager_step(i, x_static))
                    graphs.append(g)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
        except Exception as e:  # capture unsupported for some collective: measure eagerly
            sys.stderr.write(f"bench: graph capture failed ({e!r}); running eagerly\n")
            graphs, outs, use_graphs = [], [], False

    # kernels of this library per step, counted by the library (one eager step; the graphs replay the same launches):
    # forward kernels, the f32 split passes, a K-split tail launch where the launcher issues one, exchange barriers
    _l0 = sdev.launch_count()
    eager_step(0, x_static)
    sdev.synchronize()
    launches_per_step = int(sdev.launch_count() - _l0)

    def step(i, x):
        if use_graphs:
            if x is not x_static:
                x_static.copy_(x, non_blocking=True)
            graphs[i % ring].replay()
            return outs[i % ring]
        return eager_step(i, x)

    # ---- device-resident metric ----
    # The K timed steps are captured as ONE graph (step i on ring entry i % ring, as in the loop it replaces), the way a
    # model's layers reach the GPU: with the kernels' programmatic dependent launch a step's first kernel then starts
    # its prologue under the previous step's last wave instead of behind a host-side graph launch.
    timed_graph = None
    if use_graphs and not args.graph_per_step and args.steps <= 512:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                tg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(tg, stream=side):
                    for i in range(args.steps):
                        eager_step(i, x_static)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            timed_graph = tg
        except Exception as e:  # noqa: BLE001
            sys.stderr.write(f"bench: capture of the timed steps as one graph failed ({e!r}); one graph replay per step\n")
            timed_graph = None
    for i in range(args.warmup):
        step(i, x_static)
    if timed_graph is not None:
        timed_graph.replay()   # one untimed pass of the graph itself
        torch.cuda.synchronize()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = sdev.launch_count()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if timed_graph is not None:
        timed_graph.replay()          # the K steps as one graph: no host launch between them
    else:
        for i in range(args.steps):
            step(i, x_static)
    e1.record()
    barrier()
    sdev.synchronize()  # also surfaces a kernel that gave up a bounded wait
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    launches = launches_per_step * args.steps if use_graphs else sdev.launch_count() - launches0
    rows_per_step = M * (world if replicas else 1)   # replicas: every GPU processes a batch of its own
    value = rows_per_step * args.steps / (ms_total * 1e-3)

    # ---- end to end: pinned host input in, host output back, every step ----
    def e2e_step(i):
        if use_graphs:
            x_static.copy_(x_host, non_blocking=True)   # pinned host -> the graph's input buffer
            y = step(i, x_static)
        else:
            y = step(i, x_host.to(dev, non_blocking=True))
        y_host.copy_(y, non_blocking=True)              # result back to pinned host memory
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    t_e2e = torch.tensor([time.perf_counter() - t0], device=dev)
    if world > 1:
        dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
    e2e_value = rows_per_step * args.steps / float(t_e2e.item())
    e2e_info = {"mode": "sequential: torch copy in, the device entry points, torch copy out, synchronize, per step",
                "sequential_value": e2e_value}

    # ---- end to end through the library's host-buffer entry points (one GPU): the call a host-tensor caller makes ----
    # shrewq_mlp_forward_host / shrewq_linear_forward_host take pinned host x and deliver host y, copies and kernels
    # inside the call.  Sequential = one synchronising call per step.  Pipelined (the block) = the same entry point
    # asked not to synchronise: it keeps two staging slots and its own copy streams, so the copies of one step overlap
    # the kernels of the next; every step still moves its x in and its y out inside the timed region.
    if world == 1 and wl["kind"] in ("mlp", "linear"):
        try:
            from shrew_b200.quantize import mlp_forward_host
            y_pins = [torch.empty_like(y_host).pin_memory() for _ in range(2)]

            def abi_step(i, sync, out):
                m = models[i % ring]
                if wl["kind"] == "mlp":
                    return mlp_forward_host(m.gate, m.up, m.down, x_host, out=out, synchronize=sync)
                out.copy_(m.shard.forward_host(x_host))
                return out
            for i in range(3):
                abi_step(i, True, y_pins[0])
            y_ref = y_pins[0].clone()
            t0 = time.perf_counter()
            for i in range(args.steps):
                abi_step(i, True, y_pins[i & 1])
            abi_seq = M * args.steps / (time.perf_counter() - t0)
            e2e_info.update({"abi_sequential_value": abi_seq,
                             "abi_entry": "shrewq_mlp_forward_host" if wl["kind"] == "mlp" else "shrewq_linear_forward_host"})
            e2e_value, e2e_info["mode"] = abi_seq, f"{e2e_info['abi_entry']}, one synchronising call per step"
            if wl["kind"] == "mlp":
                for i in range(4):
                    abi_step(i, False, y_pins[i & 1])
                sdev.synchronize()
                same = all(torch.equal(yp, y_ref) for yp in y_pins) if ring == 1 else True
                t0 = time.perf_counter()
                for i in range(args.steps):
                    abi_step(i, False, y_pins[i & 1])
                sdev.synchronize()
                abi_pipe = M * args.steps / (time.perf_counter() - t0)
                e2e_info["abi_pipelined_value"] = abi_pipe
                if same and abi_pipe > e2e_value:
                    e2e_value = abi_pipe
                    e2e_info["mode"] = ("shrewq_mlp_forward_host without a synchronise per call (two staging slots and copy streams "
                                        "inside the library: the copies of a step overlap the kernels of its neighbours); "
                                        "one synchronise after the last step")
        except Exception as e:  # noqa: BLE001  (the torch-copy figure measured above stays)
            sys.stderr.write(f"bench: end-to-end run through the host-buffer entry points failed ({e!r})\n")
            try:
                torch.cuda.synchronize()
            except Exception:  # noqa: BLE001
                pass

    # ---- dominant kernel alone, for the roofline ----
    peaks = measured_peaks()
    iters = max(args.steps, 20)
    if wl["kind"] == "mlp":
        n_loc = models[0].gate.out_features
        hbuf = torch.empty((M, n_loc), dtype=torch.bfloat16, device=dev)
        kern = lambda i: models[i % ring].gate.forward_gate_up_silu(models[i % ring].up, x_dev, out=hbuf)  # noqa: E731
        k_flops = 2 * 2 * M * n_loc * dm
        k_bytes = 2 * n_loc * dm + 2 * 4 * n_loc + M * dm * 2 + M * n_loc * 2
        kname = models[0].gate
    elif wl["kind"] == "stack":
        # the layer whose roofline time is the longest (config 2: the vocabulary head, bound by its 823 MB f32 output)
        def roof_time(l):
            n, k, _, b = l
            return max(2 * M * n * k / (peaks["tc_sustained"] * 1e12), (n * k + 4 * n * (1 + b) + 4 * M * k + 4 * M * n) / (peaks["hbm"] * 1e9))
        li = max(range(len(layers)), key=lambda j: roof_time(layers[j]))
        n_d, k_d, relu_d, bias_d = layers[li]
        x_d = x_dev if k_d == x_dev.shape[1] else Stack.stand_ins[k_d]
        kern = lambda i: models[i % ring].layers[li][0].forward(x_d, out=Stack.bufs[li])  # noqa: E731
        k_flops = 2 * M * n_d * k_d
        k_bytes = n_d * k_d + 4 * n_d * (1 + bias_d) + 4 * M * k_d + 4 * M * n_d
        kname = models[0].layers[li][0]
    else:
        q = models[0].shard
        ybuf = torch.empty((M, q.out_features), dtype=torch.bfloat16, device=dev)
        kern = lambda i: models[i % ring].shard.forward(x_dev, out=ybuf)  # noqa: E731
        k_flops = 2 * M * q.out_features * q.in_features
        k_bytes = q.out_features * q.in_features + 4 * q.out_features + M * q.in_features * 2 + M * q.out_features * 2
        kname = q
    k_s, k_timing, k_error = None, None, None
    try:
        for i in range(3):
            kern(i)
        torch.cuda.synchronize()
        e0.record()
        for i in range(iters):
            kern(i)
        e1.record()
        torch.cuda.synchronize()
        k_s = e0.elapsed_time(e1) * 1e-3 / iters
        k_timing = "CUDA events, host-launched back to back (includes launch gaps)"
    except Exception as e:  # noqa: BLE001  (the step figures measured above are still reported)
        k_error = repr(e)
        sys.stderr.write(f"bench: timing the dominant kernel alone failed ({e!r})\n")
    # The same launches replayed from one CUDA graph: no host launch path between them, which matters for the
    # kernels of a few microseconds (batch 1).  Kept only if it ran; the shorter of the two is reported.
    if not args.no_graph and k_s is not None:
        try:
            kg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(kg):
                for i in range(iters):
                    kern(i)
            kg.replay()
            torch.cuda.synchronize()
            e0.record()
            kg.replay()
            e1.record()
            torch.cuda.synchronize()
            k_graph = e0.elapsed_time(e1) * 1e-3 / iters
            if k_graph < k_s:
                k_s, k_timing = k_graph, f"CUDA events around one graph replay of {iters} launches over the ring"
        except Exception as e:  # noqa: BLE001
            sys.stderr.write(f"bench: graph timing of the dominant kernel failed ({e!r}); keeping the host-launched figure\n")
            try:
                torch.cuda.synchronize()
            except Exception:  # noqa: BLE001  (the figures measured so far are still reported)
                pass

    # the sampler ran from the start of the device-resident timed region through the end-to-end and
    # kernel-alone timed regions: the device-resident one alone lasts ~10 ms, one nvidia-smi period
    clocks = sampler.stop() if rank == 0 else None
    kernel_family = kname.last_kernel()
    tensor_bound = M >= 128
    if wl["kind"] == "stack":   # decided by the dominant layer's own arithmetic intensity
        tensor_bound = k_flops / (peaks["tc_sustained"] * 1e12) > k_bytes / (peaks["hbm"] * 1e9)
    if tensor_bound:
        # the kernel is timed alone, in bursts of a few milliseconds: the burst figure of the measured peaks is its denominator
        roof = {"bound": "tensor", "achieved": k_flops / k_s / 1e12 if k_s else None, "peak": peaks["tc_burst"],
                "unit": "TFLOP/s", "peak_sustained": peaks["tc_sustained"]}
    else:
        roof = {"bound": "hbm", "achieved": k_bytes / k_s / 1e9 if k_s else None, "peak": peaks["hbm"], "unit": "GB/s"}
    roof["frac"] = roof["achieved"] / roof["peak"] if k_s else None
    roof.update({"traffic": KNOWN_TRAFFIC.get((args.workload, kernel_family, world)), "kernel": kernel_family,
                 "kernel_us": k_s * 1e6 if k_s else None, "peaks": peaks["source"], "timing": k_timing,
                 "algorithmic": (k_flops if tensor_bound else k_bytes)})
    if k_error:
        roof["error"] = k_error

    out = {
        "metric": "quantized_linear_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
        "scaling": "weak" if replicas else "strong", "vs_baseline": None, "dtype": ("f32" if wl["kind"] == "stack" else "bf16") + " x int8 -> f32 accumulate", "data": "synthetic",
        "config": config_line(args, wl, args.workload),
        "notes": {"sharding": "none (single GPU)" if world == 1 else f"none: {world} independent replicas, each on its own batch of {M} rows, no collective" if replicas else f"output channels over {world} GPUs, " + ("all-gather fused into the kernel epilogue (peer stores) + the library's bounded device barrier" if fused else "NCCL all-gather"),
                  "l2": f"ring of {ring} weight copies ({ring * shard_bytes / 1e6:.0f} MB per GPU)" + (" > 2x L2" if ring * shard_bytes > 2 * L2_BYTES else "; the whole configuration is smaller than L2, so the weights stay L2-resident as they would in use")},
        "tflops": flops_step * (world if replicas else 1) * args.steps / (ms_total * 1e-3) / 1e12,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": x_host.numel() * x_host.element_size() * (world if replicas else 1),
                "d2h_bytes_per_step": y_host.numel() * y_host.element_size() * (world if replicas else 1), **e2e_info},
        "gpu_launches": int(launches), "launch_mode": ("cuda graph replay (the K timed steps as one graph)" if timed_graph is not None else "cuda graph replay (one graph per ring entry)") if use_graphs else "host launches", "clocks": clocks, "roofline": roof,
    }
    if parity is not None:
        out["parity_checked"] = parity
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cstep, tokens, sample = cpu_step_factory(wl, args.granularity == "per_tensor")
        cstep()
        t0 = time.perf_counter()
        n_cpu = 0
        while n_cpu < 3 or (time.perf_counter() - t0 < 10 and n_cpu < 20):
            cstep()
            n_cpu += 1
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": tokens * n_cpu / dt, "unit": "tokens/s", "cores": torch.get_num_threads(),
                               "kind": "port", "sample": f"{n_cpu} x " + sample}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        # Every rank has its result; leave together and at once.  Collectives and symmetric-memory
        # buffers captured in CUDA graphs have kept ranks from ending in interpreter teardown on this
        # software stack (results printed, processes never exited), so after a last barrier the ranks
        # skip that teardown; the driver reclaims the context with the process.
        rc = 0
        try:
            torch.cuda.synchronize()
            dist.barrier()
        except Exception as e:  # noqa: BLE001  (the result line is out already; say what happened and leave)
            sys.stderr.write(f"bench: final barrier failed ({e!r})\n")
            rc = 1
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(rc)
    return 0


if __name__ == "__main__":
    sys.exit(main())
