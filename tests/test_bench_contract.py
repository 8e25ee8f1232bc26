"""CPU: the benchmark's reference arm prints the contract's JSON line, and the GPU arm refuses to run
without a CUDA device instead of falling back to anything."""
import json
import os
import subprocess
import sys

from tests.conftest import ROOT


def _run(*args):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, cwd=ROOT,
                          env=env, timeout=600)


def test_reference_arm_prints_the_contract_line():
    r = _run("--impl", "reference", "--steps", "1", "--warmup", "1", "--workload", "linear4096_m1")
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["metric"] == "quantized_linear_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["config"]["workload"] == "linear4096_m1"
    assert line["cpu_baseline"]["kind"] in ("port", "reference") and line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["warmup"] >= 3 and line["value"] > 0


def test_gpu_arm_has_no_cpu_fallback():
    r = _run("--steps", "1", "--warmup", "1")
    assert r.returncode != 0
    assert "no CUDA device" in (r.stderr + r.stdout)


def test_reference_arm_runs_the_small_mlp_of_config_1():
    r = _run("--impl", "reference", "--steps", "2", "--warmup", "1", "--workload", "mnist_mlp_m64")
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["config"]["workload"] == "mnist_mlp_m64" and line["config"]["activations"] == "f32"
    assert line["config"]["layers"].startswith("2 Linears") and line["value"] > 0


def test_stack_workloads_are_well_formed():
    sys.path.insert(0, ROOT)
    import bench
    for name, wl in bench.WORKLOADS.items():
        json.dumps(bench.config_of(wl))
        if wl["kind"] != "stack":
            continue
        layers = bench.stack_layers(wl)
        assert all(n > 0 and k > 0 for n, k, _, _ in layers)
        if wl["chain"]:   # each layer reads the previous one's output
            assert all(layers[i][1] == layers[i - 1][0] for i in range(1, len(layers))), name
    # config 2: 4 blocks of (4 x 256->256, 256->1024, 1024->256) and the 256->50257 head: 16,011,520 codes
    assert sum(n * k for n, k, _, _ in bench.stack_layers(bench.WORKLOADS["tinygpt_stack_m4096"])) == 16011520


def test_clock_summary_takes_the_median_of_the_samples_under_load():
    sys.path.insert(0, ROOT)
    import bench
    c = bench.ClockSampler(0)
    c.proc = type("P", (), {"terminate": lambda s: None, "wait": lambda s, timeout=0: None})()
    idle = ["0", "1965", "1965", "300.0", "0x0", "Not Active", "Not Active", "Not Active", "Not Active", "0"]
    busy = lambda mhz: ["0", str(mhz), "1965", "950.0", "0x4", "Not Active", "Not Active", "Not Active", "Active", "98"]  # noqa: E731
    c.rows = [idle, busy(1500), busy(1400), busy(1300), ["cut off"]]
    out = c.stop()
    assert out == {"sm_mhz": 1400.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3, "samples_all": 4}
    c.rows = [idle[:9] + ["[N/A]"]]      # no utilisation reported: every sample counts
    assert c.stop()["sm_mhz"] == 1965.0


def test_stack_forward_routes_inputs_and_buffers():
    # the routing of the stack workloads' step, with stand-in layers on CPU tensors
    sys.path.insert(0, ROOT)
    import torch

    import bench

    class FakeLinear:
        def __init__(self, n, k, seed):
            self.w = torch.randn(n, k, generator=torch.Generator().manual_seed(seed))

        def forward(self, src, epilogue=0, out=None):
            y = src @ self.w.t()
            out.copy_(torch.relu(y) if epilogue == 1 else y)
            return out

    M = 5
    # config 1: chained, ReLU after the first layer
    spec = bench.stack_layers(bench.WORKLOADS["mnist_mlp_m64"])
    lins = [FakeLinear(n, k, i) for i, (n, k, _, _) in enumerate(spec)]
    bufs = [torch.empty(M, n) for n, _, _, _ in spec]
    x = torch.rand(M, spec[0][1])
    y = bench.stack_forward(x, lins, spec, bufs, {}, True)
    want = torch.relu(x @ lins[0].w.t()) @ lins[1].w.t()
    assert y is bufs[-1] and torch.allclose(y, want, atol=1e-5)
    # config 2 (one block and a small head): 256-wide layers read x, the 1024-wide one its stand-in
    spec = [(256, 256, False, False)] * 4 + [(1024, 256, False, True), (256, 1024, False, True), (300, 256, False, False)]
    lins = [FakeLinear(n, k, i) for i, (n, k, _, _) in enumerate(spec)]
    bufs = [torch.empty(M, n) for n, _, _, _ in spec]
    x, s1024 = torch.randn(M, 256), torch.randn(M, 1024)
    y = bench.stack_forward(x, lins, spec, bufs, {256: torch.zeros(M, 256), 1024: s1024}, False)
    assert y is bufs[-1] and torch.allclose(y, x @ lins[-1].w.t(), atol=1e-4)
    assert torch.allclose(bufs[5], s1024 @ lins[5].w.t(), atol=1e-3) and torch.allclose(bufs[4], x @ lins[4].w.t(), atol=1e-4)


def test_reference_arm_of_a_quantize_workload_reports_bandwidth():
    r = _run("--impl", "reference", "--steps", "1", "--warmup", "1", "--workload", "quantize_1024x1024")
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["metric"] == "quantize_gb_per_s" and line["unit"] == "GB/s" and line["value"] > 0
    assert line["cpu_baseline"]["cores"] == 1 and line["config"]["rows"] == 1024


def test_reference_arm_under_torchrun_prints_one_line_from_rank_0():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", "29917", os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                        "--steps", "1", "--warmup", "1", "--workload", "mnist_mlp_m64"], capture_output=True, text=True, cwd=ROOT,
                       env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 2
