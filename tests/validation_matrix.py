"""Runs the GPU parity tests once per prepared, opt-in code path, each in a process of its own.

    python tests/validation_matrix.py [--only NAME[,NAME...]] [--list] [--timeout SECONDS] [--json PATH] [--bench]

The library's default paths are covered by `python -m pytest tests -m gpu`.  The paths that are built and
checked on the CPU model but switched off until they have passed on a GPU (environment switches, forced
kernel families, tests behind SHREWQ_TEST_UNVALIDATED=1) are listed below, safest first.  Every entry runs
as a separate pytest process, so a failure in one leaves the others standing; the run STOPS at the first
entry whose output shows a CUDA fault or a kernel that gave up a bounded wait, because whatever runs next on
that GPU would not be trustworthy, and the faulting path has to be read before it runs again.  Prints one
line per entry and, with --json, writes the same as a list of records.  With --bench every entry that PASSED and has
a timing recipe below is then timed (`python -m shrew_b200.kernel_bench mlp ...`, a process each; the benchmark's MLP
block at batch 512 and 1, plus one rank's kernels of the block sharded over 4 GPUs where sharding is what the setting is
for), so one GPU session yields both the verdict and the numbers to choose defaults by; the JSON lines go into the
record's "bench" list.

Not in the list on purpose: f16 weights beside bf16 activations in tensor memory (SHREWQ_TC_A_F16=1).  An earlier
implementation of that operand mix failed with a CUDA error on every launch, in three runs; the cause was never
established, so the path stays off the GPU until it is (its parity test has a switch of its own, SHREWQ_TEST_AF16=1).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIN = "tests/test_gpu_linear.py"

# (name, environment, pytest arguments)
MATRIX = [
    ("default", {}, ["tests"]),
    ("gemv-pdl", {"SHREWQ_GEMV_PDL": "1"}, [LIN, "-k", "gemv or config3 or config4"]),
    ("host-forward", {"SHREWQ_TEST_UNVALIDATED": "1"}, [LIN, "-k", "host_buffers"]),
    ("batch-quantize", {"SHREWQ_TEST_UNVALIDATED": "1", "SHREWQ_BATCH_QUANTIZE": "1"}, ["tests/test_gpu_quantize.py"]),
    ("shard-per-tensor", {"SHREWQ_TEST_UNVALIDATED": "1"}, ["tests/test_gpu_quantize.py", "-k", "row_shards"]),
    ("splitk-large-tiles", {"SHREWQ_TC_SPLITK_MAXTOK": "256"}, [LIN]),
    ("split-by-waves", {"SHREWQ_TC_SPLIT_WAVES": "1", "SHREWQ_TC_SPLITK_MAXTOK": "256"}, [LIN]),
    ("gated-tile-256", {"SHREWQ_TC_TOK_GATED": "256"}, [LIN, "-k", "config4 or gate"]),
    ("tile-cost-rule", {"SHREWQ_TC_TILE_RULE": "cost"}, [LIN]),
    ("tile-256-tail-split", {"SHREWQ_TC_TOK": "256", "SHREWQ_TC_TAILSPLIT": "1"}, [LIN, "-k", "config4 or config3"]),
    ("mma-bf16", {"SHREWQ_TEST_UNVALIDATED": "1"}, [LIN, "-k", "mma and not f16"]),
    ("mma-f16", {"SHREWQ_TEST_UNVALIDATED": "1"}, [LIN, "-k", "mma_f16 or mma_gated"]),
    ("mma-f16-auto", {"SHREWQ_AUTO_MMA_F16": "1", "SHREWQ_GEMV_PDL": "1"}, [LIN, "tests/test_zz_no_alloc.py"]),
    ("f32-on-tensor-cores", {"SHREWQ_TEST_UNVALIDATED": "1"}, [LIN, "-k", "f32_activations_on_tensor or config2"]),
    ("f32-on-tensor-cores-auto", {"SHREWQ_AUTO_TC_F32": "1"}, [LIN]),
    ("other-modes", {"SHREWQ_TEST_UNVALIDATED": "1"}, ["tests/test_gpu_modes.py"]),
    ("cta-pair", {"SHREWQ_TEST_UNVALIDATED": "1"}, [LIN, "-k", "cta_pair"]),
    ("cta-pair-auto", {"SHREWQ_AUTO_PAIR": "1"}, [LIN]),
    ("cta-pair-auto-tail", {"SHREWQ_AUTO_PAIR": "1", "SHREWQ_TC_TAILSPLIT": "1"}, [LIN, "-k", "config4 or config3"]),
]

# entry name -> arguments of `python -m shrew_b200.kernel_bench mlp` runs that time it (batches, setting, shards)
BENCH = {
    "default": [("512,16,1", "default", "1"), ("512", "default", "4")],
    "gemv-pdl": [("1", "pdl", "1")],
    "splitk-large-tiles": [("512", "split-large", "1"), ("512", "split-large", "4"), ("512", "split-large", "8")],
    "split-by-waves": [("512", "waves+maxtok", "1"), ("512", "waves+maxtok", "4")],
    "gated-tile-256": [("512", "gated256", "1")],
    "tile-cost-rule": [("512", "cost-rule", "1")],
    "tile-256-tail-split": [("512", "tok256+tail", "1")],
    "mma-f16-auto": [("16,1", "mma-f16+pdl", "1")],
    "cta-pair-auto": [("512", "pair", "1")],
    "cta-pair-auto-tail": [("512", "pair+tail", "1")],
}

# what in a test run's output means the GPU, or the context, can no longer be trusted
FAULT_MARKS = ("illegal memory access", "illegal instruction", "unspecified launch failure", "misaligned address",
               "device-side assert", "Xid", "gave up a bounded wait", "CUDA error: an illegal", "launch timed out")


def run_entry(name, env, args, timeout):
    cmd = [sys.executable, "-m", "pytest", *args, "-m", "gpu", "-q", "-x", "-p", "no:cacheprovider"]
    t0 = time.time()
    try:
        r = subprocess.run(cmd, cwd=ROOT, env=dict(os.environ, **env), capture_output=True, text=True, timeout=timeout)
        out, rc = r.stdout + r.stderr, r.returncode
    except subprocess.TimeoutExpired as e:
        out = ((e.stdout or b"").decode(errors="replace") if isinstance(e.stdout, bytes) else (e.stdout or "")) + "\n[timed out]"
        rc = 124
    lines = [l for l in out.strip().splitlines() if l.strip()]
    fault = next((m for m in FAULT_MARKS if m in out), None)
    if rc == 124:
        fault = fault or "timed out"
    return {"name": name, "env": env, "args": args, "rc": rc, "seconds": round(time.time() - t0, 1),
            "summary": lines[-1] if lines else "", "fault": fault,
            "tail": lines[-25:] if rc not in (0, 5) else []}      # pytest's 5 = nothing selected


def run_bench(name, timeout):
    """The timing recipes of a passed entry; returns (records, fault)."""
    out, fault = [], None
    for batches, setting, shards in BENCH.get(name, []):
        cmd = [sys.executable, "-m", "shrew_b200.kernel_bench", "mlp", batches, setting, shards]
        try:
            r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=timeout)
            text = r.stdout + r.stderr
        except subprocess.TimeoutExpired:
            text, fault = "", "timed out"
        for l in text.splitlines():
            if l.startswith("{"):
                try:
                    out.append(json.loads(l))
                except ValueError:
                    pass
        fault = fault or next((m for m in FAULT_MARKS if m in text), None)
        if fault:
            break
    return out, fault


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--timeout", type=int, default=900, help="seconds per entry")
    ap.add_argument("--json", default="")
    ap.add_argument("--bench", action="store_true", help="time every entry that passed (kernel_bench mlp, a process each)")
    a = ap.parse_args()
    names = [n for n in a.only.split(",") if n]
    unknown = [n for n in names if n not in {m[0] for m in MATRIX}]
    if unknown:
        raise SystemExit(f"unknown entries: {unknown}")
    by_name = {m[0]: m for m in MATRIX}
    todo = [by_name[n] for n in names] if names else list(MATRIX)     # --only keeps the order given
    if a.list:
        for name, env, args in todo:
            print(name, " ".join(f"{k}={v}" for k, v in env.items()), "::", " ".join(args))
        return 0
    records = []
    for name, env, args in todo:
        rec = run_entry(name, env, args, a.timeout)
        records.append(rec)
        print(f"{name:28s} rc={rec['rc']:<3d} {rec['seconds']:7.1f}s  {rec['summary']}", flush=True)
        for l in rec["tail"]:
            print("    | " + l, flush=True)
        if a.bench and rec["rc"] == 0 and not rec["fault"] and name in BENCH:
            rec["bench"], rec["fault"] = run_bench(name, a.timeout)
            for b in rec["bench"]:
                print("    # " + json.dumps(b), flush=True)
        if a.json:
            with open(a.json, "w") as f:
                json.dump(records, f, indent=1)
        if rec["fault"]:
            print(f"stopping: '{rec['fault']}' in the output of {name}; read that path before running anything else on this GPU",
                  flush=True)
            return 3
    return 0 if all(r["rc"] in (0, 5) for r in records) else 1


if __name__ == "__main__":
    sys.exit(main())
