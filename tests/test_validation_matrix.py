"""CPU: the validation matrix (tests/validation_matrix.py) names things that exist — every row selects at least one GPU
test, every timing recipe names a setting of `kernel_bench mlp` and a row of the matrix — so that a GPU session is not
spent discovering a typo."""
import importlib.util
import os
import re
import subprocess
import sys

from tests.conftest import ROOT


def _load():
    spec = importlib.util.spec_from_file_location("validation_matrix", os.path.join(ROOT, "tests", "validation_matrix.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_timing_recipes_name_settings_and_rows_that_exist():
    vm = _load()
    from shrew_b200 import kernel_bench
    settings = {name for name, _ in kernel_bench.MLP_SETTINGS}
    rows = {m[0] for m in vm.MATRIX}
    assert len(rows) == len(vm.MATRIX)
    for row, recipes in vm.BENCH.items():
        assert row in rows, row
        for batches, setting, shards in recipes:
            assert setting in settings, setting
            assert all(int(b) > 0 for b in batches.split(",")) and int(shards) >= 1


def test_environment_switches_of_the_matrix_are_read_somewhere():
    vm = _load()
    text = ""
    for d in ("shrew_b200", os.path.join("shrew_b200", "csrc"), "tests"):
        for f in os.listdir(os.path.join(ROOT, d)):
            if f.endswith((".py", ".cu", ".cuh")) and f != "validation_matrix.py" and f != "test_validation_matrix.py":
                text += open(os.path.join(ROOT, d, f), errors="replace").read()
    for _, env, _ in vm.MATRIX:
        for var in env:
            assert re.search(r'"%s"' % var, text), var


def test_every_row_selects_gpu_tests():
    from concurrent.futures import ThreadPoolExecutor
    vm = _load()

    def count(args):
        r = subprocess.run([sys.executable, "-m", "pytest", *args, "-m", "gpu", "--collect-only", "-q", "-p", "no:cacheprovider"],
                           cwd=ROOT, capture_output=True, text=True, timeout=600)
        m = re.search(r"(\d+)(?:/\d+)? tests? collected", r.stdout)
        return int(m.group(1)) if m else 0

    keys = sorted({tuple(args) for _, _, args in vm.MATRIX})
    with ThreadPoolExecutor(max_workers=8) as ex:
        counts = dict(zip(keys, ex.map(count, keys)))
    for name, _, args in vm.MATRIX:
        assert counts[tuple(args)] > 0, (name, args)
