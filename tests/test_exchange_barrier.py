"""CPU: the device barrier between GPUs (shrew_b200/csrc/exchange_kernels.cuh) run as host threads.

Every rank is a thread that writes a payload into all ranks' buffers, launches the barrier kernel and then
reads what its peers wrote: after barrier number k it must see payload k from everyone.  A rank that never
shows up must make the others' waits run out with the status block naming it, and the kernel must return
(no hang): the failure is injected on the host, nothing faults."""
import ctypes
import os
import subprocess

import pytest

from tests.conftest import ROOT

EMU_DIR = os.path.join(ROOT, "tests", "cpu_emu")
BUILD_DIR = os.path.join(EMU_DIR, "_build")


class Status(ctypes.Structure):
    _fields_ = [("timeout_flag", ctypes.c_uint), ("where", ctypes.c_uint), ("stage", ctypes.c_uint), ("parity", ctypes.c_uint)]


def _build(short_waits):
    os.makedirs(BUILD_DIR, exist_ok=True)
    src = os.path.join(EMU_DIR, "emu_exchange.cpp")
    out = os.path.join(BUILD_DIR, "libemu_exchange" + ("_short_waits" if short_waits else "") + ".so")
    deps = [src, os.path.join(EMU_DIR, "cuda_shim.h"), os.path.join(ROOT, "shrew_b200", "csrc", "exchange_kernels.cuh"),
            os.path.join(ROOT, "shrew_b200", "csrc", "ptx_small.cuh")]
    if not os.path.exists(out) or any(os.path.getmtime(d) > os.path.getmtime(out) for d in deps):
        extra = ["-DSHREWQ_EXCHANGE_FAST_POLLS=64", "-DSHREWQ_EXCHANGE_SLOW_POLLS=2000"] if short_waits else []
        subprocess.run(["g++", "-std=c++20", "-O1", "-pthread", "-fPIC", "-shared", "-Wno-unknown-pragmas", *extra, "-o", out, src],
                       check=True, cwd=EMU_DIR)
    L = ctypes.CDLL(out)
    L.emu_exchange_run.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                   ctypes.POINTER(Status)]
    return L


def _run(L, world, rounds, absent=(), delays=None):
    ab = (ctypes.c_int * world)(*[1 if r in absent else 0 for r in range(world)])
    dl = (ctypes.c_int * world)(*(delays or [0] * world))
    st = (Status * world)()
    return L.emu_exchange_run(world, rounds, ab, dl, st), st


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.timeout(300)
def test_every_rank_sees_its_peers_writes_after_the_barrier(world):
    L = _build(short_waits=False)
    rc, st = _run(L, world, 40)
    assert rc == 0
    # ranks that arrive out of step (one slow rank, one fast) still agree
    rc, st = _run(L, world, 12, delays=[(300 if r == world - 1 else 0) for r in range(world)])
    assert rc == 0


@pytest.mark.parametrize("world,missing", [(2, 1), (4, 2), (8, 0)])
@pytest.mark.timeout(300)
def test_a_rank_that_never_arrives_ends_the_wait_with_a_status(world, missing):
    L = _build(short_waits=True)
    rc, st = _run(L, world, 3, absent=(missing,))
    assert rc == 2
    for r in range(world):
        if r == missing:
            assert st[r].timeout_flag == 0
            continue
        assert st[r].timeout_flag == 3                       # the exchange's code
        assert st[r].where >> 8 == r and st[r].where & 0xFF == missing
        assert st[r].stage == 1                              # gave up at the first barrier
