"""CPU, world_size 2 over gloo: the row-shard plan and the all-gather assembly of the
multi-GPU path, with the oracle standing in for the per-rank kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from shrew_b200.sharded import ShardedLinear, assemble_gathered, plan_shards


def test_plan_covers_rows_exactly():
    for n, world in [(4096, 8), (11008, 8), (11008, 4), (50257, 8), (50257, 2), (10, 4), (3, 8), (1, 1)]:
        p = plan_shards(n, world)
        rows = [p.rows(r) for r in range(world)]
        assert rows[0][0] == 0 and max(b for _, b in rows) == n
        covered = sum(b - a for a, b in rows)
        assert covered == n
        for (a0, b0), (a1, b1) in zip(rows, rows[1:]):
            assert b0 == a1 or (a1 == n and b1 == n)
        assert all(c <= p.block for c in p.counts())
    assert plan_shards(11008, 8).counts() == [1376] * 8
    assert plan_shards(50257, 8).counts() == [6283] * 7 + [6276]


def test_assemble_gathered_layout():
    plan = plan_shards(10, 4)  # block 3: shards 3,3,3,1
    m = 5
    full = torch.arange(m * 10, dtype=torch.float32).reshape(m, 10)
    g = torch.zeros(4, m, 3)
    for r in range(4):
        a, b = plan.rows(r)
        g[r, :, :b - a] = full[:, a:b]
    assert torch.equal(assemble_gathered(g, plan), full)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n, k, m, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import shrew_oracle as oracle
        rng = np.random.default_rng(0)  # same seed on every rank: replicated inputs
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        b = rng.standard_normal(n).astype(np.float32)
        x = rng.standard_normal((m, k)).astype(np.float32)
        plan = plan_shards(n, world)
        n0, n1 = plan.rows(rank)
        # shard-local per-channel quantization is bit-identical to quantizing everything
        q_full, s_full = oracle.quantize_f32(w, oracle.PER_CHANNEL)
        q_loc, s_loc = oracle.quantize_f32(w[n0:n1], oracle.PER_CHANNEL)
        assert np.array_equal(q_loc, q_full[n0:n1]) and s_loc.tobytes() == s_full[n0:n1].tobytes()

        def local_forward(xt, out):
            y = oracle.linear_forward_f32(q_loc, s_loc, oracle.PER_CHANNEL, b[n0:n1], xt.numpy())
            out.copy_(torch.from_numpy(y))

        sl = ShardedLinear(n, local_forward)
        y = sl.forward(torch.from_numpy(x))
        ref = oracle.linear_forward_f32(q_full, s_full, oracle.PER_CHANNEL, b, x)
        ok = bool(np.array_equal(y.numpy(), ref))
        out_q.put((rank, ok, list(y.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n", [64, 37])  # even and ragged shards
def test_sharded_forward_gloo_world2(n):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n, 48, 5, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, shape in res:
        assert ok, f"rank {rank}: gathered output differs from the unsharded oracle"
        assert shape == [5, n]


# ---- per-tensor quantization of row shards: one f32 through an all-reduce(MAX) ----------------------
def _pt_worker(rank, world, port, n, k, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import shrew_oracle as oracle
        from shrew_b200.quantize import QuantConfig
        from shrew_b200.sharded import quantize_row_shard
        rng = np.random.default_rng(3)
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        w[n - 1, 0] = 0.9 if n > 1 else w[0, 0]      # the global amax sits in the LAST rank's shard
        w[0, 1] = np.nan                             # NaN is ignored by the amax on every rank
        n0, n1 = plan_shards(n, world).rows(rank)
        calls = []

        # stand-ins for the three kernels, from the oracle
        def quantize(t, cfg):
            calls.append("quantize")
            q, s = oracle.quantize_f32(t.numpy(), 1 if cfg.granularity.value == 1 else 0)
            return q, s

        def absmax(t):
            calls.append("absmax")
            a = t.numpy()
            return torch.tensor([np.fmax.reduce(np.abs(a).reshape(-1), initial=0.0)], dtype=torch.float32)

        def quantize_given_amax(t, amax):
            calls.append("given")
            # a per-tensor quantization whose amax is the supplied one: append it to the data
            aug = np.concatenate([t.numpy().reshape(-1), amax.numpy()]).astype(np.float32)
            q, s = oracle.quantize_f32(aug, oracle.PER_TENSOR)
            return q[:-1].reshape(t.shape), s

        shard = torch.from_numpy(w[n0:n1].copy())
        q_full, s_full = oracle.quantize_f32(w, oracle.PER_TENSOR)
        q, s = quantize_row_shard(shard, QuantConfig.int8(), quantize=quantize, absmax=absmax, quantize_given_amax=quantize_given_amax)
        ok_pt = bool(np.array_equal(q, q_full[n0:n1]) and s.tobytes() == s_full.tobytes()) and calls == ["absmax", "given"]
        calls.clear()
        qc_full, sc_full = oracle.quantize_f32(w, oracle.PER_CHANNEL)
        q, s = quantize_row_shard(shard, QuantConfig.int8_per_channel(), quantize=quantize, absmax=absmax,
                                  quantize_given_amax=quantize_given_amax)
        ok_pc = bool(np.array_equal(q, qc_full[n0:n1]) and s.tobytes() == sc_full[n0:n1].tobytes()) and calls == ["quantize"]
        out_q.put((rank, ok_pt, ok_pc))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n", [64, 5, 1])  # even shards, ragged shards, an empty shard on rank 1
def test_sharded_per_tensor_quantization_gloo_world2(n):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pt_worker, args=(r, 2, port, n, 24, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_pt, ok_pc in res:
        assert ok_pt, f"rank {rank}: per-tensor shard differs from the rows of the unsplit quantization"
        assert ok_pc, f"rank {rank}: per-channel shard differs"
