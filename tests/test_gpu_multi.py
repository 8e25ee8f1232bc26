"""GPU, 2 ranks (needs >= 2 GPUs): the sharded Linear with NCCL all-gather and with the
all-gather fused into the kernel epilogue (peer stores), both against the oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from oracle import shrew_oracle as oracle
        from shrew_b200 import Linear, QuantConfig, QuantizedLinear
        from shrew_b200.sharded import FusedShardedLinear, plan_shards, shard_quantized_linear
        rng = np.random.default_rng(0)
        res = {}
        for (M, N, K) in [(3, 300, 512), (200, 1000, 1024)]:
            w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
            b = (rng.standard_normal(N) * 0.1).astype(np.float32)
            x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(dev).to(torch.bfloat16)
            cfg = QuantConfig.int8_per_channel()
            wt, bt = torch.from_numpy(w).to(dev), torch.from_numpy(b).to(dev)
            q_ref, s_ref = oracle.quantize_f32(w, oracle.PER_CHANNEL)
            ref = oracle.np_linear_forward(q_ref, s_ref, oracle.PER_CHANNEL, b, x.float().cpu().numpy())
            # NCCL all-gather path
            sl = shard_quantized_linear(wt, bt, cfg)
            y = sl.forward(x)
            torch.cuda.synchronize()
            res[f"nccl_{M}"] = oracle.rel_err(y.float().cpu().numpy(), ref)
            # fused peer-store path, twice (the second call reuses the symmetric buffer)
            n0, n1 = plan_shards(N, world).rows(rank)
            shard = QuantizedLinear.from_linear(Linear(wt[n0:n1].contiguous(), bt[n0:n1].contiguous()), cfg)
            fl = FusedShardedLinear(N, shard, None, 256, torch.bfloat16)
            for it in range(2):
                yf = fl.forward(x)
                torch.cuda.synchronize()
                res[f"fused_{M}_{it}"] = oracle.rel_err(yf.float().cpu().numpy(), ref)
        # the gated MLP block with both exchanges fused (the path `bench.py --gpus N` times): a small ragged shape, then
        # the benchmark's own 4096 / 11008 block at batch 512 against the oracle on a subset of the token rows
        from shrew_b200.sharded import FusedShardedGatedMLP
        for tag, dm, dff, M, rows in (("small", 512, 1408, 96, None), ("llama", 4096, 11008, 512, [0, 1, 255, 256, 300, 511])):
            ws = [(rng.standard_normal(s, dtype=np.float32) * np.float32(0.02)) for s in ((dff, dm), (dff, dm), (dm, dff))]
            x = torch.from_numpy(rng.standard_normal((M, dm)).astype(np.float32)).to(dev).to(torch.bfloat16)
            shards = []
            for wfull in ws:
                n0, n1 = plan_shards(wfull.shape[0], world).rows(rank)
                shards.append(QuantizedLinear.from_linear(Linear(torch.from_numpy(wfull[n0:n1].copy()).to(dev), None),
                                                          QuantConfig.int8_per_channel()))
            mlp = FusedShardedGatedMLP(shards[0], shards[1], shards[2], dff, dm, M)
            for it in range(2):                    # the second step reuses the symmetric buffers
                y = mlp.forward(x)
                torch.cuda.synchronize()
            from shrew_b200.quantize import Device
            Device.get(dev).synchronize()          # surfaces a barrier that gave up
            qs = [oracle.quantize_f32(wfull, oracle.PER_CHANNEL) for wfull in ws]
            xn = x.float().cpu().numpy()
            yn = y.float().cpu().numpy()
            if rows is not None:
                xn, yn = xn[rows], yn[rows]
            g = oracle.np_linear_forward(qs[0][0], qs[0][1], 1, None, xn)
            u = oracle.np_linear_forward(qs[1][0], qs[1][1], 1, None, xn)
            h = ((g / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32) * u)
            h16 = torch.from_numpy(h).to(torch.bfloat16).float().numpy()
            ref = oracle.np_linear_forward(qs[2][0], qs[2][1], 1, None, h16)
            res[f"fused_mlp_{tag}"] = oracle.rel_err(yn, ref)
        q.put((rank, res))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_linear_two_gpus():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    try:
        for p in procs:
            p.start()
        out = [q.get(timeout=600) for _ in procs]
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        # never leave a child behind on a shared GPU, whatever failed above
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=30)
            if p.is_alive():
                p.kill()
                p.join(timeout=30)
    for rank, res in out:
        for k, err in res.items():
            assert err <= 1e-2, f"rank {rank} {k}: rel err {err:.3e}"
