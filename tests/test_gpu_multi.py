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
    for p in procs:
        p.start()
    out = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, res in out:
        for k, err in res.items():
            assert err <= 1e-2, f"rank {rank} {k}: rel err {err:.3e}"
