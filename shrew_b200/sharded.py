"""Output-channel sharding of a quantized Linear across the GPUs of one node.

The rows of W[N,K] (with their scales and bias entries) are independent, so rank r owns a
contiguous block of ceil(N/world) rows (the last block may be short).  Per-channel
quantization of a shard is bit-identical to quantizing the whole matrix
(crates/shrew/src/quantize.rs:289-308 treats each channel on its own).  Activations are
replicated; each rank computes y[:, n0:n1] and the slices are exchanged with one
all-gather over NCCL (NVLink / NVSwitch), one process per GPU.

`plan_shards` and `assemble_gathered` are pure host logic and run unchanged under the
gloo backend on CPU tensors, which is how the multi-rank path is tested without GPUs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ShardPlan:
    n: int            # full number of output channels
    world: int
    block: int        # rows per rank before the last (ceil(n / world))

    def rows(self, rank: int) -> Tuple[int, int]:
        n0 = min(rank * self.block, self.n)
        return n0, min(n0 + self.block, self.n)

    def counts(self) -> List[int]:
        return [self.rows(r)[1] - self.rows(r)[0] for r in range(self.world)]


def plan_shards(n: int, world: int) -> ShardPlan:
    if n <= 0 or world <= 0:
        raise ValueError("plan_shards: n and world must be positive")
    return ShardPlan(n, world, (n + world - 1) // world)


def assemble_gathered(gathered: torch.Tensor, plan: ShardPlan) -> torch.Tensor:
    """[world, M, block] (rank-major, short last block padded) -> [M, n] row-major."""
    world, m, block = gathered.shape
    assert world == plan.world and block == plan.block
    return gathered.permute(1, 0, 2).reshape(m, world * block)[:, :plan.n].contiguous()


def all_gather_columns(local: torch.Tensor, plan: ShardPlan, group=None) -> torch.Tensor:
    """local is this rank's [M, block] slice (padded to `block` columns if short)."""
    m = local.shape[0]
    out = torch.empty((plan.world, m, plan.block), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out.view(plan.world * m, plan.block), local.contiguous(), group=group)
    return assemble_gathered(out, plan)


class ShardedLinear:
    """A Linear whose output channels are split over the ranks of `group`.

    `local_forward(x, out)` computes this rank's slice into `out[:, :n_local]`; on GPUs it is
    QuantizedLinear.forward of the shard, in the CPU tests a stand-in."""

    def __init__(self, n: int, local_forward: Callable[[torch.Tensor, torch.Tensor], None], group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.plan = plan_shards(n, self.world)
        self.n0, self.n1 = self.plan.rows(self.rank)
        self.local_forward = local_forward

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        m = x.shape[0]
        local = torch.zeros((m, self.plan.block), dtype=out_dtype or x.dtype, device=x.device) \
            if self.n1 - self.n0 < self.plan.block else \
            torch.empty((m, self.plan.block), dtype=out_dtype or x.dtype, device=x.device)
        if self.n1 > self.n0:
            self.local_forward(x, local[:, :self.n1 - self.n0])
        if self.world == 1:
            return local[:, :self.plan.n]
        return all_gather_columns(local, self.plan, self.group)


def shard_quantized_linear(weight: torch.Tensor, bias: Optional[torch.Tensor], config, group=None) -> ShardedLinear:
    """Quantizes this rank's rows of `weight` [N,K] on its GPU and wraps the shard.
    Per-tensor granularity needs the whole tensor's amax, so every rank first takes the
    max over ranks of its local amax (one scalar all-reduce) — equivalently, quantize
    before sharding; here the per-channel case (all BASELINE multi-GPU configs) is direct."""
    from .quantize import Linear, QuantGranularity, QuantizedLinear
    if config.granularity is not QuantGranularity.PerChannel and dist.is_initialized() and dist.get_world_size(group) > 1:
        raise NotImplementedError("sharded per-tensor quantization: quantize the full tensor first, then shard the codes")
    n = weight.shape[0]
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    n0, n1 = plan_shards(n, world).rows(rank)
    b = None if bias is None else bias.reshape(-1)[n0:n1].contiguous()
    ql = QuantizedLinear.from_linear(Linear(weight[n0:n1].contiguous(), b), config)

    def local_forward(x, out, _ql=ql):
        _ql.forward(x, out=out)

    sl = ShardedLinear(n, local_forward, group)
    sl.shard = ql
    return sl


class ShardedGatedMLP:
    """h = silu(x Wg^T) * (x Wu^T), y = h Wd^T with Wg/Wu/Wd sharded by output channel:
    local gate/up -> all-gather h -> local down -> all-gather y (two gathers per block)."""

    def __init__(self, gate, up, down, n_hidden: int, n_out: int, group=None):
        # gate/up/down are this rank's QuantizedLinear shards
        self.gate, self.up, self.down = gate, up, down

        def gate_up(x, out):
            gate.forward_gate_up_silu(up, x, out=out)

        self.hidden = ShardedLinear(n_hidden, gate_up, group)
        self.out = ShardedLinear(n_out, lambda h, out: down.forward(h, out=out), group)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.out.forward(self.hidden.forward(x))
