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


def quantize_row_shard(w_shard: torch.Tensor, config, group=None, *, quantize=None, absmax=None, quantize_given_amax=None):
    """Quantizes this rank's row shard so that the result equals the matching rows of the
    unsplit tensor's quantization, bit for bit.  Per-channel: the shard alone decides
    (crates/shrew/src/quantize.rs:289-308).  Per-tensor: the scale is amax / 127 of the WHOLE tensor
    (quantize.rs:349-351), so the ranks first reduce their local amax with MAX — one f32 through an
    all-reduce, the only collective of the quantize path — and then quantize with the global value.
    The three callables default to the library's kernels; the CPU tests pass stand-ins."""
    from . import quantize as qz
    quantize = quantize or qz.quantize_tensor
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if config.granularity is qz.QuantGranularity.PerChannel or world == 1 or w_shard.dim() == 0:
        return quantize(w_shard, config)
    if not config._is_int8_symmetric():
        raise qz.ShrewError(qz._lib.ERR_UNSUPPORTED, "sharded per-tensor quantization is built for INT8 symmetric only")
    amax = (absmax or qz.absmax)(w_shard)
    dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    return (quantize_given_amax or qz.quantize_tensor_given_amax)(w_shard, amax)


def shard_quantized_linear(weight: torch.Tensor, bias: Optional[torch.Tensor], config, group=None) -> ShardedLinear:
    """Quantizes this rank's rows of `weight` [N,K] on its GPU (`quantize_row_shard`) and wraps the shard."""
    from .quantize import QuantizedLinear
    n = weight.shape[0]
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    n0, n1 = plan_shards(n, world).rows(rank)
    b = None if bias is None else bias.reshape(1, -1)[:, n0:n1].contiguous()
    ql = QuantizedLinear.new(quantize_row_shard(weight[n0:n1].contiguous().detach(), config, group), b)

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


# ---- all-gather fused into the kernel epilogue (peer stores over NVLink) ------------------
class PeerOutput:
    """The full [m_max, n] output of a sharded layer, allocated as symmetric memory so that
    every rank holds a mapping of every other rank's copy.  A shard's kernel stores its
    column slice into all copies itself; `barrier()` (the library's device-side exchange barrier on the
    current stream: shrewq_exchange_barrier, bounded waits, SHREWQ_ERR_TIMEOUT at the next synchronize
    if a peer never arrives) then makes the whole matrix readable everywhere."""

    def __init__(self, m_max: int, n: int, dtype: torch.dtype, device, group=None):
        import ctypes
        import os

        # nothing here uses multimem: keep the buffers off NVLink multicast objects where torch lets us
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm

        from . import _lib
        from .quantize import Device
        self.group = group if group is not None else dist.group.WORLD
        self.buf = symm.empty((m_max, n), dtype=dtype, device=device)
        self.hdl = symm.rendezvous(self.buf, self.group)
        self.rank, self.world = self.hdl.rank, self.hdl.world_size
        self.n = n
        self.esize = self.buf.element_size()
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        # the exchange barrier's flag block: zeroed by its owner before any rank's first barrier
        self.flags = symm.empty((_lib.EXCHANGE_FLAG_BYTES // 4,), dtype=torch.int32, device=device)
        self.flags.zero_()
        self.flag_hdl = symm.rendezvous(self.flags, self.group)
        torch.cuda.synchronize(device)
        dist.barrier(self.group)
        self.dev = Device.get(device)
        blocks = (ctypes.c_void_p * self.world)(*[int(p) for p in self.flag_hdl.buffer_ptrs])
        h = ctypes.c_void_p()
        _lib.check(_lib.lib().shrewq_exchange_create(self.dev.handle, self.rank, self.world, blocks, ctypes.byref(h)),
                   self.dev.handle)
        self._ex = h

    def slice_ptrs(self, n0: int):
        """(own pointer, [peer pointers]) of element [0, n0] in every copy."""
        off = n0 * self.esize
        own = self.ptrs[self.rank] + off
        return own, [p + off for r, p in enumerate(self.ptrs) if r != self.rank]

    def barrier(self):
        from . import _lib
        self.dev.bind_stream()
        _lib.check(_lib.lib().shrewq_exchange_barrier(self._ex), self.dev.handle)

    def __del__(self):
        try:
            from . import _lib
            if getattr(self, "_ex", None):
                _lib.lib().shrewq_exchange_destroy(self._ex)
                self._ex = None
        except Exception:
            pass


class FusedShardedLinear:
    """Row shard of a quantized Linear whose forward writes y[:, n0:n1] into every rank's
    output buffer from the kernel epilogue (shrewq_linear_forward_peers)."""

    def __init__(self, n: int, shard, up_shard, m_max: int, dtype: torch.dtype, group=None, out=None):
        import ctypes
        self.plan = plan_shards(n, dist.get_world_size(group))
        self.rank = dist.get_rank(group)
        self.n0, self.n1 = self.plan.rows(self.rank)
        self.shard, self.up = shard, up_shard
        # `out` lets several layers of the same shape share one symmetric buffer
        self.out = out if out is not None else PeerOutput(m_max, n, dtype, shard.weight_q.data.device, group)
        own, peers = self.out.slice_ptrs(self.n0)
        self._own = ctypes.c_void_p(own)
        self._peers = (ctypes.c_void_p * max(1, len(peers)))(*peers)
        self._n_peers = len(peers)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from . import _lib
        from .quantize import _DTYPE_CODE, _ptr
        m = x.shape[0]
        if m > self.out.buf.shape[0]:
            raise ValueError("FusedShardedLinear: batch larger than the symmetric output buffer")
        x = x.contiguous()
        dev = self.shard.device
        dev.bind_stream()
        if self.n1 > self.n0:
            rc = _lib.lib().shrewq_linear_forward_peers(
                self.shard._h, self.up._h if self.up is not None else None, _ptr(x), _DTYPE_CODE[x.dtype], m,
                self._own, self._peers, self._n_peers, _DTYPE_CODE[self.out.buf.dtype], self.out.n, _lib.EPILOGUE_NONE)
            _lib.check(rc, dev.handle)
        self.out.barrier()
        return self.out.buf[:m]


class FusedShardedGatedMLP:
    """The gated MLP block with both all-gathers fused into the kernels: gate/up shard ->
    peer stores of h -> barrier -> down shard -> peer stores of y -> barrier."""

    def __init__(self, gate, up, down, n_hidden: int, n_out: int, m_max: int, dtype=torch.bfloat16, group=None,
                 share=None):
        self.hidden = FusedShardedLinear(n_hidden, gate, up, m_max, dtype, group,
                                         out=None if share is None else share.hidden.out)
        self.out = FusedShardedLinear(n_out, down, None, m_max, dtype, group,
                                      out=None if share is None else share.out.out)
        self.gate, self.up, self.down = gate, up, down

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.out.forward(self.hidden.forward(x))
