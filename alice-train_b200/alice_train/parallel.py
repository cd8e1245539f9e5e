"""Partitioning of the BitLinear path across the GPUs of one box (one process per GPU).

The reference has no multi-GPU code at all (single CudaContext::new(0), src/cuda_matmul.rs:954);
the two partitionings here are the ones the target specification names:

  * data parallel over tokens: forward and dx are independent per token; dW = dy^T.x is a sum
    over tokens, so the only exchange is one all-reduce(sum) of dW per projection;
  * output-row shards of W: forward and dW are independent per row; gamma needs the global
    sum |w| (one f64 all-reduce of 8 bytes) and dx is a sum over row shards (all-reduce or
    reduce-scatter of [tokens x in]).

torch.distributed is the plumbing (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def token_shard(tokens: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced split of `tokens` (earlier ranks take the remainder)."""
    base, rem = divmod(tokens, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def row_shard(out_features: int, world: int, rank: int, align: int = 1) -> tuple[int, int]:
    """Contiguous split of W's output rows in multiples of `align` (last rank takes the tail)."""
    blocks = (out_features + align - 1) // align
    b0, b1 = token_shard(blocks, world, rank)
    return min(b0 * align, out_features), min(b1 * align, out_features)


class DwAllReducer:
    """One asynchronous all-reduce(sum) per projection, issued as soon as its dW is ready and
    waited for at the end of the step, so the exchange overlaps the remaining GEMMs."""

    def __init__(self, group=None):
        self.group = group
        self._pending = []

    def submit(self, dW: torch.Tensor):
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            self._pending.append(dist.all_reduce(dW, op=dist.ReduceOp.SUM, group=self.group, async_op=True))

    def wait(self):
        for h in self._pending:
            h.wait()
        self._pending.clear()


class SwitchBuffer:
    """A buffer in symmetric memory (every GPU of the group maps its own copy and the group's NVSwitch multicast
    address) plus the 16 bytes of barrier counters the library's exchange kernels need.  torch's symmetric-memory
    allocator provides the mapping; the transfers and the inter-GPU barriers are in the CUDA library
    (ab_switch_exchange_start / ab_dp_allreduce_wait).  Construction is collective: every rank, same sizes."""

    FLAG_BYTES = 256

    def __init__(self, ctx, nbytes: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        from . import _ffi
        self._ffi, self.ctx = _ffi, ctx
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world < 2:
            raise ValueError("a SwitchBuffer needs at least two GPUs")
        unit = 16 * self.world
        self.nbytes = (nbytes + unit - 1) // unit * unit
        self._t = symm_mem.empty(self.nbytes + self.FLAG_BYTES, dtype=torch.uint8, device=device)
        self._hdl = symm_mem.rendezvous(self._t, self.group)
        if not self._hdl.multicast_ptr:
            raise RuntimeError("this group of GPUs has no NVSwitch multicast mapping")
        self._t[nbytes:].zero_()  # padding and the barrier counters
        self._mc = self._hdl.multicast_ptr + (self._t.data_ptr() - self._hdl.buffer_ptrs[self._hdl.rank])
        self._epoch = 0
        self.bytes = self._t[:nbytes]

    def view(self, dtype, shape):
        """The buffer's first prod(shape) elements as a tensor of `dtype` (the local copy)."""
        n = 1
        for d in shape:
            n *= d
        return self._t[:n * torch.empty((), dtype=dtype).element_size()].view(dtype).view(shape)

    def start(self, op: int, out_local: torch.Tensor | None = None, ctas: int = 0):
        self._epoch += 1
        self._ffi.check(self._ffi.load().ab_switch_exchange_start(
            self.ctx.handle, op, self._mc, self._t.data_ptr(), out_local.data_ptr() if out_local is not None else None,
            self.nbytes, self._t.data_ptr() + self.nbytes, self._mc + self.nbytes, self.rank, self.world, self._epoch, int(ctas)),
            self.ctx.handle)

    @staticmethod
    def ready(buffers, device):
        """After constructing all buffers: make their zeroed counters visible on every GPU before the first exchange."""
        torch.cuda.synchronize(device)
        dist.barrier(buffers[0].group if buffers else None)
        torch.cuda.synchronize(device)


class SwitchArena:
    """Several exchange buffers carved out of ONE symmetric-memory allocation (one rendezvous instead of one per
    buffer): `sizes` are byte counts; buffer i occupies [offset[i], offset[i] + sizes[i]) rounded up to 256 * world
    bytes, and its 16 bytes of barrier counters sit in a block of 256-byte slots behind the data.  Construction is
    collective.  Pointers come back as plain integers for the C ABI (local, multicast, flags local, flags multicast)."""

    SLOT = 256

    def __init__(self, ctx, sizes, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.ctx = ctx
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world < 2:
            raise ValueError("a SwitchArena needs at least two GPUs")
        unit = 256 * self.world
        self.sizes = [int(b) for b in sizes]
        self.offsets, off = [], 0
        for b in self.sizes:
            self.offsets.append(off)
            off += (b + unit - 1) // unit * unit
        self.data_bytes = off
        self._t = symm_mem.empty(off + self.SLOT * len(self.sizes), dtype=torch.uint8, device=device)
        self._hdl = symm_mem.rendezvous(self._t, self.group)
        if not self._hdl.multicast_ptr:
            raise RuntimeError("this group of GPUs has no NVSwitch multicast mapping")
        self._t[off:].zero_()
        self.local_ptr = self._t.data_ptr()
        self.mc_ptr = self._hdl.multicast_ptr + (self._t.data_ptr() - self._hdl.buffer_ptrs[self._hdl.rank])
        self.epoch = 0

    def view(self, i: int, dtype, shape):
        n = 1
        for d in shape:
            n *= d
        nb = n * torch.empty((), dtype=dtype).element_size()
        assert nb <= self.sizes[i]
        return self._t[self.offsets[i]:self.offsets[i] + nb].view(dtype).view(shape)

    def pointers(self, i: int):
        """(local, multicast, flags_local, flags_multicast) of buffer i."""
        f = self.data_bytes + self.SLOT * i
        return (self.local_ptr + self.offsets[i], self.mc_ptr + self.offsets[i], self.local_ptr + f, self.mc_ptr + f)

    def reset_flags(self):
        """Zero the barrier counters and restart the epoch count (collective; call between two uses whose numbers of
        exchanges per buffer differ, or after a timed-out exchange)."""
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self._t[self.data_bytes:].zero_()
        self.epoch = 0
        torch.cuda.synchronize()
        dist.barrier(self.group)


class SwitchDwAllReducer:
    """dW buffers in symmetric memory, summed over the GPUs inside NVSwitch by the library's own kernel instead of
    NCCL: no staging copies and a handful of small CTAs per exchange, so the GEMMs that overlap it keep their SMs.

        red = SwitchDwAllReducer(ctx, [(out, inn), ...], device)   # collective: every rank, same shapes
        ste_dw(ctx, dy, x, red.dW[i], beta=0.0); red.submit(i); ...; red.wait()
    """

    def __init__(self, ctx, shapes, device, group=None, ctas: int = 0):
        import math
        from . import _ffi
        self._ffi, self.ctx, self.ctas = _ffi, ctx, int(ctas)
        self._bufs = [SwitchBuffer(ctx, 4 * math.prod(shape), device, group) for shape in shapes]
        self.world, self.rank = self._bufs[0].world, self._bufs[0].rank
        self.dW = [b.view(torch.float32, shape) for b, shape in zip(self._bufs, shapes)]
        SwitchBuffer.ready(self._bufs, device)

    def submit(self, i: int):
        self._bufs[i].start(self._ffi.AB_XCHG_ALLREDUCE_F32, ctas=self.ctas)

    def wait(self):
        self._ffi.check(self._ffi.load().ab_dp_allreduce_wait(self.ctx.handle), self.ctx.handle)


def global_gamma(sum_abs_local: torch.Tensor, n_total: int, group=None, floor: bool = False) -> torch.Tensor:
    """gamma of a row-sharded tensor: all-reduce the f64 shard sums of |w|, divide by the global
    element count, round to f32 (src/qwen35.rs:226-227).  Every rank gets the same bits."""
    assert sum_abs_local.dtype == torch.float64
    total = sum_abs_local.clone()
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(total, op=dist.ReduceOp.SUM, group=group)
    gamma = (total / float(n_total)).to(torch.float32)
    if floor:
        gamma = torch.clamp_min(gamma, 1e-10)
    return gamma


def global_abs_sum(sum_abs_local: torch.Tensor, group=None) -> torch.Tensor:
    """In-place all-reduce of the 8-byte f64 shard sums of |w| (the only exchange the row-sharded quantiser needs)."""
    assert sum_abs_local.dtype == torch.float64
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(sum_abs_local, op=dist.ReduceOp.SUM, group=group)
    return sum_abs_local


def gather_rows(y_local: torch.Tensor, group=None) -> torch.Tensor:
    """Forward of a row-sharded layer: concatenate the [tokens x out/g] shards along features."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return y_local
    parts = [torch.empty_like(y_local) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, y_local.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def reduce_dx(dx_partial: torch.Tensor, group=None) -> torch.Tensor:
    """Backward of a row-sharded layer: dx = sum over shards of dy[:, shard] . W_shard."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(dx_partial, op=dist.ReduceOp.SUM, group=group)
    return dx_partial
