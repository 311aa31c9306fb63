"""A 1-D tensor sharded over the GPUs of one box, one process per GPU.

The reference has no multi-GPU path (one independent OpenCL context per device, cross-
device copy unimplemented, reference src/lib/THClTensorCopy.cpp:185-220). What it does
have is the model this module keeps: each shard is an ordinary tensor on its own device,
pointwise chains run on every shard independently, and only a whole-tensor reduction
needs an exchange. That exchange is one all-gather of one float per rank over
`torch.distributed` (NCCL on GPUs), followed by a fold in rank order, so every rank
ends up with the bit-identical global value as a device-resident point tensor and
`x:div(global_sum)` can follow without a host synchronisation.

The device side is pluggable only so that the host logic (shard bounds, gather layout,
fold order) can be exercised by CPU ranks over gloo; `CudaShardOps` is the real one.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple


def shard_bounds(n: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of rank's contiguous shard; the first n % world shards get one extra element."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


class ExchangeError(RuntimeError):
    """The exchange of the per-rank partials did not complete (a rank is absent or the transport failed)."""


class CudaShardOps:
    """Device side on a GPU: per-rank partial straight into the gather buffer, fold with a kernel."""

    def __init__(self):
        import torch
        from . import tensor as T
        self.torch, self.T = torch, T
        self.device = torch.device("cuda", torch.cuda.current_device())
        # the library enqueues on torch's current stream, so NCCL orders after its kernels
        T.setDevice(torch.cuda.current_device() + 1)
        T.setStream(torch.cuda.current_stream().cuda_stream)

    def new_buffer(self, count: int):
        buf = self.torch.zeros(count, dtype=self.torch.float32, device=self.device)
        storage = self.T.ClStorage.from_device_pointer(buf.data_ptr(), count)
        return buf, storage

    def slot(self, storage, index: int):
        """0-dim tensor over element `index` of the buffer."""
        return self.T.ClTensor(storage, index + 1, [], [])

    def local_sum_into(self, slot, x) -> None:
        slot.sum(x)          # THClTensor_sumall_gpu: one launch, result written into the buffer

    def fold(self, storage, count: int, out_slot) -> None:
        L, T = self.T.lib(), self.T
        rc = L.thb200_fold_partials(C.c_void_p(T.getStream()), 0, C.c_void_p(storage.data_ptr()), count,
                                    C.c_void_p(out_slot.data_ptr()))
        if rc:
            raise T.ClError(L.thb200_last_error().decode())


class GlobalSum:
    """sum over all shards -> the same point tensor on every rank."""

    def __init__(self, ops=None, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.ops = ops if ops is not None else CudaShardOps()
        # slots [0, world): per-rank partials in rank order; slot [world]: the folded result
        self.buf, self.storage = self.ops.new_buffer(self.world + 1)
        self.mine = self.ops.slot(self.storage, self.rank)
        self.result = self.ops.slot(self.storage, self.world)
        self.exchange = "all-gather of one float per rank (torch.distributed), fold in rank order" if self.world > 1 else "none (one GPU)"
        self.launches_per_call = 2  # whole-shard reduction (one launch: its last block folds the partials), fold of the per-GPU sums

    def __call__(self, x):
        self.ops.local_sum_into(self.mine, x)
        if self.world > 1:
            partials = self.buf[: self.world]
            mine = self.buf[self.rank: self.rank + 1]
            try:
                if self.dist.get_backend(self.group) == "nccl":
                    self.dist.all_gather_into_tensor(partials, mine, group=self.group)   # in place: mine is partials[rank]
                else:
                    self.dist.all_gather([partials[r: r + 1] for r in range(self.world)], mine.clone(), group=self.group)
            except RuntimeError as e:
                # a rank that never joins ends the collective after the process group's time limit
                raise ExchangeError(f"rank {self.rank} of {self.world}: the exchange of the partial sums did not "
                                    f"complete ({str(e).splitlines()[0][:200]})") from e
        self.ops.fold(self.storage, self.world, self.result)
        return self.result
