"""A 1-D tensor sharded over the GPUs of one box, one process per GPU.

The reference has no multi-GPU path (one independent OpenCL context per device, cross-
device copy unimplemented, reference src/lib/THClTensorCopy.cpp:185-220). What it does
have is the model this module keeps: each shard is an ordinary tensor on its own device,
pointwise chains run on every shard independently, and only a whole-tensor reduction
needs an exchange. On GPUs that exchange is the library's own (`thb200_exchange_*`): the
kernel that reduces a shard stores its result straight into a cell in every GPU's memory
(plain stores over NVLink) and a one-block kernel per GPU waits, bounded, for its cells and
folds them in rank order. `exchange="nccl"` uses one all-gather of one float per rank over
`torch.distributed` and the same fold instead. Either way every rank ends up with the
bit-identical global value as a device-resident point tensor and `x:div(global_sum)` can
follow without a host synchronisation; `torch.distributed` only carries the handles once.

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

    # ---- the library's own exchange (peer stores + bounded wait) ----

    def exchange_create(self, rank: int, world: int):
        """(opaque exchange object, its 128-byte handle for the other ranks)"""
        L = self.T.lib()
        x = C.c_void_p()
        handle = C.create_string_buffer(128)
        if L.thb200_exchange_create(rank, world, C.byref(x), handle):
            raise self.T.ClError(L.thb200_last_error().decode())
        return x, handle.raw

    def exchange_connect(self, x, handles) -> None:
        L = self.T.lib()
        blob = C.create_string_buffer(b"".join(handles), 128 * len(handles))
        if L.thb200_exchange_connect(x, blob):
            raise self.T.ClError(L.thb200_last_error().decode())

    def exchange_reduce(self, x, tensor, out_slot, limit_ns: int) -> None:
        """sum of `tensor` over all ranks -> out_slot (push + fold)."""
        L, T = self.T.lib(), self.T
        n = tensor.nElement()
        need = L.thb200_reduce_all_scratch_bytes(n)
        if getattr(self, "_xscratch", None) is None or self._xscratch.size() * 4 < need:
            self._xscratch = T.ClStorage(max(need // 4, 1) + 16)
        view, keep = tensor_view(tensor)
        rc = L.thb200_exchange_reduce(C.c_void_p(T.getStream()), x, 0, C.byref(view), C.c_void_p(out_slot.data_ptr()),
                                      C.c_void_p(self._xscratch.data_ptr()), C.c_size_t(self._xscratch.size() * 4),
                                      C.c_uint64(limit_ns))
        if rc:
            raise T.ClError(L.thb200_last_error().decode())


def tensor_view(tensor):
    """thb200_tensor describing a ClTensor (0-based sizes and strides); the second value keeps the arrays alive."""
    from . import _lib
    nd = max(tensor.dim(), 1)
    size = (C.c_int64 * nd)(*tensor.size())
    stride = (C.c_int64 * nd)(*tensor.stride())
    t = _lib.thb200_tensor()
    t.data = C.cast(C.c_void_p(tensor.data_ptr()), _lib.c_float_p)
    t.ndim, t.size, t.stride = tensor.dim(), size, stride
    return t, (size, stride, tensor)


class GlobalSum:
    """sum over all shards -> the same point tensor on every rank.

    exchange: "p2p" (the library's peer-store exchange; needs device ops that offer it), "nccl" (an
    all-gather through torch.distributed) or None = "p2p" where available, else the all-gather.
    wait_limit_s bounds the device-side wait of the p2p exchange for a rank that is absent or late.
    """

    def __init__(self, ops=None, group=None, exchange: Optional[str] = None, wait_limit_s: float = 10.0):
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
        self.limit_ns = int(wait_limit_s * 1e9)
        self.x = None
        can_p2p = self.world > 1 and hasattr(self.ops, "exchange_create")
        if exchange == "p2p" and not can_p2p:
            raise ValueError("the p2p exchange needs more than one rank and device ops that provide it")
        self.why_not_p2p = None
        if can_p2p and exchange in (None, "p2p"):
            try:
                self.x, handle = self.ops.exchange_create(self.rank, self.world)
                handles = [None] * self.world
                dist.all_gather_object(handles, handle, group=group)       # host side, once
                self.ops.exchange_connect(self.x, handles)
                ok = 1
            except Exception as e:                                          # e.g. no peer access between the GPUs
                self.why_not_p2p = str(e).splitlines()[0][:200]
                ok = 0
            # every rank must take the same path
            flags = [None] * self.world
            dist.all_gather_object(flags, ok, group=group)
            if not all(flags):
                if exchange == "p2p":
                    raise ExchangeError(f"rank {self.rank}: the p2p exchange could not be set up on every rank ({self.why_not_p2p})")
                self.x = None
        if self.world == 1:
            self.exchange = "none (one GPU)"
            self.launches_per_call = 2   # whole-shard reduction (one launch), fold of the one value
        elif self.x is not None:
            self.exchange = "p2p: the reduction kernel stores its result into a cell on every GPU, a one-block kernel waits (bounded) and folds in rank order"
            self.launches_per_call = 2   # reduction + push, wait + fold
        else:
            self.exchange = "all-gather of one float per rank (torch.distributed), fold in rank order"
            self.launches_per_call = 2   # plus the collective's own kernel

    def __call__(self, x):
        if self.x is not None:
            self.ops.exchange_reduce(self.x, x, self.result, self.limit_ns)
            return self.result
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
