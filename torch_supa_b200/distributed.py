"""Row-sharded loss reduction across GPUs.

Every operator on the path is independent per row, so N GPUs each hold a contiguous block of rows and
need no communication, with one exception: ``cross_entropy`` with ``mean`` / ``sum`` reduction, which
all-reduces two scalars, the valid-row count (before the fused sweep, so that gradients are written
already scaled by 1/|V|) and the loss sum (after it).  The reference would reach BCCL through
``torch.distributed.all_reduce`` (``torch_supa/csrc/distributed/ProcessGroupBCCL.cpp:3740-3790``); here a
small NCCL communicator on raw pointers does it, because ProcessGroupNCCL only accepts CUDA tensors.
"""
from __future__ import annotations

import ctypes
import os

import torch

_REDUCTIONS = {"none": 0, "mean": 1, "sum": 2}


def shard_rows(total_rows: int, world_size: int, rank: int) -> tuple[int, int]:
    """Contiguous row block ``[begin, end)`` of ``rank``: the first ``total_rows % world_size`` ranks take
    one extra row."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"invalid rank {rank} of {world_size}")
    base, extra = divmod(total_rows, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def combine_loss(local_loss_sum: float, local_valid_rows: float, reduction: str, all_reduce_sum):
    """Host-side statement of the protocol: ``all_reduce_sum`` maps a list of floats to their sums over
    ranks.  Returns the global loss (NaN for ``mean`` when no row counts anywhere)."""
    total, count = all_reduce_sum([float(local_loss_sum), float(local_valid_rows)])
    if reduction == "sum":
        return total
    if reduction == "mean":
        return total / count if count > 0 else float("nan")
    raise ValueError("combine_loss handles the mean and sum reductions")


class LossComm:
    """NCCL communicator for supa tensors (one process per GPU)."""

    def __init__(self, rank: int, world_size: int, device_index: int, unique_id: bytes):
        from . import _check, _load

        self._host = _load()
        self.rank, self.world_size, self.device_index = rank, world_size, device_index
        handle = ctypes.c_int64(0)
        _check(self._host.supa_nccl_init(world_size, unique_id, rank, device_index, ctypes.byref(handle)))
        self.handle = handle.value

    @staticmethod
    def new_unique_id() -> bytes:
        from . import _check, _load

        buf = ctypes.create_string_buffer(128)
        _check(_load().supa_nccl_unique_id(buf))
        return buf.raw

    @classmethod
    def from_env(cls, store=None, device_index=None, key="supa_b200/nccl_id"):
        """Builds the communicator of a ``torchrun``-style job: RANK / WORLD_SIZE / LOCAL_RANK from the
        environment, the unique id shared through ``store`` (default: the store of the initialised
        ``torch.distributed`` default group, else a TCPStore on MASTER_ADDR:MASTER_PORT+1)."""
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        local = int(os.environ.get("LOCAL_RANK", "0")) if device_index is None else device_index
        if store is None:
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized():
                store = dist.distributed_c10d._get_default_store()
            else:
                store = dist.TCPStore(os.environ.get("MASTER_ADDR", "127.0.0.1"), int(os.environ.get("MASTER_PORT", "29500")) + 1,
                                      world, rank == 0)
        if rank == 0:
            store.set(key, cls.new_unique_id())
        uid = bytes(store.get(key))
        return cls(rank, world, local, uid)

    def all_reduce_(self, tensor: torch.Tensor, op: str = "sum") -> torch.Tensor:
        return torch.ops.supa_b200.all_reduce_(tensor, self.handle, {"sum": 0, "max": 1, "min": 2}[op])

    def all_reduce_ptr(self, ptr: int, count: int, dtype_code: int, op: int = 0, stream: int = 0) -> None:
        from . import _check

        _check(self._host.supa_nccl_all_reduce(ctypes.c_int64(self.handle), ctypes.c_void_p(ptr), ctypes.c_int64(count),
                                               dtype_code, op, ctypes.c_void_p(stream)))

    def abort(self) -> None:
        from . import _check

        _check(self._host.supa_nccl_abort(ctypes.c_int64(self.handle)))

    def close(self) -> None:
        if self.handle:
            self._host.supa_nccl_destroy(ctypes.c_int64(self.handle))
            self.handle = 0


def sharded_cross_entropy(logits: torch.Tensor, target: torch.Tensor, comm: LossComm | None, *, ignore_index: int = -100,
                          label_smoothing: float = 0.0, reduction: str = "mean") -> torch.Tensor:
    """``F.cross_entropy`` over rows that are sharded across the ranks of ``comm``: every rank passes its own
    row block and receives the global loss; ``loss.backward()`` leaves the local block of the gradient,
    scaled by the global 1/|V| for ``mean``."""
    handle = comm.handle if (comm is not None and comm.world_size > 1) else 0
    return torch.ops.supa_b200.sharded_cross_entropy(logits, target, _REDUCTIONS[reduction], ignore_index, label_smoothing, handle)
