"""Row-sharded loss reduction across GPUs.

Every operator on the path is independent per row, so N GPUs each hold a contiguous block of rows and
need no communication, with one exception: ``cross_entropy`` with ``mean`` / ``sum`` reduction, which
sums two scalars over the ranks, the valid-row count (before the fused sweep, so that gradients are written
already scaled by 1/|V|) and the loss sum (after it).  The reference would reach BCCL through
``torch.distributed.all_reduce`` (``torch_supa/csrc/distributed/ProcessGroupBCCL.cpp:3740-3790``).  Here the
bookkeeping kernels of the loss exchange the two values themselves through peer device memory (NVLink stores
into slot arrays mapped with CUDA IPC; ``csrc/dist/PeerExchange.h``), so no collective launch sits between the
count, the sweep and the loss; a small NCCL communicator on raw pointers is the route when the arrays cannot
be mapped (and serves ``all_reduce_`` on supa tensors in general, because ProcessGroupNCCL only accepts CUDA
tensors).  ``SUPA_B200_LOSS_EXCHANGE=nccl`` forces the NCCL route.
"""
from __future__ import annotations

import ctypes
import os

import torch

_REDUCTIONS = {"none": 0, "mean": 1, "sum": 2}
C10D_BACKEND_NAME = "supa_nccl"
_c10d_module = None


def _load_c10d_module():
    """The pybind module that lives inside the host library (PyInit__supa_c10d)."""
    global _c10d_module
    if _c10d_module is None:
        import importlib.machinery
        import importlib.util

        from . import _HOST_LIB, _load

        _load()
        loader = importlib.machinery.ExtensionFileLoader("_supa_c10d", str(_HOST_LIB))
        spec = importlib.util.spec_from_loader("_supa_c10d", loader)
        module = importlib.util.module_from_spec(spec)
        loader.exec_module(module)
        _c10d_module = module
    return _c10d_module


def _create_c10d_backend(store, rank, size, timeout):
    return _load_c10d_module().create_backend(store, rank, size, timeout)


def register_c10d_backend() -> bool:
    """Registers the ``supa_nccl`` backend of ``torch.distributed`` for the ``supa`` device, as the reference registers
    ``bccl`` when it is imported (``torch_supa/distributed/distributed_c10d.py:65-102``).  After
    ``init_process_group("cpu:gloo,supa:supa_nccl")`` (or just ``"supa_nccl"``), ``torch.distributed.all_reduce``,
    ``broadcast``, ``all_gather``, ``reduce_scatter_tensor``, ``barrier`` and DistributedDataParallel work on supa
    tensors.  Returns False when torch.distributed is not available or the name is already taken."""
    import torch.distributed as dist

    if not dist.is_available():
        return False
    if C10D_BACKEND_NAME in getattr(dist.Backend, "backend_list", []):
        return False
    dist.Backend.register_backend(C10D_BACKEND_NAME, _create_c10d_backend, devices=["supa"])
    return True


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


PEER_MAX_RANKS = 8      # SB_XCHG_MAX_RANKS
PEER_HANDLE_BYTES = 64  # sizeof(cudaIpcMemHandle_t)


def exchange_mode() -> str:
    """``peer`` (default) or ``nccl``, from SUPA_B200_LOSS_EXCHANGE."""
    mode = os.environ.get("SUPA_B200_LOSS_EXCHANGE", "peer").strip().lower()
    if mode not in ("peer", "nccl"):
        raise ValueError(f"SUPA_B200_LOSS_EXCHANGE must be 'peer' or 'nccl', got {mode!r}")
    return mode


def gather_peer_handles(store, key: str, rank: int, world_size: int, mine: bytes) -> bytes:
    """Publishes this rank's handle under ``key/rank`` and returns all handles in rank order.  ``store`` is any
    object with the ``set`` / ``get`` of a torch.distributed store (``get`` blocks until the key exists)."""
    store.set(f"{key}/{rank}", mine)
    return b"".join(bytes(store.get(f"{key}/{r}")) for r in range(world_size))


class LossComm:
    """The exchange of a row-sharded loss between supa devices (one process per GPU): an NCCL communicator
    plus, when the ranks can map each other's memory, the peer-memory slot arrays the loss kernels use."""

    def __init__(self, rank: int, world_size: int, device_index: int, unique_id: bytes):
        from . import _check, _load

        self._host = _load()
        self.rank, self.world_size, self.device_index = rank, world_size, device_index
        handle = ctypes.c_int64(0)
        _check(self._host.supa_nccl_init(world_size, unique_id, rank, device_index, ctypes.byref(handle)))
        self.handle = handle.value
        self.peer_handle = 0

    def enable_peer_exchange(self, store, key: str = "supa_b200/peer") -> bool:
        """Maps the slot arrays of all ranks (collective: every rank calls it).  Returns False, on every rank,
        and leaves the NCCL route in place when any rank could not map a peer."""
        from . import _check

        if self.world_size > PEER_MAX_RANKS:
            return False
        handle = ctypes.c_int64(0)
        _check(self._host.supa_peer_create(self.world_size, self.rank, self.device_index, ctypes.byref(handle)))
        buf = ctypes.create_string_buffer(PEER_HANDLE_BYTES)
        _check(self._host.supa_peer_export(handle, buf))
        handles = gather_peer_handles(store, key, self.rank, self.world_size, buf.raw)
        ok = self._host.supa_peer_open(handle, handles) == 0
        # agree on the outcome: one rank on the NCCL route and another waiting in a kernel would not meet
        store.set(f"{key}/ok/{self.rank}", b"1" if ok else b"0")
        all_ok = all(bytes(store.get(f"{key}/ok/{r}")) == b"1" for r in range(self.world_size))
        if all_ok:
            self.peer_handle = handle.value
        else:
            self._host.supa_peer_destroy(handle)
        return all_ok

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
        comm = cls(rank, world, local, uid)
        if world > 1 and exchange_mode() == "peer":
            comm.enable_peer_exchange(store, key + "/peer")
        return comm

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
        if self.peer_handle:
            self._host.supa_peer_destroy(ctypes.c_int64(self.peer_handle))
            self.peer_handle = 0
        if self.handle:
            self._host.supa_nccl_destroy(ctypes.c_int64(self.handle))
            self.handle = 0


def sharded_cross_entropy(logits: torch.Tensor, target: torch.Tensor, comm: LossComm | None, *, ignore_index: int = -100,
                          label_smoothing: float = 0.0, reduction: str = "mean") -> torch.Tensor:
    """``F.cross_entropy`` over rows that are sharded across the ranks of ``comm``: every rank passes its own
    row block and receives the global loss; ``loss.backward()`` leaves the local block of the gradient,
    scaled by the global 1/|V| for ``mean``."""
    sharded = comm is not None and comm.world_size > 1
    handle = comm.handle if sharded else 0
    peer = comm.peer_handle if sharded else 0
    return torch.ops.supa_b200.sharded_cross_entropy(logits, target, _REDUCTIONS[reduction], ignore_index, label_smoothing, handle, peer)
