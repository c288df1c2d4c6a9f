"""``torch.supa``: the device module of the supa backend (the subset the operator path and its tests
need; counterpart of ``torch_supa/supa/__init__.py`` in the reference)."""
from __future__ import annotations

import ctypes

import torch


def _host():
    from . import _load

    return _load()


def _check(rc):
    from . import _check as check

    check(rc)


def is_available() -> bool:
    return _host().supa_device_count() > 0


def device_count() -> int:
    return _host().supa_device_count()


def current_device() -> int:
    out = ctypes.c_int(0)
    _check(_host().supa_current_device(ctypes.byref(out)))
    return out.value


def _index(device) -> int:
    if device is None:
        return -1
    if isinstance(device, int):
        return device
    d = torch.device(device)
    if d.type != "supa":
        raise ValueError(f"expected a supa device, got {d}")
    return -1 if d.index is None else d.index


def set_device(device) -> None:
    idx = _index(device)
    if idx >= 0:
        _check(_host().supa_set_device(idx))


def synchronize(device=None) -> None:
    """Waits for all work queued on the device and raises if a kernel reported a data error
    (an out-of-range class index) since the last check."""
    _check(_host().supa_synchronize(_index(device)))


def check_error(device=None) -> None:
    """Drains the current stream and raises if the device status word is set."""
    _check(_host().supa_check_status(_index(device)))


def current_stream(device=None) -> torch.Stream:
    idx = _index(device)
    return torch._C._acc.current_stream(idx) if hasattr(torch._C, "_acc") else torch.accelerator.current_stream(idx if idx >= 0 else None)


def current_stream_handle(device=None) -> int:
    """The cudaStream_t of the calling thread's current stream (0 is the legacy default stream)."""
    out = ctypes.c_void_p(0)
    _check(_host().supa_current_stream(_index(device), ctypes.byref(out)))
    return out.value or 0


class device:
    """Context manager that changes the current supa device."""

    def __init__(self, dev):
        self.idx = _index(dev)
        self.prev = -1

    def __enter__(self):
        if self.idx >= 0:
            self.prev = current_device()
            set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            set_device(self.prev)
        return False


def _stats(dev):
    buf = (ctypes.c_int64 * 6)()
    idx = _index(dev)
    _check(_host().supa_memory_stats(idx if idx >= 0 else current_device(), buf))
    return list(buf)


def memory_stats(device=None) -> dict:
    s = _stats(device)
    return {"allocated_bytes.all.current": s[0], "allocated_bytes.all.peak": s[1], "reserved_bytes.all.current": s[2],
            "allocation.all.allocated": s[3], "allocation.all.freed": s[4], "num_ooms": s[5]}


def memory_allocated(device=None) -> int:
    return _stats(device)[0]


def max_memory_allocated(device=None) -> int:
    return _stats(device)[1]


def memory_reserved(device=None) -> int:
    return _stats(device)[2]


def reset_peak_memory_stats(device=None) -> None:
    idx = _index(device)
    _check(_host().supa_reset_peak_memory_stats(idx if idx >= 0 else current_device()))


def empty_cache() -> None:
    _check(_host().supa_empty_cache())


def host_memory_stats() -> dict:
    """Counters of the caching allocator of pinned host memory (``tensor.pin_memory()``, non-blocking copies)."""
    out = (ctypes.c_int64 * 4)()
    _check(_host().supa_host_memory_stats(out))
    return {"allocated_bytes": out[0], "reserved_bytes": out[1], "host_allocs": out[2], "cache_hits": out[3]}


def empty_host_cache() -> None:
    """Returns cached pinned host blocks to the driver."""
    _check(_host().supa_empty_pinned_cache())


def set_memory_limit(nbytes: int, device=None) -> None:
    """Caps the bytes tensors may hold on the device (0 removes the cap).  Allocations beyond it raise
    ``torch.OutOfMemoryError`` on the host without touching the GPU."""
    idx = _index(device)
    _check(_host().supa_set_memory_limit(idx if idx >= 0 else current_device(), ctypes.c_int64(nbytes)))


def memcpy_async(dst_ptr: int, src_ptr: int, nbytes: int, device=None) -> None:
    """cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDefault) on the current stream: moves bytes between
    raw addresses (used to hand data produced by other CUDA code to supa tensors without a host round trip)."""
    _check(_host().supa_memcpy_async(_index(device), ctypes.c_void_p(dst_ptr), ctypes.c_void_p(src_ptr), ctypes.c_int64(nbytes)))


def _is_in_bad_fork() -> bool:
    return False


# ---- random number generator (counterpart of torch_supa/supa/random.py:26-200) ---------------------------------------------
def _generator_control(device, op: int, value: int = 0) -> int:
    out = ctypes.c_uint64(0)
    _check(_host().supa_generator_control(_index(device), op, ctypes.c_uint64(value & 0xFFFFFFFFFFFFFFFF), ctypes.byref(out)))
    return out.value


def manual_seed(seed: int) -> None:
    """Seeds the default generator of the current device (and rewinds its offset).  Ignored when no device is present,
    so that ``torch.manual_seed`` keeps working on a machine without one."""
    if device_count() > 0:
        _generator_control(None, 0, int(seed))


def manual_seed_all(seed: int) -> None:
    for i in range(device_count()):
        _generator_control(i, 0, int(seed))


def seed() -> None:
    """Seeds the current device's default generator from a non-deterministic source."""
    if device_count() > 0:
        _generator_control(None, 1)


def seed_all() -> None:
    """One non-deterministic seed, applied to every device."""
    if device_count() > 0:
        value = _generator_control(0, 1)
        for i in range(1, device_count()):
            _generator_control(i, 0, value)


def initial_seed() -> int:
    return _generator_control(None, 2)


def get_rng_state(device="supa") -> torch.Tensor:
    """The default generator's state as a CPU byte tensor: 8 bytes of seed, 8 bytes of Philox offset."""
    out = (ctypes.c_uint8 * 16)()
    _check(_host().supa_get_rng_state(_index(device), out))
    return torch.tensor(list(out), dtype=torch.uint8)


def set_rng_state(new_state: torch.Tensor, device="supa") -> None:
    state = new_state.detach().to("cpu", torch.uint8).contiguous()
    buf = (ctypes.c_uint8 * state.numel()).from_buffer_copy(bytes(state.tolist()))
    _check(_host().supa_set_rng_state(_index(device), buf, ctypes.c_int64(state.numel())))


def get_rng_state_all() -> list:
    return [get_rng_state(i) for i in range(device_count())]


def set_rng_state_all(new_states) -> None:
    for i, state in enumerate(new_states):
        set_rng_state(state, i)


# The runtime initialises on first use; torch.utils.checkpoint reads this attribute to decide whether the device
# generator's state belongs to the state it preserves.
_initialized = True


def get_amp_supported_dtype() -> list:
    """The dtypes torch.amp.autocast accepts for this device (torch.utils.checkpoint builds a disabled autocast context for
    the device it replays on and asks for this list).  No autocast policy table is registered for supa operators."""
    return [torch.bfloat16, torch.float16]


def is_initialized() -> bool:
    return True


def _lazy_init() -> None:
    pass
