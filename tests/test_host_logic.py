"""Host-side logic that needs no GPU: registration hygiene, row sharding, the two-scalar loss protocol
over a real 2-process gloo group."""
import math
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def test_package_imports_and_registers_the_device():
    import torch_supa_b200  # noqa: F401

    assert torch._C._get_privateuse1_backend_name() == "supa"
    assert hasattr(torch, "supa") and torch.supa.device_count() >= 0
    assert torch.device("supa:0").type == "supa"


def test_no_dangling_operator_registrations():
    """Every m.impl names an existing schema (the check of test/test_dispatch_registration.py in the reference)."""
    import torch_supa_b200  # noqa: F401

    assert torch._C._dispatch_find_dangling_impls() == []


@pytest.mark.parametrize("op", ["aten::add.Tensor", "aten::add_.Tensor", "aten::add.out", "aten::mul.Tensor", "aten::mul.out",
                                "aten::gelu", "aten::gelu.out", "aten::gelu_backward", "aten::silu", "aten::silu_backward",
                                "aten::glu", "aten::glu_backward", "aten::sum.dim_IntList", "aten::sum.IntList_out", "aten::mean.dim",
                                "aten::mean.out", "aten::amax", "aten::amax.out", "aten::_log_softmax", "aten::_log_softmax.out",
                                "aten::_log_softmax_backward_data", "aten::nll_loss_forward", "aten::nll_loss_forward.output",
                                "aten::nll_loss_backward", "aten::nll_loss_backward.grad_input", "aten::cross_entropy_loss",
                                "aten::empty.memory_format", "aten::empty_strided", "aten::_copy_from", "aten::as_strided",
                                "aten::view", "aten::resize_", "aten::fill_.Scalar", "aten::zero_", "aten::_local_scalar_dense"])
def test_operator_has_a_privateuse1_kernel(op):
    import torch_supa_b200  # noqa: F401

    table = torch._C._dispatch_dump_table(op)
    line = [l for l in table.splitlines() if l.startswith("PrivateUse1:")]
    assert line and "libtorch_supa_b200" in table or "registered at" in line[0], table


def test_cross_entropy_autograd_key_falls_through():
    import torch_supa_b200  # noqa: F401

    table = torch._C._dispatch_dump_table("aten::cross_entropy_loss")
    auto = [l for l in table.splitlines() if l.startswith("AutogradPrivateUse1:")]
    assert auto and "fallthrough" in auto[0]


def test_operators_fail_loudly_without_a_device():
    import torch_supa_b200  # noqa: F401

    if torch.supa.device_count() > 0:
        pytest.skip("a device is present")
    with pytest.raises(RuntimeError):
        torch.empty(4, device="supa")


def test_seeding_without_a_device_is_ignored():
    """torch.manual_seed reaches the device module on every machine; with no device there is nothing to seed."""
    import torch_supa_b200  # noqa: F401

    if torch.supa.device_count() > 0:
        pytest.skip("a device is present")
    torch.manual_seed(3)
    torch.supa.manual_seed(3)
    torch.supa.manual_seed_all(3)
    torch.supa.seed()
    torch.supa.seed_all()
    assert torch.supa.get_rng_state_all() == []
    with pytest.raises(RuntimeError):
        torch.supa.get_rng_state()
    with pytest.raises(RuntimeError):
        torch.Generator(device="supa")


def test_shard_rows_partitions_exactly():
    from torch_supa_b200.distributed import shard_rows

    for total in (0, 1, 7, 32768, 4097):
        for world in (1, 2, 4, 8):
            blocks = [shard_rows(total, world, r) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
            sizes = [e - b for b, e in blocks]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_rows(10, 2, 2)


def test_combine_loss_rules():
    from torch_supa_b200.distributed import combine_loss

    ident = lambda v: v  # noqa: E731
    assert combine_loss(6.0, 3.0, "mean", ident) == 2.0
    assert combine_loss(6.0, 3.0, "sum", ident) == 6.0
    assert math.isnan(combine_loss(0.0, 0.0, "mean", ident))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _sharded_worker(rank, world, port, out_path):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    import torch.nn.functional as F

    from torch_supa_b200.distributed import combine_loss, shard_rows

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(0)
    rows, classes = 37, 50
    logits = torch.randn(rows, classes, generator=g) * 2
    target = torch.randint(0, classes, (rows,), generator=g)
    target[::5] = -100
    b, e = shard_rows(rows, world, rank)
    local_logits = logits[b:e].clone().requires_grad_(True)
    local_target = target[b:e]

    def all_reduce_sum(values):
        t = torch.tensor(values, dtype=torch.float64)
        dist.all_reduce(t)
        return t.tolist()

    # step 1: valid-row count first, step 2: local sums, step 3: loss sum (the protocol of the fused kernel)
    local_valid = float((local_target != -100).sum())
    (global_valid,) = all_reduce_sum([local_valid])
    local_sum = F.cross_entropy(local_logits, local_target, ignore_index=-100, label_smoothing=0.1, reduction="sum")
    loss = combine_loss(float(local_sum), local_valid, "mean", all_reduce_sum)
    (local_sum / global_valid).backward()
    ref_logits = logits.clone().requires_grad_(True)
    ref = F.cross_entropy(ref_logits, target, ignore_index=-100, label_smoothing=0.1)
    ref.backward()
    ok = abs(loss - float(ref)) <= 1e-6 * abs(float(ref)) and torch.allclose(local_logits.grad, ref_logits.grad[b:e], rtol=1e-5, atol=1e-8)
    flags = torch.tensor([1.0 if ok else 0.0], dtype=torch.float64)
    dist.all_reduce(flags)
    if rank == 0:
        Path(out_path).write_text(str(flags.item()))
    dist.destroy_process_group()


def test_two_process_gloo_sharded_loss(tmp_path):
    """World size 2 on CPU: row blocks per rank, all-reduce of (valid count) then (loss sum), gradients scaled
    by the global 1/|V|; equals the single-process result."""
    out = tmp_path / "ok.txt"
    mp.spawn(_sharded_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    assert float(out.read_text()) == 2.0


# ---- the exchange protocol of the loss kernels, restated on the host -------------------------------------------------
# The kernels publish a partial as (value, sequence number) into slot (seq % DEPTH, source rank) of every rank's array and
# add what arrives in their own array in rank order.  The same steps on shared host memory, two processes, many
# exchanges back to back: slot rows are reused every DEPTH exchanges and no rank may read a stale or a future value.
def _slot_index(seq, src_rank, depth, max_ranks):
    return (seq % depth) * max_ranks + src_rank


def _host_exchange(arrays, rank, world, seq, local, depth, max_ranks, deadline_s=20.0):
    import time

    for peer in range(world):
        slot = arrays[peer][_slot_index(seq, rank, depth, max_ranks)]
        slot[0] = local          # value first ...
        slot[1] = float(seq)     # ... then the number a reader waits for
    mine = arrays[rank]
    total = 0.0
    t0 = time.time()
    for src in range(world):
        slot = mine[_slot_index(seq, src, depth, max_ranks)]
        while slot[1] != float(seq):
            if time.time() - t0 > deadline_s:
                raise TimeoutError(f"rank {rank}: partial of rank {src} for exchange {seq} never arrived")
        total += float(slot[0])
    return total


def _exchange_worker(rank, world, port, arrays, out_path):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    from torch_supa_b200 import capi
    from torch_supa_b200.distributed import PEER_HANDLE_BYTES, gather_peer_handles

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.distributed_c10d._get_default_store()
    # the handle hand-over the GPU path uses, with stand-in bytes
    mine = bytes([rank + 1]) * PEER_HANDLE_BYTES
    handles = gather_peer_handles(store, "test/peer", rank, world, mine)
    ok = handles == b"".join(bytes([r + 1]) * PEER_HANDLE_BYTES for r in range(world))
    seq = 0
    for step in range(50):
        # count exchange, then loss exchange, as fused_forward issues them; rank 1 lags now and then
        if rank == 1 and step % 7 == 3:
            import time

            time.sleep(0.01)
        seq += 1
        count = _host_exchange(arrays, rank, world, seq, float(10 * step + rank), capi.XCHG_DEPTH, capi.XCHG_MAX_RANKS)
        seq += 1
        loss = _host_exchange(arrays, rank, world, seq, 0.5 * step + 0.25 * rank, capi.XCHG_DEPTH, capi.XCHG_MAX_RANKS)
        ok = ok and count == sum(10 * step + r for r in range(world)) and loss == sum(0.5 * step + 0.25 * r for r in range(world))
    flags = torch.tensor([1.0 if ok else 0.0], dtype=torch.float64)
    dist.all_reduce(flags)
    if rank == 0:
        Path(out_path).write_text(str(flags.item()))
    dist.destroy_process_group()


def test_two_process_slot_exchange_protocol(tmp_path):
    from torch_supa_b200 import capi

    world = 2
    arrays = [torch.zeros(capi.XCHG_DEPTH * capi.XCHG_MAX_RANKS, 2, dtype=torch.float64).share_memory_() for _ in range(world)]
    out = tmp_path / "ok.txt"
    mp.spawn(_exchange_worker, args=(world, _free_port(), arrays, str(out)), nprocs=world, join=True)
    assert float(out.read_text()) == 2.0


def test_exchange_mode_from_environment(monkeypatch):
    from torch_supa_b200.distributed import exchange_mode

    monkeypatch.delenv("SUPA_B200_LOSS_EXCHANGE", raising=False)
    assert exchange_mode() == "peer"
    monkeypatch.setenv("SUPA_B200_LOSS_EXCHANGE", "NCCL")
    assert exchange_mode() == "nccl"
    monkeypatch.setenv("SUPA_B200_LOSS_EXCHANGE", "gloo")
    with pytest.raises(ValueError):
        exchange_mode()


# ---- the c10d backend for supa tensors: registration and construction (no GPU needed) ------------------------------------
def test_c10d_backend_is_registered_for_the_supa_device():
    import torch.distributed as dist

    import torch_supa_b200  # noqa: F401

    assert "supa_nccl" in dist.Backend.backend_list
    assert dist.Backend.default_device_backend_map.get("supa") == "supa_nccl"


def test_c10d_backend_object_can_be_created_without_a_device():
    import datetime

    import torch.distributed as dist

    from torch_supa_b200.distributed import _create_c10d_backend

    backend = _create_c10d_backend(dist.HashStore(), 0, 1, datetime.timedelta(seconds=5))
    assert isinstance(backend, torch._C._distributed_c10d.Backend)
    assert backend.rank() == 0 and backend.size() == 1 and backend.name() == "supa_nccl"


def _c10d_worker(rank, world, port, out_path):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    import torch_supa_b200  # noqa: F401

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    # one backend per device type: gloo carries CPU tensors, supa_nccl is created for the supa device (its communicator
    # only comes to life with the first collective on a supa tensor)
    dist.init_process_group("cpu:gloo,supa:supa_nccl", rank=rank, world_size=world)
    pg = dist.distributed_c10d._get_default_group()
    ok = pg._get_backend(torch.device("supa")).name() == "supa_nccl" and pg._get_backend(torch.device("cpu")).name() == "gloo"
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t)
    ok = ok and t.item() == sum(range(1, world + 1))
    flags = torch.tensor([1.0 if ok else 0.0], dtype=torch.float64)
    dist.all_reduce(flags)
    if rank == 0:
        Path(out_path).write_text(str(flags.item()))
    dist.destroy_process_group()


def test_two_process_group_with_supa_backend_beside_gloo(tmp_path):
    out = tmp_path / "ok.txt"
    mp.spawn(_c10d_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    assert float(out.read_text()) == 2.0


# ---- reduction planning (host side of sb_reduce / sb_arg_reduce / sb_moments; no kernel is launched) -----------------
def _reduce_desc(sizes, in_strides, out_strides, dtype):
    from torch_supa_b200 import capi

    d = capi.ReduceDesc()
    d.op = capi.RED_SUM
    d.ndim = len(sizes)
    for i, (n, si, so) in enumerate(zip(sizes, in_strides, out_strides)):
        d.sizes[i], d.in_strides[i], d.out_strides[i] = n, si, so
    d.in_dtype = d.out_dtype = dtype
    d.in_, d.out = 0x7F0000000000, 0x7F0100000000  # never dereferenced by the planner
    return d


def test_reduce_plan_does_not_depend_on_the_order_of_the_dimensions():
    from torch_supa_b200 import capi

    # x[5000, 96].sum(0): in stride order (columns first) and as a TensorIterator lists it (the reduced dimension first)
    a = _reduce_desc([96, 5000], [1, 96], [1, 0], capi.F32)
    b = _reduce_desc([5000, 96], [96, 1], [0, 1], capi.F32)
    assert capi.reduce_path(a) == capi.reduce_path(b) == 2
    assert capi.reduce_scratch_bytes(a) == capi.reduce_scratch_bytes(b) > 0
    # x[5000, 96].sum(1): rows
    c = _reduce_desc([96, 5000], [1, 96], [0, 1], capi.F32)
    e = _reduce_desc([5000, 96], [96, 1], [1, 0], capi.F32)
    assert capi.reduce_path(c) == capi.reduce_path(e) == 0
    assert capi.reduce_scratch_bytes(c) == capi.reduce_scratch_bytes(e) == 0
    # a middle dimension of [7, 3000, 96], listed in three orders
    orders = [([96, 3000, 7], [1, 96, 288000], [1, 0, 96]), ([3000, 96, 7], [96, 1, 288000], [0, 1, 96]),
              ([7, 3000, 96], [288000, 96, 1], [96, 0, 1])]
    plans = {(capi.reduce_path(_reduce_desc(*o, capi.BF16)), capi.reduce_scratch_bytes(_reduce_desc(*o, capi.BF16))) for o in orders}
    assert len(plans) == 1 and next(iter(plans))[0] == 2
    # an expanded (stride 0) kept dimension does not take the row path away from x.sum(-1)
    f = _reduce_desc([3, 64, 1000], [0, 1, 64], [1000, 0, 1], capi.F32)
    assert capi.reduce_path(f) == 0


def test_few_long_rows_and_tall_columns_ask_for_scratch():
    from torch_supa_b200 import capi

    few_long = _reduce_desc([1 << 21, 4], [1, 1 << 21], [0, 1], capi.F32)
    assert capi.reduce_path(few_long) == 1 and capi.reduce_scratch_bytes(few_long) > 0
    assert capi.reduce_ext_scratch_bytes(capi.F32, 4, 1 << 21, 1, False) > 0       # argmax of four long rows: segments
    assert capi.reduce_ext_scratch_bytes(capi.F32, 100000, 64, 1, False) == 0      # short rows: a lane group each
    assert capi.reduce_ext_scratch_bytes(capi.F32, 1, 100000, 64, True) > 0        # var(0) of a tall matrix: row chunks
    assert capi.reduce_ext_scratch_bytes(capi.F32, 1, 32, 64, True) == 0           # too few rows to cut
    assert capi.reduce_ext_scratch_bytes(capi.F32, 70000, 100000, 3, False) == 0   # more outer slices than grid.z takes
