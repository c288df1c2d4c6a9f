"""Worker of tests/test_gpu_multi.py: one process per GPU (torchrun environment).  Every rank builds the same
seeded global problem, takes its own row block to its supa device, and checks the sharded loss and its local
gradient block against PyTorch CPU on the whole problem."""
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    import torch.distributed as dist

    import torch_supa_b200  # noqa: F401  (registers the supa device)
    from torch_supa_b200.distributed import LossComm, sharded_cross_entropy

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.supa.set_device(local)
    comm = LossComm.from_env()
    device = torch.device("supa", local)
    failures = []
    mode = os.environ.get("SUPA_B200_LOSS_EXCHANGE", "peer")
    if mode == "peer" and comm.peer_handle == 0:
        failures.append("the peer-memory exchange could not be set up (CUDA IPC mapping of the slot arrays failed)")
    if mode == "nccl" and comm.peer_handle != 0:
        failures.append("SUPA_B200_LOSS_EXCHANGE=nccl was ignored")
    for dtype, rows_per_rank, classes, eps, reduction in ((torch.float32, 37, 1000, 0.0, "mean"), (torch.float32, 64, 32000, 0.1, "mean"),
                                                          (torch.bfloat16, 16, 128256, 0.1, "mean"), (torch.float32, 19, 777, 0.0, "sum")):
        g = torch.Generator().manual_seed(1234)
        rows = rows_per_rank * world
        logits = (torch.randn(rows, classes, generator=g) * 2).to(dtype)
        target = torch.randint(0, classes, (rows,), generator=g)
        target[::7] = -100
        # rank 0's block is all ignored in one case: the global count, not the local one, must scale its gradient
        if classes == 777:
            target[:rows_per_rank] = -100
        ref_x = logits.double().requires_grad_(True)
        ref = F.cross_entropy(ref_x, target, label_smoothing=eps, reduction=reduction)
        ref.backward()
        lo, hi = rank * rows_per_rank, (rank + 1) * rows_per_rank
        x = logits[lo:hi].to(device).requires_grad_(True)
        t = target[lo:hi].to(device)
        loss = sharded_cross_entropy(x, t, comm, label_smoothing=eps, reduction=reduction)
        loss.backward()
        rtol = 2e-2 if dtype == torch.bfloat16 else 1e-5
        got, want = float(loss.float().cpu()), float(ref)
        if abs(got - want) > rtol * abs(want) + 1e-6:
            failures.append(f"loss {dtype} {reduction}: {got} vs {want}")
        gd = x.grad.cpu().double()
        gr = ref_x.grad[lo:hi]
        err = float((gd - gr).abs().max())
        tol = (2e-2 if dtype == torch.bfloat16 else 1e-5) * float(gr.abs().max()) + 1e-9
        if err > tol:
            failures.append(f"grad {dtype} {reduction}: max err {err} > {tol}")
    # several steps back to back without a host synchronisation: the slot rows of the exchange are reused every other step
    g = torch.Generator().manual_seed(99)
    rows_per_rank, classes = 64, 4096
    logits = torch.randn(rows_per_rank * world, classes, generator=g) * 2
    target = torch.randint(0, classes, (rows_per_rank * world,), generator=g)
    lo, hi = rank * rows_per_rank, (rank + 1) * rows_per_rank
    x = logits[lo:hi].to(device).requires_grad_(True)
    t = target[lo:hi].to(device)
    losses = []
    for step in range(12):
        x.grad = None
        loss = sharded_cross_entropy(x * (1.0 + 0.125 * step), t, comm)
        loss.backward()
        losses.append(loss)
    for step, loss in enumerate(losses):
        want = float(F.cross_entropy(logits.double() * (1.0 + 0.125 * step), target))
        if abs(float(loss.cpu()) - want) > 1e-5 * abs(want):
            failures.append(f"step {step}: loss {float(loss.cpu())} vs {want}")
    torch.supa.synchronize()
    # every rank reports; the job fails if any rank saw a mismatch
    flag = torch.tensor([len(failures)], dtype=torch.int64)
    dist.all_reduce(flag)
    for f in failures:
        print(f"[rank {rank}] {f}", flush=True)
    comm.close()
    dist.destroy_process_group()
    return 1 if int(flag.item()) else 0


if __name__ == "__main__":
    sys.exit(main())
