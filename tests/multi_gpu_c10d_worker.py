"""Worker of tests/test_gpu_multi.py: torch.distributed collectives and DistributedDataParallel on supa tensors through the
supa_nccl backend (one process per GPU, torchrun environment)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class Scale(torch.nn.Module):
    """A model made of operators this backend has (no dense contraction): y = sum(x * w + b)."""

    def __init__(self):
        super().__init__()
        self.w = torch.nn.Parameter(torch.arange(1.0, 9.0))
        self.b = torch.nn.Parameter(torch.zeros(8))

    def forward(self, x):
        return (x * self.w + self.b).sum(-1)


def main() -> int:
    import torch.distributed as dist

    import torch_supa_b200  # noqa: F401  (registers the device and the backend)

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.supa.set_device(local)
    dist.init_process_group("cpu:gloo,supa:supa_nccl", rank=rank, world_size=world)
    dev = torch.device("supa", local)
    failures = []

    def check(name, got, want):
        if not torch.equal(got.cpu(), want):
            failures.append(f"{name}: {got.cpu().flatten()[:6].tolist()} vs {want.flatten()[:6].tolist()}")

    total = float(sum(range(1, world + 1)))
    x = torch.full((1000,), rank + 1.0).to(dev)
    dist.all_reduce(x)
    check("all_reduce sum", x, torch.full((1000,), total))
    for op, want in ((dist.ReduceOp.MAX, float(world)), (dist.ReduceOp.MIN, 1.0), (dist.ReduceOp.AVG, total / world)):
        y = torch.full((33,), rank + 1.0).to(dev)
        dist.all_reduce(y, op=op)
        check(f"all_reduce {op}", y, torch.full((33,), want))
    i = torch.full((7,), rank + 2, dtype=torch.int64).to(dev)
    dist.all_reduce(i, op=dist.ReduceOp.PRODUCT)
    prod = 1
    for r in range(world):
        prod *= r + 2
    check("all_reduce product int64", i, torch.full((7,), prod, dtype=torch.int64))
    b = (torch.arange(10.0) * (rank + 1)).to(dev)
    dist.broadcast(b, src=world - 1)
    check("broadcast", b, torch.arange(10.0) * world)
    outs = [torch.empty(5, dtype=torch.bfloat16).to(dev) for _ in range(world)]
    dist.all_gather(outs, torch.full((5,), float(rank), dtype=torch.bfloat16).to(dev))
    for r in range(world):
        check(f"all_gather[{r}]", outs[r], torch.full((5,), float(r), dtype=torch.bfloat16))
    flat = torch.empty(world * 4).to(dev)
    dist.all_gather_into_tensor(flat, torch.full((4,), rank + 0.5).to(dev))
    check("all_gather_into_tensor", flat, torch.arange(world).repeat_interleave(4) + 0.5)
    rs_out = torch.empty(3).to(dev)
    dist.reduce_scatter_tensor(rs_out, (torch.arange(world * 3.0) + rank).to(dev))
    check("reduce_scatter_tensor", rs_out, torch.arange(rank * 3.0, rank * 3.0 + 3) * world + sum(range(world)))
    work = dist.all_reduce(x, async_op=True)
    work.wait()
    check("async all_reduce", x, torch.full((1000,), total * world))
    dist.barrier()

    # DistributedDataParallel: parameters broadcast from rank 0, gradients averaged over the ranks
    try:
        from torch.nn.parallel import DistributedDataParallel as DDP

        model = Scale()
        if rank != 0:
            with torch.no_grad():
                model.w.mul_(0)  # differs from rank 0 until DDP broadcasts
        model = model.to(dev)
        ddp = DDP(model)
        check("ddp parameter broadcast", ddp.module.w.detach(), torch.arange(1.0, 9.0))
        inp = torch.full((4, 8), rank + 1.0).to(dev)
        ddp(inp).sum().backward()
        want = torch.full((8,), 4.0 * total / world)  # d/dw of sum over the 4 rows of x * w, averaged over the ranks
        check("ddp gradient", ddp.module.w.grad, want)
        check("ddp bias gradient", ddp.module.b.grad, torch.full((8,), 4.0))
    except NotImplementedError as e:  # names the missing operator
        failures.append("DistributedDataParallel needs an operator this backend lacks: " + str(e).splitlines()[0])
    torch.supa.synchronize()
    flag = torch.tensor([len(failures)], dtype=torch.int64)
    dist.all_reduce(flag)
    for f in failures:
        print(f"[rank {rank}] {f}", flush=True)
    dist.destroy_process_group()
    return 1 if int(flag.item()) else 0


if __name__ == "__main__":
    sys.exit(main())
