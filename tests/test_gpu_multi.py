"""Row-sharded cross entropy on two GPUs of one node (needs at least two GPUs; skipped otherwise), once with the two
scalars exchanged by the loss kernels through peer memory and once through NCCL all-reduces."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode,port", [("peer", 29533), ("nccl", 29543)])
def test_sharded_cross_entropy_two_gpus(mode, port):
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "multi_gpu_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), worker]
    env = dict(os.environ, SUPA_B200_LOSS_EXCHANGE=mode)
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_c10d_collectives_and_ddp_two_gpus():
    """torch.distributed.all_reduce / broadcast / all_gather / reduce_scatter_tensor / barrier and DistributedDataParallel on
    supa tensors through the supa_nccl backend."""
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "multi_gpu_c10d_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29553", worker]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
