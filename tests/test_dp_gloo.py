"""Data-parallel host logic on CPU ranks (gloo, world_size 2): bucket assignment, launch order during backward, gradient
averaging against the single-process result on the concatenated batch, and handling of a parameter that takes no part in
a step. No GPU involved."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F
from torch import nn

from conftest import ROOT


def test_assign_buckets_fills_in_backward_order():
    from omarchy_mac_torch_b200.dp import assign_buckets
    ids, sizes = assign_buckets([10, 20, 30, 40], bucket_elems=55)
    assert ids == [2, 1, 1, 0] and sizes == [40, 50, 10]          # last parameter first; 30+20 share, 10 spills over
    ids, sizes = assign_buckets([5, 1000, 5], bucket_elems=100)    # an oversized parameter gets a bucket of its own
    assert ids == [2, 1, 0] and sizes == [5, 1000, 5]
    assert assign_buckets([], 10) == ([], [])
    # ResNet-50: 25.56 M parameters in 25 MB buckets -> 5 buckets
    from omarchy_mac_torch_b200 import models
    numels = [p.numel() for p in models.ResNet50().parameters()]
    ids, sizes = assign_buckets(numels, int(25 * (1 << 20) / 4))
    assert max(ids) + 1 == len(sizes) == 5 and sum(sizes) == sum(numels) and all(s <= 25 * (1 << 20) / 4 for s in sizes)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Conv2d(3, 8, 3, padding=1)
        self.bn = nn.BatchNorm2d(8)
        self.b = nn.Conv2d(8, 8, 3, padding=1)
        self.unused = nn.Linear(4, 4)      # never takes part in forward
        self.head = nn.Linear(8, 5)

    def forward(self, x):
        y = torch.relu(self.bn(self.a(x)))
        return self.head(self.b(y).mean((2, 3)))


def _worker(rank, world, port, out, torch_zero_grad=False):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from omarchy_mac_torch_b200.dp import DataParallel
    torch.manual_seed(7 + rank)            # deliberately different: broadcast_parameters must align the replicas
    model = Net()
    dp = DataParallel(model, bucket_mb=0.002)   # ~500 floats per bucket -> several buckets
    g = torch.Generator().manual_seed(100)
    X, Y = torch.randn(8, 3, 6, 6, generator=g), torch.randint(0, 5, (8,), generator=g)
    xs, ys = X[rank * 4:(rank + 1) * 4], Y[rank * 4:(rank + 1) * 4]
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    for _ in range(2):
        if torch_zero_grad:
            opt.zero_grad()  # torch's default set_to_none=True: the hooks must bring the new gradients back into the buckets
            dp.launch_order = []
        else:
            dp.zero_grad()
        F.cross_entropy(model(xs), ys).backward()
        order = list(dp.launch_order)
        dp.finish()
        opt.step()
    spread = dp.param_spread()  # a collective: every rank calls it
    if rank == 0:
        torch.save({"state": model.state_dict(), "order": order, "nb": len(dp.flat), "bucket_of": dp.bucket_of, "spread": spread}, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("torch_zero_grad", [False, True], ids=["dp.zero_grad", "optimizer.zero_grad"])
def test_two_ranks_match_single_process(tmp_path, torch_zero_grad):
    out = str(tmp_path / "rank0.pt")
    port = _free_port()
    mp.spawn(_worker, args=(2, port, out, torch_zero_grad), nprocs=2, join=True)
    got = torch.load(out)
    assert got["spread"] == 0.0  # the replicas hold bit-identical parameters after two steps
    # single process: same initial weights as rank 0, per-shard forward/backward (local BN statistics), averaged gradients
    torch.manual_seed(7)
    ref = Net()
    g = torch.Generator().manual_seed(100)
    X, Y = torch.randn(8, 3, 6, 6, generator=g), torch.randint(0, 5, (8,), generator=g)
    opt = torch.optim.SGD(ref.parameters(), lr=0.1)
    import copy
    for _ in range(2):
        grads, stats = [], []
        start = copy.deepcopy(ref.state_dict())
        for r in range(2):
            ref.load_state_dict(start)
            ref.zero_grad()
            F.cross_entropy(ref(X[r * 4:(r + 1) * 4]), Y[r * 4:(r + 1) * 4]).backward()
            grads.append([None if p.grad is None else p.grad.clone() for p in ref.parameters()])
            if r == 0:
                stats0 = copy.deepcopy({k: v for k, v in ref.state_dict().items() if "running" in k or "num_batches" in k})
        ref.load_state_dict(start)
        ref.load_state_dict(stats0, strict=False)   # rank 0 keeps its own running statistics
        for p, g0, g1 in zip(ref.parameters(), *grads):
            p.grad = None if g0 is None else (g0 + g1) / 2
        opt.step()
    for k, v in ref.state_dict().items():
        assert torch.allclose(got["state"][k].float(), v.float(), rtol=1e-5, atol=1e-6), k
    # buckets are launched in backward order (bucket 0 holds the last parameters); the bucket holding the parameter that
    # takes no part in the step never completes during backward, and finish() reduces it instead
    names = [n for n, _ in Net().named_parameters()]
    idle = {got["bucket_of"][i] for i, n in enumerate(names) if n.startswith("unused")}
    assert got["nb"] >= 3 and got["order"] == sorted(got["order"])
    assert set(got["order"]) == set(range(got["nb"])) - idle and idle
