"""One rank of the two-GPU data-parallel check (started by test_gpu_dp_nccl.py with RANK / LOCAL_RANK / WORLD_SIZE /
MASTER_ADDR / MASTER_PORT in the environment, like torchrun does): a small residual network on the "omarchy_mac_torch"
device, gradients reduced by omarchy_mac_torch_b200.dp over NCCL, three SGD steps on this rank's shard. Writes what rank 0
saw to the file given as argv[1]."""
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class Block(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.c1, self.b1 = nn.Conv2d(c, c, 3, padding=1, bias=False), nn.BatchNorm2d(c)
        self.c2, self.b2 = nn.Conv2d(c, c, 3, padding=1, bias=False), nn.BatchNorm2d(c)

    def forward(self, x):
        return torch.relu(self.b2(self.c2(torch.relu(self.b1(self.c1(x))))) + x)


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, 32, 3, padding=1, bias=False), nn.BatchNorm2d(32), nn.ReLU())
        self.blocks = nn.Sequential(Block(32), Block(32))
        self.head = nn.Linear(32, 10)

    def forward(self, x):
        return self.head(self.blocks(self.stem(x)).mean((2, 3)))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    import omarchy_mac_torch_b200 as omt
    from omarchy_mac_torch_b200.dp import DataParallel
    torch.manual_seed(3 + rank)                      # deliberately different: the wrapper must align the replicas
    model = Net().to(omt.DEVICE)
    dp = DataParallel(model, bucket_mb=0.05)         # several buckets
    opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    g = torch.Generator().manual_seed(11)
    X, Y = torch.randn(16, 3, 16, 16, generator=g), torch.randint(0, 10, (16,), generator=g)
    xs, ys = X[rank * 8:(rank + 1) * 8].to(omt.DEVICE), Y[rank * 8:(rank + 1) * 8].to(omt.DEVICE)
    first = [p.detach().cpu().clone() for p in model.parameters()]
    losses = []
    for _ in range(3):
        dp.zero_grad()
        loss = F.cross_entropy(model(xs), ys)
        loss.backward()
        dp.finish()
        opt.step()
        losses.append(float(loss))
    spread = dp.param_spread()                        # a collective: max over parameters of (max - min) over ranks
    moved = max(float((p.detach().cpu() - q).abs().max()) for p, q in zip(model.parameters(), first))
    omt.synchronize()
    if rank == 0:
        state = {k: v.detach().cpu().tolist() for k, v in model.state_dict().items() if v.numel() <= 64}
        json.dump({"spread": spread, "moved": moved, "losses": losses, "buckets": len(dp.flat), "small_state": state}, open(sys.argv[1], "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
