"""Data-parallel training over the GPUs of one box: one process per GPU, batch sharded across ranks, parameters
replicated, BatchNorm on local batch statistics, and one collective: a bucketed all-reduce (average) of the gradients
that overlaps with the rest of the backward pass.

The reference is single-device (csrc/device.cpp:134 deviceCount() == 1); this is the exchange step a data-parallel job
adds around its hot path. Gradients are laid out the way the reference's fused stacks lay theirs out (one flat slab with
aligned slots, csrc/plans.cpp:54-60), so a bucket is reduced in place, with no gather copy:

  * parameters are assigned to buckets of at most `bucket_mb` in reverse registration order (the order backward produces
    them); every `param.grad` is a view of its bucket's flat tensor;
  * a post-accumulate-grad hook counts arrivals; when a bucket is complete its all-reduce is launched asynchronously
    (NCCL orders it after the kernels already queued on the compute stream and runs it on its own stream, so the input-
    gradient kernels of earlier layers keep running underneath);
  * `finish()` (called before the optimizer step) makes the compute stream wait for the outstanding reductions.

Works on any device torch.distributed supports: on the "omarchy_mac_torch" device buckets are handed to NCCL through a
CUDA alias of the same memory; on CPU tensors (gloo) the same logic runs unchanged, which is how it is unit-tested."""

import torch
import torch.distributed as dist


def assign_buckets(numels, bucket_elems):
    """Bucket index for each parameter, filling buckets in reverse order (last parameter first). Returns (bucket ids in
    parameter order, sizes per bucket)."""
    ids, sizes = [0] * len(numels), []
    cur, fill = 0, 0
    for i in reversed(range(len(numels))):
        n = numels[i]
        if fill and fill + n > bucket_elems:
            sizes.append(fill)
            cur, fill = cur + 1, 0
        ids[i] = cur
        fill += n
    if fill:
        sizes.append(fill)
    return ids, sizes


def _align(n, a=64):
    return (n + a - 1) // a * a


class DataParallel:
    """Wraps a model whose parameters all live on one device. Usage per step:

        dp.zero_grad(); loss = f(model(x)); loss.backward(); dp.finish(); optimizer.step()

    `optimizer.zero_grad()` in place of `dp.zero_grad()` works too (with set_to_none=True the gradients are moved back
    into their buckets as they arrive, at the cost of one copy each).
    """

    def __init__(self, model, bucket_mb=25.0, group=None, as_comm_tensor=None):
        self.model, self.group = model, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.params = [p for p in model.parameters() if p.requires_grad]
        assert self.params, "no trainable parameters"
        dev = self.params[0].device
        assert all(p.device == dev and p.dtype == torch.float32 for p in self.params), "float32 parameters on one device"
        if as_comm_tensor is None:
            if dev.type == "omarchy_mac_torch":
                from omarchy_mac_torch_b200.native import core
                as_comm_tensor = core.as_cuda
            else:
                as_comm_tensor = lambda t: t
        ids, _ = assign_buckets([p.numel() for p in self.params], int(bucket_mb * (1 << 20) / 4))
        self.bucket_of = ids
        nb = max(ids) + 1
        # slot offsets inside each bucket: 64-float (256-byte) aligned so vectorised kernels can use the views
        offs, fill = [0] * len(self.params), [0] * nb
        for i in reversed(range(len(self.params))):
            offs[i] = fill[ids[i]]
            fill[ids[i]] += _align(self.params[i].numel())
        self.flat = [torch.zeros(max(f, 64), device=dev, dtype=torch.float32) for f in fill]
        self.comm = [as_comm_tensor(f) for f in self.flat]
        self.expected = [ids.count(b) for b in range(nb)]
        self.arrived = [0] * nb
        self.pending = []
        self.launch_order = []  # bucket ids in the order their reductions were launched during the last backward
        self.views = [self.flat[ids[i]][offs[i]:offs[i] + p.numel()].view_as(p) for i, p in enumerate(self.params)]
        for i, p in enumerate(self.params):
            p.grad = self.views[i]
            p.register_post_accumulate_grad_hook(self._make_hook(ids[i], i))
        self.broadcast_parameters()

    def broadcast_parameters(self):
        """Replicate rank 0's parameters and buffers (identical seeds make this a no-op, but it removes the assumption)."""
        if self.world <= 1:
            return
        for t in list(self.model.parameters()) + list(self.model.buffers()):
            if t.is_floating_point():
                c = self._alias(t.data)
                dist.broadcast(c, 0, group=self.group)

    def _alias(self, t):
        if t.device.type == "omarchy_mac_torch":
            from omarchy_mac_torch_b200.native import core
            return core.as_cuda(t)
        return t

    def _make_hook(self, b, i=None):
        def hook(param):
            # `optimizer.zero_grad(set_to_none=True)` (torch's default) drops the view into the bucket, and the next backward
            # then leaves a fresh gradient tensor outside it: move it back in and re-attach the view, so that what gets
            # reduced is this step's gradient.
            if i is not None and param.grad is not None and param.grad.data_ptr() != self.views[i].data_ptr():
                self.views[i].copy_(param.grad)
                param.grad = self.views[i]
            self.arrived[b] += 1
            if self.arrived[b] == self.expected[b]:
                self._reduce(b)
        return hook

    def _reduce(self, b):
        self.launch_order.append(b)
        if self.world <= 1:
            return
        op = dist.ReduceOp.AVG if self.comm[b].is_cuda else dist.ReduceOp.SUM
        work = dist.all_reduce(self.comm[b], op=op, group=self.group, async_op=True)
        self.pending.append((work, b, op))

    def zero_grad(self):
        """Zero the gradient slabs (the views stay attached to the parameters)."""
        for f in self.flat:
            f.zero_()
        self.arrived = [0] * len(self.flat)
        self.launch_order = []

    def finish(self):
        """Wait for the outstanding bucket reductions; gradients then hold the average over ranks."""
        for work, b, op in self.pending:
            work.wait()
            if op == dist.ReduceOp.SUM:
                self.flat[b].div_(self.world)
        self.pending = []
        # parameters that took no part in this backward leave their bucket incomplete: reduce those buckets now
        for b, (got, want) in enumerate(zip(self.arrived, self.expected)):
            if got != want and self.world > 1:
                dist.all_reduce(self.comm[b], op=dist.ReduceOp.SUM, group=self.group)
                self.flat[b].div_(self.world)
        # ready for the next backward whichever way the caller clears gradients (dp.zero_grad() or the optimizer's own)
        self.arrived = [0] * len(self.flat)

    def param_spread(self):
        """max - min over ranks of a float64 checksum of all parameters (sum and sum of squares): 0.0 exactly when the
        replicas are still identical after a step, which is what averaged gradients and identical optimizers must give."""
        with torch.no_grad():
            acc = torch.zeros(2, dtype=torch.float64, device=self.params[0].device)
            for p in self.params:
                d = p.detach().double()
                acc[0] += d.sum()
                acc[1] += (d * d).sum()
        if self.world <= 1:
            return 0.0
        hi, lo = self._alias(acc.clone()), self._alias(acc.clone())
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.group)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.group)
        return float((hi - lo).abs().max().item())
