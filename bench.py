"""Benchmark of the hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Prints ONE JSON line. A "step" is one pass of the hot path over one batch of synthetic input (seeded; the reference
benchmarks on random tensors too). Workloads:

  conv1     BASELINE config 1: AlexNet conv1 fwd + dgrad + wgrad, x[16,3,224,224], w[64,3,11,11], stride 4, pad 2
            (tools/gemm_bench.py "alex1"), called through the C ABI.
  plaincnn  BASELINE config 2: PlainCNN b128 training step (fwd+bwd+SGD) on the "omarchy_mac_torch" device.
  resnet18 / mobilenetv3 / resnet50   BASELINE configs 3-5, training step on the device; resnet50 is the multi-GPU one.

Timing: W >= 3 untimed warm-up steps, then K steps timed with CUDA events on the launching stream, a barrier and a
device synchronize on both sides, max over ranks; L2 is flushed between timed iterations whenever the step's working
set is smaller than L2. `value` has inputs resident in HBM; `e2e` runs the same step from pinned host buffers with the
host->device copies and the device->host read of the result inside the timed region. `--impl reference` times the
reference's CPU arm (PyTorch CPU aten, tools/acceptance.py:91) on the host cores for the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 << 20


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.t.join(timeout=2)
        sm, mx, reasons = [], None, set()
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx = float(f[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------------------
# workload: conv1 (C ABI)
# ---------------------------------------------------------------------------------------------------------------------

class Conv1:
    name = "alexnet_conv1_fwd_dgrad_wgrad"
    shape = dict(n=16, ci=3, co=64, hw=224, ks=11, stride=4, pad=2)
    flops = 3 * 2 * 16 * 64 * 55 * 55 * 3 * 11 * 11  # tools/gemm_bench.py:29, three passes
    metric, unit, higher = "conv_tflops", "TFLOP/s", True

    def host_inputs(self, seed):
        torch.manual_seed(seed)
        x = torch.randn(16, 3, 224, 224)
        conv = torch.nn.Conv2d(3, 64, 11, stride=4, padding=2)
        gy = torch.randn(16, 64, 55, 55)
        return x, conv.weight.detach().clone(), conv.bias.detach().clone(), gy

    def setup_gpu(self, seed):
        from omarchy_mac_torch_b200 import capi
        self.capi = capi
        capi.lib()
        self.h = [t.pin_memory() for t in self.host_inputs(seed)]
        self.d = [t.cuda() for t in self.h]
        self.staging = [torch.empty_like(t, device="cuda") for t in self.h]
        self.bytes_resident = sum(t.numel() * 4 for t in self.d) * 2

    def step(self, ins=None):
        c = self.capi
        x, w, b, gy = ins if ins is not None else self.d
        y = c.conv_fwd(x, w, b, 4, 2)
        dx = c.conv_dgrad(gy, w, (224, 224), 4, 2)
        dw = c.conv_wgrad(x, gy, 11, 4, 2)
        db = c.conv_bias_grad(gy)
        return y, dx, dw, db

    def e2e_step(self):
        for s, h in zip(self.staging, self.h):
            s.copy_(h, non_blocking=True)
        y, dx, dw, db = self.step(self.staging)
        return dw.sum().item()  # device->host read of a result scalar

    h2d_bytes = (16 * 3 * 224 * 224 + 64 * 3 * 121 + 64 + 16 * 64 * 55 * 55) * 4
    d2h_bytes = 4

    def value(self, ms):
        return self.flops / (ms * 1e-3) / 1e12

    def cpu_step(self, ins):
        x, w, b, gy = ins
        y = torch.nn.functional.conv2d(x, w, b, stride=4, padding=2)
        return torch.ops.aten.convolution_backward(gy, x, w, [64], [4, 4], [2, 2], [1, 1], False, [0, 0], 1, [True, True, True])

    def roofline(self, ms, peaks):
        # conv GEMMs: tensor pipe, 3xTF32-effective peak = tf32 dense (bf16/2) / 3
        peak = peaks["bf16_tflops"] / 2 / 3
        ach = self.flops / (ms * 1e-3) / 1e12
        return {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                "peak_source": f"{peaks['source']} bf16 burst / 2 (tf32) / 3 (3xTF32)"}


WORKLOADS = {"conv1": Conv1}


def dist_setup(n):
    if n <= 1:
        return 0, 1
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    return rank, world


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(v, world):
    if world <= 1:
        return v
    import torch.distributed as dist
    t = torch.tensor([v], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def time_steps(fn, steps, warmup, world, flush):
    for _ in range(warmup):
        fn()
    scratch = torch.empty(L2_BYTES * 2 // 4, device="cuda") if flush else None
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    barrier(world)
    for a, b in ev:
        if flush:
            scratch.fill_(1.0)  # evict L2 between timed iterations (outside the event pair)
        a.record()
        fn()
        b.record()
    barrier(world)
    total = sum(a.elapsed_time(b) for a, b in ev)
    return max_over_ranks(total / steps, world)


def run_reference(args, wl):
    """The reference's CPU arm: PyTorch CPU aten on all host cores (tools/acceptance.py:77,91)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ins = wl.host_inputs(0)
    for _ in range(max(1, args.warmup)):
        wl.cpu_step(ins)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        wl.cpu_step(ins)
    ms = (time.perf_counter() - t0) / args.steps * 1e3
    v = wl.value(ms)
    line = {"impl": "reference", "metric": wl.metric, "value": v, "unit": wl.unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": wl.higher, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": wl.name, **wl.shape},
            "cpu_baseline": {"value": v, "unit": wl.unit, "cores": cores, "kind": "reference",
                             "sample": f"{args.steps} full steps of PyTorch CPU aten ({torch.__version__}), {cores} threads"},
            "e2e": {"value": v, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="conv1", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    wl = WORKLOADS[args.workload]()
    if args.impl == "reference":
        return run_reference(args, wl)
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    rank, world = dist_setup(args.gpus)
    wl.setup_gpu(seed=rank)
    capi = wl.capi
    peaks = measured_peaks()
    flush = wl.bytes_resident < 2 * L2_BYTES
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    l0 = capi.lib().omt_launch_count()
    ms = time_steps(wl.step, args.steps, args.warmup, world, flush)
    launches = (capi.lib().omt_launch_count() - l0) // (args.steps + args.warmup)
    ms_e2e = time_steps(wl.e2e_step, args.steps, args.warmup, world, flush)
    clocks = sampler.stop() if rank == 0 else None
    if rank != 0:
        return
    line = {"metric": wl.metric, "value": wl.value(ms) * world, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": wl.higher, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl.name, **wl.shape, "l2": "flushed between timed iterations" if flush else "working set > L2"},
            "roofline": wl.roofline(ms, peaks),
            "e2e": {"value": wl.value(ms_e2e) * world, "unit": wl.unit, "ms_per_step": ms_e2e, "h2d_bytes_per_step": wl.h2d_bytes,
                    "d2h_bytes_per_step": wl.d2h_bytes},
            "gpu_launches": int(launches) * args.steps, "clocks": clocks}
    if not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        ins = wl.host_inputs(0)
        wl.cpu_step(ins)
        reps, t0 = 0, time.perf_counter()
        while reps < 3 or (time.perf_counter() - t0 < 10 and reps < 200):
            wl.cpu_step(ins)
            reps += 1
        cms = (time.perf_counter() - t0) / reps * 1e3
        line["cpu_baseline"] = {"value": wl.value(cms), "unit": wl.unit, "cores": cores, "kind": "reference", "ms_per_step": cms,
                                "sample": f"{reps} full steps of the same workload on PyTorch CPU aten, {cores} threads"}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
