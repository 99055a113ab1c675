"""Benchmark of the hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Prints ONE JSON line. A "step" is one pass of the hot path over one batch of synthetic input (seeded; the reference
benchmarks on random tensors too). Workloads:

  resnet50  (default) ResNet-50 training step, batch 256 per GPU, 224x224, SGD nesterov, on the "omarchy_mac_torch"
            device; with --gpus N each rank takes its own batch (weak scaling) and gradients are averaged by the
            bucketed all-reduce of omarchy_mac_torch_b200.dp. This is the configuration the metric "train ms/step at
            1/2/4/8 B200" is quoted on, and it fits one GPU. At N = 1 the line also carries a `secondary` block: the
            AlexNet-conv1 layer, the ResNet-18 step and the bandwidth-bound kernel table, each a few seconds.
  plaincnn / resnet18 / mobilenetv3   the three-block CNN (batch 128, 32x32), ResNet-18 (batch 32, 64x64) and
            MobileNetV3-Small with squeeze-excite (batch 32, 224x224) training steps on the device.
  conv1     AlexNet conv1 fwd + dgrad + wgrad, x[16,3,224,224], w[64,3,11,11], stride 4, pad 2
            (tools/gemm_bench.py "alex1"), called through the C ABI.
  conv3x3   one 256->256 3x3 layer at 28x28, batch 128, channels-last (the small case of the ncu captures).
  hbm       every bandwidth-bound kernel family on tensors far larger than L2.

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

# DRAM traffic of the tensor-core conv kernels, from the ncu capture of the `conv3x3` workload (profiles/
# conv3x3_256_28_b128_tc_kernels_ncu_full.md): dram__bytes_read.sum + dram__bytes_write.sum per launch over the
# algorithmic bytes of that launch (float32 x + y + w = 207.96 MB). Traffic grows with the activation bytes, so a step's
# conv traffic is its algorithmic conv bytes per pass times these ratios.
NCU_CONV_TRAFFIC = {"fwd": (107.8 + 59.6) / 207.96, "dgrad": (108.0 + 60.3) / 207.96, "wgrad": (205.6 + 4.5) / 207.96}
NCU_CONV_TRAFFIC_SOURCE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of conv_tc_kernel / wgrad_tc_kernel on the conv3x3 case "
                           "(fwd 167.4, dgrad 168.3, wgrad 210.1 MB per launch; 208.0 MB algorithmic), scaled by algorithmic bytes per pass")


def conv_traffic(t, reps):
    """Bytes of DRAM traffic per step for the conv calls recorded in `t` (omt_conv_timing_*), by the measured ratios."""
    return sum(v[3] / reps * NCU_CONV_TRAFFIC[k] for k, v in t.items())


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

class ConvLayer:
    """One conv layer's forward + input gradient + weight gradient (+ bias gradient) through the C ABI."""
    metric, unit, higher = "conv_tflops", "TFLOP/s", True

    def __init__(self, name, n, ci, co, hw, ks, stride, pad, channels_last):
        self.name, self.n, self.ci, self.co, self.hw, self.ks, self.stride, self.pad, self.cl = name, n, ci, co, hw, ks, stride, pad, channels_last
        self.oh = (hw + 2 * pad - ks) // stride + 1
        self.shape = dict(n=n, ci=ci, co=co, hw=hw, ks=ks, stride=stride, pad=pad, layout="channels_last" if channels_last else "nchw")
        self.flops = 3 * 2 * n * co * self.oh * self.oh * ci * ks * ks  # tools/gemm_bench.py:29, three passes
        self.h2d_bytes = (n * ci * hw * hw + co * ci * ks * ks + co + n * co * self.oh * self.oh) * 4
        self.d2h_bytes = 4

    def host_inputs(self, seed):
        torch.manual_seed(seed)
        x = torch.randn(self.n, self.ci, self.hw, self.hw)
        conv = torch.nn.Conv2d(self.ci, self.co, self.ks, stride=self.stride, padding=self.pad)
        gy = torch.randn(self.n, self.co, self.oh, self.oh)
        if self.cl:
            x, gy = x.contiguous(memory_format=torch.channels_last), gy.contiguous(memory_format=torch.channels_last)
        return x, conv.weight.detach().clone(), conv.bias.detach().clone(), gy

    def cpu_setup(self):
        return self.host_inputs(0)

    def cpu_scale(self):
        return 1.0

    def setup_gpu(self, seed, world=1):
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
        y = c.conv_fwd(x, w, b, self.stride, self.pad, cl=self.cl)
        dx = c.conv_dgrad(gy, w, (self.hw, self.hw), self.stride, self.pad, cl=self.cl)
        dw = c.conv_wgrad(x, gy, self.ks, self.stride, self.pad)
        db = c.conv_bias_grad(gy)
        return y, dx, dw, db

    def e2e_step(self):
        for s, h in zip(self.staging, self.h):
            s.copy_(h, non_blocking=True)
        y, dx, dw, db = self.step(self.staging)
        return dw.sum().item()  # device->host read of a result scalar

    def value(self, ms):
        return self.flops / (ms * 1e-3) / 1e12

    def cpu_step(self, ins):
        x, w, b, gy = ins
        y = torch.nn.functional.conv2d(x, w, b, stride=self.stride, padding=self.pad)
        return torch.ops.aten.convolution_backward(gy, x, w, [self.co], [self.stride] * 2, [self.pad] * 2, [1, 1], False, [0, 0], 1, [True, True, True])

    def roofline(self, ms, peaks):
        # conv GEMMs: tensor pipe, 3xTF32-effective peak = tf32 dense (bf16/2) / 3; per pass from the library's CUDA-event timing
        self.capi.conv_timing(True)
        for _ in range(3):
            self.step()
        torch.cuda.synchronize()
        t = self.capi.conv_timing_read(reset=True)
        self.capi.conv_timing(False)
        peak = peaks["bf16_tflops"] / 2 / 3
        ach = self.flops / (ms * 1e-3) / 1e12
        return {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                "traffic": conv_traffic(t, 3), "traffic_source": NCU_CONV_TRAFFIC_SOURCE, "algorithmic_bytes": sum(v[3] for v in t.values()) / 3,
                "peak_source": f"{peaks['source']} bf16 burst / 2 (tf32) / 3 (3xTF32)",
                "kernel": "conv fwd + dgrad + wgrad of one layer (all kernels of the three calls)",
                "per_pass": {k: {"tflops": (v[0] / (v[1] * 1e-3) / 1e12 if v[1] else None), "ms": v[1] / 3, "calls": v[2] // 3} for k, v in t.items()}}


CONV = {
    # the AlexNet conv1 shape, NCHW as the reference benchmarks it (tools/gemm_bench.py)
    "conv1": lambda: ConvLayer("alexnet_conv1_fwd_dgrad_wgrad", 16, 3, 64, 224, 11, 4, 2, False),
    # a mid-network ResNet layer, channels-last, inputs + outputs larger than L2: the small case the ncu captures use
    "conv3x3": lambda: ConvLayer("conv3x3_256_28_b128_fwd_dgrad_wgrad", 128, 256, 256, 28, 3, 1, 1, True),
}


class HbmKernels:
    """The bandwidth-bound kernels of the path, each on tensors far larger than L2, through the C ABI: achieved GB/s =
    algorithmic bytes / CUDA-event time. `value` is the geometric mean over the kernels; `roofline` reports the slowest."""
    name = "hbm_bound_kernels"
    metric, unit, higher = "hbm_kernels_gbs", "GB/s", True
    shape = dict(bn="256x64x112x112 channels-last", depthwise="128x96x56x56 3x3 and 5x5 stride 1; 64x96x112x112 -> 56x56 stride 2; channels-last", optimizer="64M parameters in 160 tensors")
    h2d_bytes = d2h_bytes = 0

    def setup_gpu(self, seed, world=1):
        from omarchy_mac_torch_b200 import capi
        self.capi = capi
        capi.lib()
        torch.manual_seed(seed)
        cl = torch.channels_last
        x = torch.randn(256, 64, 112, 112, device="cuda").contiguous(memory_format=cl)
        g = torch.randn_like(x)
        c = x.shape[1]
        gamma, beta, rm, rv = torch.rand(c, device="cuda") + 0.5, torch.randn(c, device="cuda"), torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
        mean, var, inv = (torch.empty(c, device="cuda") for _ in range(3))
        y = torch.empty_like(x)
        dx = torch.empty_like(x)
        dgb = torch.empty(2, c, device="cuda")
        n, _, h, w = x.shape
        A, P, sh = capi.act, capi.ptr, capi.stream_handle
        ne = x.numel()
        xd = torch.randn(128, 96, 56, 56, device="cuda").contiguous(memory_format=cl)
        wd = torch.randn(96, 1, 3, 3, device="cuda")
        gd = torch.randn_like(xd)
        nd = xd.numel()
        wd5 = torch.randn(96, 1, 5, 5, device="cuda")
        xs2 = torch.randn(64, 96, 112, 112, device="cuda").contiguous(memory_format=cl)   # stride-2 cases: 112^2 -> 56^2
        gs2 = torch.randn(64, 96, 56, 56, device="cuda").contiguous(memory_format=cl)
        ns2 = xs2.numel() + gs2.numel()
        params = [torch.randn(400_000, device="cuda") for _ in range(160)]
        grads = [torch.randn_like(t) for t in params]
        ms_ = [torch.zeros_like(t) for t in params]
        vs_ = [torch.zeros_like(t) for t in params]
        steps = [torch.zeros((), device="cuda") for _ in params]
        npar = sum(t.numel() for t in params)
        call = capi.call
        yp, ip = capi.maxpool_fwd(x, 3, 2, 1)   # indices and a gradient for the max-pool backward case
        gp = torch.randn_like(yp)
        self.keep_pool = (yp, ip, gp)
        self.keep = (x, g, y, dx, xd, gd, xs2, gs2, wd5, params, grads, ms_, vs_, steps)
        self.kernels = {
            # name: (callable, algorithmic bytes)
            "bn_statistics": (lambda: call("omt_bn_stats", A(x), n, c, h, w, P(mean), P(var), P(inv), P(rm), P(rv), None, None, 0.1, 1e-5, 0, sh()), 4 * ne),
            "bn_apply_relu": (lambda: call("omt_bn_apply", A(x), A(y), n, c, h, w, P(mean), P(inv), P(gamma), P(beta), capi.BN_RELU, sh()), 8 * ne),
            "bn_backward_relu": (lambda: call("omt_bn_backward", A(g), A(x), A(y), A(dx), n, c, h, w, P(mean), P(inv), P(gamma), P(dgb), 1.0, capi.BN_RELU, sh()), 24 * ne),
            "depthwise_fwd": (lambda: capi.dw_fwd(xd, wd, None, 1, 1, cl=True), 8 * nd),
            "depthwise_dgrad": (lambda: capi.dw_dgrad(gd, wd, (56, 56), 1, 1, cl=True), 8 * nd),
            "depthwise_wgrad": (lambda: capi.dw_wgrad(xd, gd, 3, 1, 1), 8 * nd),
            "depthwise5x5_fwd": (lambda: capi.dw_fwd(xd, wd5, None, 1, 2, cl=True), 8 * nd),
            "depthwise5x5_dgrad": (lambda: capi.dw_dgrad(gd, wd5, (56, 56), 1, 2, cl=True), 8 * nd),
            "depthwise5x5_wgrad": (lambda: capi.dw_wgrad(xd, gd, 5, 1, 2), 8 * nd),
            "depthwise3x3s2_fwd": (lambda: capi.dw_fwd(xs2, wd, None, 2, 1, cl=True), 4 * ns2),
            "depthwise3x3s2_dgrad": (lambda: capi.dw_dgrad(gs2, wd, (112, 112), 2, 1, cl=True), 4 * ns2),
            "depthwise3x3s2_wgrad": (lambda: capi.dw_wgrad(xs2, gs2, 3, 2, 1), 4 * ns2),
            "depthwise5x5s2_fwd": (lambda: capi.dw_fwd(xs2, wd5, None, 2, 2, cl=True), 4 * ns2),
            "maxpool3x3s2_fwd": (lambda: capi.maxpool_fwd(x, 3, 2, 1), 4 * ne + 12 * (ne // 4)),
            "maxpool3x3s2_bwd": (lambda: capi.maxpool_bwd(gp, ip, (h, w), 3, 2, 1), 4 * ne + 12 * (ne // 4)),
            "sgd_momentum": (lambda: capi.sgd(params, grads, ms_, 0.1, momentum=0.9, weight_decay=1e-4), 20 * npar),
            "adamw": (lambda: capi.adam(params, grads, ms_, vs_, steps, 1e-3, weight_decay=0.01, decoupled=True), 28 * npar),
        }
        self.bytes_resident = 1 << 40
        self.results = {}

    def step(self):
        for fn, _ in self.kernels.values():
            fn()

    e2e_step = step

    def measure(self, reps=10):
        for name, (fn, nbytes) in self.kernels.items():
            for _ in range(3):
                fn()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / reps
            self.results[name] = {"ms": ms, "gbs": nbytes / ms / 1e6, "bytes": nbytes}

    def value(self, ms):
        if not self.results:
            self.measure()
        return float(np.exp(np.mean([np.log(r["gbs"]) for r in self.results.values()])))

    def roofline(self, ms, peaks):
        if not self.results:
            self.measure()
        peak = peaks["hbm_gbs"]
        worst = min(self.results, key=lambda k: self.results[k]["gbs"])
        return {"bound": "hbm", "achieved": self.results[worst]["gbs"], "peak": peak, "unit": "GB/s", "frac": self.results[worst]["gbs"] / peak,
                "traffic": None, "kernel": worst, "peak_source": f"{peaks['source']} copy bandwidth",
                "per_kernel": {k: {"gbs": round(r["gbs"], 1), "frac": round(r["gbs"] / peak, 3), "ms": round(r["ms"], 4)} for k, r in self.results.items()}}

    def cpu_setup(self):
        return None

    def cpu_step(self, ins):
        x = torch.randn(16, 64, 112, 112)
        torch.nn.functional.batch_norm(x, None, None, training=True)

    def cpu_scale(self):
        return 1.0


# ---------------------------------------------------------------------------------------------------------------------
# training workloads on the "omarchy_mac_torch" device
# ---------------------------------------------------------------------------------------------------------------------

class Train:
    metric, unit, higher = "train_ms_per_step", "ms/step", False
    # compile=True: call the model through torch.compile(backend="omarchy_mac_torch") (fused BatchNorm/ReLU/residual graphs);
    # the small, launch-bound workloads are faster through the eager nn.Module call with the Sequential auto-fuse, and replay
    # the whole step as one CUDA graph (graph=True; omarchy_mac_torch_b200.graphs.capture). --eager / --compile / --graph /
    # --no-graph override.

    def __init__(self, name, make_model, shape, classes, make_opt, cpu_batch, note, compile=False, graph=False, regions=False):
        self.compile, self.graph, self.regions = compile, graph, regions
        self.name, self.make_model, self.in_shape, self.classes, self.make_opt = name, make_model, shape, classes, make_opt
        self.cpu_batch = min(cpu_batch, shape[0])
        self.shape = {"batch_per_gpu": shape[0], "input": list(shape[1:]), "classes": classes, "optimizer": note, "api": ""}
        self.set_api()

    def set_api(self):
        if self.compile and self.regions:
            api = 'omarchy_mac_torch_b200.compile.compile_regions(model): torch.compile(backend="omarchy_mac_torch") of the stem and of each block'
        elif self.compile:
            api = 'torch.compile(model, backend="omarchy_mac_torch")'
        else:
            api = "eager nn.Module"
        self.shape["api"] = api + (" + omarchy_mac_torch_b200.graphs.capture(step)" if self.graph else "")

    def host_inputs(self, seed, batch=None):
        g = torch.Generator().manual_seed(1000 + seed)
        b = batch or self.in_shape[0]
        return torch.randn(b, *self.in_shape[1:], generator=g), torch.randint(0, self.classes, (b,), generator=g)

    def build_model(self):
        torch.manual_seed(0)  # identical initial weights on every rank
        m = self.make_model()
        for mod in m.modules():
            if isinstance(mod, torch.nn.Dropout):
                mod.p = 0.0
        return m

    def setup_gpu(self, seed, world=1):
        import omarchy_mac_torch_b200 as omt
        from omarchy_mac_torch_b200 import capi
        from omarchy_mac_torch_b200.native import core
        self.capi, self.core, self.dev = capi, core, omt.DEVICE
        capi.lib()
        self.model = self.build_model().to(self.dev)
        # the package's compile backend: BatchNorm+ReLU(+residual add) fused in forward and backward graphs. A model that names
        # its regions is compiled region by region, so that each region's gradients reach the data-parallel hooks as soon as
        # its own backward graph is done (the bucket all-reduces then overlap the rest of the backward pass).
        if self.compile and self.regions:
            from omarchy_mac_torch_b200.compile import compile_regions
            self.fwd = compile_regions(self.model)
        else:
            self.fwd = torch.compile(self.model, backend="omarchy_mac_torch") if self.compile else self.model
        self.dp = None
        if world > 1:
            from omarchy_mac_torch_b200.dp import DataParallel
            self.dp = DataParallel(self.model, bucket_mb=25.0)
        # (AdamW inside a captured CUDA graph keeps its step counters on the device: capturable=True)
        self.opt = self.make_opt(self.model.parameters(), capturable=True) if (self.graph and "AdamW" in self.shape["optimizer"]) \
            else self.make_opt(self.model.parameters())
        xh, yh = self.host_inputs(seed)
        self.xh, self.yh = xh.pin_memory(), yh.pin_memory()
        self.x, self.y = self.xh.to(self.dev), self.yh.to(self.dev)
        self.xs, self.ys = torch.empty_like(self.x), torch.empty_like(self.y)
        self.bytes_resident = 1 << 40  # activations of a training step are far larger than L2: no flush needed
        self.h2d_bytes = self.xh.numel() * 4 + self.yh.numel() * 8
        self.d2h_bytes = 4

    def _step(self, x, y):
        if self.dp is not None:
            self.dp.zero_grad()
        else:
            self.opt.zero_grad(set_to_none=True)
        loss = torch.nn.functional.cross_entropy(self.fwd(x), y)
        loss.backward()
        if self.dp is not None:
            self.dp.finish()
        self.opt.step()
        return loss

    def step(self):
        if self.graph:
            return self._graphed()()
        return self._step(self.x, self.y)

    def _graphed(self):
        """The whole step (zero_grad, forward, backward, optimizer) as one CUDA graph over the static batch tensors."""
        if not hasattr(self, "_g"):
            from omarchy_mac_torch_b200 import graphs
            self._g = graphs.capture(lambda: self._step(self.x, self.y))
            self.launches_per_step = self._g.kernels
        return self._g

    def e2e_step(self):
        return self._e2e_prefetch()

    def _run(self, x, y):
        """One step on the device batch (x, y): the eager / compiled step, or a device-to-device copy into the recorded step's
        static batch followed by its replay."""
        if self.graph:
            g = self._graphed()
            self.x.copy_(x)
            self.y.copy_(y)
            return g()
        return self._step(x, y)

    def _e2e_prefetch(self):
        """One step fed from pinned host memory, as a prefetching data loader feeds it: this step's batch was copied to one
        of two device buffers on a side stream while the previous step computed; the copy of the next step's batch is
        issued now. Every step copies its whole batch host->device and reads its loss back, all inside the timed region."""
        if not hasattr(self, "_pf"):
            side = torch.cuda.Stream()
            bufs = [(self.xs, self.ys), (torch.empty_like(self.xs), torch.empty_like(self.ys))]
            ready = [torch.cuda.Event(), torch.cuda.Event()]   # copy into buffer k finished
            freed = [torch.cuda.Event(), torch.cuda.Event()]   # compute that read buffer k finished
            self._pf = {"side": side, "bufs": bufs, "ready": ready, "freed": freed, "i": 0}
            self._prefetch(0, first=True)
        pf = self._pf
        k = pf["i"] % 2
        torch.cuda.current_stream().wait_event(pf["ready"][k])
        self._prefetch(1 - k)
        x, y = pf["bufs"][k]
        loss = self._run(x, y)
        pf["freed"][k].record(torch.cuda.current_stream())
        pf["i"] += 1
        return loss.item()  # device->host read of the loss

    def _prefetch(self, k, first=False):
        pf = self._pf
        with torch.cuda.stream(pf["side"]):
            if not first:
                pf["side"].wait_event(pf["freed"][k])  # the step that last read this buffer (recorded before its reuse)
            x, y = pf["bufs"][k]
            x.copy_(self.xh, non_blocking=True)
            y.copy_(self.yh, non_blocking=True)
            pf["ready"][k].record(pf["side"])

    def value(self, ms):
        return ms

    def cpu_setup(self):
        self.cpu_model = self.build_model()
        self.cpu_opt = self.make_opt(self.cpu_model.parameters())
        return self.host_inputs(0, self.cpu_batch)

    def cpu_step(self, ins):
        x, y = ins
        self.cpu_opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(self.cpu_model(x), y)
        loss.backward()
        self.cpu_opt.step()
        return loss

    def cpu_scale(self):  # CPU sample batch -> full per-GPU batch
        return self.in_shape[0] / self.cpu_batch

    def roofline(self, ms, peaks):
        # conv GEMMs measured live: two extra steps with the library's per-call CUDA-event timing switched on
        if self.graph:  # the timed steps were replays: let the eager steps fill the allocator's cache for this stream first
            for _ in range(2):
                self._step(self.x, self.y)
            torch.cuda.synchronize()
        self.capi.conv_timing(True)
        for _ in range(2):
            self._step(self.x, self.y)  # eager even when the timed steps were graph replays: the timing wraps each call
        torch.cuda.synchronize()
        t = self.capi.conv_timing_read(reset=True)
        self.capi.conv_timing(False)
        flops = sum(v[0] for v in t.values()) / 2
        conv_ms = sum(v[1] for v in t.values()) / 2
        # the same work by kernel: one more step with every launch of the library bracketed by CUDA events, summed per kernel
        # name. The GEMM kernels alone (conv_tc_<tile>, wgrad_tc_<tile>) against everything a conv call launches (weight
        # re-lay, staging copies, split-K reductions included), which is what `achieved` above is computed from.
        self.core.kernel_times(True)
        self.core.debug_time_kernels(True)
        try:
            self._step(self.x, self.y)
            torch.cuda.synchronize()
            kt = self.core.kernel_times(True)
        finally:
            self.core.debug_time_kernels(False)
        helpers = ("conv_tc_weight_split", "conv_tc_stage_window", "conv_tc_splitk_epilogue", "wgrad_tc_reduce")
        gemm_ms = sum(v for k, v in kt.items() if k.startswith(("conv_tc_", "wgrad_tc_")) and k not in helpers)
        helper_ms = sum(v for k, v in kt.items() if k in helpers)
        sustained = peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]
        peak = sustained / 2 / 3
        ach = flops / (conv_ms * 1e-3) / 1e12 if conv_ms else 0.0
        return {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                "traffic": conv_traffic(t, 2), "traffic_source": NCU_CONV_TRAFFIC_SOURCE, "algorithmic_bytes": sum(v[3] for v in t.values()) / 2,
                "peak_source": f"{peaks['source']} bf16 sustained / 2 (tf32) / 3 (3xTF32)",
                "kernel": "dense conv fwd + dgrad + wgrad (all conv calls of one step)",
                "conv_flops_per_step": flops, "conv_ms_per_step": conv_ms, "conv_share_of_step": conv_ms / ms if ms else None,
                "gemm_kernels_only": {"ms_per_step": gemm_ms, "helper_kernels_ms": helper_ms,
                                      "achieved": flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms else None,
                                      "frac": flops / (gemm_ms * 1e-3) / 1e12 / peak if gemm_ms else None,
                                      "how": "per-kernel CUDA events over one extra step (omt_kernel_timing): conv_tc_<tile> + wgrad_tc_<tile> launches only"},
                "per_pass": {k: {"tflops": (v[0] / (v[1] * 1e-3) / 1e12 if v[1] else None), "ms": v[1] / 2, "calls": v[2] // 2} for k, v in t.items()}}


def _models():
    from omarchy_mac_torch_b200 import models
    return models


def _sgd(lr, **kw):
    return lambda p: torch.optim.SGD(p, lr=lr, **kw)


TRAIN = {
    "plaincnn": lambda: Train("plaincnn_b128_train", lambda: _models().PlainCNN3(), (128, 3, 32, 32), 10, _sgd(0.05, momentum=0.9), 128,
                              "SGD lr .05 momentum .9", graph=True),
    "resnet18": lambda: Train("resnet18_b32_train", lambda: _models().kaiming_normal_convs(_models().ResNet18(num_classes=1000)),
                              (32, 3, 64, 64), 1000, _sgd(0.1, momentum=0.9, weight_decay=1e-4), 32, "SGD lr .1 momentum .9 wd 1e-4", graph=True),
    "mobilenetv3": lambda: Train("mobilenetv3_small_b32_train", lambda: _models().MobileNetV3SE(), (32, 3, 224, 224), 1000,
                                 lambda p, capturable=False: torch.optim.AdamW(p, lr=1e-3, weight_decay=0.01, capturable=capturable), 32, "AdamW lr 1e-3 wd .01",
                                 graph=True),
    "resnet50": lambda: Train("resnet50_b256_train", lambda: _models().ResNet50(), (256, 3, 224, 224), 1000,
                              _sgd(0.1, momentum=0.9, nesterov=True, weight_decay=1e-4), 256, "SGD lr .1 momentum .9 nesterov wd 1e-4",
                              compile=True),
}

WORKLOADS = {**CONV, **TRAIN, "hbm": HbmKernels}


def dist_setup(n):
    if n <= 1:
        return 0, 1
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    import datetime
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()),
                            timeout=datetime.timedelta(seconds=180))  # a lost rank ends the job in minutes, not the default 10
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


def secondary(peaks):
    """Short measurements of the other named targets, carried beside the headline so that one run records them: the
    AlexNet-conv1 layer through the C ABI (TFLOP/s of fwd+dgrad+wgrad against the burst 3xTF32 peak), the PlainCNN, ResNet-18
    and MobileNetV3 training steps (ms, kernels per step) and the bandwidth-bound kernel table (GB/s against the measured copy bandwidth). Same timing rules as the
    headline (warm-up, CUDA events, L2 flushed where the working set is smaller than L2)."""
    out = {}
    for key, name, steps in (("conv1", "conv1", 30), ("plaincnn", "plaincnn", 30), ("resnet18", "resnet18", 30), ("mobilenetv3", "mobilenetv3", 20),
                             ("hbm", "hbm", 1)):
        try:
            w = WORKLOADS[name]()
            w.setup_gpu(seed=0, world=1)
            if name == "hbm":
                roof = w.roofline(0.0, peaks)
                out[key] = {"unit": "GB/s", "peak": roof["peak"], "per_kernel": roof["per_kernel"], "slowest": roof["kernel"]}
            else:
                flush = w.bytes_resident < 2 * L2_BYTES
                ms = time_steps(w.step, steps, 5, 1, flush)
                out[key] = {"workload": w.name, "ms_per_step": ms, "value": w.value(ms), "unit": w.unit, **w.shape,
                            "l2": "flushed between timed iterations" if flush else "working set > L2"}
                if name == "conv1":
                    roof = w.roofline(ms, peaks)
                    out[key].update(frac=roof["frac"], peak=roof["peak"], peak_source=roof["peak_source"], per_pass=roof["per_pass"])
                elif getattr(w, "launches_per_step", None):
                    out[key]["kernels_per_step"] = w.launches_per_step
            del w
            torch.cuda.synchronize()
        except Exception as e:  # a failure here must not take the headline line with it
            out[key] = {"error": f"{type(e).__name__}: {e}"[:300]}
    return out


def config_of(wl, world):
    """The `config` object: identical keys and values in this arm's line and in the reference arm's."""
    cfg = {"workload": wl.name, **wl.shape}
    if not wl.higher:
        cfg["parallelism"] = f"dp{world}"
    return cfg


def cpu_arm(wl, warmup, steps, budget_s):
    """Times the reference's CPU arm (PyTorch CPU aten on every host core, tools/acceptance.py:77,91) on the workload's own
    shapes. One step is always run untimed first; if `warmup + steps` steps at that step's duration fit in `budget_s`
    they all run, otherwise the remaining warm-up is dropped and as many timed steps as fit (at least 2) run. Returns
    (ms per step, timed steps, warm-up steps, threads)."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ins = wl.cpu_setup()
    t0 = time.perf_counter()
    wl.cpu_step(ins)
    first = time.perf_counter() - t0
    warm = 1
    if (warmup - 1 + steps) * first <= budget_s:
        for _ in range(warmup - 1):
            wl.cpu_step(ins)
            warm += 1
    else:
        steps = int(max(2, min(steps, (budget_s - first) // max(first, 1e-9))))
    t0 = time.perf_counter()
    for _ in range(steps):
        wl.cpu_step(ins)
    ms = (time.perf_counter() - t0) / steps * 1e3 * wl.cpu_scale()
    return ms, steps, warm, cores


def cpu_sample_text(wl, steps, warm, cores):
    return (f"{steps} timed steps after {warm} warm-up of the same workload at its full size on PyTorch CPU aten ({torch.__version__}), "
            f"{cores} threads" + (f", batch {wl.cpu_batch} scaled x{wl.cpu_scale():g} to the full batch" if wl.cpu_scale() != 1 else ""))


def run_reference(args, wl):
    """The reference's CPU arm: PyTorch CPU aten on all host cores (tools/acceptance.py:77,91)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ms, steps, warm, cores = cpu_arm(wl, args.warmup, args.steps, budget_s=240.0)
    v = wl.value(ms)
    line = {"impl": "reference", "metric": wl.metric, "value": v, "unit": wl.unit, "n_gpus": args.gpus, "steps": steps,
            "warmup": warm, "ms_per_step": ms, "higher_is_better": wl.higher, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": config_of(wl, args.gpus),
            "cpu_baseline": {"value": v, "unit": wl.unit, "cores": cores, "kind": "reference", "sample": cpu_sample_text(wl, steps, warm, cores)},
            "e2e": {"value": v, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="resnet50", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="resnet50 at N=1: skip the extra conv1 / resnet18 / hbm measurements")
    ap.add_argument("--eager", action="store_true", help="training workloads: call the nn.Module directly instead of through the compile backend")
    ap.add_argument("--compile", action="store_true", help="training workloads: call the model through the compile backend")
    ap.add_argument("--graph", action="store_true", help="training workloads on one GPU: replay the whole step as one CUDA graph")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--regions", action="store_true",
                    help="compile the model region by region (compile.compile_regions) instead of as one graph: gradient buckets then "
                         "reduce under the backward pass, at the price of some host time per region")
    ap.add_argument("--profile-step", action="store_true",
                    help="for ncu --profile-from-start off: after the warm-up run ONE step between cudaProfilerStart/Stop and exit")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    wl = WORKLOADS[args.workload]()
    if args.workload == "hbm":
        args.no_cpu_baseline = True  # a per-kernel bandwidth table has no single CPU counterpart
    if isinstance(wl, Train):
        if args.eager or args.compile:
            wl.compile = args.compile and not args.eager
        if args.regions:
            wl.regions = True
        if args.graph or args.no_graph:
            wl.graph = args.graph and not args.no_graph
        wl.set_api()
    if args.impl == "reference":
        return run_reference(args, wl)
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    rank, world = dist_setup(args.gpus)
    if isinstance(wl, Train) and world > 1 and wl.graph:
        # data-parallel steps are launched kernel by kernel: a recorded step with its NCCL all-reduces replays correctly
        # (measured on 2 GPUs), but the process then hung in its teardown
        wl.graph = False
        wl.set_api()
    wl.setup_gpu(seed=rank, world=world)
    capi = wl.capi
    peaks = measured_peaks()
    flush = wl.bytes_resident < 2 * L2_BYTES
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    if args.profile_step:
        for _ in range(args.warmup):
            wl.step()
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        wl.step()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled": wl.name, "kernel_counts": capi.kernel_counts()}))
        return
    l0 = capi.lib().omt_launch_count()
    ms = time_steps(wl.step, args.steps, args.warmup, world, flush)
    launches = (capi.lib().omt_launch_count() - l0) // (args.steps + args.warmup)
    if getattr(wl, "launches_per_step", None):  # a replayed CUDA graph: the kernels recorded at capture, per replay
        launches = wl.launches_per_step
    ms_e2e = time_steps(wl.e2e_step, args.steps, args.warmup, world, flush)
    clocks = sampler.stop() if rank == 0 else None
    roof = wl.roofline(ms, peaks)  # runs extra steps: every rank takes part (they contain the gradient all-reduce)
    spread = wl.dp.param_spread() if getattr(wl, "dp", None) is not None else None  # a collective: every rank calls it
    barrier(world)
    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return
    agg = world if wl.higher else 1  # throughput metrics aggregate over ranks; a step time does not
    line = {"metric": wl.metric, "value": wl.value(ms) * agg, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": wl.higher, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": config_of(wl, world), "l2": "flushed between timed iterations" if flush else "working set > L2",
            "roofline": roof,
            "e2e": {"value": wl.value(ms_e2e) * agg, "unit": wl.unit, "ms_per_step": ms_e2e, "h2d_bytes_per_step": wl.h2d_bytes,
                    "d2h_bytes_per_step": wl.d2h_bytes},
            "gpu_launches": int(launches) * args.steps, "clocks": clocks}
    if not wl.higher:
        line["images_per_s"] = wl.in_shape[0] * world / (ms * 1e-3)
    if spread is not None:  # replicas must end a step with bit-identical parameters: exactly 0
        line["rank_param_spread"] = spread
    if args.workload == "resnet50" and world == 1 and not args.no_secondary:
        line["secondary"] = secondary(peaks)
    if not args.no_cpu_baseline and world == 1:  # (multi-GPU runs hold their GPUs while this runs: single-GPU line only)
        # bounded sample of the same workload at its full size: one untimed step, then as many as fit in ~20 s (at least 2)
        cms, csteps, cwarm, cores = cpu_arm(wl, 1, 200, budget_s=20.0)
        line["cpu_baseline"] = {"value": wl.value(cms), "unit": wl.unit, "cores": cores, "kind": "reference", "ms_per_step": cms,
                                "sample": cpu_sample_text(wl, csteps, cwarm, cores)}
    print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
