"""Benchmark of the population-batched perturbed-layer path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (the configuration the headline metric is quoted on): ``perturbed_linear_1024``
= PerturbedLinear 1024x1024 with 1024 dense Gaussian noise matrices (4 GiB fp32), antithetic
(batch 2048), one step = population forward + fitness-weighted update.  At N > 1 every rank
owns 1024 members of a 1024*N population (weak scaling); the forward needs no communication
and the update is summed with one NCCL all-reduce.  Other workloads: ``permuted_linear_256``,
``permuted_conv_64``, ``binary_1024`` (the remaining single-layer configurations).

One JSON line is printed by rank 0.  ``value`` is member-samples per second with inputs
resident in HBM; ``e2e`` is the same through the layer API with pinned host buffers and the
host<->device copies inside the timed region; ``roofline`` describes the dominant kernel;
``cpu_baseline`` is the reference's own CPU path (its unmodified ``modules/base.py``, a copy of
which the build step keeps under ``oracle/_ref``) or, where the reference has none, the CPU
restatement under ``oracle/``, timed on the host cores on a bounded sample.  The default run adds
``sustained`` (the same step repeated for at least a second), ``es_step`` (ES steps/s of the small
CNN), ``per_config`` (the other single-layer configurations) and ``gpu_reference`` (the reference's
PyTorch layers on the same GPU); at N > 1 ``strong`` (the population of 1024 split over the GPUs)
and ``allreduce_check``.  ``--impl reference`` runs the CPU arm only.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

# stdout of this program is ONE JSON line.  Libraries write to file descriptor 1 too (NCCL prints its version
# banner there), so descriptor 1 is pointed at stderr and the JSON line goes to a private copy of the real stdout.
_JSON_OUT = os.fdopen(os.dup(1), "w")
os.dup2(2, 1)


def emit(line):
    _JSON_OUT.write(json.dumps(line) + "\n")
    _JSON_OUT.flush()


import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


# ---------------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []          # (host time when read, csv line)
        self.t_begin = self.t_end = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def wait_first_sample(self, timeout=3.0):
        t0 = time.time()
        while self.proc is not None and not self.lines and time.time() - t0 < timeout:
            time.sleep(0.02)

    def begin(self):
        self.t_begin = time.time()

    def end(self):
        self.t_end = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [l for t, l in self.lines if self.t_begin is not None and self.t_begin <= t <= (self.t_end or t) + 0.1]
        window = "timed region"
        if not inside:
            inside = [l for _, l in self.lines]
            window = "whole run (timed region shorter than the sampling period)"
        for line in inside:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "window": window,
                "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------- workloads

class Workload:
    name = ""
    dtype = "f32"
    tc = None                   # tensor-core mode override (--tc)
    units_per_step = 0          # member-samples one rank processes per step
    resident_bytes = 0          # working set touched per step (decides whether L2 must be flushed)
    cpu_cores = None            # threads the CPU sample uses when it is not torch's pool

    def mode(self):
        """Arithmetic path the layer took (its ``last_path``), or the requested mode."""
        layer = getattr(self, "layer", None)
        return getattr(layer, "last_path", None) or self.tc or "default"


class PerturbedLinear1024(Workload):
    """PerturbedLinear 1024x1024 with 1024 dense Gaussian noise matrices (4 GiB), antithetic: forward + update."""
    name = "perturbed_linear_1024"
    D, R, n = 1024, 2, 1024
    overlap_blocks = 0          # --overlap-update N: gradient in N column blocks, each all-reduced while the next streams

    def __init__(self, members=None):
        if members:
            self.D = members        # reduced member count: profiling captures only
        self.units_per_step = self.D * self.R
        self.resident_bytes = self.D * self.n * self.n * 4

    def describe(self, world):
        return {"workload": self.name, "layer": "PerturbedLinear(1024,1024)", "directions_per_gpu": self.D,
                "population": self.D * world, "batch_per_gpu": self.D * self.R, "antithetic": True,
                "noise_bytes_per_gpu": self.resident_bytes, "step": "forward + update (+ all-reduce at N>1)",
                "l2": "inputs exceed L2 (4 GiB noise streamed per phase)", "sharding": "members"}

    def setup(self, dev, rank, world):
        from nesgpu_b200 import base, dist as ndist
        self.ndist, self.world = ndist, world
        g = torch.Generator().manual_seed(1002 + rank)
        self.layer = base.PerturbedLinear(self.n, self.n, self.D, antithetic=True,
                                          options={"tc": self.tc or "3xtf32"}).to(dev)
        with torch.no_grad():
            self.layer.weight.copy_(torch.randn(self.n, self.n, generator=g) / self.n ** .5)
            self.layer.bias.zero_()
        self.layer.set_seed(5000)                       # one seed everywhere: the member offset keeps the ranks' draws apart
        self.layer.set_member_offset(rank * self.D)
        self.layer.set_noise(0.02)
        self.x_host = torch.randn(self.D * self.R, self.n, generator=g).pin_memory()
        self.w_host = (torch.rand(self.D, generator=g) * 2 - 1).pin_memory()
        self.x = self.x_host.to(dev)
        self.w = self.w_host.to(dev)
        self.y_host = torch.empty(self.D * self.R, self.n).pin_memory()
        self.grad_host = torch.empty(self.n, self.n).pin_memory()
        self.bgrad_host = torch.empty(self.n).pin_memory()
        self.bucket = None
        self.h2d = self.x_host.numel() * 4 + self.w_host.numel() * 4
        self.d2h = (self.y_host.numel() + self.grad_host.numel() + self.bgrad_host.numel()) * 4

    def _update(self, w):
        layer = self.layer
        layer.weight.grad = None
        layer.bias.grad = None
        if self.world > 1 and self.overlap_blocks:
            # column blocks of the gradient go to the all-reduce while the next block streams
            self.bucket = self.ndist.overlapped_dense_update(layer, w, self.bucket, blocks=self.overlap_blocks)
        else:
            layer.update(w)                  # from the second step on the gradients land in the bucket directly
            if self.world > 1:
                self.bucket = self.ndist.all_reduce_grads([layer.weight, layer.bias], self.bucket)
        return layer.weight.grad, layer.bias.grad

    def step(self, mark):
        with torch.no_grad():
            self.layer.perturbed_flag = True
            y = self.layer.forward(self.x)
            self.layer.perturbed_flag = False
            mark("forward")
            out = self._update(self.w)
            mark("update")
        return y, out

    def step_e2e(self):
        """Host buffers in, host buffers out.  The read-back of y runs on a copy stream while the update
        computes; everything has landed on the host when the step returns."""
        main = torch.cuda.current_stream()
        if not hasattr(self, "copy_stream"):
            self.copy_stream = torch.cuda.Stream()
        with torch.no_grad():
            self.x.copy_(self.x_host, non_blocking=True)
            self.w.copy_(self.w_host, non_blocking=True)
            self.layer.perturbed_flag = True
            y = self.layer.forward(self.x)
            self.layer.perturbed_flag = False
            self.copy_stream.wait_stream(main)
            with torch.cuda.stream(self.copy_stream):
                self.y_host.copy_(y, non_blocking=True)
                y.record_stream(self.copy_stream)
            grad, bgrad = self._update(self.w)
            self.grad_host.copy_(grad, non_blocking=True)
            self.bgrad_host.copy_(bgrad, non_blocking=True)
        main.synchronize()
        self.copy_stream.synchronize()

    def roofline(self, phase_ms, peaks):
        n, D, R = self.n, self.D, self.R
        noise = D * n * n * 4
        fwd_bytes = noise + 2 * D * R * n * 4 + n * n * 4 + D * n * 4 + n * 4       # E + x + y + W + beta + bias
        upd_bytes = noise + n * n * 4 + D * 4                                      # E + grad + weights
        upd_ms = phase_ms["update"]
        achieved = upd_bytes / (upd_ms * 1e-3) / 1e9
        return {"kernel": "weighted_noise_sum_kernel (update phase: it plus its few-microsecond partial-sum pass"
                          " and the 1024-element bias update" + ("; all-reduce included" if self.world > 1 else "") + ")",
                "bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm"], 4), "peak_source": peaks["source"],
                "algorithmic_bytes_per_launch": upd_bytes, "ms_per_launch": round(upd_ms, 4),
                # ncu dram__bytes_read+write of this kernel at 128 members (544.1 MB), scaled by members (profiles/)
                "traffic": int(544.12e6 * D / 128), "traffic_source": "ncu capture at 128 members, scaled by member count",
                "forward_phase": {"kernels": "base x.W^T (tcgen05 3xTF32 gemm_tf32_kernel + operand split, or fp32 gemm_kernel with --tc fp32) + perturbed_linear_stream_kernel",
                                  "algorithmic_bytes": fwd_bytes, "ms": round(phase_ms["forward"], 4),
                                  "achieved_GBps": round(fwd_bytes / (phase_ms["forward"] * 1e-3) / 1e9, 1),
                                  "frac": round(fwd_bytes / (phase_ms["forward"] * 1e-3) / 1e9 / peaks["hbm"], 4)}}

    def cpu_sample(self, reps):
        """CPU oracle on 128 of the 1024 members (512 MiB of noise), all host threads."""
        from oracle import perturbed_ref as O
        Ds = 128
        g = torch.Generator().manual_seed(77)
        E = torch.empty(Ds, self.n, self.n).normal_(0, 0.02, generator=g)
        beta = torch.empty(Ds, self.n).normal_(0, 0.02, generator=g)
        W = torch.randn(self.n, self.n, generator=g) / self.n ** .5
        b = torch.zeros(self.n)
        x = torch.randn(Ds * self.R, self.n, generator=g)
        w = torch.rand(Ds, generator=g) * 2 - 1

        def once():
            t0 = time.perf_counter()
            O.perturbed_linear_forward(x, W, b, E, beta, Ds, True)
            O.perturbed_update(W, E, beta, w)
            return time.perf_counter() - t0
        once()
        times = [once() for _ in range(reps)]
        return Ds * self.R, times, "128 of 1024 members (512 MiB noise): forward + update per repetition"


class PermutedLinear256(Workload):
    """PermutedLinear 256x256, 512 antithetic pairs sharing one permuted noise matrix: forward + rank-normalised update."""
    name = "permuted_linear_256"
    D, R, n = 512, 2, 256
    use_graph = True            # 134 MFLOP per step: launch-bound, so the resident-data number replays a CUDA graph
    launches_per_step = 2       # one cluster kernel (forward) + one update kernel (weight and bias gradient)

    def __init__(self):
        self.units_per_step = self.D * self.R
        self.resident_bytes = 4 * (2 * self.D * self.R * self.n + 2 * self.n * self.n + self.D * self.n) + 2 * self.D * self.n

    def describe(self, world):
        return {"workload": self.name, "layer": "PermutedLinear(256,256) auto->out", "directions_per_gpu": self.D,
                "population": self.D * world, "batch_per_gpu": self.D * self.R, "antithetic": True,
                "step": "forward + rank-normalised update", "l2": "L2 flushed between timed steps", "sharding": "members"}

    def setup(self, dev, rank, world):
        from nesgpu_b200 import base, dist as ndist
        from oracle import perturbed_ref as O
        self.ndist, self.world = ndist, world
        g = torch.Generator().manual_seed(1001 + rank)
        self.layer = base.PermutedLinear(self.n, self.n, self.D, antithetic=True).to(dev)
        with torch.no_grad():
            self.layer.weight.copy_(torch.randn(self.n, self.n, generator=g) / self.n ** .5)
            self.layer.bias.zero_()
        self.layer.set_seed(6000 + rank)
        self.layer.set_noise(0.02)
        self.x_host = torch.randn(self.D * self.R, self.n, generator=g).pin_memory()
        u = O.centered_ranks(torch.randn(self.D * self.R, generator=g))
        self.w_host = (u[:self.D] - u[self.D:]).contiguous().pin_memory()
        self.x, self.w = self.x_host.to(dev), self.w_host.to(dev)
        self.y_host = torch.empty(self.D * self.R, self.n).pin_memory()
        self.grad_host = torch.empty(self.n, self.n).pin_memory()
        self.bucket = None
        self.h2d = (self.x_host.numel() + self.w_host.numel()) * 4
        self.d2h = (self.y_host.numel() + self.grad_host.numel()) * 4

    def _update(self, w):
        self.layer.weight.grad = None
        self.layer.bias.grad = None
        self.layer.update(w)
        if self.world > 1:
            self.bucket = self.ndist.all_reduce_grads([self.layer.weight, self.layer.bias], self.bucket)
        return self.layer.weight.grad

    def step(self, mark):
        with torch.no_grad():
            self.layer.perturbed_flag = True
            y = self.layer.forward(self.x)
            self.layer.perturbed_flag = False
            mark("forward")
            g = self._update(self.w)
            mark("update")
        return y, g

    def step_e2e(self):
        with torch.no_grad():
            self.x.copy_(self.x_host, non_blocking=True)
            self.layer.perturbed_flag = True
            y = self.layer.forward(self.x)
            self.layer.perturbed_flag = False
            self.y_host.copy_(y, non_blocking=True)
            self.w.copy_(self.w_host, non_blocking=True)
            self.grad_host.copy_(self._update(self.w), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def roofline(self, phase_ms, peaks):
        flops = 2.0 * self.D * self.R * self.n * self.n
        fwd_ms = phase_ms["forward"] if "forward" in phase_ms else phase_ms["step"]
        phase_ms = dict(phase_ms, forward=fwd_ms)
        ach = flops / (fwd_ms * 1e-3) / 1e12
        peak = peaks["bf16"] / 2
        return {"kernel": "permuted_linear_out_kernel<3> (tcgen05 3xTF32, stacked [W; eps], cluster gather epilogue)" +
                          (", forward phase" if "step" not in phase_ms else "; whole graph-replayed step (forward + update) timed"),
                "bound": "tensor", "achieved": round(ach, 3), "peak": peak, "unit": "TFLOP/s",
                "frac": round(ach / peak, 5), "peak_source": peaks["source"] + " bf16 burst / 2 taken as TF32",
                "algorithmic_flops_per_launch": flops, "ms_per_launch": round(phase_ms["forward"], 4), "traffic": None,
                "note": "134 MFLOP / 3.4 MB per step: latency bound (32 blocks, 8 K stages each); the tensor pipe issues 6x the "
                        "algorithmic flops (stacked product x 3xTF32 terms)"}

    def cpu_sample(self, reps):
        from oracle import perturbed_ref as O
        layer = self.layer
        c = lambda t: t.detach().cpu()
        W, b, eps, beta, pout = c(layer.weight), c(layer.bias), c(layer.weight_noise), c(layer.bias_noise), c(layer.output_permutations)
        x, w = self.x_host.clone(), self.w_host.clone()

        def once():
            t0 = time.perf_counter()
            O.permuted_linear_forward(x, W, b, eps, beta, None, pout, self.D, True)
            O.permuted_linear_weight_grad(eps, w, None, pout, self.n, self.n)
            w @ beta
            return time.perf_counter() - t0
        once()
        return self.D * self.R, [once() for _ in range(reps)], "full configuration: forward + update per repetition"


class PermutedConv64(Workload):
    """PermutedConv2d 64 -> 64 channels, 3x3, 32x32 input, 1024 members, out_sparsity 0.5: forward + update."""
    name = "permuted_conv_64"
    D, c, hw = 1024, 64, 32

    def __init__(self, members=None):
        if members:
            self.D = members        # reduced member count: profiling captures only
        self.units_per_step = self.D
        self.resident_bytes = 2 * self.D * self.c * self.hw * self.hw * 4

    def describe(self, world):
        return {"workload": self.name, "layer": "PermutedConv2d(64,64,3,padding=1,out_sparsity=.5)",
                "directions_per_gpu": self.D, "population": self.D * world, "batch_per_gpu": self.D,
                "input": "64x32x32", "step": "forward + update", "l2": "inputs exceed L2 (256 MiB in, 256 MiB out)",
                "sharding": "members"}

    def setup(self, dev, rank, world):
        from nesgpu_b200 import base, dist as ndist
        self.ndist, self.world = ndist, world
        g = torch.Generator().manual_seed(1003 + rank)
        self.layer = base.PermutedConv2d(self.c, self.c, 3, self.D, padding=1, out_sparsity=.5,
                                         options={"tc": self.tc} if self.tc else {}).to(dev)
        with torch.no_grad():
            self.layer.weight.copy_(torch.randn(self.c, self.c, 3, 3, generator=g) * (2 / 576) ** .5)
            self.layer.bias.zero_()
        self.layer.set_seed(7000 + rank)
        self.layer.set_noise(0.02)
        self.x_host = torch.randn(self.D, self.c, self.hw, self.hw, generator=g).pin_memory()
        self.w_host = torch.randn(self.D, generator=g).pin_memory()
        self.x, self.w = self.x_host.to(dev), self.w_host.to(dev)
        self.y_host = torch.empty_like(self.x_host).pin_memory()
        self.grad_host = torch.empty(self.c, self.c, 3, 3).pin_memory()
        self.bucket = None
        self.h2d = (self.x_host.numel() + self.w_host.numel()) * 4
        self.d2h = (self.y_host.numel() + self.grad_host.numel()) * 4

    def _update(self, w):
        self.layer.weight.grad = None
        self.layer.bias.grad = None
        self.layer.update(w)
        if self.world > 1:
            self.bucket = self.ndist.all_reduce_grads([self.layer.weight, self.layer.bias], self.bucket)
        return self.layer.weight.grad

    def step(self, mark):
        with torch.no_grad():
            self.layer.perturbed_flag = True
            y = self.layer.forward(self.x)
            self.layer.perturbed_flag = False
            mark("forward")
            g = self._update(self.w)
            mark("update")
        return y, g

    def step_e2e(self):
        with torch.no_grad():
            self.x.copy_(self.x_host, non_blocking=True)
            self.layer.perturbed_flag = True
            y = self.layer.forward(self.x)
            self.layer.perturbed_flag = False
            self.y_host.copy_(y, non_blocking=True)
            self.w.copy_(self.w_host, non_blocking=True)
            self.grad_host.copy_(self._update(self.w), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def roofline(self, phase_ms, peaks):
        flops = 2.0 * self.D * self.hw * self.hw * self.c * 9 * self.c
        ach = flops / (phase_ms["forward"] * 1e-3) / 1e12
        mode = self.mode()
        bf = mode in ("bf16", "bf16x3")
        peak = peaks["bf16_sustained"] if bf else peaks["bf16_sustained"] / 2
        dense = self.name == "perturbed_conv_64"
        kernel = {"tf32": "conv_tf32_kernel (tcgen05 kind::tf32) + stage_rows_tf32_kernel",
                  "bf16": "conv_bf16_kernel<1> (tcgen05 kind::f16) + stage_rows_bf16_kernel",
                  "bf16x3": ("conv_bf16_kernel<3> (tcgen05 kind::f16, three products on bf16 hi/lo splits, operands in shared memory)"
                             if dense else
                             "conv_split_tmem_kernel (tcgen05 kind::f16, stacked hi/lo filter operand in tensor memory, two MMAs per "
                             "K step on the hi and lo input copies)") + " + stage_rows_bf16_kernel",
                  }.get(mode, "gemm_kernel<ConvProb<...>> (implicit-GEMM conv on CUDA cores)")
        note = {"tf32": "TF32 operands (stated reduced precision, bar 2e-2)", "bf16": "bf16 operands (stated reduced precision, bar 2e-2)",
                "bf16x3": "split-bf16 form: holds the fp32 bar (rel err ~5e-6); the tensor pipe executes 3-4 partial products per "
                          "algorithmic product",
                }.get(mode, "fp32 CUDA-core path (exact-fp32 parity)")
        return {"kernel": kernel + ", forward phase", "bound": "tensor", "achieved": round(ach, 2), "peak": peak, "unit": "TFLOP/s",
                "frac": round(ach / peak, 4), "peak_source": peaks["source"] + (" bf16 sustained" if bf else " bf16 sustained / 2 taken as TF32"),
                "algorithmic_flops_per_launch": flops, "ms_per_launch": round(phase_ms["forward"], 4), "traffic": None,
                "note": note + "; flops counted for the minimal form N=64"}

    def cpu_sample(self, reps):
        from oracle import perturbed_ref as O
        Ds = 128
        layer = self.layer
        c = lambda t: t.detach().cpu()
        W, b, eps = c(layer.weight), c(layer.bias), c(layer.weight_noise)
        beta, pout = c(layer.bias_noise)[:Ds].contiguous(), c(layer.output_permutations)[:Ds].contiguous()
        x, w = self.x_host[:Ds].clone(), self.w_host[:Ds].clone()

        def once():
            t0 = time.perf_counter()
            O.permuted_conv2d_forward(x, W, b, eps, beta, None, pout, Ds, 1, 1, 1, False)
            O.permuted_conv2d_weight_grad(eps, w, None, pout, self.c, self.c)
            return time.perf_counter() - t0
        once()
        return Ds, [once() for _ in range(reps)], "128 of 1024 members: forward + update per repetition"


class Binary1024(Workload):
    """Bit-packed layer: 1024 members x 1024x1024 Bernoulli weight bits, one 1024-bit input per member: sample, pack, bmm,
    weighted sum, max-pool."""
    name = "binary_1024"
    dtype = "u64"
    cpu_cores = 1
    D = n = 1024

    def __init__(self):
        self.units_per_step = self.D
        self.resident_bytes = self.D * self.n * self.n // 8

    def describe(self, world):
        return {"workload": self.name, "layer": "bit-packed 1024x1024 weights per member, one 1024-bit input per member",
                "directions_per_gpu": self.D, "population": self.D * world,
                "step": "sample_bits (Philox) + pack + bmm + weighted_sum + max_pool2d",
                "l2": "weight bits (128 MiB) exceed L2", "sharding": "members"}

    def setup(self, dev, rank, world):
        import nesgpu_b200.boolean_operations as ops
        self.ops, self.world = ops, world
        g = torch.Generator().manual_seed(1004 + rank)
        self.p = torch.rand(self.n, self.n, generator=g).half().to(dev)
        self.x_host = torch.randint(2, (self.D, self.n), generator=g).bool().pin_memory()
        self.x = self.x_host.to(dev)
        self.w_host = torch.randn(self.D, generator=g).half().pin_memory()
        self.w = self.w_host.to(dev)
        self.pool_in = torch.randint(-2 ** 62, 2 ** 62, (self.D, 32, 32, 1), generator=g).to(dev)
        self.counts_host = torch.empty(self.D, self.n, 1, dtype=torch.int32).pin_memory()
        self.ws_host = torch.empty(self.n, self.n, dtype=torch.float16).pin_memory()
        self.seed = 100 + rank
        self.h2d = self.x_host.numel() + self.w_host.numel() * 2
        self.d2h = self.counts_host.numel() * 4 + self.ws_host.numel() * 2

    def step(self, mark):
        ops = self.ops
        bits = ops.sample_bits(self.p, self.D, torch.int64, self.seed)
        mark("sample_bits")
        xb = ops.pack(self.x, torch.int64)
        counts = ops.bmm(bits, xb.view(self.D, -1, 1))
        mark("pack_bmm")
        ws = ops.weighted_sum(bits, self.w, self.n)
        mark("weighted_sum")
        mp = ops.max_pool2d(self.pool_in, 2, 2, 0, 0, 2, 2)
        mark("max_pool2d")
        return counts, ws, mp

    def step_e2e(self):
        self.x.copy_(self.x_host, non_blocking=True)
        self.w.copy_(self.w_host, non_blocking=True)
        counts, ws, _ = self.step(lambda name: None)
        self.counts_host.copy_(counts, non_blocking=True)
        self.ws_host.copy_(ws, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def roofline(self, phase_ms, peaks):
        a_bytes = self.D * self.n * self.n // 8
        nbytes = a_bytes + self.D * self.n * 4 + self.D * self.n // 8 + self.D * self.n
        ach = nbytes / (phase_ms["pack_bmm"] * 1e-3) / 1e9
        extra = {k: round(v, 4) for k, v in phase_ms.items()}
        return {"kernel": "bin_bmv_kernel (+ pack_rows_kernel), pack_bmm phase", "bound": "hbm", "achieved": round(ach, 1),
                "peak": peaks["hbm"], "unit": "GB/s", "frac": round(ach / peaks["hbm"], 4), "peak_source": peaks["source"],
                "algorithmic_bytes_per_launch": nbytes, "ms_per_launch": round(phase_ms["pack_bmm"], 4), "traffic": None,
                "phase_ms": extra,
                "sample_bits_GBps": round((a_bytes + self.n * self.n * 2) / (phase_ms["sample_bits"] * 1e-3) / 1e9, 1),
                "weighted_sum_GBps": round((a_bytes + self.n * self.n * 2) / (phase_ms["weighted_sum"] * 1e-3) / 1e9, 1)}

    def cpu_sample(self, reps):
        import numpy as np
        from oracle import binary_ref as B
        Ds = 64
        rng = np.random.default_rng(3)
        p = rng.random((self.n, self.n)).astype(np.float16)
        u = rng.random((Ds, self.n, self.n), dtype=np.float32)
        x = rng.integers(0, 2, (Ds, self.n)).astype(bool)
        w = rng.standard_normal(Ds).astype(np.float16)

        def once():
            t0 = time.perf_counter()
            bits = B.sample_bits(p, u, 64)
            B.bmm(bits, B.pack(x, 64).reshape(Ds, -1, 1))
            B.weighted_sum(bits, w, self.n)
            return time.perf_counter() - t0
        return Ds, [once() for _ in range(max(1, min(reps, 2)))], "64 of 1024 members, uniforms pre-drawn: sample_bits + pack + bmm + weighted_sum (numpy port, single thread)"



class PerturbedConv64(PermutedConv64):
    """PerturbedConv2d with one dense noise filter per member at the shape of the permuted configuration (64 -> 64, 3x3,
    32x32 input, 1024 members; 144 MiB of noise): forward + update."""
    name = "perturbed_conv_64"

    def describe(self, world):
        return dict(PermutedConv64.describe(self, world), layer="PerturbedConv2d(64,64,3,padding=1), dense noise per member")

    def setup(self, dev, rank, world):
        from nesgpu_b200 import base, dist as ndist
        self.ndist, self.world = ndist, world
        g = torch.Generator().manual_seed(1013 + rank)
        self.layer = base.PerturbedConv2d(self.c, self.c, 3, self.D, padding=1,
                                          options={"tc": self.tc} if self.tc else {}).to(dev)
        with torch.no_grad():
            self.layer.weight.copy_(torch.randn(self.c, self.c, 3, 3, generator=g) * (2 / 576) ** .5)
            self.layer.bias.zero_()
        self.layer.set_seed(7100 + rank)
        self.layer.set_noise(0.02)
        self.x_host = torch.randn(self.D, self.c, self.hw, self.hw, generator=g).pin_memory()
        self.w_host = torch.randn(self.D, generator=g).pin_memory()
        self.x, self.w = self.x_host.to(dev), self.w_host.to(dev)
        self.y_host = torch.empty_like(self.x_host).pin_memory()
        self.grad_host = torch.empty(self.c, self.c, 3, 3).pin_memory()
        self.bucket = None
        self.h2d = (self.x_host.numel() + self.w_host.numel()) * 4
        self.d2h = (self.y_host.numel() + self.grad_host.numel()) * 4

    def cpu_sample(self, reps):
        from oracle import perturbed_ref as O
        Ds = 64
        c = lambda t: t.detach().cpu()
        W, b = c(self.layer.weight), c(self.layer.bias)
        E, beta = c(self.layer.weight_noise[:Ds]), c(self.layer.bias_noise[:Ds])
        x, w = self.x_host[:Ds].clone(), self.w_host[:Ds].clone()

        def once():
            t0 = time.perf_counter()
            O.perturbed_conv2d_forward(x, W, b, E, beta, Ds, 1, 1, 1, False)
            O.perturbed_update(W, E, beta, w)
            return time.perf_counter() - t0
        once()
        return Ds, [once() for _ in range(reps)], "64 of 1024 members: forward + update per repetition"


class _Linear1024(Workload):
    """Shared scaffolding of the 1024x1024 linear layers with cheap per-member noise (batch 2048, antithetic)."""
    D, R, n = 1024, 2, 1024
    what = ""

    def __init__(self):
        self.units_per_step = self.D * self.R
        self.resident_bytes = 4 * (2 * self.D * self.R * self.n + 2 * self.n * self.n)

    def describe(self, world):
        return {"workload": self.name, "layer": self.what, "directions_per_gpu": self.D, "population": self.D * world,
                "batch_per_gpu": self.D * self.R, "antithetic": True, "step": "forward + update",
                "l2": "L2 flushed between timed steps", "sharding": "members"}

    def make_layer(self, base, dev):
        raise NotImplementedError

    def setup(self, dev, rank, world):
        from nesgpu_b200 import base
        self.world = world
        g = torch.Generator().manual_seed(1020 + rank)
        self.layer = self.make_layer(base, dev)
        with torch.no_grad():
            self.layer.weight.copy_(torch.randn(self.n, self.n, generator=g) / self.n ** .5)
            self.layer.bias.zero_()
        self.layer.set_seed(7200 + rank)
        self.layer.set_noise(0.02)
        self.x_host = torch.randn(self.D * self.R, self.n, generator=g).pin_memory()
        self.w_host = (torch.rand(self.D, generator=g) * 2 - 1).pin_memory()
        self.x, self.w = self.x_host.to(dev), self.w_host.to(dev)
        self.y_host = torch.empty(self.D * self.R, self.n).pin_memory()
        self.grad_host = torch.empty(self.n, self.n).pin_memory()
        self.h2d = (self.x_host.numel() + self.w_host.numel()) * 4
        self.d2h = (self.y_host.numel() + self.grad_host.numel()) * 4

    def step(self, mark):
        with torch.no_grad():
            self.layer.perturbed_flag = True
            y = self.layer.forward(self.x)
            self.layer.perturbed_flag = False
            mark("forward")
            self.layer.weight.grad = None
            self.layer.bias.grad = None
            self.layer.update(self.w)
            mark("update")
        return y, self.layer.weight.grad

    def step_e2e(self):
        with torch.no_grad():
            self.x.copy_(self.x_host, non_blocking=True)
            self.w.copy_(self.w_host, non_blocking=True)
            y, g = self.step(lambda name: None)
            self.y_host.copy_(y, non_blocking=True)
            self.grad_host.copy_(g, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def roofline(self, phase_ms, peaks):
        flops = 2.0 * self.D * self.R * self.n * self.n
        ach = flops / (phase_ms["forward"] * 1e-3) / 1e12
        peak = peaks["bf16"] / 2
        return {"kernel": self.kernels + ", forward phase", "bound": "tensor", "achieved": round(ach, 2), "peak": peak,
                "unit": "TFLOP/s", "frac": round(ach / peak, 4), "peak_source": peaks["source"] + " bf16 burst / 2 taken as TF32",
                "algorithmic_flops_per_launch": flops, "ms_per_launch": round(phase_ms["forward"], 4), "traffic": None,
                "note": "flops of the base product x.W^T only (4.3 GFLOP); the per-member term is O(batch * out * k)"}


class SparseLinear1024(_Linear1024):
    """SparsePerturbedLinear(1024,1024), k = 2 noise entries per member and output row (the README's sparse variant)."""
    name = "sparse_linear_1024"
    what = "SparsePerturbedLinear(1024,1024,k=2)"
    kernels = "gemm_tf32_kernel<3> (tcgen05 3xTF32 base product) + sparse_noise_kernel"

    def make_layer(self, base, dev):
        return base.SparsePerturbedLinear(self.n, self.n, self.D, antithetic=True, k=2,
                                          options={"tc": self.tc} if self.tc else {}).to(dev)

    def cpu_sample(self, reps):
        from oracle import perturbed_ref as O
        Ds = 128
        c = lambda t: t.detach().cpu()
        W, b = c(self.layer.weight), c(self.layer.bias)
        E = O.densify_sparse_noise(c(self.layer.noise_indices[:Ds]).long(), c(self.layer.weight_noise[:Ds]), self.n)
        beta = c(self.layer.bias_noise[:Ds])
        x = torch.cat([self.x_host[:Ds], self.x_host[self.D:self.D + Ds]]).clone()
        w = self.w_host[:Ds].clone()

        def once():
            t0 = time.perf_counter()
            O.perturbed_linear_forward(x, W, b, E, beta, Ds, True)
            O.perturbed_update(W, E, beta, w)
            return time.perf_counter() - t0
        once()
        return Ds * self.R, [once() for _ in range(reps)], "128 of 1024 members on the densified noise: forward + update per repetition"


class SyntheticLinear1024(_Linear1024):
    """SyntheticLinear(1024,1024): one shared noise matrix, per-member sign flips (the reference paper's fastest sampler)."""
    name = "synthetic_linear_1024"
    what = "SyntheticLinear(1024,1024) auto->out flips"
    kernels = "synthetic_linear kernels"

    def make_layer(self, base, dev):
        return base.SyntheticLinear(self.n, self.n, self.D, antithetic=True,
                                    options={"tc": self.tc} if self.tc else {}).to(dev)

    def cpu_sample(self, reps):
        from oracle import perturbed_ref as O
        c = lambda t: None if t is None else t.detach().cpu()
        L = self.layer
        W, b, eps, beta, fin, fout = c(L.weight), c(L.bias), c(L.weight_noise), c(L.bias_noise), c(L.input_flips), c(L.output_flips)
        x, w = self.x_host.clone(), self.w_host.clone()

        def once():
            t0 = time.perf_counter()
            O.synthetic_linear_forward(x, W, b, eps, beta, fin, fout, self.D, True)
            O.synthetic_weight_grad(eps, w, fin, fout)
            return time.perf_counter() - t0
        once()
        return self.D * self.R, [once() for _ in range(reps)], "full configuration: forward + update per repetition"


class BinaryBmm64(Workload):
    """General bit-packed bmm: 1024 members, 1024 x 1024-bit weights against 64 packed input columns each."""
    name = "binary_bmm_n64"
    dtype = "u64"
    cpu_cores = 1
    D, n, N = 1024, 1024, 64

    def __init__(self):
        self.units_per_step = self.D * self.N
        self.resident_bytes = self.D * self.n * self.n // 8

    def describe(self, world):
        return {"workload": self.name, "layer": "bmm of (1024, 1024, 16) by (1024, 16, 64) int64 words -> int32 counts",
                "directions_per_gpu": self.D, "population": self.D * world, "step": "bmm", "l2": "operands exceed L2",
                "sharding": "members"}

    def setup(self, dev, rank, world):
        import nesgpu_b200.boolean_operations as ops
        self.ops = ops
        g = torch.Generator().manual_seed(1030 + rank)
        self.A = torch.randint(-2 ** 62, 2 ** 62, (self.D, self.n, self.n // 64), generator=g).to(dev)
        self.B = torch.randint(-2 ** 62, 2 ** 62, (self.D, self.n // 64, self.N), generator=g).to(dev)

    def step(self, mark):
        c = self.ops.bmm(self.A, self.B)
        mark("bmm")
        return c

    def roofline(self, phase_ms, peaks):
        nbytes = self.A.numel() * 8 + self.B.numel() * 8 + self.D * self.n * self.N * 4
        ach = nbytes / (phase_ms["bmm"] * 1e-3) / 1e9
        words = self.D * self.n * (self.n // 64) * self.N
        return {"kernel": "bin_gemm_kernel (64x64 XOR-popcount tile)", "bound": "hbm", "achieved": round(ach, 1), "peak": peaks["hbm"],
                "unit": "GB/s", "frac": round(ach / peaks["hbm"], 4), "peak_source": peaks["source"],
                "algorithmic_bytes_per_launch": nbytes, "ms_per_launch": round(phase_ms["bmm"], 4), "traffic": None,
                "word_xor_popc_per_s": round(words / (phase_ms["bmm"] * 1e-3), 1),
                "note": "A 128 MiB + C 256 MiB: the int32 output dominates the traffic"}

    def cpu_sample(self, reps):
        import numpy as np
        from oracle import binary_ref as B
        Ds = 8
        rng = np.random.default_rng(4)
        A = rng.integers(-2 ** 62, 2 ** 62, (Ds, self.n, self.n // 64), dtype=np.int64)
        Bm = rng.integers(-2 ** 62, 2 ** 62, (Ds, self.n // 64, self.N), dtype=np.int64)

        def once():
            t0 = time.perf_counter()
            B.bmm(A, Bm)
            return time.perf_counter() - t0
        return Ds * self.N, [once() for _ in range(max(1, min(reps, 2)))], "8 of 1024 members (numpy port, single thread)"


class BinaryConv512(Workload):
    """Bit-packed convolution at the shape the reference's own timing script uses (booloptests.py:231-236): 128 members,
    512 -> 512 channels, 3x3, 7x7 input, padding 1."""
    name = "binary_conv_512"
    dtype = "u32"
    cpu_cores = 1
    P, cin, cout, hw = 128, 512, 512, 7

    def __init__(self):
        self.units_per_step = self.P
        self.resident_bytes = self.P * 9 * (self.cin // 32) * self.cout * 4

    def describe(self, world):
        return {"workload": self.name, "layer": "binary conv 512->512, 3x3, pad 1, 7x7 input, int32 words, per-member filters",
                "directions_per_gpu": self.P, "population": self.P * world, "step": "conv (im2col-free)",
                "l2": "L2 flushed between timed steps", "sharding": "members"}

    def setup(self, dev, rank, world):
        import nesgpu_b200.boolean_operations as ops
        self.ops = ops
        g = torch.Generator().manual_seed(1031 + rank)
        cw = self.cin // 32
        self.x = torch.randint(-2 ** 31, 2 ** 31 - 1, (self.P, self.hw, self.hw, cw), generator=g, dtype=torch.int64).int().to(dev)
        self.f = torch.randint(-2 ** 31, 2 ** 31 - 1, (self.P, 9 * cw, self.cout), generator=g, dtype=torch.int64).int().to(dev)

    def step(self, mark):
        c = self.ops.conv(self.x, self.f, 3, 3, 1, 1, 1, 1)
        mark("conv")
        return c

    def roofline(self, phase_ms, peaks):
        nbytes = self.x.numel() * 4 + self.f.numel() * 4 + self.P * self.hw * self.hw * self.cout * 4
        ach = nbytes / (phase_ms["conv"] * 1e-3) / 1e9
        words = self.P * self.hw * self.hw * 9 * (self.cin // 32) * self.cout
        return {"kernel": "bin_gemm_kernel<WindowA> (im2col-free XOR-popcount conv)", "bound": "hbm", "achieved": round(ach, 1),
                "peak": peaks["hbm"], "unit": "GB/s", "frac": round(ach / peaks["hbm"], 4), "peak_source": peaks["source"],
                "algorithmic_bytes_per_launch": nbytes, "ms_per_launch": round(phase_ms["conv"], 4), "traffic": None,
                "word_xor_popc_per_s": round(words / (phase_ms["conv"] * 1e-3), 1),
                "note": "filters 36 MiB + counts 12.3 MiB; 0.46 G word operations on 49 positions per member"}

    def cpu_sample(self, reps):
        import numpy as np
        from oracle import binary_ref as B
        Ps = 4
        rng = np.random.default_rng(5)
        cw = self.cin // 32
        x = rng.integers(-2 ** 31, 2 ** 31 - 1, (Ps, self.hw, self.hw, cw)).astype(np.int32)
        f = rng.integers(-2 ** 31, 2 ** 31 - 1, (Ps, 9 * cw, self.cout)).astype(np.int32)

        def once():
            t0 = time.perf_counter()
            B.conv(x, f, 3, 3, 1, 1, 1, 1)
            return time.perf_counter() - t0
        return Ps, [once() for _ in range(max(1, min(reps, 2)))], "4 of 128 members (numpy port, single thread)"


class EsCnn(Workload):
    """One ES step of the small CNN (Conv-ReLU-Pool x 2, two linear layers), 1024 members per GPU (8192 over 8 GPUs)."""
    name = "es_cnn_8192"
    D, R = 1024, 256
    fused = True                  # --unfused: module-by-module Conv / ReLU / MaxPool2d, per-member input copies
    FLOP_PER_PAIR = 5.262e6       # conv1 0.389 + conv2 4.461 + fc1 0.410 + fc2 0.003 MFLOP per (member, image), minimal form

    def __init__(self, members=None):
        if members:
            self.D = members
        self.units_per_step = self.D * self.R
        self.resident_bytes = 1 << 40     # activations far exceed L2

    def describe(self, world):
        return {"workload": self.name, "net": "Conv(1,32,3)-ReLU-MaxPool2-Conv(32,64,3)-ReLU-MaxPool2-Linear(1600,128)-ReLU-Linear(128,10), Permuted layers",
                "directions_per_gpu": self.D, "population": self.D * world, "images_per_member": self.R,
                "step": "set_noise + chunked population forward + CE fitness + centred ranks + update (+ all-gather / all-reduce at N>1)",
                "l2": "activations exceed L2", "sharding": "members", "sigma": 0.02, "fused_layers": self.fused,
                "precision": {None: "tf32", "tf32": "tf32 operands, fp32 accumulation (stated mode, rel err ~1e-3 per layer)",
                              "bf16": "bf16 operands in conv2 and the linear layers (rel err ~3e-3 per layer), fp32 accumulation (stated mode)",
                              "fp32": "fp32 bar (rel err <= 1e-4): conv1 exact fp32, conv2 split-bf16 three-product form, linear layers 3xTF32"
                              }.get(self.tc, self.tc)}

    def setup(self, dev, rank, world):
        from nesgpu_b200 import base, es
        self.es, self.world, self.dev = es, world, dev
        D = self.D
        torch.manual_seed(1005)       # same initial weights on every rank
        if self.tc is None:
            self.tc = "tf32"       # default for this workload: the stated TF32 tensor-core mode (--tc fp32 holds the fp32 bar)
        self.dtype = {"tf32": "tf32", "bf16": "bf16"}.get(self.tc, "f32")
        opts = {"tc": self.tc} if self.tc in ("tf32", "bf16") else {}
        lin = {"tc": self.tc} if self.tc in ("tf32", "bf16") else {}  # the stated reduced-precision modes cover the linear layers
        if self.fused:
            # Conv -> ReLU -> MaxPool2 blocks as fused layers; the first one is told that the images are shared
            pair = self.tc == "bf16" and D % 2 == 0          # two images per tensor-core instruction in layer 2
            o1 = {"shared_input": True, "fuse": "relu_maxpool2", "out_dtype": "bf16x2" if pair else (self.tc if opts else "fp32")}
            if pair:
                opts = dict(opts, in_layout="bf16x2")
            if self.tc == "fp32":
                # the fp32 bar on the tensor cores: layer 1 (exact fp32) hands layer 2 its activations as bf16 hi + lo
                # parts, layer 2 runs the three-product split form, the linear layers their 3xTF32 default
                o1["out_dtype"] = "bf16x3"
                opts = {"tc": "bf16x3"}
            self.net = torch.nn.Sequential(
                base.PermutedConv2d(1, 32, 3, D, options=o1),
                base.PermutedConv2d(32, 64, 3, D, options=dict(opts, fuse="relu_maxpool2")), torch.nn.Flatten(),
                base.PermutedLinear(1600, 128, D, options=lin), torch.nn.ReLU(),
                base.PermutedLinear(128, 10, D, options=lin)).to(dev)
        else:
            self.net = torch.nn.Sequential(
                base.PermutedConv2d(1, 32, 3, D), torch.nn.ReLU(), torch.nn.MaxPool2d(2),
                base.PermutedConv2d(32, 64, 3, D, options=opts), torch.nn.ReLU(), torch.nn.MaxPool2d(2), torch.nn.Flatten(),
                base.PermutedLinear(1600, 128, D), torch.nn.ReLU(), base.PermutedLinear(128, 10, D)).to(dev)
        self.pm = base.PerturbedModel(self.net, D)
        self.pm.set_noise_scale(0.02)
        import random
        random.seed(9000)                               # the per-step seeds agree on all ranks ...
        self.pm.set_member_offset(rank * D)             # ... and the member offset keeps their members apart
        g = torch.Generator().manual_seed(2005)
        self.images_host = torch.rand(self.R, 1, 28, 28, generator=g).pin_memory()
        self.labels_host = torch.randint(10, (self.R,), generator=g).pin_memory()
        self.images, self.labels = self.images_host.to(dev), self.labels_host.to(dev)
        self.fit_host = torch.empty(D).pin_memory()
        self.nparams = sum(p.numel() for p in self.net.parameters())
        self.grad_host = torch.empty(self.nparams).pin_memory()
        self.bucket = None
        self.h2d = self.images_host.numel() * 4 + self.labels_host.numel() * 8
        self.d2h = (D + self.nparams) * 4

    def step(self, mark):
        pm, es = self.pm, self.es
        pm.set_seed()             # new seeds every step, as the reference's trainer does (mnisttest.py:128-131)
        pm.set_noise()
        mark("set_noise")
        fit = es.population_fitness(pm, self.images, self.labels, self.D, streams=2 if self.tc == "bf16" else 1)
        mark("forward")
        _, self.bucket = self._update(fit)
        mark("update")
        return fit

    def _update(self, fit):
        from nesgpu_b200 import dist as ndist
        sizes = [self.D] * self.world if self.world > 1 else None      # equal slices: no size exchange, no host sync
        everyone = ndist.gather_fitness(fit, sizes=sizes)
        w_all = self.es.update_weights(everyone, 0.02)
        rank = torch.distributed.get_rank() if self.world > 1 else 0
        lo, hi = ndist.member_slice(everyone.numel(), rank, self.world)
        for p in self.net.parameters():
            p.grad = None
        with torch.no_grad():
            self.pm.update(w_all[lo:hi].contiguous())
        return fit, ndist.all_reduce_grads(self.net.parameters(), self.bucket)

    def step_e2e(self):
        self.images.copy_(self.images_host, non_blocking=True)
        self.labels.copy_(self.labels_host, non_blocking=True)
        fit = self.step(lambda name: None)
        self.fit_host.copy_(fit, non_blocking=True)
        if self.bucket is not None:
            self.grad_host.copy_(self.bucket.flat, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def roofline(self, phase_ms, peaks):
        flops = self.FLOP_PER_PAIR * self.D * self.R
        ach = flops / (phase_ms["forward"] * 1e-3) / 1e12
        peak = peaks["bf16_sustained"] / 2
        kernels = ("shared_conv_pool_kernel, conv_pool_tc_kernel / conv_pool_pair_kernel, permuted_operand_kernel + gemm_tf32_kernel, CE"
                   if self.fused else "conv1, conv2, fc1, fc2 kernels + torch ReLU / MaxPool / CE")
        return {"kernel": "population forward (%s), forward phase" % kernels,
                "bound": "tensor", "achieved": round(ach, 2), "peak": peak, "unit": "TFLOP/s", "frac": round(ach / peak, 4),
                "peak_source": peaks["source"] + " bf16 sustained / 2 taken as TF32",
                "algorithmic_flops_per_launch": flops, "ms_per_launch": round(phase_ms["forward"], 3), "traffic": None,
                "es_steps_per_s": round(1e3 / sum(phase_ms.values()), 3),
                "note": "flops for the minimal one-product form (5.262 MFLOP per member-image pair); the fused conv2 kernel "
                        "evaluates the two-product form (stacked filter [W; eps]), i.e. about twice these flops on the tensor pipe"}

    def cpu_sample(self, reps):
        """CPU oracle on 16 members x 32 images of the same net (forward + CE + ranks + update)."""
        from oracle import perturbed_ref as O
        import torch.nn.functional as F
        Ds, Rs = 16, 32
        g = torch.Generator().manual_seed(5)
        shapes = [("conv", 1, 32), ("conv", 32, 64), ("lin", 1600, 128), ("lin", 128, 10)]
        layers = []
        for kind, cin, cout in shapes:
            p_in, p_out, isp, osp = O.resolve_permutation(cin, cout)
            tail = (3, 3) if kind == "conv" else ()
            layers.append(dict(kind=kind, cin=cin, cout=cout,
                               W=torch.randn(cout, cin, *tail, generator=g) * 0.05, b=torch.zeros(cout),
                               eps=0.02 * torch.randn(osp, isp, *tail, generator=g), beta=0.02 * torch.randn(Ds, cout, generator=g),
                               pin=torch.stack([torch.randperm(cin, generator=g) for _ in range(Ds)]).short() if p_in else None,
                               pout=torch.stack([torch.randperm(cout, generator=g) for _ in range(Ds)]).short() if p_out else None))
        images = torch.rand(Rs, 1, 28, 28, generator=g)
        labels = torch.randint(10, (Rs,), generator=g)

        def once():
            t0 = time.perf_counter()
            x = images.unsqueeze(1).expand(Rs, Ds, 1, 28, 28).reshape(Rs * Ds, 1, 28, 28)
            for i, L in enumerate(layers):
                if L["kind"] == "conv":
                    x = O.permuted_conv2d_forward(x, L["W"], L["b"], L["eps"], L["beta"], L["pin"], L["pout"], Ds)
                    x = F.max_pool2d(F.relu(x), 2)
                else:
                    x = O.permuted_linear_forward(x.reshape(Rs * Ds, -1), L["W"], L["b"], L["eps"], L["beta"], L["pin"], L["pout"], Ds)
                    if i == 2:
                        x = F.relu(x)
            ce = F.cross_entropy(x, labels.repeat_interleave(Ds), reduction="none").view(Rs, Ds)
            w = O.centered_ranks(-ce.mean(0))
            for L in layers:
                if L["kind"] == "conv":
                    O.permuted_conv2d_weight_grad(L["eps"], w, L["pin"], L["pout"], L["cin"], L["cout"])
                else:
                    O.permuted_linear_weight_grad(L["eps"], w, L["pin"], L["pout"], L["cin"], L["cout"])
            return time.perf_counter() - t0
        once()
        return Ds * Rs, [once() for _ in range(reps)], "16 members x 32 images of the same net: forward + CE + ranks + update per repetition"


WORKLOADS = {w.name: w for w in (PerturbedLinear1024, PermutedLinear256, PermutedConv64, PerturbedConv64, SparseLinear1024,
                                 SyntheticLinear1024, Binary1024, BinaryBmm64, BinaryConv512, EsCnn)}


# ---------------------------------------------------------------------------------- runs

UNIT = "member-samples/s"
METRIC = "perturbed-member samples/sec per layer (forward + update)"


def bind_to_gpu_numa_node(local_rank):
    """Run this process on the CPUs of the NUMA node its GPU hangs off, so that the pinned host buffers it allocates
    afterwards (first touch) and its copy threads are local to that GPU.  Returns the node, or a string that
    says why nothing was bound."""
    try:
        props = torch.cuda.get_device_properties(local_rank)
        bdf = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        node = int(open("/sys/bus/pci/devices/%s/numa_node" % bdf).read().strip())
        if node < 0:
            return "no NUMA node reported for %s" % bdf
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            return node
        return "node %d has no CPU this process may use" % node
    except (OSError, ValueError, AttributeError) as exc:
        return "%s: %s" % (type(exc).__name__, exc)


def _sync_all(world):
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def _max_over_ranks(ms, dev, world):
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return t.item()


def _flush_buffer(wl, dev):
    """L2 flush between timed steps for workloads whose working set fits in L2 twice over."""
    if wl.resident_bytes < 2 * L2_BYTES:
        return torch.empty(2 * L2_BYTES // 4, dtype=torch.float32, device=dev)
    return None


def time_steps(wl, steps, warmup, dev, world, use_graph=True, sampler=None):
    """W untimed steps, then exactly K timed steps between barriers, CUDA events on the launching stream; the time
    is the max over ranks.  Launch-bound workloads (``wl.use_graph``) replay a captured CUDA graph at N = 1."""
    from nesgpu_b200 import _cabi
    flush = _flush_buffer(wl, dev)
    null_mark = lambda name: None
    for _ in range(warmup):
        wl.step(null_mark)
        if flush is not None:
            flush.fill_(1.0)
    _sync_all(world)
    graph = None
    if getattr(wl, "use_graph", False) and world == 1 and use_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            wl.step(null_mark)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            wl.step(null_mark)
        for _ in range(3):
            graph.replay()
        _sync_all(world)
    if sampler:
        sampler.wait_first_sample()
    names, events = [], []
    launches0 = _cabi.lib.nes_launch_count()
    _sync_all(world)
    if sampler:
        sampler.begin()
    t_wall0 = time.perf_counter()
    for i in range(steps):
        ev = [torch.cuda.Event(enable_timing=True)]
        ev[0].record()

        def mark(name, ev=ev, i=i):
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            ev.append(e)
            if i == 0:
                names.append(name)
        if graph is not None:
            graph.replay()
            mark("step")
        else:
            wl.step(mark)
        events.append(ev)
        if flush is not None:
            flush.fill_(1.0)
    _sync_all(world)
    wall = time.perf_counter() - t_wall0
    if sampler:
        sampler.end()
    launches = _cabi.lib.nes_launch_count() - launches0
    total_ms = sum(ev[0].elapsed_time(ev[-1]) for ev in events)
    if flush is None:      # contiguous region: first start to last end
        total_ms = events[0][0].elapsed_time(events[-1][-1])
    phase_ms = {n: statistics.mean(ev[j].elapsed_time(ev[j + 1]) for ev in events) for j, n in enumerate(names)}
    total_ms = _max_over_ranks(total_ms, dev, world)
    _cabi.check_device_errors()
    return {"ms_per_step": total_ms / steps, "phase_ms": phase_ms, "graph": graph, "flush": flush, "wall": wall,
            "launches": int(launches) if graph is None else int(wl.launches_per_step * steps)}


def time_sustained(wl, timing, ms_per_step, dev, world, local_rank, rank, seconds=1.0):
    """The same step repeated until the block spans at least ``seconds`` (the step count is derived from the
    headline time, so every rank runs the same number of steps), with clock samples taken inside it."""
    graph, flush = timing["graph"], timing["flush"]
    steps = max(10, int(seconds * 1e3 / max(ms_per_step, 1e-3)) + 1)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        sampler.wait_first_sample()
    null_mark = lambda name: None
    _sync_all(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler:
        sampler.begin()
    e0.record()
    for _ in range(steps):
        if graph is not None:
            graph.replay()
        else:
            wl.step(null_mark)
        if flush is not None:
            flush.fill_(1.0)
    e1.record()
    _sync_all(world)
    if sampler:
        sampler.end()
    ms = _max_over_ranks(e0.elapsed_time(e1), dev, world) / steps
    out = {"steps": steps, "ms_per_step": round(ms, 4), "seconds": round(ms * steps * 1e-3, 3),
           "value": round(wl.units_per_step * world / (ms * 1e-3), 1),
           "clocks": sampler.stop() if sampler else None}
    if flush is not None:
        out["note"] = "includes the L2 flush between steps (the headline times the steps only)"
    return out


def time_e2e(wl, steps, dev, world):
    for _ in range(2):
        wl.step_e2e()
    _sync_all(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(3, min(steps, 20))
    e0.record()
    for _ in range(e2e_steps):
        wl.step_e2e()
    e1.record()
    _sync_all(world)
    return _max_over_ranks(e0.elapsed_time(e1), dev, world) / e2e_steps, e2e_steps


def es_step_extra(dev, rank, world):
    """The metric's second half, ES steps/s: one ES step of the small CNN (1024 members x 256 images per GPU) timed the
    same way (5 steps after 3 warm-up steps, barrier on both sides, max over ranks) at the fp32 bar and in the two
    stated reduced-precision modes."""
    out = {"workload": "es_cnn_8192", "images_per_member": EsCnn.R, "directions_per_gpu": EsCnn.D,
           "population": EsCnn.D * world, "steps": 5, "warmup": 3}
    null_mark = lambda name: None
    for mode in ("fp32", "tf32", "bf16"):
        try:
            es = EsCnn()
            es.tc = mode
            es.setup(dev, rank, world)
            for _ in range(3):
                es.step(null_mark)
            _sync_all(world)
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(5):
                es.step(null_mark)
            a1.record()
            _sync_all(world)
            ms = _max_over_ranks(a0.elapsed_time(a1), dev, world) / 5
            out[mode] = {"ms_per_step": round(ms, 3), "es_steps_per_s": round(1e3 / ms, 2),
                         "member_image_pairs_per_s": round(es.D * es.R * world / (ms * 1e-3), 1)}
            del es
        except Exception as exc:      # the headline line must not depend on this extra
            out[mode] = {"error": "%s: %s" % (type(exc).__name__, exc)}
    torch.cuda.empty_cache()
    return out


# the other single-layer configurations, measured in the default run next to the headline (N = 1)
PER_CONFIG = [
    ("permuted_linear_256", "permuted_linear_256", None, 200),
    ("permuted_conv_64", "permuted_conv_64", None, 20),
    ("permuted_conv_64_tf32", "permuted_conv_64", "tf32", 20),
    ("permuted_conv_64_bf16", "permuted_conv_64", "bf16", 20),
    ("perturbed_conv_64", "perturbed_conv_64", None, 20),
    ("sparse_linear_1024", "sparse_linear_1024", None, 50),
    ("synthetic_linear_1024", "synthetic_linear_1024", None, 50),
    ("binary_1024", "binary_1024", None, 30),
    ("binary_bmm_n64", "binary_bmm_n64", None, 30),
    ("binary_conv_512", "binary_conv_512", None, 30),
]


def per_config_extra(dev, rank, peaks):
    out = {}
    for key, name, tc, steps in PER_CONFIG:
        if name not in WORKLOADS:
            continue
        try:
            wl = WORKLOADS[name]()
            wl.tc = tc
            wl.setup(dev, rank, 1)
            t = time_steps(wl, steps, 3, dev, 1)
            e2e_ms, _ = time_e2e(wl, 10, dev, 1) if hasattr(wl, "step_e2e") else (None, 0)
            entry = {"config": wl.describe(1), "precision_mode": wl.mode(), "steps": steps,
                     "ms_per_step": round(t["ms_per_step"], 4),
                     "value": round(wl.units_per_step / (t["ms_per_step"] * 1e-3), 1), "unit": UNIT,
                     "phase_ms": {k: round(v, 4) for k, v in t["phase_ms"].items()}, "cuda_graph": t["graph"] is not None,
                     "gpu_launches_per_step": t["launches"] / steps, "roofline": wl.roofline(t["phase_ms"], peaks)}
            if e2e_ms:
                entry["e2e"] = {"value": round(wl.units_per_step / (e2e_ms * 1e-3), 1), "ms_per_step": round(e2e_ms, 4),
                                "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h}
            out[key] = entry
            del wl, t
        except Exception as exc:
            out[key] = {"error": "%s: %s" % (type(exc).__name__, exc)}
        torch.cuda.empty_cache()
    return out


# ---- the reference's own layer file (oracle/_ref, a copy made by the build step where a checkout exists)

def reference_module():
    from oracle import reference_copy
    return reference_copy.load()


def reference_state(ref, name, dev, members=None):
    """A layer of the reference's ``modules/base.py`` on ``dev`` with seeded noise / permutation tensors assigned
    (``set_noise`` is bypassed: its generator is device-specific), plus a closure that runs one forward + update.
    Returns (units per step, step function, description)."""
    g = torch.Generator().manual_seed(4242)
    if name == "perturbed_linear_1024":
        n, R = 1024, 2
        D = members or 1024
        layer = ref.PerturbedLinear(n, n, D, antithetic=True).to(dev)
        with torch.no_grad():
            layer.weight.copy_(torch.randn(n, n, generator=g) / n ** .5)
            layer.bias.zero_()
        layer.weight_noise = torch.empty(D, n, n, device=dev).normal_(0, 0.02)
        layer.bias_noise = torch.empty(D, n, device=dev).normal_(0, 0.02)
        x = torch.randn(D * R, n, generator=g).to(dev)
        w = (torch.rand(D, generator=g) * 2 - 1).to(dev)
        units, what = D * R, "%d of 1024 members, PerturbedLinear(1024,1024) antithetic: forward + update" % D
    elif name == "permuted_linear_256":
        n, R, D = 256, 2, 512
        layer = ref.PermutedLinear(n, n, D, antithetic=True).to(dev)
        with torch.no_grad():
            layer.weight.copy_(torch.randn(n, n, generator=g) / n ** .5)
            layer.bias.zero_()
        layer.weight_noise = (0.02 * torch.randn(n, n, generator=g)).to(dev)
        layer.bias_noise = (0.02 * torch.randn(D, n, generator=g)).to(dev)
        layer.output_permutations = torch.stack([torch.randperm(n, generator=g) for _ in range(D)]).short().to(dev)
        x = torch.randn(D * R, n, generator=g).to(dev)
        w = torch.randn(D, generator=g).to(dev)
        units, what = D * R, "full configuration, PermutedLinear(256,256) x 512 antithetic pairs: forward + update"
    elif name == "permuted_conv_64":
        c, hw = 64, 32
        D = members or 1024
        layer = ref.PermutedConv2d(c, c, 3, D, padding=1, out_sparsity=.5).to(dev)
        with torch.no_grad():
            layer.weight.copy_(torch.randn(c, c, 3, 3, generator=g) * (2 / 576) ** .5)
            layer.bias.zero_()
        layer.weight_noise = (0.02 * 2 ** .5 * torch.randn(32, c, 3, 3, generator=g)).to(dev)
        layer.bias_noise = (0.02 * torch.randn(D, c, generator=g)).to(dev)
        layer.output_permutations = torch.stack([torch.randperm(c, generator=g) for _ in range(D)]).short().to(dev)
        x = torch.randn(D, c, hw, hw, generator=g).to(dev)
        w = torch.randn(D, generator=g).to(dev)
        units, what = D, "%d of 1024 members, PermutedConv2d(64,64,3,padding=1,out_sparsity=.5) on 32x32: forward + update" % D
    else:
        return None

    def step():
        with torch.no_grad():
            layer.perturbed_flag = True
            y = layer.forward(x)
            layer.perturbed_flag = False
            layer.weight.grad = None
            if layer.bias is not None:
                layer.bias.grad = None
            layer.update(w)
        return y
    return units, step, what


def gpu_reference_extra(dev):
    """Informational: the reference's own PyTorch layers (cuBLAS / cuDNN / ATen chains) on the same GPU for the three
    fp32 single-layer configurations -- the library chains the kernels of this repository replace."""
    ref = reference_module()
    if ref is None:
        return {"unavailable": "no copy of the reference's modules/base.py under oracle/_ref on this machine"}
    out = {"kind": "reference (modules/base.py, unmodified) on cuda", "statistic": "median of 20 after 5 warm-up steps, CUDA events"}
    for name in ("permuted_linear_256", "perturbed_linear_1024", "permuted_conv_64"):
        try:
            units, step, what = reference_state(ref, name, dev)
            for _ in range(5):
                step()
            torch.cuda.synchronize()
            times = []
            for _ in range(20):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                step()
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            med = statistics.median(times)
            out[name] = {"ms_per_step": round(med, 4), "value": round(units / (med * 1e-3), 1), "unit": UNIT, "sample": what}
            del step
        except Exception as exc:
            out[name] = {"error": "%s: %s" % (type(exc).__name__, exc)}
        torch.cuda.empty_cache()
    return out


def cpu_baseline(wl, reps, unit):
    """The CPU arm beside the GPU number: the reference's own layer file where a copy exists and covers the workload
    (``kind: "reference"``), else the CPU restatement under oracle/ (``kind: "port"``); all host cores."""
    ref = reference_module()
    state = reference_state(ref, wl.name, "cpu", members=128 if wl.name != "permuted_linear_256" else None) if ref else None
    if state is not None:
        units, step, what = state
        step()
        times = []
        for _ in range(reps):
            t0 = time.perf_counter()
            step()
            times.append(time.perf_counter() - t0)
        med = statistics.median(times)
        return {"value": round(units / med, 2), "unit": unit, "cores": torch.get_num_threads(), "kind": "reference",
                "sample": what, "seconds_per_repetition": round(med, 4), "repetitions": len(times)}
    units, times, sample = wl.cpu_sample(reps)
    med = statistics.median(times)
    cores = getattr(wl, "cpu_cores", None) or torch.get_num_threads()
    return {"value": round(units / med, 2), "unit": unit, "cores": cores, "kind": "port",
            "sample": sample, "seconds_per_repetition": round(med, 4), "repetitions": len(times)}


def run_reference(args, rank, world):
    """The reference arm: the reference's own CPU implementation of the workload on the host cores (its unmodified
    ``modules/base.py`` from oracle/_ref with seeded tensors assigned, the whole configuration when it fits the host's
    memory), else the CPU restatement under oracle/.  Rank 0 alone runs it."""
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    wl = WORKLOADS[args.workload]()
    ref = reference_module()
    state = None
    if ref is not None:
        try:
            import psutil
            roomy = psutil.virtual_memory().available > 12 * 2 ** 30
        except Exception:
            roomy = False
        members = None if (roomy or args.workload == "permuted_linear_256") else 128
        state = reference_state(ref, args.workload, "cpu", members=members)
    if state is not None:
        units, step, sample = state
        kind = "reference"
        for _ in range(max(1, args.warmup)):
            step()
        times = []
        budget = time.perf_counter() + 150.0            # the whole arm ends within a few minutes
        for _ in range(args.steps):
            t0 = time.perf_counter()
            step()
            times.append(time.perf_counter() - t0)
            if time.perf_counter() > budget:
                break
        cores = torch.get_num_threads()
        note = ("the reference's own modules/base.py (unmodified copy under oracle/_ref) on the host cores with seeded "
                "noise and permutation tensors assigned; each step is one forward + update of the sample")
    else:
        kind = "port"
        if args.workload in ("permuted_linear_256", "permuted_conv_64"):
            _cpu_layer_state(wl)
        units, times, sample = wl.cpu_sample(args.steps + args.warmup)
        times = times[args.warmup:] if len(times) > args.warmup else times
        cores = getattr(wl, "cpu_cores", None) or torch.get_num_threads()
        note = ("CPU restatement (oracle/) of the reference's algorithm on the host cores: the reference has no CPU path "
                "for this workload or no copy of it exists on this machine; each step is the bounded sample")
    total = sum(times)
    value = units * len(times) / total
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": args.gpus,
            "steps": len(times), "warmup": args.warmup, "ms_per_step": round(1e3 * total / len(times), 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": wl.describe(1),
            "cpu_baseline": {"value": round(value, 2), "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": round(value, 2), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "note": note}
    if args.workload == "perturbed_linear_1024" and not args.no_es:
        # the ES step of the small CNN on the host cores, next to the es_step entry of the GPU arm
        try:
            es_units, es_times, es_sample = EsCnn().cpu_sample(2)
            med = statistics.median(es_times)
            line["es_step"] = {"workload": "es_cnn_8192", "member_image_pairs_per_s": round(es_units / med, 1),
                               "seconds_per_repetition": round(med, 4), "cores": torch.get_num_threads(), "kind": "port",
                               "sample": es_sample}
        except Exception as exc:
            line["es_step"] = {"error": "%s: %s" % (type(exc).__name__, exc)}
    emit(line)


def _cpu_layer_state(wl):
    """Layer state for the CPU-only port arm, drawn with torch's CPU generator."""
    g = torch.Generator().manual_seed(4242)

    class S:
        pass
    s = S()
    if wl.name == "permuted_linear_256":
        n, D = wl.n, wl.D
        s.weight = torch.randn(n, n, generator=g) / n ** .5
        s.bias = torch.zeros(n)
        s.weight_noise = 0.02 * torch.randn(n, n, generator=g)
        s.bias_noise = 0.02 * torch.randn(D, n, generator=g)
        s.output_permutations = torch.stack([torch.randperm(n, generator=g) for _ in range(D)]).short()
        wl.x_host = torch.randn(D * wl.R, n, generator=g)
        wl.w_host = torch.randn(D, generator=g)
    else:
        c, D = wl.c, wl.D
        s.weight = torch.randn(c, c, 3, 3, generator=g) * (2 / 576) ** .5
        s.bias = torch.zeros(c)
        s.weight_noise = 0.02 * 2 ** .5 * torch.randn(32, c, 3, 3, generator=g)
        s.bias_noise = 0.02 * torch.randn(D, c, generator=g)
        s.output_permutations = torch.stack([torch.randperm(c, generator=g) for _ in range(D)]).short()
        wl.x_host = torch.randn(128, c, wl.hw, wl.hw, generator=g)
        wl.w_host = torch.randn(D, generator=g)
    wl.layer = s


def allreduce_check(wl, dev, world):
    """Correctness of the NCCL path: the all-reduced weight gradient against the sum of the ranks' all-gathered partial
    gradients, on the first 4096 entries."""
    import torch.distributed as dist
    layer = wl.layer
    with torch.no_grad():
        layer.weight.grad = None
        layer.bias.grad = None
        partial = layer.weight_grad(wl.w).flatten()[:4096].double().contiguous()
        parts = [torch.empty_like(partial) for _ in range(world)]
        dist.all_gather(parts, partial)
        want = torch.stack(parts).sum(dim=0)
        grad, _ = wl._update(wl.w)
        got = grad.flatten()[:4096].double()
    err = ((got - want).abs().max() / want.abs().max().clamp_min(1e-30)).item()
    return {"entries": 4096, "max_rel_err": err, "ranks": world}


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    numa_node = bind_to_gpu_numa_node(local_rank) if world > 1 else None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    wl = WORKLOADS[args.workload](args.members) if args.members else WORKLOADS[args.workload]()
    wl.tc = args.tc
    if args.unfused:
        wl.fused = False
    if args.overlap_update:
        wl.overlap_blocks = args.overlap_update
    wl.setup(dev, rank, world)
    peaks = measured_peaks()
    default_run = args.workload == "perturbed_linear_1024" and not args.members

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    timing = time_steps(wl, args.steps, args.warmup, dev, world, use_graph=not args.no_graph, sampler=sampler)
    clocks = sampler.stop() if sampler else None
    ms_per_step = timing["ms_per_step"]
    e2e_ms, e2e_steps = time_e2e(wl, args.steps, dev, world)
    sustained = time_sustained(wl, timing, ms_per_step, dev, world, local_rank, rank) if not args.no_extras else None

    extras = {}
    if world > 1 and args.workload == "perturbed_linear_1024" and not args.no_extras:
        try:
            extras["allreduce_check"] = allreduce_check(wl, dev, world)
        except Exception as exc:
            extras["allreduce_check"] = {"error": "%s: %s" % (type(exc).__name__, exc)}
        try:
            # strong scaling: the configuration's own population of 1024 members split over the GPUs
            sw = PerturbedLinear1024(max(1, 1024 // world))
            sw.tc = args.tc
            sw.setup(dev, rank, world)
            st = time_steps(sw, min(args.steps, 200), args.warmup, dev, world)
            extras["strong"] = {"population": sw.D * world, "members_per_gpu": sw.D, "ms_per_step": round(st["ms_per_step"], 4),
                                "value": round(sw.units_per_step * world / (st["ms_per_step"] * 1e-3), 1), "unit": UNIT,
                                "phase_ms": {k: round(v, 4) for k, v in st["phase_ms"].items()}}
            del sw, st
            torch.cuda.empty_cache()
        except Exception as exc:
            extras["strong"] = {"error": "%s: %s" % (type(exc).__name__, exc)}
    if default_run and not args.no_es:
        extras["es_step"] = es_step_extra(dev, rank, world)
    roofline = wl.roofline(timing["phase_ms"], peaks) if rank == 0 else None
    config = wl.describe(world)
    mode = wl.mode()
    h2d, d2h = getattr(wl, "h2d", None), getattr(wl, "d2h", None)
    timing["graph"] = timing["flush"] = None
    if default_run and world == 1 and not args.no_extras:
        del wl                                    # 4 GiB of noise: the other configurations get a clean device
        torch.cuda.empty_cache()
        extras["per_config"] = per_config_extra(dev, rank, peaks)
        extras["gpu_reference"] = gpu_reference_extra(dev)
        wl = WORKLOADS[args.workload]()           # for the CPU baseline below (no device state needed)

    if rank == 0:
        value = wl.units_per_step * world / (ms_per_step * 1e-3)
        line = {"metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": config, "precision_mode": mode,
                "e2e": {"value": round(wl.units_per_step * world / (e2e_ms * 1e-3), 1), "unit": UNIT,
                        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": round(e2e_ms, 4), "steps": e2e_steps},
                "gpu_launches": timing["launches"], "cuda_graph": timing["launches"] is not None and getattr(wl, "use_graph", False) and world == 1 and not args.no_graph,
                "phase_ms": {k: round(v, 4) for k, v in timing["phase_ms"].items()},
                "wall_s_timed_region": round(timing["wall"], 4), "clocks": clocks, "roofline": roofline}
        if sustained is not None:
            line["sustained"] = sustained
        if numa_node is not None:
            line["numa_node_rank0"] = numa_node
        line.update(extras)
        if world == 1 and not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count() or 1)
            line["cpu_baseline"] = cpu_baseline(wl, 5, UNIT)
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="perturbed_linear_1024", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="permuted_linear_256: launch every step from Python instead of replaying a captured CUDA graph")
    ap.add_argument("--tc", default=None, choices=["fp32", "tf32", "3xtf32", "bf16", "bf16x3", "auto"],
                    help="tensor-core mode of the layer (default: the layer's own default, which holds the fp32 bar)")
    ap.add_argument("--no-es", action="store_true",
                    help="default workload: skip the extra ES-step measurement (es_step in the JSON line)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the sustained block, the other configurations (per_config), the same-GPU run of the "
                         "reference's layers (gpu_reference) and, at N > 1, the strong-scaling and all-reduce checks")
    ap.add_argument("--overlap-update", type=int, default=0,
                    help="perturbed_linear_1024 at N > 1: form the gradient in this many column blocks and all-reduce each "
                         "while the next one streams (default 0: one update kernel, one in-place all-reduce)")
    ap.add_argument("--unfused", action="store_true",
                    help="es_cnn_8192: separate Conv / ReLU / MaxPool2d modules and per-member input copies instead of the fused layers")
    ap.add_argument("--members", type=int, default=0,
                    help="members per GPU instead of 1024 (small case for ncu captures; not for binary_1024 / permuted_linear_256)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
