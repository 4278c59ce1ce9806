#!/usr/bin/env python
"""Benchmark of the hinge forest evaluation path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c3|c3b|c2|c1|c4|c5|c5tc|c5f]

A step is one pass of the hot path over one batch of seeded synthetic input.  The default
workload (c3) is the large-batch forest inference configuration: x [1048576,128] ~ N(0,1), 1024
trees of depth 8, thresholds U(-3,3), feature indices U[0,127], leaf weights N(0,1).  With N GPUs
every rank evaluates its own batch of that size against replicated parameters (weak scaling; the
forward has no communication, the training workloads all-reduce the parameter gradients once per
step).  Rank 0 prints ONE JSON line:

  value         tree-evals/s, whole job, inputs resident in HBM, CUDA events, max over ranks
  e2e           the same metric through the reference-facing operators / modules with HOST buffers:
                pinned input copied in and the result copied back inside the timed region
  roofline      algorithmic bytes of one step / measured step time, against the measured HBM peak
  cpu_baseline  the C restatement of the reference algorithm on all host threads (bounded sample)
  fwd_bwd       (c3 only) forward + backward of the same shape, device resident: a training step, in which the
                forward keeps its traversal for the backward; a 64-row slice of it is checked against the port
  cuda_graph    (c1, c2) the same step captured once and replayed as a CUDA graph
  workloads     (c3 at N = 1) the other configurations c1, c2, c4, c5 (and c5tc: c5 with this library's tensor-core
                Linear + BatchNorm front; c5f: front and forest as one step, the normalised activations never
                written), a few device-resident steps each, with a slice of each result checked
                against the port in the CPU leg
  strong, train (c3 at N > 1) the large batch split over the ranks (no collective; shards compared with the
                whole on rank 0), and training steps of c2 and c5 with the NCCL all-reduce of the parameter
                gradients inside the timed region
  reference_gpu (c3 at N = 1, when oracle/_ref holds the reference built with its CUDA kernels) the reference's own
                GPU kernels on the same device and tensors: c1 and c2 steps and the c3 forward on a 65 536-row
                chunk, each with this library's time for the same call and whether the results are equal
  gpu_launches  kernels of this library launched inside the timed region (the library's own counter)

Other workloads: c1 (the reference's speedtest shape, fwd+bwd), c2 (ferns, fwd+bwd), c4 (2-D
convolution, fwd+bwd), c5 (Linear -> BatchNorm1d -> sequential-ordinal forest training step).
`--impl reference` times the reference's own CPU implementation (oracle/_ref when it was built,
else the C restatement) on all host cores, on a bounded sample per step.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "c3": dict(op="forest", kind="tree", B=1048576, C=128, T=1024, depth=8, M=0, x="randn", bwd=False,
               name="C3 large-batch forest inference x[1048576,128] T=1024 depth=8"),
    "c3b": dict(op="forest", kind="tree", B=1048576, C=128, T=1024, depth=8, M=0, x="randn", bwd=True,
                name="C3 shape, forward + backward x[1048576,128] T=1024 depth=8"),
    "c2": dict(op="forest", kind="fern", B=4096, C=256, T=500, depth=10, M=10, x="randn", bwd=True,
               name="C2 fern fwd+bwd x[4096,256] T=500 depth=10 extra_outputs=10"),
    "c1": dict(op="forest", kind="tree", B=100, C=1000, T=100, depth=7, M=1, x="rand", bwd=True,
               name="C1 forest fwd+bwd x[100,1000] T=100 depth=7 extra_outputs=1"),
    "c4": dict(op="conv", kind="tree", B=64, C=64, T=128, depth=5, M=0, x="randn", bwd=True, H=64, W=64,
               name="C4 HingeTreeConv2d fwd+bwd x[64,64,64,64] 3x3 s1 p1, 128x64 trees depth 5"),
    "c5": dict(op="pipeline", kind="tree", B=8192, C=784, T=100, depth=7, M=0, x="rand", bwd=True, hidden=12700,
               name="C5 Linear(784->12700) -> BatchNorm1d -> forest(100 trees depth 7, sequential ordinals) train step"),
    "c5f": dict(op="pipeline", kind="tree", B=8192, C=784, T=100, depth=7, M=0, x="rand", bwd=True, hidden=12700, front="fused",
                name="C5 as one step of this library: LinearBatchNormForest (tcgen05 TF32 projection + statistics, forest on "
                     "the unmaterialised normalisation, one-pass batch-norm input gradient) train step"),
    "c5tc": dict(op="pipeline", kind="tree", B=8192, C=784, T=100, depth=7, M=0, x="rand", bwd=True, hidden=12700, front="tc",
                 name="C5 with this library's tensor-core front: LinearBatchNorm1d (tcgen05 TF32 projection + statistics) "
                      "-> forest(100 trees depth 7, sequential ordinals) train step"),
    # the other operator families, for the profiler (--kernel-only): sizes whose tensors exceed L2
    "a5": dict(op="family", family="linear", kind="tree", B=262144, C=784, T=100, depth=7, M=0, O=10, bwd=True,
               name="A5 tree_fused_linear forward + backward x[262144,784] T=100 depth=7 O=10"),
    "a6": dict(op="family", family="fusion", kind="tree", B=2048, C=32, Cv=16, T=64, depth=6, M=0, bwd=True,
               name="A6 tree_fusion forward + backward img[2048,32,16,16] vec[2048,16] T=64 depth=6"),
    "a7": dict(op="family", family="sparse", kind="tree", B=65536, C=256, T=256, depth=7, M=0, bwd=True,
               name="A7 sparse_tree_backward x[65536,256] T=256 depth=7"),
    "a8": dict(op="family", family="contract", kind="tree", B=64, C=64, T=0, depth=1, M=0, H=256, W=256, bwd=False,
               name="A8 contract + expand x[64,64,256,256] float32 window 2x2"),
    "a9": dict(op="family", family="trie", kind="tree", B=131072, C=256, T=256, depth=7, M=0, bwd=True,
               name="A9 trie forward + backward x[131072,256] T=256 depth=7"),
}


# DRAM bytes (read + write) of one full-size launch of the c3 tile kernel, from an Nsight Compute capture of that
# launch with the two DRAM byte counters alone (one pass, nothing saved or restored):
# dram__bytes_read.sum 574.28 MB + dram__bytes_write.sum 4.24 GB.
C3_DRAM_BYTES_PER_LAUNCH = 574.28e6 + 4.24e9


def decisions(kind, depth):
    return depth if kind == "fern" else 2 ** depth - 1


def evals_per_step(wl, B):
    if wl["op"] == "family":
        inner = 256 if wl["family"] == "fusion" else 1
        return B * max(wl["T"], 1) * inner
    if wl["op"] == "conv":
        return B * wl["H"] * wl["W"] * wl["T"] * wl["C"]  # one tree per (out channel, in channel, position)
    return B * wl["T"]


def algorithmic_bytes(wl, B, backward):
    """Compulsory traffic with the API's dtypes (fp32 data, int64 ordinals), each tensor touched once."""
    depth, M = wl["depth"], max(wl["M"], 1)
    N, L = decisions(wl["kind"], depth), 2 ** depth
    if wl["op"] == "conv":
        trees = wl["T"] * wl["C"]
        x_bytes, out_bytes = 4 * B * wl["C"] * wl["H"] * wl["W"], 4 * B * wl["T"] * wl["H"] * wl["W"] * M
    else:
        C = wl["hidden"] if wl["op"] == "pipeline" else wl["C"]
        trees = wl["T"]
        x_bytes, out_bytes = 4 * B * C, 4 * B * wl["T"] * M
    params = 12 * trees * N + 4 * trees * L * M
    fwd = x_bytes + params + out_bytes
    if not backward:
        return fwd
    return fwd + (x_bytes + params + out_bytes) + (x_bytes + 4 * trees * N + 4 * trees * L * M)


def make_params(wl, seed=0):
    import torch
    gen = torch.Generator().manual_seed(seed)
    N, L = decisions(wl["kind"], wl["depth"]), 2 ** wl["depth"]
    extra = (wl["M"],) if wl["M"] else ()
    if wl["op"] == "conv":
        thr = torch.rand((wl["T"], wl["C"], N), generator=gen) * 6 - 3
        ord_ = torch.randint(0, 9, (wl["T"], wl["C"], N), generator=gen)
        w = torch.randn((wl["T"], wl["C"], L) + extra, generator=gen)
        return thr, ord_, w
    C = wl["hidden"] if wl["op"] == "pipeline" else wl["C"]
    thr = torch.rand((wl["T"], N), generator=gen) * 6 - 3
    if wl["op"] == "pipeline":
        ord_ = (torch.arange(wl["T"] * N) % C).view(wl["T"], N)
    else:
        ord_ = torch.randint(0, C, (wl["T"], N), generator=gen)
    w = torch.randn((wl["T"], L) + extra, generator=gen)
    return thr, ord_, w


def make_x(wl, rows, seed, channels=None):
    import torch
    gen = torch.Generator().manual_seed(1000 + seed)
    C = channels or wl["C"]
    shape = (rows, C, wl["H"], wl["W"]) if wl["op"] == "conv" else (rows, C)
    return torch.rand(shape, generator=gen) if wl["x"] == "rand" else torch.randn(shape, generator=gen)


# ---- clocks -------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---- CPU legs ------------------------------------------------------------------------------

def cpu_channels(wl):
    """Feature count the trees see on the CPU legs (the pipeline's forest stage reads the hidden activations)."""
    return wl["hidden"] if wl["op"] == "pipeline" else wl["C"]


def _cpu_forward_port(job):
    from oracle import hinge_oracle as ho
    op, kind, x, thr, ord_, w = job
    if op == "conv":
        return ho.conv_forward(kind, x, thr, ord_, w, (3, 3), (1, 1), (1, 1), (1, 1)).shape[0]
    return ho.forward(kind, x, thr, ord_, w).shape[0]


def cpu_port_rate(wl, rows, threads):
    """The C restatement (forward) on `threads` host threads (ctypes releases the GIL), rows split evenly."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor
    from oracle import hinge_oracle as ho
    ho.lib()
    thr, ord_, w = [t.numpy() for t in make_params(wl)]
    x = make_x(wl, rows, 0, cpu_channels(wl)).numpy()
    parts = [p for p in np.array_split(x, threads) if len(p)]
    jobs = [(wl["op"], wl["kind"], p, thr, ord_, w) for p in parts]
    with ThreadPoolExecutor(max_workers=threads) as ex:
        t0 = time.perf_counter()
        list(ex.map(_cpu_forward_port, jobs))
        dt = time.perf_counter() - t0
    return evals_per_step(wl, rows) / dt, dt


def cpu_sample_rows(wl, cores, seconds=12.0):
    """Rows whose forward takes about `seconds` of wall time on `cores` cores at ~80 ns per tree evaluation."""
    per_row = evals_per_step(wl, 1) * 80e-9
    return int(max(min(cores, wl["B"]), min(wl["B"], seconds * cores / per_row)))


_REF_STATE = {}


def _ref_worker_init(op, kind, thr, ord_, w):
    import torch
    torch.set_num_threads(1)
    from oracle import build_ref
    _REF_STATE["mod"] = build_ref.load()
    _REF_STATE["args"] = (op, kind, thr, ord_, w)


def _ref_worker_run(x):
    op, kind, thr, ord_, w = _REF_STATE["args"]
    mod = _REF_STATE["mod"]
    if op == "conv":
        out = getattr(mod, kind + "_conv2d_forward")(x, thr, ord_, w, [3, 3], [1, 1], [1, 1], [1, 1])
    else:
        out = getattr(mod, kind + "_forward")(x, thr, ord_, w)
    return out.shape[0]


def reference_arm(a, wl):
    """The reference's own CPU implementation (forward) on all host cores, bounded sample per step."""
    import torch
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cores = os.cpu_count() or 1
    rows = cpu_sample_rows(wl, cores, seconds=0.5)
    rows = max(cores, rows - rows % cores) if rows >= cores else rows
    thr, ord_, w = make_params(wl)
    x = make_x(wl, rows, 0, cpu_channels(wl))
    kind_used = "reference"
    try:
        from oracle import build_ref
        build_ref.load()
    except Exception:
        kind_used = "port"
    times = []
    if kind_used == "reference":
        import multiprocessing as mp
        ctx = mp.get_context("fork")
        with ctx.Pool(cores, initializer=_ref_worker_init, initargs=(wl["op"], wl["kind"], thr, ord_, w)) as pool:
            chunks = [c for c in torch.chunk(x, cores) if c.shape[0]]
            for step in range(a.warmup + a.steps):
                t0 = time.perf_counter()
                pool.map(_ref_worker_run, chunks)
                dt = time.perf_counter() - t0
                if step >= a.warmup:
                    times.append(dt)
    else:
        for step in range(a.warmup + a.steps):
            _, dt = cpu_port_rate(wl, rows, cores)
            if step >= a.warmup:
                times.append(dt)
    total = sum(times)
    value = evals_per_step(wl, rows) * len(times) / total
    sample = "forward of %d of %d rows per step on %d cores" % (rows, wl["B"], cores)
    line = {
        "impl": "reference", "metric": "tree-evals/sec fwd", "value": value, "unit": "tree-evals/s",
        "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["name"], "sample": sample},
        "cpu_baseline": {"value": value, "unit": "tree-evals/s", "cores": cores, "kind": kind_used, "sample": sample},
        "e2e": {"value": value, "unit": "tree-evals/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- our arm: one runner per kind of workload ------------------------------------------------

class ForestRunner:
    """Plain forest / fern through the C ABI (device resident) and through hingetree_cpp (end to end)."""

    def __init__(self, wl, B, device, rank, world=1):
        import torch
        from hingetreefortorch_b200 import _cabi
        from hingetreefortorch_b200._ext import hingetree_cpp
        self.wl, self.B, self.device, self.torch, self.ext = wl, B, device, torch, hingetree_cpp
        self.world = world
        self.thr, self.ord, self.w = [t.to(device) for t in make_params(wl)]
        self.x_host = make_x(wl, B, rank)
        self.x = self.x_host.to(device)
        self.forest = _cabi.Forest(wl["kind"], self.x, self.w)
        self.out = torch.empty(self.forest.out_shape, dtype=torch.float32, device=device)
        self.g = None
        # a training step keeps the forward's traversal for the backward where the library offers it
        self.keep = self.forest.saves_forward()

    def enable_backward(self):
        torch = self.torch
        if self.g is None:
            self.g = torch.randn(self.forest.out_shape, generator=torch.Generator(device=self.device).manual_seed(5),
                                 device=self.device)
            # threshold and leaf-weight gradients side by side in one buffer: one all-reduce per step at N > 1
            self.param_grads = torch.empty(self.thr.numel() + self.w.numel(), dtype=torch.float32, device=self.device)
            n = self.thr.numel()
            self.grads = (torch.empty_like(self.x), self.param_grads[:n].view_as(self.thr),
                          self.param_grads[n:].view_as(self.w))

    def step(self, backward, reduce=True):
        keep = backward and self.keep
        self.forest.forward(self.x, self.thr, self.ord, self.w, out=self.out, save=keep)
        if backward:
            self.forest.backward(self.x, self.thr, self.ord, self.w, self.g, outs=self.grads, saved=keep)
            if self.world > 1 and reduce:  # a training step: parameter gradients summed over the ranks
                import torch.distributed as dist
                dist.all_reduce(self.param_grads)

    def check(self):
        if self.forest.ordinal_flags() != 0:
            raise SystemExit("bench.py: device status word set (ordinal range or pipeline timeout)")

    def prepare_e2e(self):
        torch, B = self.torch, self.B
        self.chunk = min(B, 65536)
        self.x_pinned = self.x_host.pin_memory()
        self.out_pinned = torch.empty(self.forest.out_shape, dtype=torch.float32).pin_memory()
        self.copy_in, self.copy_out = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)
        self.fwd = getattr(self.ext, self.wl["kind"] + "_forward")
        self.bwd = getattr(self.ext, self.wl["kind"] + "_backward")
        if self.wl["bwd"]:
            self.g_pinned = self.g.cpu().pin_memory()
            self.gx_pinned = torch.empty_like(self.x_host).pin_memory()
        elem = 4 * max(self.wl["M"], 1)
        h2d, d2h = 4 * B * self.wl["C"], elem * B * self.wl["T"]
        if self.wl["bwd"]:
            h2d, d2h = h2d + d2h, d2h + 4 * B * self.wl["C"]
        return h2d, d2h, ("hingetree_cpp.%s_forward%s on %d-row chunks, pinned host buffers, 3 streams"
                          % (self.wl["kind"], "/_backward" if self.wl["bwd"] else "", self.chunk))

    def e2e_step(self):
        torch, B, chunk = self.torch, self.B, self.chunk
        compute = torch.cuda.current_stream(self.device)
        keep = []
        for lo in range(0, B, chunk):
            hi = min(B, lo + chunk)
            with torch.cuda.stream(self.copy_in):
                xc = self.x_pinned[lo:hi].to(self.device, non_blocking=True)
                gc = self.g_pinned[lo:hi].to(self.device, non_blocking=True) if self.wl["bwd"] else None
                ready = torch.cuda.Event()
                ready.record(self.copy_in)
            compute.wait_event(ready)
            oc = self.fwd(xc, self.thr, self.ord, self.w)
            gxc = None
            if self.wl["bwd"]:
                gxc = self.bwd(xc, True, self.thr, True, self.ord, False, self.w, True, gc)[0]
                gc.record_stream(compute)
            xc.record_stream(compute)
            done = torch.cuda.Event()
            done.record(compute)
            self.copy_out.wait_event(done)
            with torch.cuda.stream(self.copy_out):
                self.out_pinned[lo:hi].copy_(oc, non_blocking=True)
                oc.record_stream(self.copy_out)
                if gxc is not None:
                    self.gx_pinned[lo:hi].copy_(gxc, non_blocking=True)
                    gxc.record_stream(self.copy_out)
            keep.append((oc, gxc))
        self.copy_out.synchronize()

    def verify_e2e(self):
        if not self.torch.equal(self.out_pinned[:256], self.out[:256].cpu()):
            raise SystemExit("bench.py: end-to-end output differs from the device-resident output")

    def release_e2e(self):
        self.x_pinned = self.out_pinned = None
        if self.wl["bwd"]:
            self.g_pinned = self.gx_pinned = None


class ModuleRunner:
    """Workloads driven through the nn.Module surface: convolution (c4) and the Linear->BN->forest pipeline (c5)."""

    def __init__(self, wl, B, device, rank, world):
        import torch
        import torch.nn as nn
        from hingetreefortorch_b200 import RandomHingeForest as R
        self.wl, self.B, self.device, self.torch, self.world = wl, B, device, torch, world
        torch.manual_seed(0)
        thr, ord_, w = make_params(wl)
        if wl["op"] == "conv":
            module = R.HingeTreeConv2d(wl["C"], wl["T"], wl["depth"], 3, stride=1, padding=1)
            self.model = module
        else:
            module = R.RandomHingeForest(wl["hidden"], wl["T"], wl["depth"], init_type="sequential")
            if wl.get("front") == "fused":
                self.model = R.LinearBatchNormForest(R.LinearBatchNorm1d(wl["C"], wl["hidden"]), module)
            elif wl.get("front") == "tc":
                self.model = nn.Sequential(R.LinearBatchNorm1d(wl["C"], wl["hidden"]), module)
            else:
                self.model = nn.Sequential(nn.Linear(wl["C"], wl["hidden"], bias=False),
                                           nn.BatchNorm1d(wl["hidden"], affine=False), module)
        with torch.no_grad():
            module.thresholds.copy_(thr)
            module.ordinals.copy_(ord_)
            module.weights.copy_(w)
        self.model = self.model.to(device)
        self.x_host = make_x(wl, B, rank)
        self.x = self.x_host.to(device).requires_grad_(wl["op"] == "conv")
        self.bucket = None
        if world > 1:
            from hingetreefortorch_b200.distributed import GradientBucket
            self.bucket = GradientBucket([p for p in self.model.parameters() if p.requires_grad])

    def enable_backward(self):
        pass

    def _train_step(self, x, reduce=True):
        for p in self.model.parameters():
            p.grad = None
        if x.grad is not None:
            x.grad = None
        loss = self.model(x).sum()
        loss.backward()
        if self.bucket is not None and reduce:
            self.bucket.all_reduce()
        return loss

    def step(self, backward, reduce=True):
        self._train_step(self.x, reduce)

    def check(self):
        pass

    def prepare_e2e(self):
        self.x_pinned = self.x_host.pin_memory()
        self.loss_host = self.torch.empty((), dtype=self.torch.float32).pin_memory()
        return self.x_host.numel() * 4, 4, "nn.Module forward + loss.backward(), pinned host input, loss read back"

    def e2e_step(self):
        x = self.x_pinned.to(self.device, non_blocking=True).requires_grad_(self.wl["op"] == "conv")
        loss = self._train_step(x)
        self.loss_host.copy_(loss.detach(), non_blocking=True)
        self.torch.cuda.current_stream(self.device).synchronize()

    def verify_e2e(self):
        if not self.torch.isfinite(self.loss_host):
            raise SystemExit("bench.py: end-to-end loss is not finite")

    def release_e2e(self):
        self.x_pinned = None


class FamilyRunner:
    """One of the other operator families of the reference's surface through hingetree_cpp, device resident, at a
    size whose tensors exceed L2: fused linear (A5), image + vector fusion (A6), sparse backward (A7), contract /
    expand (A8), trie (A9).  These legs exist for the profiler (bench.py --workload a5 ... --kernel-only)."""

    def __init__(self, wl, B, device, rank, world=1):
        import torch
        from hingetreefortorch_b200._ext import hingetree_cpp as ext
        self.wl, self.B, self.device, self.torch = wl, B, device, torch
        gen = torch.Generator().manual_seed(3)
        family, kind, C, T, depth = wl["family"], wl["kind"], wl["C"], wl["T"], wl["depth"]
        N, L = decisions(kind, depth), 2 ** depth

        def dev(t):
            return t.to(device)

        if family == "contract":
            x = dev(torch.randn((B, C, wl["H"], wl["W"]), generator=gen))
            self.run = lambda: ext.expand(ext.contract(x, [2, 2], [0, 0]), [0, 0])
            return
        thr = dev(torch.rand((T, N), generator=gen) * 6 - 3)
        if family == "linear":
            x = dev(torch.rand((B, C), generator=gen))
            ord_ = dev(torch.randint(0, C, (T, N), generator=gen))
            w = dev(torch.randn((T, L), generator=gen))
            lin, bias = dev(torch.randn((wl["O"], T), generator=gen)), dev(torch.randn((wl["O"],), generator=gen))
            g = dev(torch.randn((B, wl["O"]), generator=gen))
            fwd, bwd = getattr(ext, kind + "_fused_linear_forward"), getattr(ext, kind + "_fused_linear_backward")
            self.run = lambda: (fwd(x, thr, ord_, w, lin, bias),
                                bwd(x, True, thr, True, ord_, False, w, True, lin, True, bias, True, g))
        elif family == "fusion":
            img = dev(torch.randn((B, C, 16, 16), generator=gen))
            vec = dev(torch.randn((B, wl["Cv"]), generator=gen))
            ord_ = dev(torch.randint(0, C + wl["Cv"], (T, N), generator=gen))
            w = dev(torch.randn((T, L), generator=gen))
            g = dev(torch.randn((B, T, 16, 16), generator=gen))
            fwd, bwd = getattr(ext, kind + "_fusion_forward"), getattr(ext, kind + "_fusion_backward")
            self.run = lambda: (fwd(img, vec, thr, ord_, w), bwd(img, True, vec, True, thr, True, ord_, False, w, True, g))
        elif family == "sparse":
            x = dev(torch.randn((B, C), generator=gen))
            ord_ = dev(torch.randint(0, C, (T, N), generator=gen))
            w = dev(torch.randn((T, L), generator=gen))
            g = dev(torch.randn((B, T), generator=gen))
            bwd = getattr(ext, "sparse_" + kind + "_backward")
            self.run = lambda: bwd(x, True, thr, True, ord_, False, w, True, g)
        elif family == "trie":
            x = dev(torch.randn((B, C), generator=gen))
            ord_ = dev(torch.randint(0, C, (T, N), generator=gen))
            w = dev(torch.randn((T, N), generator=gen))  # a weight per internal vertex
            g = dev(torch.randn((B, T), generator=gen))
            self.run = lambda: (ext.trie_forward(x, thr, ord_, w), ext.trie_backward(x, True, thr, True, ord_, False, w, True, g))
        else:
            raise SystemExit("bench.py: unknown family " + family)

    def enable_backward(self):
        pass

    def step(self, backward, reduce=True):
        self.run()

    def check(self):
        pass


def launch_count():
    """Kernels the library has launched so far in this process (its own counter)."""
    from hingetreefortorch_b200 import _cabi
    return int(_cabi.library().ht_launch_count())


def make_runner(wl, B, device, rank, world):
    if wl["op"] == "family":
        return FamilyRunner(wl, B, device, rank, world)
    runner = ForestRunner(wl, B, device, rank, world) if wl["op"] == "forest" else ModuleRunner(wl, B, device, rank, world)
    if wl["bwd"]:
        runner.enable_backward()
    return runner


class Timer:
    """Times steps with CUDA events on the current stream, bracketed by a barrier and a device synchronisation on
    both sides; the figure is the maximum over the ranks."""

    def __init__(self, device, world):
        import torch
        self.torch, self.device, self.world = torch, device, world

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        self.torch.cuda.synchronize()

    def run(self, step, steps):
        """Returns (elapsed ms of all steps, max over ranks; per-step ms on this rank; launches of the library)."""
        torch = self.torch
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        before = launch_count()
        begin.record()
        for s, e in events:
            s.record()
            step()
            e.record()
        end.record()
        self.barrier()
        launches = launch_count() - before
        t = torch.tensor([begin.elapsed_time(end)], dtype=torch.float64, device=self.device)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), [s.elapsed_time(e) for s, e in events], launches


def side_workload(key, device, timer, peak, steps=8):
    """One of the other configurations, device resident, a few steps: what the driver's single run records of it.
    Returns the figures and what the CPU leg needs to check a slice of the result against the port."""
    import torch
    wl = WORKLOADS[key]
    runner = make_runner(wl, wl["B"], device, 0, 1)
    for _ in range(3):
        runner.step(wl["bwd"])
    ms, _, launches = timer.run(lambda: runner.step(wl["bwd"]), steps)
    ms /= steps
    evals = evals_per_step(wl, wl["B"])
    nbytes = algorithmic_bytes(wl, wl["B"], wl["bwd"])
    figures = {"workload": wl["name"], "ms_per_step": ms, "value": evals / (ms * 1e-3), "unit": "tree-evals/s",
               "steps": steps, "bytes_per_step": nbytes, "achieved_gbs": nbytes / (ms * 1e-3) / 1e9,
               "frac": nbytes / (ms * 1e-3) / 1e9 / peak, "gpu_launches_per_step": launches / steps}
    check = None
    rows = min(64, wl["B"])
    if wl["op"] == "forest":
        runner.step(True)
        torch.cuda.synchronize()
        check = {"kind": wl["kind"], "op": "forest", "x": runner.x[:rows].cpu().numpy(), "thr": runner.thr.cpu().numpy(),
                 "ord": runner.ord.cpu().numpy(), "w": runner.w.cpu().numpy(), "g": runner.g[:rows].cpu().numpy(),
                 "out": runner.out[:rows].cpu().numpy(), "gx": runner.grads[0][:rows].cpu().numpy()}
    elif wl["op"] == "conv":
        module = runner.model
        x1 = runner.x[:1].detach()
        with torch.no_grad():
            out1 = module(x1)
        check = {"kind": wl["kind"], "op": "conv", "x": x1.cpu().numpy(), "thr": module.thresholds.detach().cpu().numpy(),
                 "ord": module.ordinals.cpu().numpy(), "w": module.weights.detach().cpu().numpy(), "out": out1.cpu().numpy()}
    else:  # the pipeline's forest stage on the normalised activations the model itself produced
        fused = wl.get("front") == "fused"
        forest = runner.model.forest if fused else runner.model[-1]
        front = runner.model.front if fused else runner.model[:-1]
        with torch.no_grad():
            z = front(runner.x)[:rows].contiguous()
            out = forest(z)
        check = {"kind": wl["kind"], "op": "forest", "x": z.cpu().numpy(), "thr": forest.thresholds.detach().cpu().numpy(),
                 "ord": forest.ordinals.cpu().numpy(), "w": forest.weights.detach().cpu().numpy(), "out": out.cpu().numpy()}
    del runner
    torch.cuda.empty_cache()
    return figures, check


def check_against_port(check):
    """CPU leg: a slice of a workload's device result against the C restatement of the reference algorithm.
    Forward bit for bit; the x gradient (where kept) within 1e-5 of the summed term magnitudes."""
    import numpy as np
    from oracle import hinge_oracle as ho
    if check["op"] == "conv":
        want = ho.conv_forward(check["kind"], check["x"], check["thr"], check["ord"], check["w"], (3, 3), (1, 1), (1, 1), (1, 1))
    else:
        want = ho.forward(check["kind"], check["x"], check["thr"], check["ord"], check["w"])
    ok = bool(np.array_equal(want.reshape(check["out"].shape), check["out"]))
    if ok and "gx" in check:
        ref = ho.backward(check["kind"], check["x"], check["thr"], check["ord"], check["w"], check["g"])[0]
        mag = ho.magnitudes(ho.backward, check["kind"], check["x"], check["thr"], check["ord"], check["w"], check["g"])[0]
        ok = bool(np.all(np.abs(check["gx"].astype(np.float64) - ref) <= 1e-5 * mag + 1e-30))
    return ok


def reference_gpu_leg(device, steps=5):
    """The reference's own CUDA kernels (the unmodified reference built with ``-DWITH_CUDA=1`` by
    ``oracle/build_ref.py --gpu``) on the same GPU and the same tensors, as a second baseline beside the CPU one:
    C1 and C2 steps, and the C3 forward on 65 536-row chunks (the reference launches ``gridDim.y = B / 8`` unchecked,
    hingetree_gpu.cu:491-495, so B stays far below 524 280).  Each figure comes with this library's time on
    the same call and whether the two results are equal bit for bit.  None when the build is not there."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    try:
        import build_ref
        ref = build_ref.load_gpu()
    except Exception:
        return None
    from hingetreefortorch_b200._ext import hingetree_cpp as ours

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(steps):
            fn()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / steps

    legs = {}
    for key, rows in (("c1", None), ("c2", None), ("c3", 65536)):
        wl = WORKLOADS[key]
        B = rows or wl["B"]
        thr, ord_, w = (t.to(device) for t in make_params(wl))
        x = make_x(wl, B, 0).to(device)
        fwd_ref = getattr(ref, wl["kind"] + "_forward")
        fwd_ours = getattr(ours, wl["kind"] + "_forward")
        out_ref, out_ours = fwd_ref(x, thr, ord_, w), fwd_ours(x, thr, ord_, w)
        leg = {"workload": wl["name"] if rows is None else "C3 forward on a %d-row chunk" % B,
               "forward_equal": bool(torch.equal(out_ref, out_ours))}
        if wl["bwd"]:
            g = torch.randn(out_ref.shape, generator=torch.Generator().manual_seed(7)).to(device)
            bwd_ref = getattr(ref, wl["kind"] + "_backward")
            bwd_ours = getattr(ours, wl["kind"] + "_backward")
            g_ref = bwd_ref(x, True, thr, True, ord_, False, w, True, g)
            g_ours = bwd_ours(x, True, thr, True, ord_, False, w, True, g)
            scale = [float(t.abs().max()) for t in (g_ref[0], g_ref[1], g_ref[3])]
            leg["backward_max_difference_over_max"] = max(
                float((a - b).abs().max()) / max(s_, 1e-30)
                for a, b, s_ in zip((g_ref[0], g_ref[1], g_ref[3]), (g_ours[0], g_ours[1], g_ours[3]), scale))
            t_ref = timed(lambda: (fwd_ref(x, thr, ord_, w), bwd_ref(x, True, thr, True, ord_, False, w, True, g)))
            t_ours = timed(lambda: (fwd_ours(x, thr, ord_, w), bwd_ours(x, True, thr, True, ord_, False, w, True, g)))
        else:
            t_ref = timed(lambda: fwd_ref(x, thr, ord_, w))
            t_ours = timed(lambda: fwd_ours(x, thr, ord_, w))
        evals = evals_per_step(wl, B)
        leg.update({"reference_ms": t_ref, "ours_ms": t_ours, "reference_value": evals / (t_ref * 1e-3),
                    "ours_value": evals / (t_ours * 1e-3), "unit": "tree-evals/s", "ratio": t_ref / t_ours})
        legs[key] = leg
        del x, thr, ord_, w, out_ref, out_ours
        torch.cuda.empty_cache()
    legs["call"] = "hingetree_cpp operators of both libraries (allocation and the reference's per-call host sync included)"
    return legs


def bind_to_gpu_numa_node(local):
    """Best effort: run this rank (and first-touch its pinned buffers) on the host cores next to its GPU.
    Returns what was done, for the end-to-end record."""
    try:
        import torch
        props = torch.cuda.get_device_properties(local)
        bus = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        node = int(open("/sys/bus/pci/devices/%s/numa_node" % bus).read())
        if node < 0:
            return {"node": None}
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        usable = cpus & os.sched_getaffinity(0)
        if usable:
            os.sched_setaffinity(0, usable)
        return {"node": node, "cpus": len(usable)}
    except Exception as exc:  # no sysfs entry, no such attribute: leave the affinity alone
        return {"node": None, "why": type(exc).__name__}


def scale_legs(a, device, rank, world, timer, peak):
    """N > 1 only.  `strong`: the large-batch forward with its 1 048 576 rows split over the ranks (no communication),
    checked by comparing sampled rows of every shard with rank 0's evaluation of the whole batch.  `train`: training
    steps of the fern and the pipeline configurations with the all-reduce of the parameter gradients inside the timed
    region, next to the same step without it and the all-reduce alone."""
    import torch
    import torch.distributed as dist
    from hingetreefortorch_b200 import _cabi
    from hingetreefortorch_b200.distributed import shard_bounds
    out = {}
    wl = WORKLOADS["c3"]
    B = wl["B"]
    lo, hi = shard_bounds(B, rank, world)
    gen = torch.Generator().manual_seed(4242)
    x_all = torch.randn((B, wl["C"]), generator=gen)  # the same batch on every rank
    thr, ord_, w = [t.to(device) for t in make_params(wl)]
    x = x_all[lo:hi].to(device)
    forest = _cabi.Forest(wl["kind"], x, w, backward_workspace=False)
    res = torch.empty(forest.out_shape, dtype=torch.float32, device=device)
    step = lambda: forest.forward(x, thr, ord_, w, out=res)
    for _ in range(3):
        step()
    steps = max(3, min(a.steps, 20))
    ms, _, _ = timer.run(step, steps)
    ms /= steps
    # sampled rows of every shard against the whole batch evaluated on rank 0
    picks = torch.linspace(0, hi - lo - 1, 64).long().to(device)
    mine = torch.cat([res[picks], (picks + lo).float().unsqueeze(1)], dim=1)
    gathered = [torch.empty_like(mine) for _ in range(world)] if rank == 0 else None
    dist.gather(mine, gathered, dst=0)
    equal = None
    if rank == 0:
        xg = x_all.to(device)
        whole = _cabi.Forest(wl["kind"], xg, w, backward_workspace=False).forward(xg, thr, ord_, w)
        equal = all(bool(torch.equal(t[:, :-1], whole[t[:, -1].long()])) for t in gathered)
        del whole, xg
    nbytes = algorithmic_bytes(wl, B, False)
    out["strong"] = {"workload": wl["name"], "rows_per_gpu": hi - lo, "ms_per_step": ms, "steps": steps,
                     "value": B * wl["T"] / (ms * 1e-3), "unit": "tree-evals/s", "collective": None,
                     "achieved_gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_n_gpus": nbytes / (ms * 1e-3) / 1e9 / (peak * world),
                     "shards_equal_whole": equal}
    del forest, res, x, x_all
    torch.cuda.empty_cache()

    train = {}
    for key in ("c2", "c5", "c5tc", "c5f"):
        twl = WORKLOADS[key]
        runner = make_runner(twl, twl["B"], device, rank, world)
        for _ in range(3):
            runner.step(True)
        steps = 10
        with_ms, _, _ = timer.run(lambda: runner.step(True), steps)
        without_ms, _, _ = timer.run(lambda: runner.step(True, reduce=False), steps)
        bucket = runner.param_grads if twl["op"] == "forest" else runner.bucket.flat
        alone_ms, _, _ = timer.run(lambda: dist.all_reduce(bucket), steps)
        nbytes = bucket.numel() * 4
        train[key] = {"workload": twl["name"], "rows_per_gpu": twl["B"], "ms_per_step": with_ms / steps,
                      "ms_per_step_without_allreduce": without_ms / steps, "allreduce_alone_ms": alone_ms / steps,
                      "bucket_bytes": nbytes, "value": evals_per_step(twl, twl["B"]) * world / (with_ms / steps * 1e-3),
                      "unit": "tree-evals/s (weak: every rank its own batch)",
                      "allreduce_bus_gbs": 2 * (world - 1) / world * nbytes / (alone_ms / steps * 1e-3) / 1e9}
        del runner
        torch.cuda.empty_cache()
    out["train"] = train
    return out


def our_arm(a, wl):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product arm has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    numa = bind_to_gpu_numa_node(local) if world > 1 else None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    B = a.rows or wl["B"]
    if a.linear == "tf32":
        torch.backends.cuda.matmul.allow_tf32 = True
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    timer = Timer(device, world)
    runner = make_runner(wl, B, device, rank, world)
    if a.rewalk and wl["op"] == "forest":
        runner.keep = False

    for _ in range(a.warmup):
        runner.step(wl["bwd"])
    timer.barrier()
    runner.check()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    elapsed_ms, per_step_ms, launches = timer.run(lambda: runner.step(wl["bwd"]), a.steps)
    clocks = sampler.stop() if rank == 0 else None
    evals = evals_per_step(wl, B)
    value = evals * world * a.steps / (elapsed_ms * 1e-3)

    if a.kernel_only or wl["op"] == "family":  # the operator-family legs are device-resident timings only
        if rank == 0:
            print(json.dumps({"kernel_only": True, "rows": B, "ms_per_step": elapsed_ms / a.steps, "value": value}))
        if world > 1:
            dist.destroy_process_group()
        return

    checks = {}  # slices of device results for the CPU leg to compare with the port

    # forward + backward of the inference shape (a training step: the forward keeps its traversal for the
    # backward), as a second device-resident figure
    fwd_bwd = None
    if wl["op"] == "forest" and not wl["bwd"]:
        runner.enable_backward()
        runner.step(True, reduce=False)
        fb_steps = max(1, min(a.steps, 5))
        fb_ms, _, fb_launches = timer.run(lambda: runner.step(True, reduce=False), fb_steps)
        fb_bytes = algorithmic_bytes(wl, B, True)
        fwd_bwd = {"value": evals * world * fb_steps / (fb_ms * 1e-3), "unit": "tree-evals/s",
                   "ms_per_step": fb_ms / fb_steps, "steps": fb_steps, "bytes_per_step": fb_bytes,
                   "achieved_gbs": fb_bytes / (fb_ms / fb_steps * 1e-3) / 1e9, "gpu_launches": fb_launches,
                   "forward_keeps_traversal": bool(runner.keep)}
        fwd_bwd["frac"] = fwd_bwd["achieved_gbs"] / peak
        if rank == 0 and world == 1:
            rows = 64
            checks["fwd_bwd"] = {"kind": wl["kind"], "op": "forest", "x": runner.x[:rows].cpu().numpy(),
                                 "thr": runner.thr.cpu().numpy(), "ord": runner.ord.cpu().numpy(), "w": runner.w.cpu().numpy(),
                                 "g": runner.g[:rows].cpu().numpy(), "out": runner.out[:rows].cpu().numpy(),
                                 "gx": runner.grads[0][:rows].cpu().numpy()}
        runner.g = runner.grads = runner.param_grads = None
        torch.cuda.empty_cache()

    # the launch-latency workloads once more as one CUDA-graph replay per step: the C ABI neither
    # allocates nor synchronises, so a step is capturable as it stands
    cuda_graph = None
    if wl["op"] == "forest" and B * wl["T"] <= 4096 * 1024 and world == 1:
        cuda_graph = graph_replay(runner, wl, evals, a.steps)

    # ---- end to end through the reference-facing surface, host buffers in and out -------------
    h2d, d2h, call = runner.prepare_e2e()
    e2e_steps = max(1, min(a.steps, 5))
    for _ in range(2):
        runner.e2e_step()
    timer.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        runner.e2e_step()
    torch.cuda.synchronize()
    t = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = evals * world * e2e_steps / float(t.item())
    runner.verify_e2e()
    runner.release_e2e()

    # ---- what else one run records: the other configurations (N = 1), the collective and the split (N > 1) ----
    workloads, scale, reference_gpu = None, None, None
    if a.workload == "c3" and not a.rows and not a.lean:
        del runner
        torch.cuda.empty_cache()
        if world == 1:
            workloads = {}
            for key in ("c1", "c2", "c4", "c5", "c5tc", "c5f"):
                workloads[key], checks[key] = side_workload(key, device, timer, peak)
            reference_gpu = reference_gpu_leg(device)
        else:
            scale = scale_legs(a, device, rank, world, timer, peak)

    if rank == 0:
        launch_ms = statistics.mean(per_step_ms)
        bytes_per_step = algorithmic_bytes(wl, B, wl["bwd"])
        achieved = bytes_per_step / (launch_ms * 1e-3) / 1e9
        # CPU leg: the port timed on the host cores, and, as the checker, slices of this run's device results
        cores = os.cpu_count() or 1
        sample_rows = cpu_sample_rows(wl, cores)
        cpu_value, cpu_dt = cpu_port_rate(wl, sample_rows, cores)
        parity = {name: check_against_port(c) for name, c in checks.items() if c is not None}
        if fwd_bwd is not None and "fwd_bwd" in parity:
            fwd_bwd["slice_matches_port"] = parity.pop("fwd_bwd")
        for key, ok in parity.items():
            workloads[key]["slice_matches_port"] = ok
        line = {
            "metric": "tree-evals/sec " + ("fwd+bwd" if wl["bwd"] else "fwd"),
            "value": value, "unit": "tree-evals/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": elapsed_ms / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["name"] + ("" if B == wl["B"] else " (rows overridden)") +
                       (" [Linear in tf32]" if a.linear == "tf32" and wl["op"] == "pipeline" else ""), "rows_per_gpu": B,
                       "l2": "inputs and outputs exceed L2 (126 MB): no flush between iterations" if bytes_per_step > 126e6
                       else "working set fits L2 (126 MB); launch-latency regime",
                       "parallelism": "batch-sharded x%d, replicated parameters%s"
                       % (world, ", one NCCL all-reduce of parameter gradients per step"
                          if world > 1 and wl["bwd"] else "")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": C3_DRAM_BYTES_PER_LAUNCH if a.workload == "c3" and B == wl["B"] else None,
                         "peak_source": peak_src, "bytes_per_launch": bytes_per_step,
                         "launch_ms": launch_ms, "frac_of_8TBs": achieved / 8000.0},
            "cpu_baseline": {"value": cpu_value, "unit": "tree-evals/s", "cores": cores, "kind": "port",
                             "sample": "forward of %d of %d rows, %.1f s" % (sample_rows, wl["B"], cpu_dt)},
            "e2e": {"value": e2e_value, "unit": "tree-evals/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "call": call},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if numa is not None:
            line["e2e"]["host_binding"] = numa
        if fwd_bwd is not None:
            line["fwd_bwd"] = fwd_bwd
        if cuda_graph is not None:
            line["cuda_graph"] = cuda_graph
        if workloads is not None:
            line["workloads"] = workloads
        if scale is not None:
            line.update(scale)
        if reference_gpu is not None:
            line["reference_gpu"] = reference_gpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def graph_replay(runner, wl, evals, steps):
    import torch
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        runner.step(wl["bwd"])
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        runner.step(wl["bwd"])
    for _ in range(3):
        graph.replay()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    replays = max(steps, 50)
    torch.cuda.synchronize()
    begin.record()
    for _ in range(replays):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    graph_ms = begin.elapsed_time(end) / replays
    runner.check()
    return {"ms_per_step": graph_ms, "value": evals / (graph_ms * 1e-3), "unit": "tree-evals/s", "steps": replays}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--rows", type=int, default=0, help="rows per GPU instead of the workload's (profiler captures)")
    ap.add_argument("--linear", default="fp32", choices=["fp32", "tf32"],
                    help="c5 only: arithmetic of torch's Linear (cuBLAS); the forest stage is fp32 either way")
    ap.add_argument("--rewalk", action="store_true",
                    help="forest workloads: the forward keeps nothing and the backward walks the trees again")
    ap.add_argument("--lean", action="store_true",
                    help="c3 only: skip the other configurations (N = 1) and the strong-scaling / training legs (N > 1)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="time the device-resident step only (profiler captures): no end-to-end and no CPU leg")
    a = ap.parse_args()
    if a.impl == "ours":
        a.warmup = max(a.warmup, 3)
    wl = WORKLOADS[a.workload]
    if a.impl == "reference":
        reference_arm(a, wl)
    else:
        our_arm(a, wl)


if __name__ == "__main__":
    main()
