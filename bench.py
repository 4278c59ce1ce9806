#!/usr/bin/env python
"""Benchmark of the hinge forest evaluation path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c3|c2|c1]

A step is one pass of the hot path over one batch of seeded synthetic input.  The default
workload is the large-batch forest inference configuration (x [1048576,128] ~ N(0,1), 1024
trees of depth 8, thresholds U(-3,3), feature indices U[0,127], leaf weights N(0,1)); with N
GPUs every rank evaluates its own batch of that size against replicated parameters (weak
scaling, no communication in the data path).  Rank 0 prints ONE JSON line:

  value      tree-evals/s, whole job, inputs resident in HBM, timed with CUDA events, max over ranks
  e2e        the same metric through the reference-facing operator (hingetree_cpp.tree_forward) with
             HOST buffers: pinned input copied in, full output copied back, inside the timed region
  roofline   algorithmic bytes of one forward / measured launch time, against the measured HBM peak
  cpu_baseline   the CPU restatement of the reference algorithm on this machine's host cores
                 (bounded sample of the same workload)

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
    # name: kind, B, C, T, depth, M (0 = no inner weight dim), backward
    "c3": dict(kind="tree", B=1048576, C=128, T=1024, depth=8, M=0, x="randn", bwd=False,
               name="C3 large-batch forest inference x[1048576,128] T=1024 depth=8"),
    "c2": dict(kind="fern", B=4096, C=256, T=500, depth=10, M=10, x="randn", bwd=True,
               name="C2 fern fwd+bwd x[4096,256] T=500 depth=10 extra_outputs=10"),
    "c1": dict(kind="tree", B=100, C=1000, T=100, depth=7, M=1, x="rand", bwd=True,
               name="C1 forest fwd+bwd x[100,1000] T=100 depth=7 extra_outputs=1"),
}


def decisions(kind, depth):
    return depth if kind == "fern" else 2 ** depth - 1


def algorithmic_bytes(wl, B, backward=False):
    """Compulsory traffic with the API's dtypes (fp32 data, int64 ordinals), each tensor touched once."""
    C, T, depth, M = wl["C"], wl["T"], wl["depth"], max(wl["M"], 1)
    N, L = decisions(wl["kind"], depth), 2 ** depth
    fwd = 4 * B * C + 12 * T * N + 4 * T * L * M + 4 * B * T * M
    if not backward:
        return fwd
    bwd = (4 * B * C + 12 * T * N + 4 * T * L * M + 4 * B * T * M) + (4 * B * C + 4 * T * N + 4 * T * L * M)
    return fwd + bwd


def make_params(wl, seed=0):
    import torch
    gen = torch.Generator().manual_seed(seed)
    N, L = decisions(wl["kind"], wl["depth"]), 2 ** wl["depth"]
    thr = torch.rand((wl["T"], N), generator=gen) * 6 - 3
    ord_ = torch.randint(0, wl["C"], (wl["T"], N), generator=gen)
    wshape = (wl["T"], L) + ((wl["M"],) if wl["M"] else ())
    w = torch.randn(wshape, generator=gen)
    return thr, ord_, w


def make_x(wl, rows, seed):
    import torch
    gen = torch.Generator().manual_seed(1000 + seed)
    if wl["x"] == "rand":
        return torch.rand((rows, wl["C"]), generator=gen)
    return torch.randn((rows, wl["C"]), generator=gen)


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
                                          "--format=csv,noheader,nounits", "-lms", "100"],
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
        # samples taken under load are the upper half of the clock readings when the region is short
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---- CPU legs ------------------------------------------------------------------------------

def _cpu_forward_port(args):
    kind, x, thr, ord_, w = args
    from oracle import hinge_oracle as ho
    return ho.forward(kind, x, thr, ord_, w).shape[0]


def cpu_port_rate(wl, rows, threads):
    """The C restatement on `threads` host threads (ctypes releases the GIL), rows split evenly."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor
    from oracle import hinge_oracle as ho
    ho.lib()
    thr, ord_, w = [t.numpy() for t in make_params(wl)]
    x = make_x(wl, rows, 0).numpy()
    parts = [p for p in np.array_split(x, threads) if len(p)]
    jobs = [(wl["kind"], p, thr, ord_, w) for p in parts]
    with ThreadPoolExecutor(max_workers=threads) as ex:
        t0 = time.perf_counter()
        list(ex.map(_cpu_forward_port, jobs))
        dt = time.perf_counter() - t0
    return rows * wl["T"] / dt, dt


_REF_STATE = {}


def _ref_worker_init(kind, thr, ord_, w):
    import torch
    torch.set_num_threads(1)
    from oracle import build_ref
    _REF_STATE["mod"] = build_ref.load()
    _REF_STATE["args"] = (kind, thr, ord_, w)


def _ref_worker_run(x):
    kind, thr, ord_, w = _REF_STATE["args"]
    out = getattr(_REF_STATE["mod"], kind + "_forward")(x, thr, ord_, w)
    return out.shape[0]


def reference_arm(a, wl):
    """The reference's own CPU implementation on all host cores, bounded sample per step."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    rows_per_core = max(1, min(wl["B"] // cores, 512 if wl["T"] * wl["depth"] >= 4096 else wl["B"]))
    rows = rows_per_core * cores
    thr, ord_, w = make_params(wl)
    x = make_x(wl, rows, 0)
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
        with ctx.Pool(cores, initializer=_ref_worker_init, initargs=(wl["kind"], thr, ord_, w)) as pool:
            chunks = list(torch.chunk(x, cores))
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
    value = rows * wl["T"] * len(times) / total
    sample = "%d of %d rows per step (%d per core), all %d trees" % (rows, wl["B"], rows_per_core, wl["T"])
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


# ---- our arm --------------------------------------------------------------------------------

def our_arm(a, wl):
    import torch
    import torch.distributed as dist
    from hingetreefortorch_b200 import _cabi
    from hingetreefortorch_b200._ext import hingetree_cpp

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this benchmark has no CPU path for the product arm")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    B = a.rows or wl["B"]
    thr, ord_, w = [t.to(device) for t in make_params(wl)]
    x_host = make_x(wl, B, rank)
    x = x_host.to(device)
    forest = _cabi.Forest(wl["kind"], x, w)
    out = torch.empty(forest.out_shape, dtype=torch.float32, device=device)
    g = gx = gthr = gw = None
    if wl["bwd"]:
        g = torch.randn(forest.out_shape, generator=torch.Generator(device=device).manual_seed(5), device=device)
        gx, gthr, gw = torch.empty_like(x), torch.empty_like(thr), torch.empty_like(w)

    def step():
        forest.forward(x, thr, ord_, w, out=out)
        if wl["bwd"]:
            forest.backward(x, thr, ord_, w, g, outs=(gx, gthr, gw))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(a.warmup):
        step()
    barrier()
    if forest.ordinal_flags() != 0:
        raise SystemExit("bench.py: ordinals out of range")
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(a.steps)]
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for s, e in events:
        s.record()
        step()
        e.record()
    end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    elapsed_ms = begin.elapsed_time(end)
    per_step_ms = [s.elapsed_time(e) for s, e in events]
    t = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    evals = B * wl["T"]
    value = evals * world * a.steps / (elapsed_ms * 1e-3)

    if a.kernel_only:
        if rank == 0:
            print(json.dumps({"kernel_only": True, "rows": B, "ms_per_step": elapsed_ms / a.steps, "value": value}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end through the reference-facing operator, host buffers in and out -----------
    fwd_op = getattr(hingetree_cpp, wl["kind"] + "_forward")
    chunk = min(B, 65536)
    n_chunks = (B + chunk - 1) // chunk
    x_pinned = x_host.pin_memory()
    out_pinned = torch.empty(forest.out_shape, dtype=torch.float32).pin_memory()
    copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    compute = torch.cuda.current_stream(device)

    def e2e_step():
        staged = []
        for c in range(n_chunks):
            lo, hi = c * chunk, min(B, (c + 1) * chunk)
            with torch.cuda.stream(copy_in):
                xc = x_pinned[lo:hi].to(device, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(copy_in)
            compute.wait_event(ready)
            oc = fwd_op(xc, thr, ord_, w)
            xc.record_stream(compute)
            done = torch.cuda.Event()
            done.record(compute)
            copy_out.wait_event(done)
            with torch.cuda.stream(copy_out):
                out_pinned[lo:hi].copy_(oc, non_blocking=True)
                oc.record_stream(copy_out)
            staged.append(oc)
        copy_out.synchronize()

    e2e_steps = max(1, min(a.steps, 5))
    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    t = torch.tensor([e2e_s], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = evals * world * e2e_steps / float(t.item())
    # the end-to-end output must be the resident-path output
    if not torch.equal(out_pinned[:1024], out[:1024].cpu()):
        raise SystemExit("bench.py: end-to-end output differs from the device-resident output")

    if rank == 0:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(peaks_path):
            peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
        else:
            peak, peak_src = 6650.0, "fallback"
        launch_ms = statistics.mean(per_step_ms)
        bytes_per_launch = algorithmic_bytes(wl, B, wl["bwd"])
        achieved = bytes_per_launch / (launch_ms * 1e-3) / 1e9
        cores = os.cpu_count() or 1
        sample_rows = min(B, max(cores * 8, int(15.0 * cores / (wl["T"] * 80e-9))))
        cpu_value, cpu_dt = cpu_port_rate(wl, sample_rows, cores)
        elem = 4 * (wl["M"] or 1)
        line = {
            "metric": "tree-evals/sec " + ("fwd+bwd" if wl["bwd"] else "fwd"),
            "value": value, "unit": "tree-evals/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": elapsed_ms / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["name"] + ("" if B == wl["B"] else " (rows overridden)"), "rows_per_gpu": B, "l2": "inputs and outputs exceed L2 (126 MB)"
                       if bytes_per_launch > 4 * 126e6 else "working set fits L2",
                       "parallelism": "batch-sharded x%d, replicated parameters" % world},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": peak_src, "bytes_per_launch": bytes_per_launch,
                         "launch_ms": launch_ms, "frac_of_8TBs": achieved / 8000.0},
            "cpu_baseline": {"value": cpu_value, "unit": "tree-evals/s", "cores": cores, "kind": "port",
                             "sample": "%d of %d rows, all %d trees, %.1f s" % (sample_rows, B, wl["T"], cpu_dt)},
            "e2e": {"value": e2e_value, "unit": "tree-evals/s", "h2d_bytes_per_step": 4 * B * wl["C"],
                    "d2h_bytes_per_step": elem * B * wl["T"], "steps": e2e_steps,
                    "call": "hingetree_cpp.%s_forward on %d-row chunks, pinned host buffers, 3 streams" % (wl["kind"], chunk)},
            "gpu_launches": a.steps * (2 + (2 if wl["bwd"] else 0)),
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--rows", type=int, default=0, help="rows per GPU instead of the workload's (profiler captures)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="time the device-resident step only (profiler captures): no end-to-end and no CPU leg")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3) if a.impl == "ours" else a.warmup
    wl = WORKLOADS[a.workload]
    if a.impl == "reference":
        reference_arm(a, wl)
    else:
        our_arm(a, wl)


if __name__ == "__main__":
    main()
