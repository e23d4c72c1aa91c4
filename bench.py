#!/usr/bin/env python
"""Benchmark of the grouped-GEMM hot path on B200.

    python bench.py --gpus 1 --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W    # CPU per-expert loop
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

One JSON line on stdout (rank 0).  Workloads (synthetic, seeded; bf16):

* N = 1: Mixtral-8x7B expert up-projection, z=8, 32768 rows (16384 tokens x
  top-2), k=4096, n=14336, batch sizes multinomial(Dirichlet(1), seed 1).  A step
  is forward (a@b) + dgrad (grad@b^T) + wgrad (a^T@grad): three kernel launches.
* N > 1: expert-parallel projection, z=64 experts sharded evenly, 65536 tokens x
  top-4 = 262144 rows, hidden 6144, ffn 10752, uniform routing seed 3.  A step is
  dispatch -> forward -> combine, then dispatch of the output gradient -> dgrad +
  wgrad -> combine.  Rows move between GPUs with the library's peer-memory push
  kernel (--exchange nccl: NCCL all-to-all instead).  Total work is fixed
  ("strong" scaling); the line also carries the same workload timed on one GPU.

``value`` is TFLOP/s over the timed steps with inputs resident in HBM, timed with
CUDA events (max over ranks).  ``e2e`` is the same step driven from pinned host
buffers with the host<->device copies inside the timed region.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "gmm bf16 throughput, fwd+dgrad+wgrad"
UNIT = "TFLOP/s"


# ----------------------------------------------------------------------------- workloads
def mixtral_batch_sizes():
    """benchmark configuration 2: multinomial(32768, Dirichlet(alpha=1)), seed 1."""
    rng = np.random.default_rng(1)
    p = rng.dirichlet(np.ones(8))
    return [int(v) for v in rng.multinomial(32768, p)]


def fine_grained_batch_sizes():
    """benchmark configuration 4: 256 experts, Zipf(1.1) popularity, 51 forced empty, 65536 rows, seed 2."""
    rng = np.random.default_rng(2)
    perm = rng.permutation(256)
    w = np.zeros(256)
    w[perm] = 1.0 / np.arange(1, 257) ** 1.1
    zero = rng.choice(256, 51, replace=False)
    w[zero] = 0
    w /= w.sum()
    return [int(v) for v in rng.multinomial(65536, w)]


def ep_routing(tokens=65536, experts=64, top_k=4):
    """benchmark configuration 5: uniform-random top-k distinct experts per token, seed 3."""
    rng = np.random.default_rng(3)
    idx = np.argsort(rng.random((tokens, experts)), axis=1)[:, :top_k]
    return torch.from_numpy(np.ascontiguousarray(idx)).to(torch.int64)


MIXTRAL = dict(z=8, rows=32768, k=4096, n=14336)
EP = dict(z=64, tokens=65536, top_k=4, hidden=6144, ffn=10752)


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a region runs.
    Read-only: never sets a clock or any other device state."""

    REASONS = {
        0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting",
    }

    def __init__(self, index, period=0.01):
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [v for v in visible.split(",") if v.strip() != ""]
                if index < len(ids) and ids[index].strip().isdigit():
                    phys = int(ids[index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------- helpers
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"source": "measured", "hbm_gbs": p["hbm_gbs"], "burst": p["bf16_tflops"],
                "sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"])}
    return {"source": "fallback", "hbm_gbs": 6650.0, "burst": 1590.0, "sustained": 1400.0}


def dist_info():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return world, rank, local


def timed_region(fn, steps, world):
    """Barrier + synchronize, K steps between two CUDA events on the current
    stream, synchronize + barrier; returns the max-over-ranks milliseconds."""
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.barrier()
    return float(ms.item())


# ----------------------------------------------------------------------------- CPU baseline
def cpu_workload(n_gpus):
    """Shapes the CPU reference runs: the N=1 workload (Mixtral up-projection) or,
    for N>1, the expert-parallel projection with a subset of its 64 experts (all
    of them would need 8 GB of host weights for no change in the per-row rate)."""
    if n_gpus == 1:
        return {"name": "mixtral up-projection", "sizes": mixtral_batch_sizes(), "k": MIXTRAL["k"],
                "n": MIXTRAL["n"], "experts_total": MIXTRAL["z"]}
    counts = torch.bincount(ep_routing().reshape(-1), minlength=EP["z"]).tolist()
    return {"name": "expert-parallel projection, first 8 of 64 experts", "sizes": counts[:8],
            "k": EP["hidden"], "n": EP["ffn"], "experts_total": EP["z"]}


def cpu_sample_inputs(work, frac):
    """The workload with each expert's rows cut to ``frac`` of its size (full k
    and n, full weights of the sampled experts)."""
    sizes = [max(1, int(s * frac)) for s in work["sizes"]]
    rows = sum(sizes)
    g = torch.Generator().manual_seed(1)
    a = torch.randn(rows, work["k"], generator=g).bfloat16()
    b = (torch.randn(len(sizes), work["k"], work["n"], generator=g) * 0.02).bfloat16()
    grad = torch.randn(rows, work["n"], generator=g).bfloat16()
    return sizes, a, b, grad


def cpu_step(sizes, a, b, grad):
    """Reference CPU path: the per-expert torch.matmul loop of the reference's
    tests, forward + dgrad + wgrad."""
    from oracle import gmm_oracle
    bs = torch.tensor(sizes)
    gmm_oracle.torch_loop_bf16(a, b, bs, trans_b=False)
    gmm_oracle.torch_loop_bf16(grad, b, bs, trans_b=True)
    gmm_oracle.torch_loop_tn_bf16(a, grad, bs)
    return 3 * 2.0 * sum(sizes) * a.shape[1] * grad.shape[1]


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use the host."""
    cores = os.cpu_count() or 1
    if torch.get_num_threads() < cores:
        torch.set_num_threads(cores)


def pick_cpu_sample(work, target_s):
    """Inputs of the CPU sample whose step takes about ``target_s`` seconds on
    this host (at most the full workload).  Small samples run far below the
    host's large-matrix rate, so the sample is grown until one step is long
    enough.  Returns (frac, sizes, a, b, grad, seconds of the last step)."""
    frac = 1.0 / 256
    while True:
        sizes, a, b, grad = cpu_sample_inputs(work, frac)
        cpu_step(sizes, a, b, grad)  # warm-up (thread pool, primitive caches)
        t0 = time.perf_counter()
        cpu_step(sizes, a, b, grad)
        dt = max(time.perf_counter() - t0, 1e-3)
        if dt >= 0.6 * target_s or frac >= 1.0:
            return frac, sizes, a, b, grad, dt
        frac = min(1.0, frac * min(8.0, target_s / dt))


def cpu_sample_text(work, sizes, frac):
    return (f"per-expert torch.matmul loop (bf16, CPU), {work['name']}: {sum(sizes)} of {sum(work['sizes'])} rows "
            f"of {len(sizes)} experts (each cut to {frac:.4f} of its rows), k={work['k']} n={work['n']}, "
            "full weights of those experts, fwd+dgrad+wgrad")


def cpu_baseline(target_s=12.0):
    use_all_host_threads()
    work = cpu_workload(1)
    frac, sizes, a, b, grad, _ = pick_cpu_sample(work, target_s)
    t0 = time.perf_counter()
    flops = cpu_step(sizes, a, b, grad)
    dt = time.perf_counter() - t0
    return {
        "value": flops / dt / 1e12, "unit": UNIT, "cores": torch.get_num_threads(),
        "host_cpus": os.cpu_count(), "kind": "port",
        "sample": cpu_sample_text(work, sizes, frac) + f", one pass of {dt:.1f} s",
    }


def run_reference(args):
    """--impl reference: the reference's CPU-runnable path (its test oracle's
    per-expert matmul loop; the CUDA extension itself cannot be built without
    the CUTLASS submodule and has no CPU code) on the host cores."""
    world, rank, _ = dist_info()
    if rank != 0:
        return
    use_all_host_threads()
    work = cpu_workload(args.gpus)
    frac, sizes, a, b, grad, _ = pick_cpu_sample(work, 3.0)
    for _ in range(args.warmup):
        cpu_step(sizes, a, b, grad)
    t0 = time.perf_counter()
    flops = 0.0
    for _ in range(args.steps):
        flops += cpu_step(sizes, a, b, grad)
    dt = time.perf_counter() - t0
    value = flops / dt / 1e12
    sample = cpu_sample_text(work, sizes, frac) + ", per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(),
                         "host_cpus": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- our arm
def workload_config(n_gpus):
    if n_gpus == 1:
        return {"workload": "mixtral-8x7b expert up-projection fwd+dgrad+wgrad (configs[2] of the baseline spec, on "
                            "configs[1] shapes): z=8 rows=32768 k=4096 n=14336, batch_sizes "
                            "multinomial(Dirichlet(1), seed 1), on device",
                "batch_sizes": mixtral_batch_sizes(),
                "l2": "inputs larger than L2 (2.1 GB read per pass, no flush)"}
    return {"workload": f"expert-parallel projection fwd+dgrad+wgrad (configs[4] of the baseline spec): z=64 sharded over "
                        f"{n_gpus} ranks, 65536 tokens x top-4 = 262144 rows, hidden 6144, ffn 10752, uniform "
                        "routing seed 3, dispatch/combine over NVLink",
            "parallelism": f"ep{n_gpus}",
            "l2": "inputs larger than L2 (per-rank operands of several GB, no flush)"}


def time_loop(fn, iters):
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def median_rounds(fn, iters, rounds):
    """``rounds`` timed loops of ``iters`` calls each; ms per call: median, min, max."""
    vals = sorted(time_loop(fn, iters) for _ in range(rounds))
    return {"ms": vals[len(vals) // 2], "ms_min": vals[0], "ms_max": vals[-1], "rounds": rounds, "iters": iters}


def library_loop_fns(a, b, grad, sizes):
    """The reference's default GPU path on the same tensors: one library GEMM per
    expert (what csrc/grouped_gemm.cu:396-435 of the reference does through
    cublasGemmEx), here as ``torch.matmul`` on row slices.  Needs batch sizes on
    the host, as the reference's cuBLAS build does."""
    offs = [0]
    for v in sizes:
        offs.append(offs[-1] + v)
    z = len(sizes)
    c = torch.empty(a.shape[0], b.shape[2], device=a.device, dtype=a.dtype)
    dx = torch.empty_like(a)
    dw = torch.empty_like(b)

    def fwd():
        for i in range(z):
            if sizes[i]:
                torch.matmul(a[offs[i]:offs[i + 1]], b[i], out=c[offs[i]:offs[i + 1]])

    def dgrad():
        for i in range(z):
            if sizes[i]:
                torch.matmul(grad[offs[i]:offs[i + 1]], b[i].t(), out=dx[offs[i]:offs[i + 1]])

    def wgrad():
        for i in range(z):
            torch.matmul(a[offs[i]:offs[i + 1]].t(), grad[offs[i]:offs[i + 1]], out=dw[i])

    return {"fwd": fwd, "dgrad": dgrad, "wgrad": wgrad}


def compare_passes(ours, loop, flops, iters, rounds):
    """Each pass of this library and of the per-expert library loop, timed in turn
    inside every round so that both see the same clocks; medians over the rounds."""
    acc = {name: {"ours": [], "loop": []} for name in ours}
    for fn in list(ours.values()) + list(loop.values()):
        fn()
    for _ in range(rounds):
        for name in ours:
            acc[name]["ours"].append(time_loop(ours[name], iters))
            acc[name]["loop"].append(time_loop(loop[name], iters))
    passes, lib = {}, {}
    for name, v in acc.items():
        o, l = sorted(v["ours"]), sorted(v["loop"])
        om, lm = o[len(o) // 2], l[len(l) // 2]
        passes[name] = {"ms": om, "ms_min": o[0], "ms_max": o[-1], "tflops": flops / om / 1e9}
        lib[name] = {"ms": lm, "ms_min": l[0], "ms_max": l[-1], "tflops": flops / lm / 1e9, "ours_over_loop": lm / om}
    return passes, lib


def run_single(args):
    from grouped_gemm_b200 import _capi, backend
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    z, rows, k, n = MIXTRAL["z"], MIXTRAL["rows"], MIXTRAL["k"], MIXTRAL["n"]
    sizes = mixtral_batch_sizes()
    g = torch.Generator(device=dev).manual_seed(1)
    a = torch.randn(rows, k, device=dev, generator=g).bfloat16()
    b = (torch.randn(z, k, n, device=dev, generator=g) * 0.02).bfloat16()
    grad = torch.randn(rows, n, device=dev, generator=g).bfloat16()
    bs = torch.tensor(sizes, dtype=torch.int64, device=dev)
    flops_pass = 2.0 * rows * k * n

    def fwd():
        return backend.gmm(a, b, bs)

    def dgrad():
        return backend.gmm(grad, b, bs, trans_b=True)

    def wgrad():
        return backend.gmm(a, grad, bs, trans_a=True)

    def step():
        fwd(); dgrad(); wgrad()

    for _ in range(args.warmup):
        step()
    # K steps per round, timed on the device; the value is the median round
    launches0 = _capi.launch_count()
    round_ms = []
    with ClockSampler(0) as clocks:
        for _ in range(args.rounds):
            round_ms.append(timed_region(step, args.steps, 1) / args.steps)
    launches = (_capi.launch_count() - launches0) // args.rounds
    ms_step = sorted(round_ms)[len(round_ms) // 2]
    value = 3 * flops_pass / ms_step / 1e9

    # per-pass device times, each against the per-expert library loop on the same
    # tensors (the dominant kernel's figure feeds the roofline)
    iters = max(args.steps // 2, 5)
    passes, library = compare_passes({"fwd": fwd, "dgrad": dgrad, "wgrad": wgrad},
                                     library_loop_fns(a, b, grad, sizes), flops_pass, iters, args.rounds)
    torch.cuda.empty_cache()
    peaks = measured_peaks()
    top = max(passes, key=lambda p: passes[p]["ms"])
    kernel_of = {"fwd": "gmm_kernel<NN>", "dgrad": "gmm_kernel<NT>", "wgrad": "gmm_kernel<TN>"}
    traffic, traffic_source = measured_traffic(kernel_of[top])
    roofline = {
        "bound": "tensor", "kernel": kernel_of[top], "achieved": passes[top]["tflops"],
        "peak": peaks["burst"], "unit": "TFLOP/s", "frac": passes[top]["tflops"] / peaks["burst"],
        "peak_source": f"{peaks['source']} cuBLAS bf16 burst (kernel timed alone)",
        "step_frac_of_sustained": value / peaks["sustained"],
        "flops_per_launch": flops_pass, "ms_per_launch": passes[top]["ms"],
        "traffic": traffic, "traffic_source": traffic_source,
        "algorithmic_bytes": 2.0 * (rows * k + z * k * n + rows * n),
    }
    gpu_library_loop = {"what": "per-expert torch.matmul (cuBLAS) loop on the same tensors, batch sizes on the host; "
                                "timed in turn with this library's pass inside each round",
                        "mixtral_up": library}

    # benchmark configuration 3 also names the down-projection, b [8, 14336, 4096]
    down, library_down = down_projection(backend, dev, bs, sizes, iters, args.rounds)
    gpu_library_loop["mixtral_down"] = library_down

    # small-M, HBM-bound group shapes (benchmark configuration 4): report GB/s
    del a, b, grad
    torch.cuda.empty_cache()
    hbm, library_fine = fine_grained_hbm(backend, dev, peaks, args.rounds)
    gpu_library_loop["fine_grained"] = library_fine

    # end to end: pinned host buffers in and out, copies inside the timed region
    g = torch.Generator(device=dev).manual_seed(1)
    a = torch.randn(rows, k, device=dev, generator=g).bfloat16()
    b = (torch.randn(z, k, n, device=dev, generator=g) * 0.02).bfloat16()
    grad = torch.randn(rows, n, device=dev, generator=g).bfloat16()
    e2e = e2e_single(backend, a, b, grad, bs, flops_pass, max(4, min(args.steps, 8)))

    fused = None
    if args.fused:
        del a, b, grad
        fused = fused_neighbours(backend, dev, bs)
    scaling_base = None if args.no_scaling_base else ep_value_single(args.steps, dev)
    baseline = cpu_baseline() if not args.no_cpu_baseline else None

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(1),
        "rounds": {"count": args.rounds, "ms_per_step_min": min(round_ms), "ms_per_step_max": max(round_ms)},
        "passes": passes, "down_projection": down, "roofline": roofline, "hbm_bound_case": hbm,
        "gpu_library_loop": gpu_library_loop,
        "cpu_baseline": baseline,
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks.summary(),
        "frac_of_nominal_2250": value / 2250.0, "device_status": backend.device_status(),
    }
    if scaling_base is not None:
        line["scaling_base"] = scaling_base
    if fused is not None:
        line["fused_neighbours"] = fused
    print(json.dumps(line), flush=True)


TRAFFIC_FILE = os.path.join(ROOT, "bench_traffic.json")


def measured_traffic(kernel):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the
    named kernel at the benchmark's size, from the file ``--traffic-from`` wrote out
    of an ncu capture of ``--profile`` runs of this build; (None, reason) without it."""
    if not os.path.exists(TRAFFIC_FILE):
        return None, "no ncu capture recorded for this build (bench.py --traffic-from)"
    with open(TRAFFIC_FILE) as f:
        rec = json.load(f)
    entry = rec.get("kernels", {}).get(kernel)
    if entry is None:
        return None, f"{os.path.basename(TRAFFIC_FILE)} has no entry for {kernel}"
    return entry["dram_bytes"], rec.get("source", "ncu")


def record_traffic(paths):
    """--traffic-from CSV [CSV ...]: read ncu --csv logs (metrics dram__bytes_read.sum,
    dram__bytes_write.sum) of ``--profile`` runs and write the bytes per launch of
    each gmm_kernel layout, last captured launch of each, to bench_traffic.json."""
    import csv
    layouts = {"0": "gmm_kernel<NN>", "1": "gmm_kernel<NT>", "2": "gmm_kernel<TN>"}
    found = {}
    for path in paths:
        header = None
        per_id = {}
        with open(path, newline="") as f:
            for row in csv.reader(f):
                if row and row[0] == "ID":
                    header = row
                    continue
                if header is None or len(row) != len(header):
                    continue
                d = dict(zip(header, row))
                name = d["Kernel Name"]
                if "gmm_kernel<" not in name:
                    continue
                mode = name.split("gmm_kernel<")[1].split(",")[0].strip().replace("(b200gmm::Mode)", "")
                if d["Metric Name"] in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
                    value = float(d["Metric Value"].replace(",", ""))
                    unit = d["Metric Unit"].lower()
                    scale = {"byte": 1.0, "kbyte": 1e3, "mbyte": 1e6, "gbyte": 1e9}.get(unit, 1.0)
                    rec = per_id.setdefault(d["ID"], {"mode": mode, "bytes": 0.0})
                    rec["bytes"] += value * scale
        for _, rec in sorted(per_id.items(), key=lambda kv: int(kv[0])):
            if rec["mode"] in layouts:
                found[layouts[rec["mode"]]] = {"dram_bytes": rec["bytes"], "capture": os.path.basename(path)}
    out = {"source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, one launch at the benchmark's size "
                     "(bench.py --profile PASS under ncu, then bench.py --traffic-from)",
           "kernels": found}
    with open(TRAFFIC_FILE, "w") as f:
        json.dump(out, f, indent=1)
        f.write("\n")
    print(json.dumps(out))


def fused_neighbours(backend, dev, bs, rounds=6):
    """The caller-side passes either side of gmm, fused into the kernel, each timed
    against the same work done with separate torch kernels (Mixtral shapes; rounds
    interleaved so that both sides see the same clocks; median and min in ms)."""
    z, rows, k, n = MIXTRAL["z"], MIXTRAL["rows"], MIXTRAL["k"], MIXTRAL["n"]
    g = torch.Generator(device=dev).manual_seed(5)
    F = torch.nn.functional

    def compare(cases):
        for _, fn in cases:
            fn()
        acc = {name: [] for name, _ in cases}
        for _ in range(rounds):
            for name, fn in cases:
                fn()
                acc[name].append(time_loop(fn, 5))
        return {name: {"median_ms": sorted(v)[len(v) // 2], "min_ms": min(v)} for name, v in acc.items()}

    out = {"workload": "mixtral shapes, z=8, 32768 rows; up-projection k=4096 n=14336, down-projection k=14336 n=4096"}
    # sort-by-expert fused into the A-tile load
    tokens = rows // 2
    x = torch.randn(tokens, k, device=dev, generator=g).bfloat16()
    idx = torch.randint(0, tokens, (rows,), device=dev, generator=g)
    b_gate = (torch.randn(z, k, n, device=dev, generator=g) * 0.02).bfloat16()
    c = torch.empty(rows, n, device=dev, dtype=torch.bfloat16)
    a = x.index_select(0, idx)
    out["gather"] = compare((
        ("gmm_gather", lambda: backend.gmm_gather(x, idx, b_gate, bs, c=c)),
        ("index_select + gmm", lambda: backend.gmm(x.index_select(0, idx), b_gate, bs, c=c)),
        ("gmm on rows already sorted", lambda: backend.gmm(a, b_gate, bs, c=c))))
    # gate and up products with the activation in the epilogue
    b_up = (torch.randn(z, k, n, device=dev, generator=g) * 0.02).bfloat16()
    h1 = torch.empty(rows, n, device=dev, dtype=torch.bfloat16)

    def two_launches():
        backend.gmm(a, b_gate, bs, c=c)
        backend.gmm(a, b_up, bs, c=h1)
        return F.silu(c) * h1

    out["swiglu"] = compare((
        ("gmm_swiglu", lambda: backend.gmm_swiglu(a, b_gate, b_up, bs, c=c)),
        ("2 gmm + silu * mul", two_launches)))
    # the same with its backward: the gated product as an autograd function (products
    # recomputed in the backward kernel) against two ops.gmm and torch's elementwise ops
    from grouped_gemm_b200 import fused, ops
    grad_h = torch.randn(rows, n, device=dev, generator=g).bfloat16()
    leaves = [t.detach().requires_grad_(True) for t in (a, b_gate, b_up)]

    def fused_fwd_bwd():
        for t in leaves:
            t.grad = None
        fused.gmm_swiglu(leaves[0], leaves[1], leaves[2], bs).backward(grad_h)

    def separate_fwd_bwd():
        for t in leaves:
            t.grad = None
        (F.silu(ops.gmm(leaves[0], leaves[1], bs)) * ops.gmm(leaves[0], leaves[2], bs)).backward(grad_h)

    out["swiglu_fwd_bwd"] = compare((
        ("fused.gmm_swiglu forward + backward", fused_fwd_bwd),
        ("2 ops.gmm + silu * mul, forward + backward", separate_fwd_bwd)))
    del b_gate, b_up, h1, x, a, leaves, grad_h
    # weighted top-2 combine in the epilogue of the down-projection
    a2 = torch.randn(rows, n, device=dev, generator=g).bfloat16()
    b_down = (torch.randn(z, n, k, device=dev, generator=g) * 0.02).bfloat16()
    token_of_row = torch.randint(0, tokens, (rows,), device=dev, generator=g)
    weight = torch.rand(rows, device=dev, generator=g)
    y = torch.empty(rows, k, device=dev, dtype=torch.bfloat16)
    result = torch.zeros(tokens, k, device=dev, dtype=torch.bfloat16)

    def fused_combine():
        result.zero_()
        backend.gmm_scatter(a2, b_down, bs, result, token_of_row, row_weight=weight, accumulate=True)

    def separate_combine():
        backend.gmm(a2, b_down, bs, c=y)
        result.zero_()
        result.index_add_(0, token_of_row, (y.float() * weight[:, None]).bfloat16())

    out["combine"] = compare((
        ("gmm_scatter(row_weight, accumulate)", fused_combine),
        ("gmm + weight + index_add_", separate_combine),
        ("gmm alone", lambda: backend.gmm(a2, b_down, bs, c=y))))
    return out


def down_projection(backend, dev, bs, sizes, iters, rounds):
    """The three passes on the down-projection shapes (k=14336, n=4096), each
    against the per-expert library loop."""
    z, rows, k, n = MIXTRAL["z"], MIXTRAL["rows"], MIXTRAL["n"], MIXTRAL["k"]
    g = torch.Generator(device=dev).manual_seed(4)
    a = torch.randn(rows, k, device=dev, generator=g).bfloat16()
    b = (torch.randn(z, k, n, device=dev, generator=g) * 0.02).bfloat16()
    grad = torch.randn(rows, n, device=dev, generator=g).bfloat16()
    flops = 2.0 * rows * k * n
    ours = {"fwd": lambda: backend.gmm(a, b, bs),
            "dgrad": lambda: backend.gmm(grad, b, bs, trans_b=True),
            "wgrad": lambda: backend.gmm(a, grad, bs, trans_a=True)}
    passes, library = compare_passes(ours, library_loop_fns(a, b, grad, sizes), flops, iters, rounds)
    out = {"workload": "b [8, 14336, 4096], a [32768, 14336], same batch sizes"}
    out.update(passes)
    return out, library


def fine_grained_hbm(backend, dev, peaks, rounds):
    """benchmark configuration 4 (z=256, k=7168, n=2048, 65536 rows, ~20 % empty experts;
    median group 59 rows): the weights (forward, dgrad) or the per-expert outputs
    (wgrad) dominate the traffic, so these passes are judged against the HBM
    roofline.  Algorithmic bytes: operands + weights of non-empty experts +
    output; wgrad writes all 256 output blocks."""
    sizes = fine_grained_batch_sizes()
    z, k, n, rows = 256, 7168, 2048, 65536
    g = torch.Generator(device=dev).manual_seed(2)
    a = torch.randn(rows, k, device=dev, generator=g).bfloat16()
    b = (torch.randn(z, k, n, device=dev, generator=g) * 0.02).bfloat16()
    grad = torch.randn(rows, n, device=dev, generator=g).bfloat16()
    bs = torch.tensor(sizes, dtype=torch.int64, device=dev)
    nonempty = sum(1 for s in sizes if s > 0)
    flops = 2.0 * rows * k * n
    nbytes = {"fwd": 2.0 * (rows * k + nonempty * k * n + rows * n),
              "dgrad": 2.0 * (rows * n + nonempty * k * n + rows * k),
              "wgrad": 2.0 * (rows * k + rows * n + z * k * n)}
    c_w = torch.empty(z, k, n, device=dev, dtype=torch.bfloat16)
    ours = {"fwd": lambda: backend.gmm(a, b, bs),
            "dgrad": lambda: backend.gmm(grad, b, bs, trans_b=True),
            "wgrad": lambda: backend.gmm(a, grad, bs, trans_a=True, c=c_w)}
    passes, library = compare_passes(ours, library_loop_fns(a, b, grad, sizes), flops, 5, rounds)
    out = {"workload": "config 4: z=256 k=7168 n=2048 rows=65536, 51 empty experts, median 59 rows"}
    for name, rec in passes.items():
        tensor_ms = flops / peaks["burst"] / 1e9
        hbm_ms = nbytes[name] / peaks["hbm_gbs"] / 1e6
        rec.update({"gbs": nbytes[name] / rec["ms"] / 1e6, "hbm_frac": nbytes[name] / rec["ms"] / 1e6 / peaks["hbm_gbs"],
                    "algorithmic_bytes": nbytes[name],
                    "roofline_ms": max(tensor_ms, hbm_ms), "roofline_frac": max(tensor_ms, hbm_ms) / rec["ms"]})
        out[name] = rec
    return out, library


def e2e_single(backend, a, b, grad, bs, flops_pass, steps):
    """The step driven from pinned host memory: every step copies that step's a,
    b and grad to the device, runs forward, dgrad and wgrad through
    ``backend.gmm`` and copies c, dgrad and wgrad back.  Copies run on their own
    streams with double-buffered device inputs, so the upload of step i+1 and the
    download of step i overlap the GEMMs of the neighbouring steps (PCIe is full
    duplex); nothing is skipped or cached between steps."""
    dev = a.device
    host_in = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for t in (a, b, grad)]
    dev_in = [[torch.empty_like(t) for t in (a, b, grad)] for _ in range(2)]
    outs_shape = [(a.shape[0], b.shape[2]), (a.shape[0], a.shape[1]), tuple(b.shape)]
    host_out = [torch.empty(s, dtype=torch.bfloat16, pin_memory=True) for s in outs_shape]
    h2d = sum(t.numel() * 2 for t in host_in)
    d2h = sum(t.numel() * 2 for t in host_out)
    compute = torch.cuda.current_stream(dev)
    up, down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def run(n_steps):
        in_free = [None, None]     # event: the GEMMs that read this input set are done
        for i in range(n_steps):
            da, db, dg = dev_in[i % 2]
            with torch.cuda.stream(up):
                if in_free[i % 2] is not None:
                    up.wait_event(in_free[i % 2])
                da.copy_(host_in[0], non_blocking=True)
                db.copy_(host_in[1], non_blocking=True)
                dg.copy_(host_in[2], non_blocking=True)
                ready = up.record_event()
            compute.wait_event(ready)
            c = backend.gmm(da, db, bs)
            dx = backend.gmm(dg, db, bs, trans_b=True)
            dw = backend.gmm(da, dg, bs, trans_a=True)
            done = compute.record_event()
            in_free[i % 2] = done
            with torch.cuda.stream(down):
                down.wait_event(done)
                for dst, src in zip(host_out, (c, dx, dw)):
                    dst.copy_(src, non_blocking=True)
                    src.record_stream(down)
        compute.wait_stream(up)
        compute.wait_stream(down)

    run(2)
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    up.wait_stream(compute)
    e0.record()
    run(steps)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"value": 3 * flops_pass / ms / 1e9, "unit": UNIT, "ms_per_step": ms, "steps": steps,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "what": "pinned host a, b, grad -> device; fwd+dgrad+wgrad through grouped_gemm_b200.backend.gmm; "
                    "c, dgrad, wgrad -> pinned host; uploads, GEMMs and downloads of neighbouring steps overlap "
                    "(three streams, double-buffered inputs)"}


def ep_setup(world, rank, dev):
    from grouped_gemm_b200 import expert_parallel as ep
    ids = ep_routing(EP["tokens"], EP["z"], EP["top_k"])
    per = EP["tokens"] // world
    local_ids = ids[rank * per:(rank + 1) * per].to(dev)
    plan = ep.build_plan(local_ids, EP["z"])
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(per, EP["hidden"], device=dev, generator=g).bfloat16()
    w = (torch.randn(EP["z"] // world, EP["hidden"], EP["ffn"], device=dev, generator=g) * 0.02).bfloat16()
    grad = torch.randn(per * EP["top_k"], EP["ffn"], device=dev, generator=g).bfloat16()
    return ep, plan, x, w, grad


def ep_flops():
    return 3 * 2.0 * EP["tokens"] * EP["top_k"] * EP["hidden"] * EP["ffn"]


def ep_value_single(steps, dev):
    """The multi-GPU workload on one GPU (all 64 experts local, rows only
    permuted), timed with the step function the multi-GPU lines use: the
    denominator for their strong-scaling efficiency."""
    from grouped_gemm_b200 import backend, expert_parallel as ep
    ids = ep_routing(EP["tokens"], EP["z"], EP["top_k"]).to(dev)
    g = torch.Generator(device=dev).manual_seed(100)
    x = torch.randn(EP["tokens"], EP["hidden"], device=dev, generator=g).bfloat16()
    w = (torch.randn(EP["z"], EP["hidden"], EP["ffn"], device=dev, generator=g) * 0.02).bfloat16()
    grad = torch.randn(EP["tokens"] * EP["top_k"], EP["ffn"], device=dev, generator=g).bfloat16()
    px = ep.PeerExchange(ids, EP["z"], EP["hidden"], EP["ffn"], single_rank=True)
    gmm_fn = lambda a_, b_, bs_, ta, tb: backend.gmm(a_, b_, bs_, trans_a=ta, trans_b=tb)
    step = lambda: px.step_fused(x, w, grad, gmm_fn, x_next=x)
    for _ in range(3):
        step()
    steps = max(steps, 2)
    ms = time_loop(step, steps)
    out = {"workload": workload_config(2)["workload"].replace("over 2 ranks", "over 1 rank"),
           "value": ep_flops() / ms / 1e9, "unit": UNIT, "ms_per_step": ms, "steps": steps,
           "step": "PeerExchange.step_fused, as in the multi-GPU lines"}
    del x, w, grad, px
    torch.cuda.empty_cache()
    return out


def ep_parity(ep, px, plan, x, w, grad, gmm_fn, backend, rank):
    """Before anything is timed: one step over peer memory against the same step
    over NCCL all-to-all (bit for bit, every element of out_rows, dx, dw), and the
    local GEMMs of this rank against an fp32 CPU product on sampled rows."""
    want = ep.expert_parallel_step(x, w, grad, plan, gmm_fn)
    differs = []
    for tag, in_kernel, nxt in (("step_fused", True, None), ("step_fused announcing the next activations", True, x),
                                ("step_fused on activations sent ahead", True, x),
                                ("step_fused on activations sent ahead, none announced", True, None),
                                ("step_fused with the gradient push as its own kernel", False, None)):
        got = px.step_fused(x, w, grad, gmm_fn, push_in_kernel=in_kernel, x_next=nxt)
        torch.cuda.synchronize()
        for name, u, v in zip(("out_rows", "dx", "dw"), got, want):
            if u.shape != v.shape or not torch.equal(u, v):
                differs.append(f"{tag}: {name}")
    same = not differs
    # local GEMMs vs fp32 on the host: 64 rows of the forward and of dgrad, 8 rows of one expert's wgrad
    a = ep.dispatch(x, plan)
    gl = ep.dispatch_rows(grad, plan)
    sizes = plan.batch_sizes_host
    starts = np.concatenate([[0], np.cumsum(sizes)])
    rng = np.random.default_rng(7 + rank)
    rows = np.sort(rng.choice(int(starts[-1]), size=min(64, int(starts[-1])), replace=False))
    expert_of = np.searchsorted(starts, rows, side="right") - 1
    c = backend.gmm(a, w, plan.batch_sizes)
    da = backend.gmm(gl, w, plan.batch_sizes, trans_b=True)
    dw = backend.gmm(a, gl, plan.batch_sizes, trans_a=True)
    max_err = 0.0
    ok = True
    for e in np.unique(expert_of):
        sel = torch.from_numpy(rows[expert_of == e]).to(a.device)
        we = w[int(e)].float().cpu()
        for got_rows, ref in ((c[sel], a[sel].float().cpu() @ we), (da[sel], gl[sel].float().cpu() @ we.t())):
            err = (got_rows.float().cpu() - ref).abs()
            max_err = max(max_err, float(err.max()))
            ok = ok and bool((err <= 1e-2 + 1e-2 * ref.abs()).all())
    e0 = int(np.argmax(sizes))
    sl = slice(int(starts[e0]), int(starts[e0 + 1]))
    krows = torch.from_numpy(rng.choice(EP["hidden"], size=8, replace=False)).to(a.device)
    ref = a[sl][:, krows].float().cpu().t() @ gl[sl].float().cpu()
    err = (dw[e0][krows].float().cpu() - ref).abs()
    max_err = max(max_err, float(err.max()))
    ok = ok and bool((err <= 1e-2 * float(ref.abs().max()) + 1e-2 * ref.abs()).all())
    return {"checked": True, "peer_path_equals_nccl_path_bitwise": bool(same), "differs": differs,
            "local_gemms_within_tolerance": bool(ok),
            "max_abs_err_vs_fp32": max_err, "rows_sampled": int(len(rows))}


class StdoutToStderr:
    """Send file descriptor 1 to stderr while libraries initialise (NCCL prints
    its version banner on stdout), so that stdout carries the JSON line only."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)
        return self

    def __exit__(self, *exc):
        sys.stdout.flush()
        os.dup2(self.saved, 1)
        os.close(self.saved)


def run_multi(args):
    with StdoutToStderr():
        line = measure_multi(args)
    if line is not None:
        print(json.dumps(line), flush=True)


def measure_multi(args):
    import torch.distributed as dist
    from grouped_gemm_b200 import _capi, backend
    world, rank, local = dist_info()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    # Same workload on one GPU first (rank 0 alone; the others wait): the
    # denominator a reader needs for strong-scaling efficiency.
    scaling_base = None
    if rank == 0 and not args.no_scaling_base:
        scaling_base = ep_value_single(args.steps, dev)
    dist.barrier()
    ep, plan, x, w, grad = ep_setup(world, rank, dev)
    gmm_fn = lambda a_, b_, bs_, ta, tb: backend.gmm(a_, b_, bs_, trans_a=ta, trans_b=tb)
    exchange_note = ""
    px = None
    if args.exchange == "peer":
        per = EP["tokens"] // world
        try:
            px = ep.PeerExchange(ep_routing()[rank * per:(rank + 1) * per].to(dev), EP["z"], EP["hidden"], EP["ffn"])
            failed = 0
        except Exception as exc:  # noqa: BLE001  (symmetric memory unavailable)
            exchange_note = f" (peer-memory setup failed, NCCL exchange used instead: {type(exc).__name__}: {exc})"[:300]
            failed = 1
        # every rank takes the same path
        agree = torch.tensor([failed], device=dev)
        dist.all_reduce(agree, op=dist.ReduceOp.MAX)
        if int(agree.item()):
            px = None
            args.exchange = "nccl"
            exchange_note = exchange_note or " (peer-memory setup failed on another rank, NCCL exchange used instead)"
    parity = None
    if px is not None:
        if not args.no_parity:
            parity = ep_parity(ep, px, plan, x, w, grad, gmm_fn, backend, rank)
        if args.no_fused_combine:
            step = lambda: px.step(x, w, grad, gmm_fn)
        else:
            step = lambda: px.step_fused(x, w, grad, gmm_fn, push_in_kernel=not args.no_push_in_kernel,
                                         x_next=None if args.no_push_in_kernel else x)
        exchange_step = step
    else:
        step = lambda: ep.expert_parallel_step(x, w, grad, plan, gmm_fn)
        exchange_step = step
    for _ in range(max(args.warmup, 3)):
        step()
    launches0 = _capi.launch_count()
    round_ms = []
    with ClockSampler(local) as clocks:
        for _ in range(args.rounds):
            round_ms.append(timed_region(step, args.steps, world) / args.steps)
    launches = (_capi.launch_count() - launches0) * world // args.rounds
    ms_step = sorted(round_ms)[len(round_ms) // 2]
    value = ep_flops() / ms_step / 1e9

    # where a step's time goes on this rank's main stream (one more step, marked with events)
    phases = None
    if px is not None and not (args.no_fused_combine):
        px.step_fused(x, w, grad, gmm_fn, timeline=True, push_in_kernel=not args.no_push_in_kernel,
                      x_next=None if args.no_push_in_kernel else x)
        phases = px.phase_times()

    # the same step with NCCL all-to-all as the exchange (the baseline of this path)
    nccl_exchange = None
    if px is not None and not args.no_nccl_compare:
        nccl_step = lambda: ep.expert_parallel_step(x, w, grad, plan, gmm_fn)
        for _ in range(2):
            nccl_step()
        n_steps = max(2, min(args.steps, 5))
        ms_nccl = timed_region(nccl_step, n_steps, world) / n_steps
        nccl_exchange = {"value": ep_flops() / ms_nccl / 1e9, "unit": UNIT, "ms_per_step": ms_nccl, "steps": n_steps}
        torch.cuda.empty_cache()

    # split: local GEMMs alone (max over ranks), to show the exchange share
    a = ep.dispatch(x, plan)
    gl = ep.dispatch_rows(grad, plan)

    def gemms():
        backend.gmm(a, w, plan.batch_sizes)
        backend.gmm(gl, w, plan.batch_sizes, trans_b=True)
        backend.gmm(a, gl, plan.batch_sizes, trans_a=True)

    gemms()
    ms_gemm = timed_region(gemms, args.steps, world) / args.steps
    del a, gl

    # end to end from pinned host buffers
    hx = torch.empty(x.shape, dtype=x.dtype, pin_memory=True).copy_(x)
    hg = torch.empty(grad.shape, dtype=grad.dtype, pin_memory=True).copy_(grad)
    ho = torch.empty(grad.shape, dtype=grad.dtype, pin_memory=True)
    hdx = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
    hdw = torch.empty(w.shape, dtype=w.dtype, pin_memory=True)

    def e2e_step():
        x.copy_(hx, non_blocking=True)
        grad.copy_(hg, non_blocking=True)
        out_rows, dx, dw = exchange_step()
        ho.copy_(out_rows, non_blocking=True)
        hdx.copy_(dx, non_blocking=True)
        hdw.copy_(dw, non_blocking=True)

    e2e_step()
    e2e_steps = min(args.steps, 3)
    ms_e2e = timed_region(e2e_step, e2e_steps, world) / e2e_steps
    peaks = measured_peaks()
    status = torch.tensor([backend.device_status(dev)], device=dev)
    dist.all_reduce(status, op=dist.ReduceOp.MAX)
    if parity is not None:
        # a rank that disagrees makes the whole line disagree
        flags = torch.tensor([0 if parity["peer_path_equals_nccl_path_bitwise"] else 1,
                              0 if parity["local_gemms_within_tolerance"] else 1], device=dev)
        dist.all_reduce(flags, op=dist.ReduceOp.MAX)
        err = torch.tensor([parity["max_abs_err_vs_fp32"]], device=dev)
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        parity["peer_path_equals_nccl_path_bitwise"] = not bool(flags[0].item())
        parity["local_gemms_within_tolerance"] = not bool(flags[1].item())
        parity["max_abs_err_vs_fp32"] = float(err.item())
        parity["ranks"] = world
    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world),
            "roofline": {"bound": "tensor", "kernel": "gmm_kernel<NN|NT|TN> (local GEMMs of one step)",
                         "achieved": ep_flops() / world / ms_gemm / 1e9, "peak": peaks["sustained"],
                         "unit": "TFLOP/s", "frac": ep_flops() / world / ms_gemm / 1e9 / peaks["sustained"],
                         "peak_source": f"{peaks['source']} cuBLAS bf16 sustained (per GPU)", "traffic": None},
            "exchange": (("peer memory over NVLink (symmetric memory): "
                          + ("4 row pushes per step" if args.no_fused_combine else
                             "both combines written by the GEMM epilogues straight into the token owners' buffers; "
                             + ("2 row pushes (dispatch) per step" if args.no_push_in_kernel else
                                "the gradient dispatch done by push warps inside the forward GEMM kernel and the "
                                "next step's activation dispatch by push warps inside the dgrad kernel: no "
                                "exchange pass of its own is left in a step"))
                          )
                         if args.exchange == "peer" else "NCCL all_to_all_single + index gathers" + exchange_note),
            "rounds": {"count": args.rounds, "ms_per_step_min": min(round_ms), "ms_per_step_max": max(round_ms)},
            "parity": parity, "nccl_exchange": nccl_exchange, "phases_ms_rank0": phases,
            "exchange_share": 1.0 - ms_gemm / ms_step, "ms_gemm_per_step": ms_gemm,
            "scaling_base": scaling_base,
            "cpu_baseline": None,
            "e2e": {"value": ep_flops() / ms_e2e / 1e9, "unit": UNIT, "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": (hx.numel() + hg.numel()) * 2 * world,
                    "d2h_bytes_per_step": (ho.numel() + hdx.numel() + hdw.numel()) * 2 * world},
            "gpu_launches": launches, "clocks": clocks.summary(), "device_status": int(status.item()),
        }
    dist.destroy_process_group()
    return line


def run_profile_case(args):
    """--profile PASS: allocate only that pass's operands (Mixtral size, or
    benchmark configuration 4 with --profile-workload fine) and launch it a few times;
    meant to be wrapped in ncu (one kernel, one captured launch).  Prints the
    CUDA-event time of the last launch."""
    from grouped_gemm_b200 import backend
    dev = torch.device("cuda", 0)
    if args.profile_workload == "fine":
        z, rows, k, n = 256, 65536, 7168, 2048
        sizes = fine_grained_batch_sizes()
    elif args.profile_workload == "fine64":
        # a quarter of benchmark configuration 4 (its first 64 experts, same size
        # distribution): under 3 GB on the device, for captures with many passes
        sizes = fine_grained_batch_sizes()[:64]
        z, rows, k, n = 64, sum(sizes), 7168, 2048
    elif args.profile_workload == "down":
        z, rows, k, n = MIXTRAL["z"], MIXTRAL["rows"], MIXTRAL["n"], MIXTRAL["k"]
        sizes = mixtral_batch_sizes()
    else:
        z, rows, k, n = MIXTRAL["z"], MIXTRAL["rows"], MIXTRAL["k"], MIXTRAL["n"]
        sizes = mixtral_batch_sizes()
    g = torch.Generator(device=dev).manual_seed(1)
    bs = torch.tensor(sizes, dtype=torch.int64, device=dev)
    if args.profile == "fwd":
        a = torch.randn(rows, k, device=dev, generator=g).bfloat16()
        b = (torch.randn(z, k, n, device=dev, generator=g) * 0.02).bfloat16()
        c = torch.empty(rows, n, device=dev, dtype=torch.bfloat16)
        fn = lambda: backend.gmm(a, b, bs, c=c)
    elif args.profile == "dgrad":
        a = torch.randn(rows, n, device=dev, generator=g).bfloat16()
        b = (torch.randn(z, k, n, device=dev, generator=g) * 0.02).bfloat16()
        c = torch.empty(rows, k, device=dev, dtype=torch.bfloat16)
        fn = lambda: backend.gmm(a, b, bs, trans_b=True, c=c)
    elif args.profile == "gather":
        x = torch.randn(rows // 2, k, device=dev, generator=g).bfloat16()
        idx = torch.randint(0, rows // 2, (rows,), device=dev, generator=g)
        b = (torch.randn(z, k, n, device=dev, generator=g) * 0.02).bfloat16()
        c = torch.empty(rows, n, device=dev, dtype=torch.bfloat16)
        fn = lambda: backend.gmm_gather(x, idx, b, bs, c=c)
    elif args.profile == "swiglu":
        a = torch.randn(rows, k, device=dev, generator=g).bfloat16()
        b = (torch.randn(z, k, n, device=dev, generator=g) * 0.02).bfloat16()
        b2 = (torch.randn(z, k, n, device=dev, generator=g) * 0.02).bfloat16()
        c = torch.empty(rows, n, device=dev, dtype=torch.bfloat16)
        fn = lambda: backend.gmm_swiglu(a, b, b2, bs, c=c)
    elif args.profile == "push":
        # The forward product with its rows scattered through a table and, inside the same
        # launch, a row transfer of the size of its output (here into a local buffer: the
        # kernel is the one the expert-parallel step runs, the destination table has one entry).
        from grouped_gemm_b200 import _capi
        lib = _capi.load()
        a = torch.randn(rows, k, device=dev, generator=g).bfloat16()
        b = (torch.randn(z, k, n, device=dev, generator=g) * 0.02).bfloat16()
        c = torch.empty(rows, n, device=dev, dtype=torch.bfloat16)
        src = torch.randn(rows, n, device=dev, generator=g).bfloat16()
        dst = torch.empty_like(src)
        dest = torch.randperm(rows, device=dev) * (n * 2) + c.data_ptr()
        src_row = torch.randperm(rows, device=dev).to(torch.int32)
        dst_row = torch.randperm(rows, device=dev).to(torch.int64)
        dst_rank = torch.zeros(rows, dtype=torch.int32, device=dev)
        table = torch.tensor([dst.data_ptr()], dtype=torch.int64, device=dev)
        ws_bytes = _capi.workspace_bytes(z)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        status = backend.backend.device_status(dev).data_ptr()

        def fn():
            rc = lib.b200gmm_run_scatter_push(
                a.data_ptr(), b.data_ptr(), dest.data_ptr(), c.data_ptr(), c.numel() * 2, bs.data_ptr(), 1, z, rows, k, n,
                0, src.data_ptr(), n * 2, rows, src_row.data_ptr(), dst_rank.data_ptr(), dst_row.data_ptr(),
                table.data_ptr(), ws.data_ptr(), ws_bytes, status, torch.cuda.current_stream(dev).cuda_stream)
            _capi.check(rc, "b200gmm_run_scatter_push")
    else:
        a = torch.randn(rows, k, device=dev, generator=g).bfloat16()
        b = torch.randn(rows, n, device=dev, generator=g).bfloat16()
        c = torch.empty(z, k, n, device=dev, dtype=torch.bfloat16)
        fn = lambda: backend.gmm(a, b, bs, trans_a=True, c=c)
    for _ in range(args.profile_launches - 1):
        fn()
    ms = time_loop(fn, 1)
    print(json.dumps({"profile": args.profile, "launches": args.profile_launches, "last_ms": ms,
                      "device_status": backend.device_status()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--profile", choices=["fwd", "dgrad", "wgrad", "gather", "swiglu", "push"], default=None,
                    help="launch one pass of the Mixtral workload a few times and exit (for ncu)")
    ap.add_argument("--profile-launches", type=int, default=2)
    ap.add_argument("--profile-workload", choices=["mixtral", "down", "fine", "fine64"], default="mixtral")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--rounds", type=int, default=5,
                    help="timed rounds of --steps steps each; the value is the median round")
    ap.add_argument("--traffic-from", nargs="+", default=None, metavar="NCU_CSV",
                    help="record DRAM bytes per launch from ncu --csv logs of --profile runs and exit")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                    help="multi-GPU row exchange: peer-memory pushes (default) or NCCL all-to-all")
    ap.add_argument("--no-parity", action="store_true",
                    help="multi-GPU runs: skip the check against the NCCL path and the fp32 products before timing")
    ap.add_argument("--no-nccl-compare", action="store_true",
                    help="multi-GPU runs: skip timing the same step with NCCL all-to-all as the exchange")
    ap.add_argument("--no-push-in-kernel", action="store_true",
                    help="multi-GPU runs: dispatch the gradient rows and the activations with row pushes of their own "
                         "between the GEMMs instead of from inside the forward / dgrad GEMM kernels")
    ap.add_argument("--no-fused-combine", action="store_true",
                    help="multi-GPU runs: combine with separate push kernels instead of from the GEMM epilogues")
    ap.add_argument("--no-scaling-base", action="store_true",
                    help="skip timing the multi-GPU workload on one GPU (rank 0's) alone")
    ap.add_argument("--fused", action="store_true",
                    help="also time gmm_gather, gmm_swiglu and the weighted combine against separate torch kernels")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.traffic_from:
        return record_traffic(args.traffic_from)
    args.rounds = max(args.rounds, 1)
    if args.impl == "reference":
        return run_reference(args)
    world, _, _ = dist_info()
    if args.profile:
        return run_profile_case(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path "
                         "(use --impl reference for the CPU baseline)")
    if world > 1 or args.gpus > 1:
        if world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
        return run_multi(args)
    return run_single(args)


if __name__ == "__main__":
    main()
