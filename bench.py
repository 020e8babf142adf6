#!/usr/bin/env python
"""ResNet-50 v1.5 inference throughput through the ODLA C ABI of libodla_b200.so.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun, one rank per GPU)
    python bench.py --impl reference ...                      (the reference's CPU kernels on the host cores)

    python bench.py --inlib-gpus N                            (one process; one execute sharded over N GPUs by the library)

One step = one odla_ExecuteComputation over a batch of 256 synthetic NHWC fp16 images (ResNet-50
v1.5 at 224 x 224, random He-normal weights with folded batch norm).  `value` is measured with the
inputs already resident in HBM (device pointers bound), `e2e` with pinned host buffers bound, so the
host-to-device copy of the images and the device-to-host copy of the probabilities are inside the
timed region (wall clock around the synchronous call).  Device times come from CUDA events recorded
by the library on the stream its kernels run on; multi-rank numbers take the maximum over ranks.
Each rank owns one GPU and a full copy of the weights; there is no collective on the data path
(weak scaling).  The same network in int8 quantise/dequantise form is measured the same way and
reported as the `int8` object of the line.
"""
import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = "heterogeneity-aware-lowering-and-optimization_b200"
sys.path.insert(0, ROOT)

BATCH = 256
METRIC = "resnet50_v1.5_inference_throughput"
UNIT = "img/s"


# ------------------------------------------------------------------ multi-rank helpers ----
def _dist():
    import torch.distributed as dist
    return dist if dist.is_available() and dist.is_initialized() else None


def max_over_ranks(x):
    d = _dist()
    if d is None:
        return float(x)
    import torch
    t = torch.tensor([float(x)], dtype=torch.float64, device="cuda" if d.get_backend() == "nccl" else "cpu")
    d.all_reduce(t, op=d.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x):
    d = _dist()
    if d is None:
        return x
    import torch
    t = torch.tensor([float(x)], dtype=torch.float64, device="cuda" if d.get_backend() == "nccl" else "cpu")
    d.all_reduce(t, op=d.ReduceOp.SUM)
    return type(x)(t.item())


def rank_seed(base, rank):
    return base * 1000003 + 7919 * rank


def barrier():
    d = _dist()
    if d is not None:
        d.barrier()


# ------------------------------------------------------------------------- clocks ----
class ClockSampler(threading.Thread):
    """Samples the SM clock, the power draw and the throttle reasons while the timed region runs: through NVML in this
    process every 2 ms when the binding is there (a 4 ms step is invisible to a tool that is spawned every 200 ms),
    else through nvidia-smi every 200 ms.  Reading only; nothing about the GPU is changed."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag = index, [], threading.Event()
        self.nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nvml = None

    def run(self):
        if self.nvml is not None:
            nv, h = self.nvml, self.handle
            bits = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20}
            while not self.stop_flag.is_set():
                try:
                    sm = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                    pw = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                    try:
                        r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                    except Exception:
                        r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                    self.samples.append((sm, self.sm_max, pw, [k for k, b in bits.items() if r & b]))
                except Exception:
                    pass
                self.stop_flag.wait(0.002)
            return
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                f = [x.strip() for x in out.split(",")]
                if len(f) >= 7 and f[0].replace(".", "").isdigit():
                    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                    self.samples.append((float(f[0]), float(f[1]), float(f[2]) if f[2].replace(".", "").isdigit() else 0.0,
                                         [n for i, n in enumerate(names) if f[3 + i].lower().startswith("active")]))
            except Exception:
                pass
            self.stop_flag.wait(0.2)

    def summary(self):
        self.stop_flag.set()
        self.join(timeout=6)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        # "under load": samples whose power draw is in the upper half of what was seen (the L2 flush and the host-side
        # gaps between steps draw little)
        pmax = max(s[2] for s in self.samples)
        busy = [s for s in self.samples if s[2] >= 0.5 * pmax] or self.samples
        sm = sorted(s[0] for s in busy)
        reasons = sorted({r for s in self.samples for r in s[3]})
        return {"sm_mhz": sm[len(sm) // 2], "sm_min_mhz": sm[0], "sm_max_mhz": self.samples[0][1], "power_w_max": round(pmax, 1), "reasons": reasons,
                "samples": len(self.samples), "samples_under_load": len(busy), "source": "nvml, 2 ms" if self.nvml is not None else "nvidia-smi, 200 ms"}


# ------------------------------------------------------------------- the two arms ----
def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def run_reference(args, rank, world):
    """The reference's own CPU kernels (runtime/generic, compiled into oracle/_ref) driven through the oracle ODLA
    platform: every step runs one image per host thread (the reference kernels are single-threaded per image) through
    the same fp32 ResNet-50 graph.  The run is bounded in time: steps beyond the budget are not executed and the line
    reports the number that were."""
    if rank != 0:
        return
    pkg = importlib.import_module(PKG)
    odla = pkg.odla
    rn = importlib.import_module(PKG + ".halo_models.resnet50")
    ref_path = os.path.join(ROOT, "oracle", "libodla_cpuref.so")
    if not os.path.exists(ref_path):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "libodla_cpuref.so"], check=True, stdout=subprocess.DEVNULL)
    ref = odla.OdlaLib(ref_path)
    cores = ref.cpuref_Threads()
    kind = "reference" if ref.cpuref_UsesReference() else "port"
    w = rn.weights()
    sample = cores
    g = odla.Graph(ref, "resnet50")
    rn.build(g, sample, w)
    x = rn.inputs(sample, seed=11)
    budget = float(os.environ.get("BENCH_REFERENCE_BUDGET_S", "300"))
    t_begin = time.time()
    t0 = time.time()
    g.run(x)                                   # warm-up (page-in, thread start); also tells how long a step takes
    first = time.time() - t0
    warm = 1
    steps, dt = 0, 0.0
    while steps < args.steps and (steps == 0 or (time.time() - t_begin) + first < budget):
        t0 = time.time()
        g.run(x)
        dt += time.time() - t0
        steps += 1
    g.close()
    value = sample * steps / dt
    desc = "%d images (one per host thread) of the 256-image batch per step, fp32, %s kernels on %d host threads; %d of %d steps ran inside the %.0f s budget" % (
        sample, "runtime/generic" if kind == "reference" else "restated", cores, steps, args.steps, budget)
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps, "warmup": warm,
                      "steps_requested": args.steps, "warmup_requested": args.warmup,
                      "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                      "data": "synthetic", "config": {"workload": "resnet50_v1.5_nhwc_fp16_b%d" % BATCH, "sample_images_per_step": sample,
                                                      "note": "same graph and weights as the GPU arm, evaluated in fp32 on a sample of the batch"},
                      "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": desc},
                      "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def cpu_baseline_leg(pkg, rn, w, seconds=20.0):
    """The oracle timed on this box's host cores on a bounded sample (rank 0, N=1 only)."""
    odla = pkg.odla
    ref = odla.OdlaLib(os.path.join(ROOT, "oracle", "libodla_cpuref.so"))
    cores = ref.cpuref_Threads()
    kind = "reference" if ref.cpuref_UsesReference() else "port"
    sample = max(1, min(cores, 8))
    g = odla.Graph(ref, "resnet50")
    rn.build(g, sample, w)
    x = rn.inputs(sample, seed=11)
    t0 = time.time()
    n = 0
    while True:
        g.run(x)
        n += 1
        if time.time() - t0 > seconds or n >= 3:
            break
    dt = time.time() - t0
    g.close()
    return {"value": sample * n / dt, "unit": UNIT, "cores": min(cores, sample), "kind": kind,
            "sample": "%d pass(es) over %d images (fp32, one image per host thread, %d threads busy)" % (n, sample, min(cores, sample))}


def bind_to_gpu_numa_node(index):
    """Pins this process to the CPUs next to GPU `index` (NVML's affinity mask) before any pinned buffer is allocated,
    so that eight ranks' host-to-device copies do not all cross the same socket.  Best effort; returns what it did."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = [64 * i + b for i, wd in enumerate(words) for b in range(64) if (wd >> b) & 1]
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if allowed:
            os.sched_setaffinity(0, allowed)
            return "%d cpus near gpu %d" % (len(allowed), index)
    except Exception as e:   # no NVML, no permission: leave the affinity alone
        return "unchanged (%s)" % type(e).__name__
    return "unchanged"


# ResNet-50 dram__bytes_read.sum + dram__bytes_write.sum of the tensor-core kernel, summed over its launches of one
# execute and divided by their number: one ncu capture at a smaller batch (the full batch breaks the capture-size rule),
# scaled in proportion to the batch (activation traffic grows with it; the 25 / 51 MB of weights do not, which makes the
# scaled figure a slight over-estimate).  See profiles/.
NCU_TRAFFIC = {"f16": {"bytes_per_launch": 9.8226e7, "launches": 54, "at_batch": 128, "source": "ncu capture of all 54 launches at B=128 (4.066 GB read + 1.238 GB written), scaled by batch / 128"},
               "s8": {"bytes_per_launch": 4.1931e7, "launches": 54, "at_batch": 128, "source": "ncu capture of all 54 launches at B=128 (1.975 GB read + 0.290 GB written), scaled by batch / 128"}}


def tensor_roofline(prof, ms_per_step, peaks, peak_kind, clocks, int8, batch):
    """Roofline of the tensor-core kernel from the timed step: its share of the step comes from a pass that brackets
    every launch with events (serialised, so only the SHARE is used), its time is that share of the measured
    ms_per_step -- never more than the step it sits in."""
    fam = {}
    for p in prof:
        f = fam.setdefault(p["op"], {"launches": 0, "ms": 0.0, "flops": 0.0, "bytes": 0.0})
        f["launches"] += 1
        f["ms"] += p["ms"]
        f["flops"] += p["flops"]
        f["bytes"] += p["bytes"]
    tc = [f for k, f in fam.items() if k.endswith("_umma")]
    all_ms = max(sum(f["ms"] for f in fam.values()), 1e-9)
    share = sum(f["ms"] for f in tc) / all_ms
    tc_flops = sum(f["flops"] for f in tc)
    tc_bytes = sum(f["bytes"] for f in tc)
    tc_launches = sum(f["launches"] for f in tc)
    kernel_ms = ms_per_step * share
    mult = 2.0 if int8 else 1.0
    burst, sustained = mult * float(peaks.get("bf16_tflops", 0)), mult * float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops", 0)))
    sm, sm_max = clocks.get("sm_mhz"), clocks.get("sm_max_mhz")
    regime = "burst" if (sm and sm_max and sm >= 0.93 * sm_max) else "sustained"
    peak = burst if regime == "burst" else sustained
    achieved = tc_flops / (kernel_ms * 1e-3) / 1e12 if kernel_ms > 0 else 0.0
    tr = NCU_TRAFFIC["s8" if int8 else "f16"]
    roof = {"bound": "tensor", "kernel": "umma_conv_kernel (tcgen05 implicit-GEMM conv / GEMM, %d launches per step)" % tc_launches,
            "achieved": achieved, "peak": peak, "unit": "TOP/s" if int8 else "TFLOP/s", "frac": achieved / peak if peak else None,
            "peak_source": ("2 x " if int8 else "") + peak_kind + " bf16 " + regime + (" (no int8 peak is measured; the tensor pipe runs kind::i8 at twice the 16-bit rate)" if int8 else ""),
            "regime": regime, "frac_vs_burst": achieved / burst if burst else None, "frac_vs_sustained": achieved / sustained if sustained else None,
            "flops_per_step": tc_flops, "kernel_ms_per_step": kernel_ms, "share_of_step": share, "avg_launch_ms": kernel_ms / max(tc_launches, 1),
            "whole_step_achieved": tc_flops / (ms_per_step * 1e-3) / 1e12,
            "ms_per_step_x_sm_mhz": ms_per_step * sm if sm else None,
            "algorithmic_bytes_per_launch": tc_bytes / max(tc_launches, 1),
            "traffic": tr["bytes_per_launch"] * batch / tr["at_batch"] if tr else None,
            "traffic_source": tr["source"] if tr else None,
            "hbm_view": {"achieved_gbs": tc_bytes / (kernel_ms * 1e-3) / 1e9 if kernel_ms > 0 else 0.0, "peak_gbs": float(peaks.get("hbm_gbs", 0))}}
    families = {k: {"launches": v["launches"], "share": round(v["ms"] / all_ms, 4)} for k, v in sorted(fam.items(), key=lambda kv: -kv[1]["ms"])}
    return roof, families


def run_b200(args, rank, world, local_rank):
    numa = bind_to_gpu_numa_node(local_rank) if world > 1 else "single rank: not pinned"
    import torch
    pkg = importlib.import_module(PKG)
    odla = pkg.odla
    rn = importlib.import_module(PKG + ".halo_models.resnet50")
    inlib = args.inlib_gpus
    if not inlib:
        os.environ["ODLA_B200_DEVICE"] = str(local_rank)
        os.environ["ODLA_B200_NUM_GPUS"] = "1"
    torch.cuda.set_device(local_rank)
    lib = pkg.load()
    if lib.b200_DeviceCount() < 1:
        raise RuntimeError("bench.py needs a CUDA device: libodla_b200 has no CPU fallback")
    n_lib_gpus = inlib if inlib else 1
    w = rn.weights()
    BATCH = args.batch * n_lib_gpus
    peaks, peak_kind = measured_peaks()
    flush = [torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda:%d" % d) for d in (range(n_lib_gpus) if inlib else [local_rank])]   # larger than the 126 MB L2
    x_np = rn.inputs(BATCH, seed=rank_seed(10 + BATCH, rank), dtype=np.float16)["input"]
    x_host = torch.from_numpy(x_np).pin_memory()
    x_host2 = x_host.clone().pin_memory()     # the second context's own buffers (same images: results must agree)
    x_dev = x_host.cuda()
    h2d = x_host.numel() * 2
    total_images = sum_over_ranks(BATCH * args.steps)

    def measure(build, tag, int8):
        """value (device-resident), e2e (pinned host buffers) and the roofline for one form of the network."""
        g = odla.Graph(lib, "resnet50_" + tag, fp16=not int8, n_gpus=n_lib_gpus)
        build(g)
        g.context()   # odla_CreateContext attaches to the most recently created computation: make it now
        # a second context of the same computation (a lane of its own in the library) for the pipelined end-to-end leg;
        # with two executes in flight a whole step's input copy hides under the other step, so no sub-batches there
        ctx2 = g.extra_context() if args.contexts > 1 else None
        # The end-to-end leg binds host buffers; there the library pipelines the batch over sub-batches
        # (ODLA_BATCHES_PER_STEP) so that one sub-batch's input copy runs under another's kernels.
        g_host = g
        if args.sub_batches > 1:
            g_host = odla.Graph(lib, "resnet50_%s_host" % tag, fp16=not int8, n_gpus=n_lib_gpus, sub_batches=args.sub_batches)
            build(g_host)
            g_host.context()
        # the probabilities come back in the graph's own output type: fp16 for the fp16 graph fed fp16 images, fp32 for
        # the quantise/dequantise form
        y_dt = {odla.FLOAT16: torch.float16, odla.FLOAT32: torch.float32}[g.dtypes["prob"]]
        y_host = torch.zeros((BATCH, 1000), dtype=y_dt).pin_memory()
        y_host2 = torch.zeros((BATCH, 1000), dtype=y_dt).pin_memory()
        y_dev = torch.zeros((BATCH, 1000), dtype=y_dt, device="cuda")
        d2h = y_host.numel() * y_host.element_size()

        def step(gg):
            for f in flush:
                f.zero_()
            for d in range(len(flush)):
                torch.cuda.synchronize(flush[d].device)
            t0 = time.perf_counter()
            st = gg.execute()
            wall = time.perf_counter() - t0
            if st != 0:
                raise RuntimeError("odla_ExecuteComputation failed with status %d" % st)
            return gg.device_ms(), wall * 1e3

        def timed(gg, device_resident, sampler=None):
            gg.bind_input("input", x_dev.data_ptr() if device_resident else x_host.data_ptr())
            gg.bind_output("prob", y_dev.data_ptr() if device_resident else y_host.data_ptr())
            for _ in range(args.warmup):
                step(gg)
            barrier()
            torch.cuda.synchronize()
            if sampler:
                sampler.start()
            dev = wall = 0.0
            for _ in range(args.steps):
                d, wl = step(gg)
                dev += d
                wall += wl
            torch.cuda.synchronize()
            barrier()
            return max_over_ranks(dev), max_over_ranks(wall)

        def timed_pipelined(ctxs, bufs):
            """K steps with `len(ctxs)` executes in flight: step i is started with odla_AsyncExecuteComputation on context
            i mod n as soon as that context's previous step has delivered its outputs.  Every step still copies its own
            input from pinned host memory and its result back; the copies of one step run under the kernels of another.
            No L2 flush is possible between overlapping steps: each step streams 77 MB of fresh input and ~1.5 GB of
            activations through the 126 MB L2."""
            for c, (xh, yh) in zip(ctxs, bufs):
                c.bind_input("input", xh.data_ptr())
                c.bind_output("prob", yh.data_ptr())
            def run(n):
                for i in range(n):
                    c = ctxs[i % len(ctxs)]
                    if c.wait() != 0 or c.execute_async() != 0:
                        raise RuntimeError("asynchronous execute failed")
                for c in ctxs:
                    if c.wait() != 0:
                        raise RuntimeError("asynchronous execute failed")
            run(max(args.warmup, len(ctxs)))
            barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            run(args.steps)
            wall = (time.perf_counter() - t0) * 1e3
            torch.cuda.synchronize()
            barrier()
            return max_over_ranks(wall)

        sampler = ClockSampler(local_rank)
        dev_ms, _ = timed(g, True, sampler)
        clocks = sampler.summary()
        launches = g.launches() * args.steps
        e2e_dev_ms, e2e_wall_ms = timed(g_host, False)
        top1 = int(y_host.float().argmax(dim=1)[0])
        if abs(float(y_host.float().sum(dim=1).mean()) - 1.0) > 1e-2:
            raise RuntimeError("probabilities do not sum to one")
        e2e = {"value": total_images / (e2e_wall_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_wall_ms / args.steps, "device_ms_per_step": e2e_dev_ms / args.steps, "sub_batches": args.sub_batches,
               "h2d_gbs_per_rank": h2d / (e2e_wall_ms / args.steps * 1e-3) / 1e9, "executes_in_flight": 1,
               "timing": "wall clock around the synchronous odla_ExecuteComputation, max over ranks"}
        if ctx2 is not None:
            pipe_ms = timed_pipelined([g, ctx2], [(x_host, y_host), (x_host2, y_host2)])
            if not torch.equal(y_host, y_host2):
                raise RuntimeError("the two contexts disagree on the same input")
            e2e = {"value": total_images / (pipe_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                   "ms_per_step": pipe_ms / args.steps, "sub_batches": 1, "h2d_gbs_per_rank": h2d / (pipe_ms / args.steps * 1e-3) / 1e9,
                   "executes_in_flight": 2,
                   "timing": "wall clock over K steps issued with odla_AsyncExecuteComputation on two contexts of one computation (each step copies its "
                             "own input from pinned host memory and its result back; step i+1's input copy runs under step i's kernels), max over ranks",
                   "one_at_a_time": e2e}
        g.bind_input("input", x_dev.data_ptr())
        g.bind_output("prob", y_dev.data_ptr())
        prof = g.profile(runs=max(2, min(5, args.steps)))
        roof, families = tensor_roofline(prof, dev_ms / args.steps, peaks, peak_kind, clocks, int8, args.batch)
        g.close()
        if g_host is not g:
            g_host.close()
        return {"value": total_images / (dev_ms / 1e3), "ms_per_step": dev_ms / args.steps,
                "e2e": e2e,
                "gpu_launches": launches, "clocks": clocks, "roofline": roof, "families": families, "top1": top1}

    if args.only_int8:   # profiling aid: the int8 form alone, printed as a line of its own
        scales = rn.calibrate(w, n_images=8)
        r8 = measure(lambda g: rn.build_int8(g, BATCH, w, rn.quantize_weights(w), scales, input_type=odla.FLOAT16), "int8", True)
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": r8["value"], "unit": UNIT, "dtype": "s8", "config": {"workload": "resnet50_v1.5_nhwc_int8_b%d" % args.batch},
                              "ms_per_step": r8["ms_per_step"], "e2e": r8["e2e"], "roofline": r8["roofline"], "clocks": r8["clocks"]}))
        return
    fp16 = measure(lambda g: rn.build(g, BATCH, w, input_type=odla.FLOAT16), "fp16", False)
    int8 = None
    if not args.no_int8:
        scales = rn.calibrate(w, n_images=8)
        wq = rn.quantize_weights(w)
        r8 = measure(lambda g: rn.build_int8(g, BATCH, w, wq, scales, input_type=odla.FLOAT16), "int8", True)
        int8 = {"value": r8["value"], "unit": UNIT, "ms_per_step": r8["ms_per_step"], "dtype": "s8 (int32 accumulate; per-channel weight scales, per-tensor activation scales)",
                "e2e": r8["e2e"], "gpu_launches": r8["gpu_launches"], "clocks": r8["clocks"], "roofline": r8["roofline"], "kernel_families_share": r8["families"],
                "check": {"top1_of_first_image": r8["top1"]}}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not inlib:
        cpu = cpu_baseline_leg(pkg, rn, w)
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": fp16["value"], "unit": UNIT, "n_gpus": world * n_lib_gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": fp16["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": "resnet50_v1.5_nhwc_fp16_b%d" % args.batch, "batch_per_gpu": args.batch, "global_batch": BATCH * world, "input": "NHWC fp16 N(0,1)",
                       "weights": "He-normal, folded BN, random init", "l2": "256 MiB buffer written between steps",
                       "parallelism": ("one process, odla_ExecuteComputation shards dim 0 over %d GPUs" % inlib) if inlib else "dp%d (one process per GPU)" % world,
                       "timing": "CUDA events on the library's stream around each odla_ExecuteComputation, summed over the steps, max over ranks",
                       "host_affinity": numa},
            "e2e": fp16["e2e"], "gpu_launches": fp16["gpu_launches"], "clocks": fp16["clocks"], "roofline": fp16["roofline"],
            "kernel_families_share": fp16["families"], "int8": int8, "cpu_baseline": cpu, "check": {"top1_of_first_image": fp16["top1"]}}))


def run_ops(args, rank, world, local_rank):
    """The memory-bound kernels one at a time, each as a single-op ODLA graph at the shape it has in the ResNet-50 /
    YOLOv3 / BERT-base workloads: device-resident tensors, CUDA events around the kernel's own launch, achieved GB/s =
    algorithmic bytes (input + output, each once) / time against the measured copy bandwidth."""
    import torch
    pkg = importlib.import_module(PKG)
    odla = pkg.odla
    os.environ["ODLA_B200_DEVICE"] = str(local_rank)
    os.environ["ODLA_B200_NUM_GPUS"] = "1"
    torch.cuda.set_device(local_rank)
    lib = pkg.load()
    if lib.b200_DeviceCount() < 1:
        raise RuntimeError("bench.py needs a CUDA device: libodla_b200 has no CPU fallback")
    peaks, peak_kind = measured_peaks()
    hbm = float(peaks["hbm_gbs"])
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    F16, F32, I8, I32 = odla.FLOAT16, odla.FLOAT32, odla.INT8, odla.INT32
    NHWC = odla.CHANNELS_LAST
    tdt = {F16: torch.float16, F32: torch.float32, I8: torch.int8, I32: torch.int32}
    B = args.batch
    sc = lambda g: g.Constant("scale", np.array([0.05], np.float32))
    cases = [
        ("maxpool 3x3/2 [%d,112,112,64] f16" % B, "maxpool", True, [("x", (B, 112, 112, 64), F16)],
         lambda g, a: g.MaxPool(a[0], NHWC, (3, 3), (2, 2), (1, 1), (1, 1), (B, 56, 56, 64), "y")),
        ("maxpool 3x3/2 [%d,112,112,64] s8" % B, "maxpool", False, [("x", (B, 112, 112, 64), I8)],
         lambda g, a: g.MaxPool(a[0], NHWC, (3, 3), (2, 2), (1, 1), (1, 1), (B, 56, 56, 64), "y")),
        ("reduce_mean (1,2) [%d,7,7,2048] f16" % B, "reduce_mean", True, [("x", (B, 7, 7, 2048), F16)],
         lambda g, a: g.ReduceMean(a[0], (1, 2), True, (B, 1, 1, 2048), "y")),
        ("dequantize+reduce_mean (1,2) [%d,7,7,2048] s8" % B, "reduce_mean", False, [("x", (B, 7, 7, 2048), I8)],
         lambda g, a: g.ReduceMean(g.Dequantize(a[0], sc(g), None, 0, F32, "xd"), (1, 2), True, (B, 1, 1, 2048), "y")),
        ("softmax rows [%d,128] f16 (BERT scores, B=%d)" % (B // 4 * 12 * 128, B // 4), "softmax", True, [("x", (B // 4 * 12 * 128, 128), F16)],
         lambda g, a: g.Softmax(a[0], -1, "y")),
        ("softmax rows [%d,1000] f32 (classifier)" % B, "softmax", False, [("x", (B, 1000), F32)], lambda g, a: g.Softmax(a[0], -1, "y")),
        ("layernorm rows [%d,768] f16 (BERT, B=%d)" % (B // 4 * 128, B // 4), "layernorm", True, [("x", (B // 4 * 128, 768), F16)],
         lambda g, a: g.LayerNorm(a[0], (-1,), 1e-12, g.Constant("g", np.ones(768, np.float32)), g.Constant("b", np.zeros(768, np.float32)), "y")),
        ("quantize f16->s8 [%d,224,224,3]" % B, "quantize", False, [("x", (B, 224, 224, 3), F16)], lambda g, a: g.Quantize(a[0], sc(g), None, 0, I8, "y")),
        ("dequantize s8->f32 [%d,56,56,256]" % (B // 4), "dequantize", False, [("x", (B // 4, 56, 56, 256), I8)], lambda g, a: g.Dequantize(a[0], sc(g), None, 0, F32, "y")),
        ("resize nearest x2 [%d,26,26,256] f16 (YOLOv3, B=%d)" % (B // 4, B // 4), "resize", True, [("x", (B // 4, 26, 26, 256), F16)],
         lambda g, a: g.Resize(a[0], (B // 4, 52, 52, 256), "y")),
        ("concat channels [%d,52,52,128+256] f16 (YOLOv3)" % (B // 4), "concat", True, [("a", (B // 4, 52, 52, 128), F16), ("b", (B // 4, 52, 52, 256), F16)],
         lambda g, a: g.Concat([a[0], a[1]], 3, (B // 4, 52, 52, 384), "y")),
        ("gather rows [30522,768]->[%d,768] f16 (BERT embedding)" % (B // 4 * 128), "gather", True, [("ids", (B // 4, 128), I32)],
         lambda g, a: g.Gather(g.Constant("emb", (np.arange(30522 * 768, dtype=np.float32) % 97).astype(np.float16).reshape(30522, 768)), a[0], 0, (B // 4, 128, 768), "y")),
        ("transpose (0,2,1,3) [%d,128,12,64] f16 (BERT heads)" % (B // 4), "transpose", True, [("x", (B // 4, 128, 12, 64), F16)],
         lambda g, a: g.Transpose(a[0], (0, 2, 1, 3), (B // 4, 12, 128, 64), "y")),
        ("add same shape [%d,56,56,256] f16" % (B // 4), "binary", True, [("a", (B // 4, 56, 56, 256), F16), ("b", (B // 4, 56, 56, 256), F16)],
         lambda g, a: g.Add(a[0], a[1], "y")),
    ]
    rows = []
    for title, op, fp16, arg_specs, build in cases:
        g = odla.Graph(lib, "op", fp16=fp16, n_gpus=1)
        a = [g.Argument(n, shp, dt) for n, shp, dt in arg_specs]
        out = build(g, a)
        # the output keeps the storage type so that no conversion kernel runs: declare it in that type
        g.Output(out)
        ins = {n: (torch.randint(0, 30522, shp, dtype=torch.int32, device="cuda") if dt == I32 else
                   torch.randint(-100, 100, shp, dtype=torch.int8, device="cuda") if dt == I8 else torch.randn(shp, device="cuda").to(tdt[dt])) for n, shp, dt in arg_specs}
        on = g.out_names[0]
        y = torch.empty(g.shapes[on], dtype=tdt[g.dtypes[on]], device="cuda")
        for n, t in ins.items():
            g.bind_input(n, t.data_ptr())
        g.bind_output(on, y.data_ptr())
        ms, prof, other = [], [], []
        for i in range(args.warmup + args.steps):
            flush.zero_()
            torch.cuda.synchronize()
            entries = g.profile(runs=1)      # plain launches, each bracketed by CUDA events on the library's stream
            prof = [q for q in entries if q["op"] == op]
            other = [q["op"] for q in entries if q["op"] != op]
            if i >= args.warmup:
                ms.append(sum(q["ms"] for q in prof))
        g.close()
        t = sorted(ms)[len(ms) // 2]
        nbytes = sum(q["bytes"] for q in prof)
        rows.append({"kernel": title, "launch_op": op, "other_launches": other, "ms": round(t, 5), "algorithmic_mb": round(nbytes / 1e6, 2),
                     "gbs": round(nbytes / (t * 1e-3) / 1e9, 1), "frac_of_hbm": round(nbytes / (t * 1e-3) / 1e9 / hbm, 3)})
    if rank == 0:
        print(json.dumps({"metric": "memory_bound_kernels_achieved_bandwidth", "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                          "peak": hbm, "peak_source": peak_kind + " copy bandwidth", "data": "synthetic",
                          "config": {"workload": "single-op graphs at the shapes of the ResNet-50 (B=%d) / YOLOv3 / BERT-base workloads" % B,
                                     "timing": "CUDA events around the kernel's launch(es) on the library's stream, median; 256 MiB L2 flush before each execute (the execute's own device-to-device copy of the bound input into the arena then leaves up to 126 MB of it in L2)"},
                          "kernels": rows}))


def run_secondary(args, rank, world, local_rank):
    """The other two networks (YOLOv3-416, BERT-base S=128) through the same path and timing
    method as the ResNet-50 line: fp16 storage, device-resident `value`, host-bound `e2e`, tensor-core roofline."""
    import torch
    pkg = importlib.import_module(PKG)
    odla = pkg.odla
    os.environ["ODLA_B200_DEVICE"] = str(local_rank)
    os.environ["ODLA_B200_NUM_GPUS"] = "1"
    torch.cuda.set_device(local_rank)
    lib = pkg.load()
    if lib.b200_DeviceCount() < 1:
        raise RuntimeError("bench.py needs a CUDA device: libodla_b200 has no CPU fallback")
    if args.workload == "yolov3":
        m = importlib.import_module(PKG + ".halo_models.yolov3")
        batch = args.batch if args.batch != BATCH else 16
        w = m.weights()
        x_np = m.inputs(batch)
        build = lambda g: m.build(g, batch, w)
        unit, metric, mac, name = "img/s", "yolov3_416_inference_throughput", m.MAC_PER_IMAGE_416, "yolov3_416_nhwc_fp16_b%d" % batch
    else:
        m = importlib.import_module(PKG + ".halo_models.bert")
        batch = args.batch if args.batch != BATCH else 64
        w = m.weights(m.BASE)
        x_np = m.inputs(m.BASE, batch)
        build = lambda g: m.build(g, batch, m.BASE, w)
        unit, metric, mac, name = "seq/s", "bert_base_s128_encoder_throughput", m.MAC_PER_SEQUENCE_BASE, "bert_base_s128_fp16_b%d" % batch
    g = odla.Graph(lib, args.workload, fp16=True, n_gpus=1)
    build(g)
    g.context()
    ctx2 = g.extra_context() if args.contexts > 1 else None   # a second context (own lane) for the pipelined end-to-end leg
    g_host = odla.Graph(lib, args.workload + "_host", fp16=True, n_gpus=1, sub_batches=args.sub_batches)
    build(g_host)
    g_host.context()
    x_host = {k: torch.from_numpy(v).pin_memory() for k, v in x_np.items()}
    x_dev = {k: v.cuda() for k, v in x_host.items()}
    np_dt = {odla.FLOAT32: torch.float32, odla.FLOAT16: torch.float16, odla.INT32: torch.int32, odla.INT8: torch.int8}
    y_host = {n: torch.empty(g.shapes[n], dtype=np_dt[g.dtypes[n]]).pin_memory() for n in g.out_names}
    y_dev = {n: torch.empty(g.shapes[n], dtype=np_dt[g.dtypes[n]], device="cuda") for n in g.out_names}
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    h2d = sum(v.numel() * v.element_size() for v in x_host.values())
    d2h = sum(v.numel() * v.element_size() for v in y_host.values())

    def timed(gg, xs, ys, sampler=None):
        for k, v in xs.items():
            gg.bind_input(k, v.data_ptr())
        for k, v in ys.items():
            gg.bind_output(k, v.data_ptr())

        def step():
            flush.zero_()
            torch.cuda.synchronize()
            if gg.execute() != 0:
                raise RuntimeError("odla_ExecuteComputation failed")
            return gg.device_ms()
        for _ in range(args.warmup):
            step()
        barrier()
        if sampler:
            sampler.start()
        ms = sum(step() for _ in range(args.steps))
        barrier()
        return max_over_ranks(ms)

    def timed_pipelined(ctxs, bufs):
        """K steps with two executes in flight (odla_AsyncExecuteComputation on two contexts of one computation), every
        step copying its own inputs from pinned host memory and its outputs back; wall clock, max over ranks."""
        for c, (xs, ys) in zip(ctxs, bufs):
            for k, v in xs.items():
                c.bind_input(k, v.data_ptr())
            for k, v in ys.items():
                c.bind_output(k, v.data_ptr())

        def run(n):
            for i in range(n):
                c = ctxs[i % len(ctxs)]
                if c.wait() != 0 or c.execute_async() != 0:
                    raise RuntimeError("asynchronous execute failed")
            for c in ctxs:
                if c.wait() != 0:
                    raise RuntimeError("asynchronous execute failed")
        run(max(args.warmup, len(ctxs)))
        barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        run(args.steps)
        wall = (time.perf_counter() - t0) * 1e3
        barrier()
        return max_over_ranks(wall)

    sampler = ClockSampler(local_rank)
    dev_ms = timed(g, x_dev, y_dev, sampler)
    clocks = sampler.summary()
    launches = g.launches() * args.steps
    e2e_ms = timed(g_host, x_host, y_host)
    total = sum_over_ranks(batch * args.steps)
    e2e = {"value": total / (e2e_ms / 1e3), "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps,
           "sub_batches": args.sub_batches, "executes_in_flight": 1}
    if ctx2 is not None:
        x_host2 = {k: v.clone().pin_memory() for k, v in x_host.items()}
        y_host2 = {k: torch.empty_like(v).pin_memory() for k, v in y_host.items()}
        pipe_ms = timed_pipelined([g, ctx2], [(x_host, y_host), (x_host2, y_host2)])
        for k in y_host:
            if not torch.equal(y_host[k], y_host2[k]):
                raise RuntimeError("the two contexts disagree on the same input")
        e2e = {"value": total / (pipe_ms / 1e3), "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": pipe_ms / args.steps,
               "sub_batches": 1, "executes_in_flight": 2, "one_at_a_time": e2e}
    prof = g.profile(runs=2)
    tc = [q for q in prof if q["op"].endswith("_umma") or q["op"] == "attention"]   # every launch that runs on the tensor cores
    tc_ms, tc_flops = sum(q["ms"] for q in tc), sum(q["flops"] for q in tc)
    all_ms = sum(q["ms"] for q in prof)
    peaks, peak_kind = measured_peaks()
    peak = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops")))
    achieved = tc_flops / (tc_ms * 1e-3) / 1e12 if tc_ms else 0.0
    fam = {}
    for q in prof:
        f = fam.setdefault(q["op"], {"launches": 0, "ms": 0.0})
        f["launches"] += 1
        f["ms"] = round(f["ms"] + q["ms"], 4)
    int8 = None
    if args.workload == "bert" and not args.no_int8:
        # the same encoder in its int8-GEMM form (Quantize / Dequantize around the six dense layers of every block,
        # soft-max / LayerNorm / attention products in fp16), device-resident
        q = m.quantize(m.BASE, w, n_sequences=2)
        g8 = odla.Graph(lib, "bert_int8", fp16=True, n_gpus=1)
        m.build(g8, batch, m.BASE, w, quant=q)
        g8.context()
        ms8 = timed(g8, x_dev, y_dev)
        prof8 = g8.profile(runs=2)
        fam8 = {}
        for q8 in prof8:
            f = fam8.setdefault(q8["op"], {"launches": 0, "ms": 0.0})
            f["launches"] += 1
            f["ms"] = round(f["ms"] + q8["ms"], 4)
        int8 = {"value": total / (ms8 / 1e3), "unit": unit, "ms_per_step": ms8 / args.steps, "dtype": "s8 GEMMs (int32 accumulate), f16 elsewhere",
                "kernel_families_ms_per_step": dict(sorted(fam8.items(), key=lambda kv: -kv[1]["ms"]))}
        g8.close()
    if rank == 0:
        print(json.dumps({
            "int8": int8,
            "metric": metric, "value": total / (dev_ms / 1e3), "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": name, "batch_per_gpu": batch, "l2": "256 MiB buffer written between steps", "parallelism": "dp%d" % world,
                       "work_per_unit_gflop": 2 * mac / 1e9},
            "e2e": e2e,
            "gpu_launches": launches, "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "umma_conv_kernel / attn_kernel (%d tensor-core launches per step)" % len(tc), "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak if peak else None, "peak_source": peak_kind + " bf16 sustained", "share_of_step": tc_ms / max(all_ms, 1e-9),
                         "traffic": None},
            "kernel_families_ms_per_step": dict(sorted(fam.items(), key=lambda kv: -kv[1]["ms"])),
            "cpu_baseline": None}))
    g.close()
    g_host.close()

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-int8", action="store_true", help="skip the secondary int8 measurement")
    ap.add_argument("--only-int8", action="store_true", help="measure only the int8 form (for profiling one of its kernels)")
    ap.add_argument("--workload", default="resnet50", choices=["resnet50", "yolov3", "bert", "ops"],
                    help="resnet50 is the benchmark line; yolov3 (B=16) and bert (B=64) are the other two networks; ops times every memory-bound kernel on its own")
    ap.add_argument("--sub-batches", type=int, default=2, help="ODLA_BATCHES_PER_STEP of the end-to-end (host-bound) leg; 1 = off")
    ap.add_argument("--contexts", type=int, default=2, choices=[1, 2],
                    help="executes in flight in the end-to-end leg: 2 = two contexts driven with odla_AsyncExecuteComputation (the one-at-a-time figure is reported beside it)")
    ap.add_argument("--batch", type=int, default=BATCH, help="images per GPU per step (256 = the benchmark configuration; smaller values are for profiling)")
    ap.add_argument("--inlib-gpus", type=int, default=0, help="single process: one odla_ExecuteComputation shards a batch of N x --batch images over N GPUs inside the library")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else max(args.warmup, 1)
    rank, world, local_rank = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.workload == "resnet50":
            run_b200(args, rank, world, local_rank)
        elif args.workload == "ops":
            run_ops(args, rank, world, local_rank)
        else:
            run_secondary(args, rank, world, local_rank)
    finally:
        d = _dist()
        if d is not None:
            d.destroy_process_group()


if __name__ == "__main__":
    main()
