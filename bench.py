#!/usr/bin/env python
"""ResNet-50 v1.5 inference throughput through the ODLA C ABI of libodla_b200.so.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun, one rank per GPU)
    python bench.py --impl reference ...                      (the reference's CPU kernels on the host cores)

One step = one odla_ExecuteComputation over a batch of 256 synthetic NHWC fp16 images (BASELINE
config 2).  `value` is measured with the inputs already resident in HBM (device pointers bound),
`e2e` with pinned host buffers bound, so the host-to-device copy of the images and the
device-to-host copy of the probabilities are inside the timed region.  Times come from CUDA events
recorded by the library on the stream its kernels run on; multi-rank numbers take the maximum over
ranks.  Each rank owns one GPU and a full copy of the weights; there is no collective on the data
path (weak scaling).
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
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag = index, [], threading.Event()

    def run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                f = [x.strip() for x in out.split(",")]
                if len(f) >= 7:
                    self.samples.append(f)
            except Exception:
                pass
            self.stop_flag.wait(0.2)

    def summary(self):
        self.stop_flag.set()
        self.join(timeout=6)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = sorted(float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit())
        reasons = []
        for i, name in enumerate(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]):
            if any(s[3 + i].lower().startswith("active") for s in self.samples):
                reasons.append(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": float(self.samples[0][1]) if self.samples[0][1].replace(".", "").isdigit() else None,
                "reasons": reasons, "samples": len(self.samples)}


# ------------------------------------------------------------------- the two arms ----
def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def run_reference(args, rank, world):
    """The reference's own CPU kernels (runtime/generic, compiled into oracle/_ref) driven through
    the oracle ODLA platform on every host thread; a bounded sample of the workload per step."""
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

    def make(batch):
        g = odla.Graph(ref, "resnet50")
        rn.build(g, batch, w)
        return g, rn.inputs(batch, seed=11)

    # One image per host thread runs each image through the reference's scalar kernels; if that
    # cannot finish in a few minutes fall back to one image split by output rows over the threads.
    sample = cores if kind == "reference" else 1
    g, x = make(sample)
    t0 = time.time()
    g.run(x)
    first = time.time() - t0
    budget = 200.0
    if first * (args.steps + args.warmup) > budget and sample > 1:
        g.close()
        sample = 1
        os.environ["ODLA_CPUREF_NO_REFLIB"] = "1"
        g, x = make(sample)
        kind = "port"
    for _ in range(max(args.warmup - 1, 0)):
        g.run(x)
    t0 = time.time()
    for _ in range(args.steps):
        g.run(x)
    dt = time.time() - t0
    g.close()
    value = sample * args.steps / dt
    desc = "%d image(s) of the 256-image batch per step, fp32, %s kernels on %d host threads" % (sample, "runtime/generic" if kind == "reference" else "restated", cores)
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                      "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                      "data": "synthetic", "config": {"workload": "resnet50_v1.5_nhwc_b256", "sample_images_per_step": sample},
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
    return {"value": sample * n / dt, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": "%d pass(es) over %d images (fp32, one image per host thread)" % (n, sample)}


def run_b200(args, rank, world, local_rank):
    import torch
    pkg = importlib.import_module(PKG)
    odla = pkg.odla
    rn = importlib.import_module(PKG + ".halo_models.resnet50")
    os.environ["ODLA_B200_DEVICE"] = str(local_rank)
    os.environ["ODLA_B200_NUM_GPUS"] = "1"
    torch.cuda.set_device(local_rank)
    lib = pkg.load()
    if lib.b200_DeviceCount() < 1:
        raise RuntimeError("bench.py needs a CUDA device: libodla_b200 has no CPU fallback")
    w = rn.weights()
    BATCH = args.batch
    g = odla.Graph(lib, "resnet50", fp16=True, n_gpus=1)
    rn.build(g, BATCH, w, input_type=odla.FLOAT16)
    x_host = torch.from_numpy(rn.inputs(BATCH, seed=rank_seed(10 + BATCH, rank), dtype=np.float16)["input"]).pin_memory()
    y_host = torch.empty((BATCH, 1000), dtype=torch.float32).pin_memory()
    x_dev = x_host.cuda()
    y_dev = torch.empty((BATCH, 1000), dtype=torch.float32, device="cuda")
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")   # larger than the 126 MB L2
    h2d, d2h = x_host.numel() * 2, y_host.numel() * 4

    # The end-to-end leg binds host buffers; there the library pipelines the batch over sub-batches
    # (ODLA_BATCHES_PER_STEP) so that one sub-batch's input copy runs under another's kernels.
    g.context()   # odla_CreateContext attaches to the most recently created computation: make it now
    g_host = g
    if args.sub_batches > 1:
        g_host = odla.Graph(lib, "resnet50_host", fp16=True, n_gpus=1, sub_batches=args.sub_batches)
        rn.build(g_host, BATCH, w, input_type=odla.FLOAT16)
        g_host.context()

    def bind(device_resident):
        gg = g if device_resident else g_host
        gg.bind_input("input", x_dev.data_ptr() if device_resident else x_host.data_ptr())
        gg.bind_output("prob", y_dev.data_ptr() if device_resident else y_host.data_ptr())
        return gg

    def step(gg):
        flush.zero_()
        torch.cuda.synchronize()
        st = gg.execute()
        if st != 0:
            raise RuntimeError("odla_ExecuteComputation failed with status %d" % st)
        return gg.device_ms()

    def timed(device_resident, sampler=None):
        gg = bind(device_resident)
        for _ in range(args.warmup):
            step(gg)
        barrier()
        torch.cuda.synchronize()
        if sampler:
            sampler.start()
        t0 = time.time()
        ms = sum(step(gg) for _ in range(args.steps))
        torch.cuda.synchronize()
        wall = time.time() - t0
        barrier()
        return max_over_ranks(ms), max_over_ranks(wall * 1e3)

    sampler = ClockSampler(local_rank)
    dev_ms, wall_ms = timed(True, sampler)
    clocks = sampler.summary()
    launches = g.launches() * args.steps
    e2e_ms, _ = timed(False)
    total_images = sum_over_ranks(BATCH * args.steps)
    value = total_images / (dev_ms / 1e3)
    e2e_value = total_images / (e2e_ms / 1e3)
    top1 = int(y_host.argmax(dim=1)[0])

    # per-kernel durations: a pass with every launch bracketed by CUDA events on the library's stream
    bind(True)
    prof = g.profile(runs=max(2, min(5, args.steps)))
    fam = {}
    for p in prof:
        f = fam.setdefault(p["op"], {"launches": 0, "ms": 0.0, "flops": 0.0, "bytes": 0.0})
        f["launches"] += 1
        f["ms"] += p["ms"]
        f["flops"] += p["flops"]
        f["bytes"] += p["bytes"]
    tc = [f for k, f in fam.items() if k.endswith("_umma")]
    tc_ms = sum(f["ms"] for f in tc)
    tc_flops = sum(f["flops"] for f in tc)
    tc_launches = sum(f["launches"] for f in tc)
    peaks, peak_kind = measured_peaks()
    peak = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops")))
    achieved = tc_flops / (tc_ms * 1e-3) / 1e12 if tc_ms > 0 else 0.0
    roofline = {"bound": "tensor", "kernel": "umma_conv_kernel (tcgen05 implicit-GEMM conv / GEMM, %d launches per step)" % tc_launches,
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak if peak else None, "peak_source": peak_kind + " bf16 sustained",
                "avg_launch_ms": tc_ms / max(tc_launches, 1), "share_of_step": tc_ms / max(sum(f["ms"] for f in fam.values()), 1e-9),
                # dram__bytes_read.sum + dram__bytes_write.sum of this kernel, average per launch: one ncu capture of all 54
                # launches at B=128 (5.321 GB; activations already exceed the 126 MB L2 there), scaled by 2 to B=256.
                "traffic": 1.9707e8 * (BATCH / 256.0), "traffic_unit": "bytes per launch (54 launches per step)",
                "algorithmic_bytes_per_launch": sum(f["bytes"] for f in tc) / max(tc_launches, 1),
                "hbm_view": {"achieved_gbs": sum(f["bytes"] for f in tc) / (tc_ms * 1e-3) / 1e9 if tc_ms > 0 else 0.0, "peak_gbs": float(peaks.get("hbm_gbs", 0))}}
    families = {k: {"launches": v["launches"], "ms": round(v["ms"], 4)} for k, v in sorted(fam.items(), key=lambda kv: -kv[1]["ms"])}
    g.close()

    # Secondary measurement: the same network in int8 quantise/dequantise form (BASELINE config 3),
    # device-resident fp32 input, same timing method.  int8 tensor peak is taken as 2x the measured bf16 figure.
    int8 = None
    if not args.no_int8:
        scales = rn.calibrate(w, n_images=8)
        wq = rn.quantize_weights(w)
        g8 = odla.Graph(lib, "resnet50_int8", n_gpus=1)
        rn.build_int8(g8, BATCH, w, wq, scales)
        x8 = x_host.float().cuda()
        g8.bind_input("input", x8.data_ptr())
        g8.bind_output("prob", y_dev.data_ptr())

        def step8():
            flush.zero_()
            torch.cuda.synchronize()
            if g8.execute() != 0:
                raise RuntimeError("int8 execute failed")
            return g8.device_ms()
        for _ in range(args.warmup):
            step8()
        barrier()
        ms8 = max_over_ranks(sum(step8() for _ in range(args.steps)))
        prof8 = g8.profile(runs=2)
        tc8 = [q for q in prof8 if q["op"].endswith("_umma")]
        tc8_ms, tc8_ops = sum(q["ms"] for q in tc8), sum(q["flops"] for q in tc8)
        int8 = {"value": total_images / (ms8 / 1e3), "unit": UNIT, "ms_per_step": ms8 / args.steps, "dtype": "s8 (int32 accumulate)",
                "roofline": {"bound": "tensor", "achieved": tc8_ops / (tc8_ms * 1e-3) / 1e12 if tc8_ms else 0.0, "peak": 2 * peak, "unit": "TOP/s",
                             "frac": (tc8_ops / (tc8_ms * 1e-3) / 1e12) / (2 * peak) if tc8_ms else None, "peak_source": "2 x " + peak_kind + " bf16 sustained (no int8 measurement available)"}}
        g8.close()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_leg(pkg, rn, w)
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "wall_ms_per_step": wall_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": "resnet50_v1.5_nhwc_fp16_b%d" % BATCH, "batch_per_gpu": BATCH, "global_batch": BATCH * world, "input": "NHWC fp16 N(0,1)",
                       "weights": "He-normal, folded BN, random init", "l2": "256 MiB buffer written between steps", "parallelism": "dp%d" % world,
                       "timing": "CUDA events on the library's stream around each odla_ExecuteComputation, summed over the steps, max over ranks"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps,
                    "sub_batches": args.sub_batches},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "kernel_families_ms_per_step": families,
            "int8": int8, "cpu_baseline": cpu, "check": {"top1_of_first_image": top1}}))



def run_secondary(args, rank, world, local_rank):
    """The other BASELINE configurations (YOLOv3-416, BERT-base S=128) through the same path and timing
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

    sampler = ClockSampler(local_rank)
    dev_ms = timed(g, x_dev, y_dev, sampler)
    clocks = sampler.summary()
    launches = g.launches() * args.steps
    e2e_ms = timed(g_host, x_host, y_host)
    total = sum_over_ranks(batch * args.steps)
    prof = g.profile(runs=2)
    tc = [q for q in prof if q["op"].endswith("_umma")]
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
    if rank == 0:
        print(json.dumps({
            "metric": metric, "value": total / (dev_ms / 1e3), "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": name, "batch_per_gpu": batch, "l2": "256 MiB buffer written between steps", "parallelism": "dp%d" % world,
                       "work_per_unit_gflop": 2 * mac / 1e9},
            "e2e": {"value": total / (e2e_ms / 1e3), "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps,
                    "sub_batches": args.sub_batches},
            "gpu_launches": launches, "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "umma_conv_kernel (%d launches per step)" % len(tc), "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
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
    ap.add_argument("--workload", default="resnet50", choices=["resnet50", "yolov3", "bert"],
                    help="resnet50 is the benchmark line; yolov3 (B=16) and bert (B=64) are the secondary BASELINE configurations")
    ap.add_argument("--sub-batches", type=int, default=2, help="ODLA_BATCHES_PER_STEP of the end-to-end (host-bound) leg; 1 = off")
    ap.add_argument("--batch", type=int, default=BATCH, help="images per GPU per step (256 = the benchmark configuration; smaller values are for profiling)")
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
        else:
            run_secondary(args, rank, world, local_rank)
    finally:
        d = _dist()
        if d is not None:
            d.destroy_process_group()


if __name__ == "__main__":
    main()
