"""Throughput of the fused 1080p -> 224x224 pre-processing path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Workload (per GPU): the classification pre-processing batch -- 256 uint8 NHWC 1080x1920x3 images (seeded uniform
bytes, synthetic) -> bilinear resize to 256x256 -> centre crop 224x224 -> per-channel (v - mean) * (1/std) ->
float32 NCHW. One step = one pass over the batch = one fused kernel launch. The batch (1.59 GB) is far larger
than the 126 MB L2, so every step reads its source rows from HBM; no flush is needed between steps.

One JSON line is printed by rank 0. `value` = images/s with inputs resident in HBM (device-timed with CUDA
events on the launching stream, max over ranks). `e2e` = the same metric from page-locked HOST buffers to a
page-locked HOST result through the library's C entry point, transfers inside the timed region. `roofline` relates
the kernel's algorithmic bytes to the measured HBM copy bandwidth of this pool. `cpu_baseline` times the CPU
checker on a bounded sample on this box's host cores.

`--impl reference` times the reference's own CPU implementation of the path (its golden functions compiled into
oracle/_ref when available, else the C restatement) on all host cores; under torchrun only rank 0 runs it.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "images/sec, 1080p->224x224 fused preproc (resize 256 bilinear, crop 224, mean/std, f32 NCHW)"
UNIT = "images/s"
BATCH = 256
SRC_H, SRC_W = 1080, 1920
RESIZE = (256, 256)
CROP = (16, 16)
OUT = (224, 224)
MEAN = (123.675, 116.28, 103.53)
STD = (58.395, 57.12, 57.375)
# Algorithmic bytes per image: distinct 32-byte source sectors tapped (448 rows x 5056 B = 2,265,088 B, computed by
# oracle_resize_source_bytes and pinned by a CPU test) + the float32 NCHW output (3*224*224*4 = 602,112 B).
ALG_SRC_BYTES = 2265088
ALG_OUT_BYTES = 3 * 224 * 224 * 4
ALG_BYTES = ALG_SRC_BYTES + ALG_OUT_BYTES
# DRAM traffic per image of the staged kernel from the ncu capture summarised in
# profiles/resize_staged_linear_f32_1080p_to_224.md (full-size launch of 256 images, one-pass capture).
NCU_TRAFFIC_BYTES_PER_IMAGE = 736304128 / 256
FALLBACK_HBM_GBS = 6650.0


def inv_std():
    import numpy as np
    return tuple(float(np.float32(1.0) / np.float32(s)) for s in STD)


def workload_config(n_gpus: int) -> dict:
    return {
        "workload": "classification preproc, dense batch: 256 x 1080x1920x3 u8 NHWC per GPU -> resize 256x256 "
                    "linear -> crop 224x224 @ (16,16) -> (v-mean)*(1/std) per channel -> f32 NCHW",
        "images_per_gpu": BATCH, "global_batch": BATCH * n_gpus, "sharding": f"by sample, {n_gpus} x {BATCH}",
        "collective": "none", "l2": "input 1.59 GB per GPU >> 126 MB L2, no flush needed",
        "src_cast": False,
    }


# ------------------------------------------------------------------------------------------------ clocks

class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------ CPU legs

def cpu_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def time_cpu(images_total: int, repeats: int, warm: int = 0):
    """Times the CPU implementation of the workload on `images_total` images with every host thread.
    Returns (images_per_second_list, kind, cores, description)."""
    import numpy as np
    from oracle import oracle as O  # the checker, timed here as the CPU baseline -- never on the product path

    threads = cpu_threads()
    rng = np.random.default_rng(1234)
    src = rng.integers(0, 256, (images_total, SRC_H, SRC_W, 3), dtype=np.uint8)
    ref = O.ref()
    rates = []
    if ref is not None:
        # The reference's own golden function. It has one scalar scale/offset pair (its operator cannot express
        # per-channel constants), so channel 0's constants stand in: same taps, same operation count.
        kind = "reference"
        scale, offset = 1.0 / STD[0], -MEAN[0] / STD[0]
        from concurrent.futures import ThreadPoolExecutor
        bounds = [(images_total * t // threads, images_total * (t + 1) // threads) for t in range(threads)]
        bounds = [b for b in bounds if b[1] > b[0]]

        def work(b):
            O.ref_rccr(src[b[0]:b[1]], RESIZE, CROP, OUT, 1, 0, scale, offset, False, np.float32, True)

        with ThreadPoolExecutor(max_workers=len(bounds)) as ex:
            for i in range(warm + repeats):
                t0 = time.perf_counter()
                list(ex.map(work, bounds))
                dt = time.perf_counter() - t0
                if i >= warm:
                    rates.append(images_total / dt)
        what = "reference golden ResizeCropConvert (tests/cvcuda/system/TestOpResizeCropConvertReformat.cpp:76-172), " \
               "scalar scale/offset of channel 0"
    else:
        kind = "port"
        spec = O.ResizeSpec(resize=RESIZE, crop=CROP, out_size=OUT, interp=O.LINEAR, src_cast=False, base=MEAN,
                            mul=inv_std())
        imgs = list(src)
        for i in range(warm + repeats):
            t0 = time.perf_counter()
            O.resize_crop(imgs, spec, np.float32, True, nthreads=threads)
            dt = time.perf_counter() - t0
            if i >= warm:
                rates.append(images_total / dt)
        what = "C restatement of the reference golden (oracle/preproc_oracle.c)"
    sample = f"{images_total} of the {BATCH} images per pass, {repeats} timed passes, {threads} threads; {what}"
    return rates, kind, threads, sample


def run_reference(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = cpu_threads()
    images = max(threads * 4, 32)  # one step = a bounded sample of the batch, a few images per thread
    t0 = time.perf_counter()
    rates, kind, cores, sample = time_cpu(images, args.steps, warm=args.warmup)
    value = statistics.mean(rates)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 * images / value, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------------ GPU arm

def run_native(args) -> int:
    import numpy as np
    import torch
    import torch.distributed as dist

    import __graft_entry__ as ge

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = ge.load_package()  # raises when libcvcuda_b200.so is missing: there is no fallback path

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        return pkg.sharding.max_over_ranks(ms, dev)

    # seeded synthetic batch, generated on the device (each rank its own shard of the global batch)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    src = torch.randint(0, 256, (BATCH, SRC_H, SRC_W, 3), dtype=torch.uint8, device=dev, generator=gen)
    out = torch.empty((BATCH, 3, OUT[1], OUT[0]), dtype=torch.float32, device=dev)
    mul = inv_std()

    def step(dst, source):
        pkg.fused_preprocess_into(dst, source, resize_dim=RESIZE, interp=pkg.Interp.LINEAR, crop_pos=CROP, layout="NCHW",
                                  base=MEAN, mul=mul, srcCast=False)

    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()

    # ---- device-resident throughput
    for _ in range(max(args.warmup, 3)):
        step(out, src)
    barrier()
    launches0 = pkg.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(out, src)
    e1.record()
    barrier()
    launches = pkg.launch_count() - launches0
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_per_step = ms_total / args.steps
    value = world * BATCH * args.steps / (ms_total / 1000.0)
    if pkg.read_device_error() != 0:
        raise RuntimeError("device error word set: a kernel gave up on a bounded wait")

    # ---- end to end from page-locked host memory to a page-locked host result
    host_src = torch.empty((BATCH, SRC_H, SRC_W, 3), dtype=torch.uint8).pin_memory()
    host_src.copy_(src.cpu())
    host_out = torch.empty((BATCH, 3, OUT[1], OUT[0]), dtype=torch.float32).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_copy_step():
        # whole batch host -> device, fused kernel, result device -> host
        src.copy_(host_src, non_blocking=True)
        step(out, src)
        host_out.copy_(out, non_blocking=True)

    def e2e_direct_step():
        # the kernel pulls only the source rows it taps straight out of the page-locked host buffer
        # (bulk copies into shared memory), result device -> host
        step(out, host_src)
        host_out.copy_(out, non_blocking=True)

    def e2e_zero_copy_step():
        # one launch and nothing else: tapped source rows come in over PCIe by bulk copy, result rows go out as
        # full-line stores into the page-locked host result
        step(host_out, host_src)

    e2e_modes = {"h2d_copy+kernel+d2h": (e2e_copy_step, host_src.numel()),
                 "kernel reads pinned host rows directly + d2h": (e2e_direct_step, ALG_SRC_BYTES * BATCH),
                 "kernel reads pinned host rows and writes the pinned host result": (e2e_zero_copy_step,
                                                                                    ALG_SRC_BYTES * BATCH)}
    e2e_results = {}
    for name, (fn, h2d_bytes) in e2e_modes.items():
        for _ in range(2):
            fn()
        barrier()
        e0.record()
        for _ in range(e2e_steps):
            fn()
        e1.record()
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1))
        e2e_results[name] = {"value": world * BATCH * e2e_steps / (ms / 1000.0), "ms_per_step": ms / e2e_steps,
                             "h2d_bytes_per_step": int(h2d_bytes)}
    if pkg.read_device_error() != 0:
        raise RuntimeError("device error word set during the end-to-end runs")
    check = host_out[:2].numpy().copy()
    best = max(e2e_results, key=lambda k: e2e_results[k]["value"])

    # ---- the reference project's own CUDA kernel (compiled for sm_100a from the reference sources into oracle/_ref),
    # same GPU, same source batch: a reported baseline, like the CPU one. Its operator has one scalar scale/offset, so
    # channel 0's constants stand in and the per-channel Normalize pass its pipeline would still need is not timed.
    ref_cuda = None
    if rank == 0:
        from oracle import ref_cuda as RC
        if RC.lib() is not None:
            out_ref = torch.empty_like(out)
            n_ref = max(3, min(args.steps, 50))

            def ref_step():
                RC.rccr_tensor(src, out_ref, True, RESIZE, 1, CROP, 0, mul[0], -MEAN[0] * mul[0], False)

            for _ in range(3):
                ref_step()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(n_ref):
                ref_step()
            e1.record()
            torch.cuda.synchronize()
            ref_ms = e0.elapsed_time(e1) / n_ref
            ref_cuda = {"value": BATCH / (ref_ms / 1000.0), "unit": UNIT + " on one GPU", "ms_per_step": ref_ms,
                        "launches": n_ref,
                        "kind": "reference resizeCrop_bilinear kernel (src/cvcuda/priv/OpResizeCropConvertReformat.cu:158-198), "
                                "its 16x16 launch shape, built for sm_100a; scalar scale/offset of channel 0, float32 NCHW; "
                                "the Normalize pass its pipeline needs for per-channel constants is not included"}
            del out_ref

    clock_info = clocks.stop() if rank == 0 else None
    if world > 1:
        dist.barrier()

    if rank == 0:
        # the result that came back to the host must be the real one: check two images against the CPU checker
        from oracle import oracle as O
        spec = O.ResizeSpec(resize=RESIZE, crop=CROP, out_size=OUT, interp=O.LINEAR, src_cast=False, base=MEAN, mul=mul)
        want = O.resize_crop(list(host_src[:2].numpy()), spec, np.float32, True, nthreads=2)
        parity = float(np.abs(check.astype(np.float64) - want).max())
        if parity > 1e-5:
            raise RuntimeError(f"bench output differs from the CPU checker by {parity}")

        peak_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(peak_path):
            peak, peak_kind = float(json.load(open(peak_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        else:
            peak, peak_kind = FALLBACK_HBM_GBS, "fallback"
        achieved = ALG_BYTES * BATCH / (ms_per_step / 1000.0) / 1e9  # per GPU: one launch processes BATCH images
        cpu_rates, kind, cores, sample = time_cpu(max(cpu_threads() * 4, 32), 3, warm=1)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(world),
            "gb_per_s_algorithmic_per_gpu": achieved,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "frac_of_nominal_8000": achieved / 8000.0,
                         "alg_bytes_per_image": ALG_BYTES, "images_per_launch": BATCH,
                         "traffic": NCU_TRAFFIC_BYTES_PER_IMAGE * BATCH if NCU_TRAFFIC_BYTES_PER_IMAGE else None,
                         "kernel": "resize_staged_kernel<LINEAR,F32,planar>"},
            "e2e": {"value": e2e_results[best]["value"], "unit": UNIT, "mode": best,
                    "h2d_bytes_per_step": e2e_results[best]["h2d_bytes_per_step"],
                    "d2h_bytes_per_step": int(host_out.numel() * 4), "steps": e2e_steps, "all_modes": e2e_results},
            "reference_cuda_baseline": ref_cuda,
            "cpu_baseline": {"value": statistics.mean(cpu_rates), "unit": UNIT, "cores": cores, "kind": kind,
                             "sample": sample},
            "gpu_launches": int(launches), "clocks": clock_info, "parity_max_abs_diff": parity,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", choices=("native", "reference"), default="native")
    args = ap.parse_args()
    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 5
        args.warmup = args.warmup if args.warmup is not None else 1
        return run_reference(args)
    args.steps = args.steps if args.steps is not None else 2000
    args.warmup = args.warmup if args.warmup is not None else 20
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            # convenience: relaunch under torchrun, one rank per GPU
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", "29541", os.path.abspath(__file__), "--gpus",
                   str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup)]
            return subprocess.call(cmd)
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    return run_native(args)


if __name__ == "__main__":
    sys.exit(main())
