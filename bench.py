"""Throughput of the fused image pre-processing path on B200, for every benchmark configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 2|3|4|5-linear|5-nearest|cfnr]
                    [--scaling weak|strong] [--impl native|reference] [--images M] [--kernel-only]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Default workload (`--config 2`, per GPU): the classification pre-processing batch -- 256 uint8 NHWC 1080x1920x3 images
(seeded uniform bytes, synthetic) -> bilinear resize to 256x256 -> centre crop 224x224 -> per-channel (v - mean) * (1/std)
-> float32 NCHW. One step = one pass over the batch = one fused kernel launch. Every configuration's source batch is far
larger than the 126 MB L2, so every step reads its source rows from HBM; no flush is needed between steps.

Other configurations: 3 = variable-shape batch of 128 images, one random rectangle each -> 224x224 bilinear -> horizontal
flip p = 0.5 -> mean/std -> float16 NCHW; 4 = letterbox of 64 1080p images into a 640x640 canvas; 5-linear / 5-nearest =
4K -> 512x512 -> 448x448 -> mean/std -> float16 (weak scaling: 128 images per GPU; `--scaling strong`: 1024 images split
evenly over the GPUs); cfnr = CropFlipNormalizeReformat alone on 32 1080p images.

One JSON line is printed by rank 0. `value` = images/s with inputs resident in HBM, device-timed with CUDA events on the
launching stream, max over ranks; with fewer than 200 steps the timed window of exactly `steps` passes is repeated
(`repeats`) and the median window is reported with the spread. The timed steps are issued twice: one library call per
step from Python (`eager_ms_per_step`) and the same launches replayed from one CUDA graph (`launch_mode`; `value` and
`ms_per_step` are the replay's, `--no-graph` keeps the first). `e2e` = the same metric from page-locked HOST buffers to a
page-locked HOST result through the library's C entry point, transfers inside the timed region, with the measured
concurrent host<->device copy bandwidth of the same buffers beside it. `roofline` relates the kernel's algorithmic bytes
to the measured HBM copy bandwidth. `cpu_baseline` times the CPU implementation on a bounded sample on the host cores.
`reference_cuda_baseline` / `handle_api` (rank 0): the reference's own operators built for sm_100a, chained the way its
users have to chain them, and this library driven through the reference's C++ wrappers on real nvcv handles, both timed
by the same harness in child processes.

`--impl reference` times the reference's own CPU implementation of the path on all host cores; under torchrun only rank 0
runs it.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

UNIT = "images/s"
MEAN = (123.675, 116.28, 103.53)
STD = (58.395, 57.12, 57.375)
FALLBACK_HBM_GBS = 6650.0
SEED = 1234

# DRAM traffic per image from the ncu captures summarised under profiles/ (bytes read + written per launch / images).
NCU_TRAFFIC_BYTES_PER_IMAGE = {"2": 736304128 / 256}


def inv_std():
    import numpy as np
    return tuple(float(np.float32(1.0) / np.float32(s)) for s in STD)


# ------------------------------------------------------------------------------------------------ algorithmic bytes

def tapped_source_bytes(src_w: int, src_h: int, pitch: int, resize, crop, out, interp: int, roi=None) -> int:
    """Distinct 32-byte sectors of one packed RGB uint8 image (row pitch `pitch`, base on a sector boundary) that hold a
    byte addressed by a tap of the resize formula, times 32: float32 coordinates exactly as the operator computes them
    (scale = size / resize; nearest floor(scale * (d + crop + 0.5)); linear floor(scale * (d + crop + 0.5) - 0.5) and the
    next pixel, clamped to the image or to the rectangle `roi` = (x, y, w, h))."""
    import numpy as np
    f32 = np.float32
    x0, y0, w, h = (0, 0, src_w, src_h) if roi is None else (int(v) for v in roi)

    def taps(n_out, c0, size, rs):
        scale = f32(size) / f32(rs)
        d = (np.arange(n_out, dtype=np.float32) + f32(c0)) + f32(0.5)
        if interp == 0:
            return np.unique(np.floor(scale * d).astype(np.int64))
        s0 = np.floor(scale * d - f32(0.5)).astype(np.int64)
        return np.unique(np.concatenate([np.maximum(s0, 0), np.minimum(s0 + 1, size - 1)]))

    cols, rows = taps(out[0], crop[0], w, resize[0]), taps(out[1], crop[1], h, resize[1])
    start = (y0 + rows) * pitch + x0 * 3
    first = (start[:, None] + cols[None, :] * 3) // 32
    last = (start[:, None] + cols[None, :] * 3 + 2) // 32
    both = np.sort(np.concatenate([first, last], axis=1), axis=1)
    distinct = 1 + (np.diff(both, axis=1) != 0).sum(axis=1)
    return int(distinct.sum()) * 32


# ------------------------------------------------------------------------------------------------ configurations

class Config:
    """One benchmark configuration: what a step is, its sizes, and its algorithmic bytes per image."""

    def __init__(self, key: str):
        self.key = key
        k = key
        self.varshape = k == "3"
        self.interp = 0 if k == "5-nearest" else 1
        if k == "2":
            self.images, self.h, self.w, self.resize, self.crop, self.out = 256, 1080, 1920, (256, 256), (16, 16), (224, 224)
            self.out_dtype, self.kernel = "f32", "resize_staged_kernel<LINEAR,F32,planar>"
            self.metric = "images/sec, 1080p->224x224 fused preproc (resize 256 bilinear, crop 224, mean/std, f32 NCHW)"
            self.text = ("classification preproc, dense batch: {n} x 1080x1920x3 u8 NHWC per GPU -> resize 256x256 linear -> "
                         "crop 224x224 @ (16,16) -> (v-mean)*(1/std) per channel -> f32 NCHW")
        elif k == "4":
            self.images, self.h, self.w, self.resize, self.crop, self.out = 64, 1080, 1920, (640, 360), (0, 0), (640, 360)
            self.canvas, self.top = (640, 640), 140
            self.out_dtype, self.kernel = "f32", "resize_staged_kernel<LINEAR,F32,planar> (letterbox)"
            self.metric = "images/sec, 1080p letterbox into 640x640 (resize 640x360 bilinear, pad 114, BGR, x/255, f32 NCHW)"
            self.text = ("detection letterbox: {n} x 1080x1920x3 u8 NHWC per GPU -> resize 640x360 linear -> rows 140..499 of a "
                         "640x640 canvas padded with 114 -> BGR -> x/255 -> f32 NCHW")
        elif k in ("5-linear", "5-nearest"):
            self.images, self.h, self.w, self.resize, self.crop, self.out = 128, 2160, 3840, (512, 512), (32, 32), (448, 448)
            name = "nearest" if self.interp == 0 else "linear"
            self.out_dtype, self.kernel = "f16", f"resize_staged_kernel<{name.upper()},F16,planar>"
            self.metric = f"images/sec, 4K->448x448 fused preproc (resize 512 {name}, crop 448, mean/std, f16 NCHW)"
            self.text = ("4K throughput sweep: {n} x 2160x3840x3 u8 NHWC per GPU -> resize 512x512 " + name +
                         " -> crop 448x448 @ (32,32) -> (v-mean)*(1/std) per channel -> f16 NCHW")
        elif k == "3":
            self.images, self.resize, self.crop, self.out = 128, (224, 224), (0, 0), (224, 224)
            self.out_dtype, self.kernel = "f16", "resize_rowwalk_kernel<LINEAR,F16,planar> (per-sample geometry)"
            self.metric = "images/sec, variable-shape random crop -> 224x224 bilinear, flip p=0.5, mean/std, f16 NCHW"
            self.text = ("variable-shape batch: {n} RGB u8 images per GPU, H in [360,2160], W in [480,3840], one random rectangle "
                         "each (8-100 % of the area, aspect 3/4..4/3) -> resize 224x224 linear (rounded to u8) -> horizontal flip "
                         "p=0.5 -> (v-mean)*(1/std) -> f16 NCHW")
        elif k == "cfnr":
            self.images, self.h, self.w, self.out = 32, 1080, 1920, (1920, 1080)
            self.out_dtype, self.kernel = "f32", "slice_u8x3_kernel<F32>"
            self.metric = "images/sec, CropFlipNormalizeReformat 1080p RGB u8 -> f32 NCHW (whole image, flip both, reflect-101)"
            self.text = ("CropFlipNormalizeReformat alone: {n} x 1080x1920 RGB u8 images per GPU, crop = whole image, flip both "
                         "axes, REFLECT101, (v-mean)/std -> f32 NCHW")
        else:
            raise SystemExit(f"unknown --config {key}")
        self.out_elem = 4 if self.out_dtype == "f32" else 2

    def out_shape(self, n):
        w, h = getattr(self, "canvas", self.out)
        return (n, 3, h, w)

    def out_bytes_per_image(self) -> int:
        _, c, h, w = self.out_shape(1)
        return c * h * w * self.out_elem

    def varshape_inputs(self, n: int, rank: int):
        """Seeded sizes, rectangles (the reference's RandomResizedCrop procedure) and flip codes of `n` images."""
        import numpy as np
        import __graft_entry__ as ge
        rng = np.random.default_rng(SEED + 1000 * rank)
        sizes = [(int(rng.integers(480, 3841)), int(rng.integers(360, 2161))) for _ in range(n)]
        rects = np.array(ge.load_package().random_crop_rects(sizes, seed=SEED + rank), np.int32)
        flips = np.where(rng.random(n) < 0.5, 1, 2).astype(np.int32)
        return sizes, rects, flips

    def alg_bytes(self, sizes=None, rects=None) -> float:
        """Algorithmic bytes per image: tapped source sectors + output bytes (the mean over the batch for config 3)."""
        if self.key == "cfnr":
            return self.h * self.w * 3 + self.out_bytes_per_image()
        if self.varshape:
            total = 0
            for (w, h), r in zip(sizes, rects):
                total += tapped_source_bytes(w, h, (w * 3 + 31) // 32 * 32, self.resize, self.crop, self.out, 1, roi=r)
            return total / len(sizes) + self.out_bytes_per_image()
        return tapped_source_bytes(self.w, self.h, self.w * 3, self.resize, self.crop, self.out, self.interp) \
            + self.out_bytes_per_image()


def per_gpu_images(cfg: Config, args, world: int) -> int:
    if args.images:
        return args.images
    if args.scaling == "strong":
        total = 1024 if cfg.key.startswith("5") else cfg.images
        if total % world:
            raise SystemExit(f"{total} images do not split evenly over {world} GPUs")
        return total // world
    return cfg.images


def workload_config(cfg: Config, n: int, world: int, scaling: str) -> dict:
    return {"workload": cfg.text.format(n=n), "config": cfg.key, "images_per_gpu": n, "global_batch": n * world,
            "sharding": f"by sample, {world} x {n}", "scaling": scaling, "collective": "none",
            "l2": "source batch per GPU >> 126 MB L2, no flush needed"}


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


def bind_to_gpu_numa_node(local: int):
    """Runs this rank on the host cores next to its GPU (as `nvidia-smi topo -m` reports them), so that page-locked
    buffers it touches first land in that NUMA node's memory. Returns what was done, for the record."""
    try:
        text = subprocess.run(["nvidia-smi", "topo", "-m"], capture_output=True, text=True, timeout=20).stdout
        header = next(ln for ln in text.splitlines() if "CPU Affinity" in ln)
        cols = [c.strip() for c in header.replace("\x1b[4m", "").replace("\x1b[0m", "").split("\t")]
        row = next(ln for ln in text.splitlines() if ln.replace("\x1b[4m", "").startswith(f"GPU{local}\t")
                   or ln.replace("\x1b[4m", "").startswith(f"GPU{local} "))
        cells = [c.strip() for c in row.replace("\x1b[4m", "").replace("\x1b[0m", "").split("\t")]
        spec = cells[cols.index("CPU Affinity")]
        cpus = set()
        for part in spec.split(","):
            a, _, b = part.partition("-")
            cpus.update(range(int(a), int(b or a) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return {"bound": False, "why": f"GPU{local} cores {spec} are outside this process's cpuset"}
        os.sched_setaffinity(0, allowed)
        return {"bound": True, "cores": spec, "count": len(allowed)}
    except Exception as e:  # noqa: BLE001 - best effort: the measurement still runs unbound
        return {"bound": False, "why": f"{type(e).__name__}: {e}"[:160]}


# ------------------------------------------------------------------------------------------------ CPU legs

def cpu_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def time_cpu(cfg: Config, images_total: int, repeats: int, warm: int = 0):
    """Times the CPU implementation of the configuration on `images_total` images with every host thread.
    Returns (images_per_second_list, kind, cores, description)."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle as O  # the checker, timed here as the CPU baseline -- never on the product path

    threads = cpu_threads()
    rng = np.random.default_rng(SEED)
    ref = O.ref()
    mul = inv_std()
    bounds = [(images_total * t // threads, images_total * (t + 1) // threads) for t in range(threads)]
    bounds = [b for b in bounds if b[1] > b[0]]
    if cfg.key == "cfnr":
        src = rng.integers(0, 256, (images_total, cfg.h, cfg.w, 3), dtype=np.uint8)
        if ref is not None:
            kind, what = "reference", "reference golden CropFlipNormalizeReformat (tests/cvcuda/system/" \
                                      "TestOpCropFlipNormalizeReformat.cpp:43-149), one image per thread at a time"

            def work(b):
                for i in range(*b):
                    O.ref_cfnr(src[i], False, (0, 0, cfg.w, cfg.h), -1, cfg.out, np.float32, True, 4, 0.0, MEAN, STD, 1.0, 0.0, 0.0, 1)
        else:
            kind, what = "port", "C restatement of the reference golden (oracle/preproc_oracle.c)"
            rect = np.tile(np.array([0, 0, cfg.w, cfg.h], np.int32), (images_total, 1))

            def work(b):
                O.crop_flip_normalize(list(src[b[0]:b[1]]), False, rect[b[0]:b[1]], np.full(b[1] - b[0], -1, np.int32), cfg.out,
                                      np.float32, True, 4, 0.0, np.array(MEAN, np.float32), np.array(STD, np.float32), 1.0, 0.0,
                                      0.0, 1)
    elif cfg.varshape or cfg.key == "4" or ref is None:
        # no single reference golden expresses these passes: the C restatement (pinned to chains of the goldens by the tests)
        kind, what = "port", "C restatement of the reference golden (oracle/preproc_oracle.c)"
        if cfg.varshape:
            sizes, rects, flips = cfg.varshape_inputs(images_total, 0)
            imgs = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for (w, h) in sizes]
            spec = O.ResizeSpec(resize=cfg.resize, out_size=cfg.out, interp=1, src_cast=True, base=MEAN, mul=mul)

            def work(b):
                O.resize_crop(imgs[b[0]:b[1]], spec, np.float16, True, roi=rects[b[0]:b[1]], flip=flips[b[0]:b[1]])
        else:
            src = rng.integers(0, 256, (images_total, cfg.h, cfg.w, 3), dtype=np.uint8)
            if cfg.key == "4":
                spec = O.ResizeSpec(resize=cfg.resize, out_size=cfg.out, interp=1, src_cast=True, manip=1, scale=1.0 / 255.0,
                                    canvas=cfg.canvas, dst_pos=(0, cfg.top), pad_value=114.0)
                odt = np.float32
            else:
                spec = O.ResizeSpec(resize=cfg.resize, crop=cfg.crop, out_size=cfg.out, interp=cfg.interp, src_cast=False,
                                    base=MEAN, mul=mul)
                odt = np.float32 if cfg.out_dtype == "f32" else np.float16

            def work(b):
                O.resize_crop(list(src[b[0]:b[1]]), spec, odt, True)
    else:
        # The reference's own golden function. It has one scalar scale/offset pair (its operator cannot express
        # per-channel constants) and float32 output, so channel 0's constants stand in: same taps, same operation count.
        kind = "reference"
        what = "reference golden ResizeCropConvert (tests/cvcuda/system/TestOpResizeCropConvertReformat.cpp:76-172), " \
               "scalar scale/offset of channel 0, float32 output"
        src = rng.integers(0, 256, (images_total, cfg.h, cfg.w, 3), dtype=np.uint8)
        scale, offset = 1.0 / STD[0], -MEAN[0] / STD[0]

        def work(b):
            O.ref_rccr(src[b[0]:b[1]], cfg.resize, cfg.crop, cfg.out, cfg.interp, 0, scale, offset, False, np.float32, True)

    rates = []
    with ThreadPoolExecutor(max_workers=len(bounds)) as ex:
        for i in range(warm + repeats):
            t0 = time.perf_counter()
            list(ex.map(work, bounds))
            dt = time.perf_counter() - t0
            if i >= warm:
                rates.append(images_total / dt)
    sample = f"{images_total} images per pass, {repeats} timed passes, {threads} threads; {what}"
    return rates, kind, threads, sample


def cpu_sample_images(cfg: Config) -> int:
    per_thread = {"2": 4, "4": 2, "3": 2, "cfnr": 1}.get(cfg.key, 1)
    return max(cpu_threads() * per_thread, 16)


def run_reference(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cfg = Config(args.config)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    images = cpu_sample_images(cfg)  # one step = a bounded sample of the batch, a few images per thread
    t0 = time.perf_counter()
    rates, kind, cores, sample = time_cpu(cfg, images, args.steps, warm=args.warmup)
    value = statistics.mean(rates)
    line = {
        "impl": "reference", "metric": cfg.metric, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 * images / value, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": cfg.out_dtype, "data": "synthetic",
        "config": workload_config(cfg, per_gpu_images(cfg, args, max(world, args.gpus)), max(world, args.gpus), args.scaling),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------------ harness legs

def run_harness_leg(args) -> int:
    """Child process of the GPU arm: times one configuration through the harness over the reference's C++ API
    (oracle/ref_ops_harness.cpp), against the reference's own operators (`ref`) or this library (`b200`)."""
    from oracle import ref_ops as R
    cfg = Config(args.config)
    L = R.load(args.harness_leg)
    if L is None:
        print("HARNESS " + json.dumps({"unavailable": "harness library not built"}))
        return 0
    n, it, wu = args.images or cfg.images, max(3, min(args.steps, 50)), 3
    res = {"images": n}
    modes = [("chain", True)] + ([("one_pass", False)] if args.harness_leg == "b200" and cfg.key != "cfnr" else [])
    for name, chain in modes:
        try:
            if cfg.key in ("2", "5-linear", "5-nearest"):
                # the reference refuses inputs above 2 GiB per call: at most 86 4K images (or 345 1080p images) a time
                per_call = (2 ** 31 - 1) // (cfg.h * cfg.w * 3)
                ms, launches = R.time_classify(L, n, cfg.h, cfg.w, cfg.resize, cfg.crop, cfg.out, cfg.interp, chain, per_call, wu, it)
            elif cfg.key == "4":
                ms, launches = R.time_letterbox(L, n, cfg.h, cfg.w, cfg.resize, cfg.canvas, cfg.top, chain, wu, it)
            elif cfg.key == "3":
                sizes, rects, flips = cfg.varshape_inputs(n, 0)
                ms, launches = R.time_varshape(L, sizes, cfg.out, rects, flips, chain, wu, it)
            else:
                ms, launches = R.time_cfnr(L, n, cfg.h, cfg.w, wu, it)
            res[name] = {"ms_per_step": ms, "value": n / (ms / 1000.0), "launches_per_step": launches}
        except R.HarnessError as e:
            res[name] = {"unavailable": str(e)[:300]}
    # the operators of the chain one at a time (same tensors, the others not run inside the timed region)
    stage_names = {"2": ["ResizeCropConvertReformat f32 NHWC", "Normalize f32", "Reformat NHWC->NCHW"],
                   "4": ["Resize u8", "CopyMakeBorder u8", "ConvertTo u8->f32", "Reformat NHWC->NCHW"]}.get(cfg.key)
    if stage_names and "ms_per_step" in res.get("chain", {}):
        stages = {}
        try:
            for i, name in enumerate(stage_names):
                R.select_stage(L, i)
                if cfg.key == "2":
                    ms, _ = R.time_classify(L, n, cfg.h, cfg.w, cfg.resize, cfg.crop, cfg.out, cfg.interp, True,
                                            (2 ** 31 - 1) // (cfg.h * cfg.w * 3), wu, it)
                else:
                    ms, _ = R.time_letterbox(L, n, cfg.h, cfg.w, cfg.resize, cfg.canvas, cfg.top, True, wu, it)
                stages[name] = ms
        except R.HarnessError as e:
            stages["unavailable"] = str(e)[:200]
        finally:
            R.select_stage(L, -1)
        res["chain"]["stage_ms"] = stages
    if cfg.key == "2":
        # the stock variable-shape operator on an image list of equal-sized images (the same call in both libraries)
        try:
            ms = R.time_rccr_list(L, 64, cfg.h, cfg.w, cfg.resize, cfg.crop, cfg.out, cfg.interp, 1.0 / 255.0, wu, it)
            res["image_list"] = {"ms_per_step": ms, "value": 64 / (ms / 1000.0), "images": 64,
                                 "workload": "stock ResizeCropConvertReformat on a 64-image list, x/255, float32 NCHW"}
        except R.HarnessError as e:
            res["image_list"] = {"unavailable": str(e)[:300]}
    if args.harness_leg == "b200" and cfg.key in ("2", "5-linear", "5-nearest"):
        # end to end through the handle API: nvcv tensors that wrap page-locked host memory, at most 2 GiB of source per call
        try:
            m = min(n, (2 ** 31 - 1) // (cfg.h * cfg.w * 3))
            ms = R.time_classify_e2e_host(L, m, cfg.h, cfg.w, cfg.resize, cfg.crop, cfg.out, cfg.interp, 2, max(3, min(args.steps, 10)))
            res["e2e_host_tensors"] = {"ms_per_step": ms, "value": m / (ms / 1000.0), "images": m, "output": "float32 NCHW"}
        except R.HarnessError as e:
            res["e2e_host_tensors"] = {"unavailable": str(e)[:300]}
    print("HARNESS " + json.dumps(res))
    return 0


def harness_child(which: str, cfg: Config, n: int, steps: int):
    """Runs run_harness_leg in a child process (the harness must not share a process with another object-model library)."""
    try:
        p = subprocess.run([sys.executable, os.path.abspath(__file__), "--harness-leg", which, "--config", cfg.key, "--images",
                            str(n), "--steps", str(steps)], capture_output=True, text=True, timeout=600)
        line = next((ln for ln in p.stdout.splitlines() if ln.startswith("HARNESS ")), None)
        if line is None:
            return {"unavailable": f"child exited {p.returncode}: {p.stderr[-300:]}"}
        return json.loads(line[len("HARNESS "):])
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}


HARNESS_NOTES = {
    "2": "ResizeCropConvertReformat (float32 NHWC) -> Normalize (per-channel, stddev flag) -> Reformat (NHWC -> NCHW)",
    "5-linear": "ResizeCropConvertReformat in calls of at most 86 images (float32 NHWC) -> Normalize -> Reformat; float32 "
                "(the reference has no float16 output)",
    "5-nearest": "ResizeCropConvertReformat in calls of at most 86 images (float32 NHWC) -> Normalize -> Reformat; float32 "
                 "(the reference has no float16 output)",
    "4": "Resize -> CopyMakeBorder (constant 114) -> ConvertTo (x 1/255, float32) -> Reformat (NHWC -> NCHW); the channel "
         "swap would be a fifth operator and is left out",
    "3": "RandomResizedCrop (variable-shape, draws its own rectangles: an equal-work stand-in) -> CropFlipNormalizeReformat; "
         "float32 (no float16 output)",
    "cfnr": "CropFlipNormalizeReformat, one call",
}


# ------------------------------------------------------------------------------------------------ GPU arm

def run_native(args) -> int:
    import numpy as np
    import torch
    import torch.distributed as dist

    import __graft_entry__ as ge

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    all_cores = os.sched_getaffinity(0)
    affinity = bind_to_gpu_numa_node(local) if not args.kernel_only else None
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = ge.load_package()  # raises when libcvcuda_b200.so is missing: there is no fallback path
    if args.path:
        pkg.set_kernel_path(args.path)
    cfg = Config(args.config)
    n = per_gpu_images(cfg, args, world)
    mul = inv_std()
    tdt = torch.float32 if cfg.out_dtype == "f32" else torch.float16

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        return pkg.sharding.max_over_ranks(ms, dev)

    # ---- seeded synthetic batch, generated on the device (each rank its own shard of the global batch)
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + rank)
    out = torch.empty(cfg.out_shape(n), dtype=tdt, device=dev)
    sizes = rects = flips = None
    def image_arena(sizes_wh):
        """One allocation holding every image of a variable-shape batch (rows padded to 32 bytes, images on 256-byte
        boundaries, as the reference's allocator lays images out), filled with seeded bytes; returns (arena, views, offsets)."""
        offs, total = [], 0
        for (w, h) in sizes_wh:
            offs.append(total)
            total += ((w * 3 + 31) // 32 * 32 * h + 255) // 256 * 256
        arena = torch.empty((total,), dtype=torch.uint8, device=dev)
        for i in range(0, total, 1 << 27):
            arena[i:i + (1 << 27)] = torch.randint(0, 256, (min(1 << 27, total - i),), dtype=torch.uint8, device=dev, generator=gen)
        return arena, image_views(arena, sizes_wh, offs), offs

    def image_views(arena, sizes_wh, offs):
        views = []
        for (w, h), o in zip(sizes_wh, offs):
            pitch = (w * 3 + 31) // 32 * 32
            views.append(arena[o:o + pitch * h].view(h, pitch)[:, : w * 3].unflatten(1, (w, 3)))
        return views

    arena = arena_offsets = None
    if cfg.varshape:
        sizes, rects, flips = cfg.varshape_inputs(n, rank)
        arena, images, arena_offsets = image_arena(sizes)
        src = pkg.ImageBatchVarShape(images)
        t_rects, t_flips = torch.from_numpy(rects).to(dev), torch.from_numpy(flips).to(dev)
        src_bytes = sum(w * h * 3 for (w, h) in sizes)
    elif cfg.key == "cfnr":
        sizes = [(cfg.w, cfg.h)] * n
        arena, images, arena_offsets = image_arena(sizes)
        src = pkg.ImageBatchVarShape(images)
        t_rects = torch.tensor([[0, 0, cfg.w, cfg.h]] * n, dtype=torch.int32, device=dev).reshape(n, 1, 1, 4)
        t_flips = torch.full((n,), -1, dtype=torch.int32, device=dev)
        t_base = torch.tensor(MEAN, dtype=torch.float32, device=dev).reshape(1, 1, 1, 3)
        t_scale = torch.tensor(STD, dtype=torch.float32, device=dev).reshape(1, 1, 1, 3)
        src_bytes = n * cfg.h * cfg.w * 3
    else:
        src = torch.empty((n, cfg.h, cfg.w, 3), dtype=torch.uint8, device=dev)
        for i in range(0, n, 64):  # in slices: randint makes an int64 temporary eight times the size of its result
            src[i:i + 64] = torch.randint(0, 256, (min(64, n - i), cfg.h, cfg.w, 3), dtype=torch.uint8, device=dev, generator=gen)
        src_bytes = src.numel()

    def step(dst, source):
        if cfg.key == "cfnr":
            pkg.crop_flip_normalize_reformat_into(dst, source, t_rects, t_flips, t_base, t_scale, 1.0, 0.0, 0.0, 1,
                                                  pkg.Border.REFLECT101, 0.0, layout="NCHW")
        elif cfg.varshape:
            pkg.fused_preprocess_into(dst, source, resize_dim=cfg.resize, interp=1, layout="NCHW", base=MEAN, mul=mul,
                                      srcCast=True, roi=t_rects, flip_code=t_flips)
        elif cfg.key == "4":
            pkg.fused_preprocess_into(dst, source, resize_dim=cfg.resize, interp=1, layout="NCHW", manip=1, scale=1.0 / 255.0,
                                      srcCast=True, dst_pos=(0, cfg.top), region_size=cfg.resize, pad_value=114.0)
        else:
            pkg.fused_preprocess_into(dst, source, resize_dim=cfg.resize, interp=cfg.interp, crop_pos=cfg.crop, layout="NCHW",
                                      base=MEAN, mul=mul, srcCast=False)

    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()

    # ---- device-resident throughput: windows of exactly `steps` passes
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step(out, src)
    repeats = 1 if args.steps >= 200 else max(1, min(9, math.ceil(200 / args.steps)))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed_windows(run_window):
        got = []
        for _ in range(repeats):
            barrier()
            e0.record()
            run_window()
            e1.record()
            barrier()
            got.append(max_over_ranks(e0.elapsed_time(e1)))
        return got

    def eager_window():
        for _ in range(args.steps):
            step(out, src)

    launches0 = pkg.launch_count()
    eager_window()
    launches = pkg.launch_count() - launches0  # kernels of one window, counted by the library at launch time
    eager = timed_windows(eager_window)
    # The same `steps` launches replayed from one CUDA graph: no host work between the kernels, which is how a serving loop
    # that cares about the last microseconds issues them (the host side of a call is 20 us of Python here). Every rank must
    # take the same branch: the windows hold barriers.
    windows, launch_mode = eager, "one library call per step from Python"
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                eager_window()
            graph.replay()
            torch.cuda.synchronize()
            captured = 1
        except Exception as exc:  # noqa: BLE001 - the eager figure stands
            captured = 0
            if rank == 0:
                print(f"bench: CUDA graph capture failed ({exc}); reporting the eager loop", file=sys.stderr)
        if int(max_over_ranks(float(1 - captured))) == 0:
            windows, launch_mode = timed_windows(graph.replay), "CUDA graph replay of the timed steps"
    ms_total = statistics.median(windows)
    ms_per_step = ms_total / args.steps
    value = world * n * args.steps / (ms_total / 1000.0)
    if pkg.read_device_error() != 0:
        raise RuntimeError("device error word set: a kernel gave up on a bounded wait")

    peak_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peak_path):
        peak, peak_kind = float(json.load(open(peak_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_kind = FALLBACK_HBM_GBS, "fallback"
    alg = cfg.alg_bytes(sizes, rects)
    achieved = alg * n / (ms_per_step / 1000.0) / 1e9  # per GPU: one launch processes n images
    traffic = NCU_TRAFFIC_BYTES_PER_IMAGE.get(cfg.key)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_kind": peak_kind, "frac_of_nominal_8000": achieved / 8000.0, "alg_bytes_per_image": alg,
                "images_per_launch": n, "traffic": traffic * n if traffic else None, "kernel": cfg.kernel,
                "whole_source_plus_output_gbs": (src_bytes + cfg.out_bytes_per_image() * n) / (ms_per_step / 1000.0) / 1e9}
    line = {
        "metric": cfg.metric, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": cfg.out_dtype, "data": "synthetic", "config": workload_config(cfg, n, world, args.scaling),
        "repeats": repeats, "window_ms_per_step": {"median": ms_per_step, "min": min(windows) / args.steps,
                                                   "max": max(windows) / args.steps},
        "gb_per_s_algorithmic_per_gpu": achieved, "roofline": roofline, "gpu_launches": int(launches),
        "launch_mode": launch_mode, "eager_ms_per_step": statistics.median(eager) / args.steps,
    }
    if args.kernel_only:
        if rank == 0:
            line["clocks"] = clocks.stop()
            print(json.dumps(line))
        if world > 1:
            dist.destroy_process_group()
        return 0

    # ---- end to end from page-locked host memory to a page-locked host result. Large batches go through a bounded
    # page-locked staging batch (at most 2 GiB of source), passed as many times as the batch needs.
    host_batch = None
    if cfg.varshape or cfg.key == "cfnr":
        # the whole batch lives in one page-locked arena with the device arena's layout: one copy call moves it
        m = n
        host_arena = torch.empty((arena.numel(),), dtype=torch.uint8).pin_memory()
        host_arena.copy_(arena)
        host_images = image_views(host_arena, sizes, arena_offsets)
        host_batch = pkg.ImageBatchVarShape(host_images)
        dev_src, host_src = src, None
        h2d_full = host_arena.numel()
    else:
        m = min(n, max(1, (2 ** 31) // (cfg.h * cfg.w * 3)))
        host_src = torch.empty((m, cfg.h, cfg.w, 3), dtype=torch.uint8).pin_memory()
        host_src.copy_(src[:m])
        dev_src = src[:m]
        h2d_full = host_src.numel()
    host_out = torch.empty(cfg.out_shape(m), dtype=tdt).pin_memory()
    dev_out = out[:m]
    passes = (n + m - 1) // m
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_copy_step():
        # whole batch host -> device, fused kernel, result device -> host
        for _ in range(passes):
            if host_src is None:
                arena.copy_(host_arena, non_blocking=True)
            else:
                dev_src.copy_(host_src, non_blocking=True)
            step(dev_out, dev_src)
            host_out.copy_(dev_out, non_blocking=True)

    e2e_modes = {"h2d_copy+kernel+d2h": (e2e_copy_step, h2d_full * passes)}
    if host_src is not None:
        tapped = int(alg - cfg.out_bytes_per_image()) * m * passes

        def e2e_direct_step():
            # the kernel pulls only the source rows it taps straight out of the page-locked host buffer (bulk copies into
            # shared memory), result device -> host
            for _ in range(passes):
                step(dev_out, host_src)
                host_out.copy_(dev_out, non_blocking=True)

        def e2e_zero_copy_step():
            # one launch and nothing else: tapped source rows come in over PCIe by bulk copy, result rows go out as
            # full-line stores into the page-locked host result
            for _ in range(passes):
                step(host_out, host_src)

        e2e_modes["kernel reads pinned host rows directly + d2h"] = (e2e_direct_step, tapped)
        e2e_modes["kernel reads pinned host rows and writes the pinned host result"] = (e2e_zero_copy_step, tapped)
    if cfg.varshape:
        # per-sample geometry from host memory: the staged kernel's bulk copies fetch exactly the tapped row segments over
        # PCIe (the row-walk kernel's byte loads would cross the link one sector at a time)
        tapped = int((alg - cfg.out_bytes_per_image()) * n)

        def e2e_varshape_direct():
            prev = pkg.set_kernel_path(2)
            try:
                step(dev_out, host_batch)
            finally:
                pkg.set_kernel_path(prev)
            host_out.copy_(dev_out, non_blocking=True)

        def e2e_varshape_zero_copy():
            prev = pkg.set_kernel_path(2)
            try:
                step(host_out, host_batch)
            finally:
                pkg.set_kernel_path(prev)

        e2e_modes["kernel reads pinned host rows directly + d2h"] = (e2e_varshape_direct, tapped)
        e2e_modes["kernel reads pinned host rows and writes the pinned host result"] = (e2e_varshape_zero_copy, tapped)
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
        e2e_results[name] = {"value": world * n * e2e_steps / (ms / 1000.0), "ms_per_step": ms / e2e_steps,
                             "h2d_bytes_per_step": int(h2d_bytes)}
    if pkg.read_device_error() != 0:
        raise RuntimeError("device error word set during the end-to-end runs")
    check = host_out[:2].numpy().copy()
    best = max(e2e_results, key=lambda k: e2e_results[k]["value"])
    d2h_bytes = int(host_out.numel() * host_out.element_size()) * passes

    # ---- the ceiling of any end-to-end number: plain copies of the same page-locked buffers, every rank at once
    pcie = {}
    if host_src is not None:
        s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()

        def copies(up: bool, down: bool):
            barrier()
            t0 = time.perf_counter()
            for _ in range(3):
                if up:
                    with torch.cuda.stream(s_up):
                        dev_src.copy_(host_src, non_blocking=True)
                if down:
                    with torch.cuda.stream(s_down):
                        host_out.copy_(dev_out, non_blocking=True)
            barrier()
            return (time.perf_counter() - t0) / 3

        copies(True, True)
        t_up, t_down, t_both = copies(True, False), copies(False, True), copies(True, True)
        up_b, down_b = host_src.numel(), host_out.numel() * host_out.element_size()
        pcie = {"h2d_gbs_per_rank": up_b / t_up / 1e9, "d2h_gbs_per_rank": down_b / t_down / 1e9,
                "both_directions_gbs_per_rank": (up_b + down_b) / t_both / 1e9, "ranks_copying_at_once": world,
                "how": "cudaMemcpyAsync of the bench's own page-locked source and result buffers, 3 copies, host clock "
                       "between barriers; this rank's figures (rank 0)"}
        bw = e2e_results[best]
        moved = (bw["h2d_bytes_per_step"] + d2h_bytes) / world * 1.0
        pcie["best_mode_gbs_per_rank"] = (bw["h2d_bytes_per_step"] + d2h_bytes) / (bw["ms_per_step"] / 1000.0) / 1e9
        pcie["best_mode_frac_of_both_directions_copy"] = pcie["best_mode_gbs_per_rank"] / pcie["both_directions_gbs_per_rank"]
        del moved

    clock_info = clocks.stop() if rank == 0 else None
    if world > 1:
        dist.barrier()

    if rank == 0:
        # the result that came back to the host must be the real one: check two images against the CPU checker
        from oracle import oracle as O
        if cfg.key == "cfnr":
            two = [host_images[i].numpy() for i in range(2)]
            want = O.crop_flip_normalize(two, False, np.array([[0, 0, cfg.w, cfg.h]] * 2, np.int32), np.array([-1, -1], np.int32),
                                         cfg.out, np.float32, True, 4, 0.0, np.array(MEAN, np.float32), np.array(STD, np.float32),
                                         1.0, 0.0, 0.0, 1, nthreads=2)
        elif cfg.varshape:
            spec = O.ResizeSpec(resize=cfg.resize, out_size=cfg.out, interp=1, src_cast=True, base=MEAN, mul=mul)
            want = O.resize_crop([host_images[i].numpy() for i in range(2)], spec, np.float16, True, roi=rects[:2], flip=flips[:2],
                                 nthreads=2)
        elif cfg.key == "4":
            spec = O.ResizeSpec(resize=cfg.resize, out_size=cfg.out, interp=1, src_cast=True, manip=1, scale=1.0 / 255.0,
                                canvas=cfg.canvas, dst_pos=(0, cfg.top), pad_value=114.0)
            want = O.resize_crop(list(host_src[:2].numpy()), spec, np.float32, True, nthreads=2)
        else:
            spec = O.ResizeSpec(resize=cfg.resize, crop=cfg.crop, out_size=cfg.out, interp=cfg.interp, src_cast=False, base=MEAN,
                                mul=mul)
            want = O.resize_crop(list(host_src[:2].numpy()), spec, np.float32 if cfg.out_dtype == "f32" else np.float16, True,
                                 nthreads=2)
        parity = float(np.abs(check.astype(np.float64) - want.astype(np.float64)).max())
        if parity > (1e-5 if cfg.out_dtype == "f32" else 2e-3):
            raise RuntimeError(f"bench output differs from the CPU checker by {parity}")

        # baselines, none of them the optimisation target; the CPU one gets every host core back
        os.sched_setaffinity(0, all_cores)
        cpu_rates, kind, cores, sample = time_cpu(cfg, cpu_sample_images(cfg), 3, warm=1)
        n_h = min(n, 256 if cfg.key == "2" else 128)
        ref_leg = harness_child("ref", cfg, n_h, args.steps)
        own_leg = harness_child("b200", cfg, n_h, args.steps)
        ref_cuda = {"kind": "the reference's own operators (libcvcuda built for sm_100a from its sources), through its C++ "
                            "wrappers on real nvcv tensors / image batches, device-resident, CUDA events",
                    "chain": HARNESS_NOTES[cfg.key], "unit": UNIT + " on one GPU", **ref_leg}
        handle_api = {"kind": "this library through the same wrappers and real nvcv handles: `one_pass` = the extended entry "
                              "point (cvcudaB200FusedPreprocess[VarShape]Submit), `chain` = the same operator chain as the "
                              "reference's, `e2e_host_tensors` = one_pass on nvcv tensors that wrap page-locked host memory "
                              "(source rows pulled over PCIe, result written to the host)", "unit": UNIT + " on one GPU", **own_leg}
        line.update({
            "e2e": {"value": e2e_results[best]["value"], "unit": UNIT, "mode": best,
                    "h2d_bytes_per_step": e2e_results[best]["h2d_bytes_per_step"], "d2h_bytes_per_step": d2h_bytes,
                    "steps": e2e_steps, "staging_batch_images": m, "passes_per_step": passes, "all_modes": e2e_results,
                    "pcie_peak_gbs": pcie or None, "host_affinity": affinity},
            "reference_cuda_baseline": ref_cuda, "handle_api": handle_api,
            "cpu_baseline": {"value": statistics.mean(cpu_rates), "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
            "clocks": clock_info, "parity_max_abs_diff": parity,
        })
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
    ap.add_argument("--config", default="2", choices=("2", "3", "4", "5-linear", "5-nearest", "cfnr"))
    ap.add_argument("--scaling", default="weak", choices=("weak", "strong"),
                    help="weak: the configuration's batch on every GPU; strong: the whole job (1024 images for 5-*) split evenly")
    ap.add_argument("--images", type=int, default=0, help="images per GPU, overriding the configuration (small profiling runs)")
    ap.add_argument("--no-graph", action="store_true", help="time one library call per step from Python only (default: also replay "
                    "the timed steps from a CUDA graph and report that)")
    ap.add_argument("--kernel-only", action="store_true", help="device-resident timing only: no end-to-end, CPU or reference legs")
    ap.add_argument("--path", type=int, default=0, choices=(0, 1, 2, 3),
                    help="kernel choice of the resize path for profiling runs: 0 automatic, 1 per-pixel gather, 2 staged, 3 row walk")
    ap.add_argument("--harness-leg", choices=("ref", "b200"), default=None, help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.harness_leg:
        args.steps = args.steps or 20
        return run_harness_leg(args)
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
                   "--master-addr", "127.0.0.1", "--master-port", "29541", os.path.abspath(__file__)] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    return run_native(args)


if __name__ == "__main__":
    sys.exit(main())
