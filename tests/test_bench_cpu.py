"""CPU: the bench's own bookkeeping -- algorithmic bytes per image against the oracle's sector bitmap and the figures the
configurations are specified with, the configuration table, and the reference arm's JSON line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


@pytest.mark.parametrize("key,src_bytes,total", [("2", 2265088, 2867200), ("4", 4147200, 9062400),
                                                 ("5-linear", 9060352, 10264576), ("5-nearest", 4530176, 5734400)])
def test_algorithmic_bytes_of_the_dense_configurations(oracle, key, src_bytes, total):
    cfg = bench.Config(key)
    got = bench.tapped_source_bytes(cfg.w, cfg.h, cfg.w * 3, cfg.resize, cfg.crop, cfg.out, cfg.interp)
    spec = oracle.ResizeSpec(resize=cfg.resize, crop=cfg.crop, out_size=cfg.out, interp=cfg.interp)
    assert got == src_bytes == oracle.resize_source_bytes(cfg.w, cfg.h, cfg.w * 3, spec)
    assert cfg.alg_bytes() == total


def test_algorithmic_bytes_with_rectangles_match_the_oracle_bitmap(oracle):
    rng = np.random.default_rng(5)
    for _ in range(12):
        w, h = int(rng.integers(480, 3841)), int(rng.integers(360, 2161))
        cw, ch = int(rng.integers(40, w + 1)), int(rng.integers(40, h + 1))
        roi = (int(rng.integers(0, w - cw + 1)), int(rng.integers(0, h - ch + 1)), cw, ch)
        pitch = (w * 3 + 31) // 32 * 32
        spec = oracle.ResizeSpec(resize=(224, 224), out_size=(224, 224), interp=1)
        assert bench.tapped_source_bytes(w, h, pitch, (224, 224), (0, 0), (224, 224), 1, roi=roi) \
            == oracle.resize_source_bytes(w, h, pitch, spec, roi=np.array(roi, np.int32))
    spec = oracle.ResizeSpec(resize=(50, 41), crop=(9, 11), out_size=(33, 20), interp=0)
    assert bench.tapped_source_bytes(37, 29, 111, (50, 41), (9, 11), (33, 20), 0) == oracle.resize_source_bytes(37, 29, 111, spec)


def test_strong_scaling_splits_the_whole_job():
    class A:
        images, scaling = 0, "strong"
    assert [bench.per_gpu_images(bench.Config("5-linear"), A, w) for w in (1, 2, 4, 8)] == [1024, 512, 256, 128]
    A.scaling = "weak"
    assert bench.per_gpu_images(bench.Config("5-linear"), A, 8) == 128 and bench.per_gpu_images(bench.Config("2"), A, 4) == 256


def test_reference_arm_prints_one_json_line(built):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "images/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["config"]["config"] == "2"
