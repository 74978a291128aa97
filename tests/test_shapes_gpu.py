"""GPU: the staged kernel under launch shapes other than the defaults (rows per work unit, ring depth, consumer teams,
consumer warps), chosen through the library's tuning variables. The variables are read once per process, so every
shape runs the seeded random sweep of test_random_gpu.py in a child process."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))

SHAPES = [
    {"B200PP_UNIT_ROWS": "1"},
    {"B200PP_UNIT_ROWS": "2", "B200PP_STAGES": "4", "B200PP_TEAMS": "2"},
    {"B200PP_UNIT_ROWS": "3", "B200PP_STAGES": "4", "B200PP_TEAMS": "4", "B200PP_MAX_CONSUMERS": "256"},
    {"B200PP_UNIT_ROWS": "4", "B200PP_STAGES": "2", "B200PP_MAX_CONSUMERS": "64"},
    # a team count that does not divide the ring depth must be reduced by the library, never launched
    {"B200PP_UNIT_ROWS": "1", "B200PP_STAGES": "3", "B200PP_TEAMS": "2"},
    {"B200PP_UNIT_ROWS": "2", "B200PP_STAGES": "6", "B200PP_TEAMS": "3", "B200PP_MAX_CTAS_PER_SM": "1"},
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: ",".join(f"{k[7:].lower()}={v}" for k, v in s.items()))
def test_random_sweep_under_launch_shape(shape):
    env = dict(os.environ)
    env.update(shape)
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(HERE, "test_random_gpu.py"), "-m", "gpu", "-x", "-q",
                        "-p", "no:cacheprovider"], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, (r.stdout[-3000:] + r.stderr[-1000:])
