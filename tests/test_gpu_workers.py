"""The walk's workers that are not the default ones, held to the same tests.

Which worker walks a GQA group (`HKB_MMA_MIN_GROUP`), stream or fixed-split grid
(`HKB_FIXED_SPLITS`) and joined or separate step launches (`HKB_STEP_UNFUSED`) are read from the
environment; each setting runs the decode and step tests in a child process of its own. The
defaults are what every other GPU test runs."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]
PICK = "lens_by_splits or gqa_shapes or fp8_cache or head_dim_64 or nan_past or graph_padding or hybrid"


@pytest.mark.parametrize("env", [
    {"HKB_MMA_MIN_GROUP": "8"},                               # CUDA cores below a group of 8, bf16 and fp8
    {"HKB_MMA_MIN_GROUP": "1"},                               # tensor-core tiles at every group
    {"HKB_FIXED_SPLITS": "1"},                                # one CTA a (sequence, kv head, split)
    {"HKB_STEP_UNFUSED": "1"},                                # hkb_decode_step as three launches
], ids=lambda e: ",".join(f"{k}={v}" for k, v in e.items()))
def test_decode_and_step_tests_under_another_worker(env):
    files = ["tests/test_gpu_decode.py", "tests/test_gpu_step.py"]
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider", *files, "-k",
           PICK + " or one_launch_equals or many_pieces or padding_and_empty"]
    r = subprocess.run(cmd, cwd=ROOT, env={**os.environ, **env}, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stdout[-3000:]
