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


@pytest.mark.parametrize("env", [
    {"HKB_PREFILL_NO_TMA": "1"},                              # K, V and the query tiles by cp.async / vector loads
    {"HKB_PREFILL_MMA_SYNC": "1"},                            # the mma.sync form at head_dim 128 too
], ids=lambda e: ",".join(f"{k}={v}" for k, v in e.items()))
def test_prefill_tests_under_the_other_forms(env):
    """The tensor-memory prefill kernel without TMA (its cp.async gather and the softmax warps' own staging
    of the query rows, which in the persistent grid wait for the item before), and the mma.sync kernel in
    its place: the prefill tests in a child process of each setting (the test that asks which kernel runs
    sets the variable itself and is left out)."""
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider", "tests/test_gpu_prefill.py", "tests/test_gpu_f16.py",
           "-k", "not which_kernel and not both_kernel_forms"]
    r = subprocess.run(cmd, cwd=ROOT, env={**os.environ, **env}, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stdout[-3000:]
