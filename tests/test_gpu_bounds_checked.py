"""The ragged-shape kernel tests once more against the range-checking build of the library (-DAB_BOUNDS_CHECK): every
guarded index of the kernels must stay inside its array (a violation is recorded in the device status word and the
access is skipped, so nothing faults). This is the memory checker of this code base where compute-sanitizer is not
available."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_ragged_shapes_stay_in_bounds_in_the_checked_build():
    from albatross_b200 import build
    lib = build.LIB_CHECKED       # built ahead of time (`python -m albatross_b200.build --bounds-check`, or build())
    assert os.path.exists(lib), "the range-checking build of the library is missing"

    env = dict(os.environ, AB_BOUNDS_CHECK="1")
    cmd = [sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
           os.path.join(ROOT, "tests", "test_gpu_kernels.py"),
           os.path.join(ROOT, "tests", "test_gpu_model.py"),
           "-k", "gemv_against_oracle or batched_product or wkv7_operator_against or zero_and_linearity or "
                 "single_token_path or batch_path or sequence_path or unequal_length"]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    tail = (res.stdout + res.stderr)[-2000:]
    assert res.returncode == 0, tail
    assert "passed" in res.stdout and "AB_BOUNDS_CHECK: a kernel recorded" not in res.stdout, tail
