"""The opt-in Q4_K tensor-core GEMM with the activation scales folded into the operand (IZB_GEMM_FOLD=1): same results as
the CUDA-core GEMM and the oracle within 1e-5 of max|ref|.  Runs in a child process because the switch is read once."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_folded_scale_gemm_matches_core_gemm_and_oracle():
    env = dict(os.environ, IZB_GEMM_FOLD="1")
    r = subprocess.run([sys.executable, os.path.join(os.path.dirname(__file__), "tc_fold_worker.py")], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "fold ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
