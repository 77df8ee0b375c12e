"""The FMA division by a shared divisor (csrc/common.cuh, SharedDivisor) against the IEEE quotient, on the GPU.

The AdamW kernels divide sixteen numerators per lane by one block scale; they take the correctly rounded reciprocal once and
correct each quotient twice.  tests/shared_divisor_probe.cu runs that code beside `a / b` for every 64th divisor mantissa at
three exponents (plus the all-ones and all-zero mantissas), with numerators placed on and next to the rounding boundaries:
about 6 x 10^8 quotients, none may differ."""
import shutil
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_shared_divisor_division_is_the_ieee_quotient(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        pytest.skip("nvcc is needed to build the probe")
    exe = tmp_path / "shared_divisor_probe"
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--fmad=false",
                    "-I", str(ROOT / "sm120-nvfp4-training_b200" / "csrc"), "-I", str(ROOT / "include"),
                    str(ROOT / "tests" / "shared_divisor_probe.cu"), "-o", str(exe)], check=True, capture_output=True, text=True)
    out = subprocess.run([str(exe), "64", "128"], check=True, capture_output=True, text=True, timeout=600).stdout.split()
    assert out[0] == "mismatches" and int(out[3]) > 5e8, out
    assert int(out[1]) == 0, out
