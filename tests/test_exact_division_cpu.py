"""The division-free forms of the quantiser's block-scale arithmetic equal the IEEE quotients (tests/exact_division.c).
The suite samples the bit patterns with an odd stride; `exact_division 1` walks all of them."""
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent


def test_fma_quotients_equal_ieee_division(tmp_path):
    exe = tmp_path / "exact_division"
    subprocess.run(["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-mfma", str(HERE / "exact_division.c"), "-lm", "-o", str(exe)], check=True)
    out = subprocess.run([str(exe), "257"], check=True, capture_output=True, text=True, timeout=600).stdout.split()
    assert out[0] == "div6" and out[3] == "e4m3"
    # a / 6: the forms only differ where the quotient is subnormal, below 2^-125 (bit pattern 0x01000000)
    assert int(out[2]) < 0x01000000
    assert int(out[4]) == 0


def test_division_free_round_up_test_of_the_variance_code(tmp_path):
    """tests/exact_threshold.c: u < ((z - lo)(z + lo)) / (2 lo + 1) against its FMA form (AdamW kernels, rounds_up) over
    every 97th float z of [0, 255] and [0, 15] and the uniforms around the turning point.  The full enumeration (stride 1,
    1.4 x 10^10 cases, 20 s on 16 cores) was run when the form was adopted: no difference."""
    exe = tmp_path / "exact_threshold"
    subprocess.run(["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-mfma", str(HERE / "exact_threshold.c"), "-lm", "-o", str(exe)],
                   check=True)
    out = subprocess.run([str(exe), "97"], check=True, capture_output=True, text=True).stdout.split()
    assert out[0] == "threshold" and int(out[1]) == 0 and int(out[2]) > 1e8, out
