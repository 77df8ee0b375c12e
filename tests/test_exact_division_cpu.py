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
