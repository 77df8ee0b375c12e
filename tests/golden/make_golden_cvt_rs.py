"""Samples the dumps of tests/golden/cvt_rs_probe.cu (run on a B200) into cvt_rs_e2m1x4.npz:

    python tests/golden/make_golden_cvt_rs.py <directory holding rs_probe1.bin and rs_probe2.bin>

Each record is (a, b, c, d, rbits) -> the 16-bit result of cvt.rs.satfinite.e2m1x4.f32 {a, b, c, d}, rbits.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def main():
    src = Path(sys.argv[1])
    rng = np.random.default_rng(5)
    raw = (src / "rs_probe1.bin").read_bytes()
    n = int(np.frombuffer(raw[:4], np.int32)[0])
    xs = np.frombuffer(raw[4:4 + 4 * n], np.float32)
    table = np.frombuffer(raw[4 + 4 * n:], np.uint16).reshape(n, 4, 4, 256)
    picks = 5
    i = np.repeat(np.arange(n), picks)
    pos, byte, b = (rng.integers(0, k, i.size) for k in (4, 4, 256))
    ops = np.zeros((4, i.size), dtype=np.float32)
    ops[pos, np.arange(i.size)] = xs[i]
    rbits = (b.astype(np.uint32) << (8 * byte).astype(np.uint32)).astype(np.uint32)
    out = table[i, pos, byte, b]
    raw = (src / "rs_probe2.bin").read_bytes()
    m = int(np.frombuffer(raw[:4], np.int32)[0])
    x = np.frombuffer(raw[4:4 + 4 * m], np.float32)
    r = np.frombuffer(raw[4 + 4 * m:4 + 8 * m], np.uint32)
    o = np.frombuffer(raw[4 + 8 * m:], np.uint16)
    keep = 20000
    ops2 = np.stack([x[:keep], -x[:keep], x[:keep] * np.float32(0.5), x[:keep] * np.float32(2)])
    np.savez_compressed(HERE / "cvt_rs_e2m1x4.npz", a=np.concatenate([ops[0], ops2[0]]), b=np.concatenate([ops[1], ops2[1]]),
                        c=np.concatenate([ops[2], ops2[2]]), d=np.concatenate([ops[3], ops2[3]]),
                        rbits=np.concatenate([rbits, r[:keep]]), out=np.concatenate([out, o[:keep]]))
    print("wrote", HERE / "cvt_rs_e2m1x4.npz", i.size + keep, "records")


if __name__ == "__main__":
    main()
