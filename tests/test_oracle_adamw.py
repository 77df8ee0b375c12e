"""The AdamW oracle against golden vectors produced by the reference's own Triton kernels (CPU interpreter)."""
import numpy as np
import pytest

import oracle as O
from conftest import GOLDEN

FORMATS = ["half16_v8", "half16_v8b128", "split24_v8", "tile32", "sr16_v8", "half16_m4v4_sqrt", "float8_m4v4_sqrt", "half16_m8v4",
           "split24_m4", "sr16_m4", "sr16_m4v4", "float8_v8"]


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN / "adamw_reference.npz")


def hyper_for(gold, t):
    lr, b1, b2, eps, wd = (float(x) for x in gold["hyper"])
    return O.adam_hyper(lr, (b1, b2), eps, wd, t)


def run_oracle_steps(gold, fmt, check):
    master, vb, mb = O.FORMATS[fmt]
    rows, cols, stride = (int(x) for x in gold["meta"])
    n = rows * cols
    width = O.state_block(fmt)
    p = gold[f"{fmt}_p0"].copy()
    tail = gold[f"{fmt}_tail0"].copy() if master == 24 else None
    unit = gold[f"{fmt}_unit0"].copy() if master == 8 else None
    m = np.zeros((n + 1) // 2 if mb == 4 and vb != 4 else n, dtype=np.uint8 if mb == 4 else np.int8)
    ms = np.zeros(-(-n // (64 if mb == 4 else width)), dtype=np.float32)
    vs = np.zeros(-(-n // (64 if vb == 4 else width)), dtype=np.float32)
    v = None
    if vb != 4 or mb != 4:
        v = np.zeros(-(-n // 2) if vb == 4 else n, dtype=np.uint8 if vb < 16 else np.uint16)
    sa, sb = (float(x) for x in gold["scales"])
    for t in (1, 2, 3):
        packed = t < 3
        grad = gold[f"raw{t - 1}"] if packed else gold["dense"]
        part = O.adam_update(fmt, p, grad, m, v, ms, vs, step=t, key=12345 + 7919 * 3, hyper=hyper_for(gold, t), tail=tail,
                             unit=unit, grad_kind=2 if packed else 0, grad_cols=cols if packed else 1,
                             grad_stride=stride if packed else 1, sa=sa, sb=sb, extra=gold["extra"] if t == 2 else None)
        check(t, dict(p=p, m=m, v=v, ms=ms, vs=vs, tail=tail, unit=unit, part=part, scale=np.array([O.finish_scale(part)])))


@pytest.mark.parametrize("fmt", FORMATS)
def test_update_matches_reference(gold, fmt):
    def check(t, state):
        for name, got in state.items():
            if got is None:
                continue
            want = gold[f"{fmt}_s{t}_{name}"]
            same = np.array_equal(got.view(np.uint8) if got.dtype != np.uint8 else got, want.view(np.uint8) if want.dtype != np.uint8 else want)
            assert same, f"{fmt} step {t} {name}: {(got != want).sum()} of {got.size} differ"
    run_oracle_steps(gold, fmt, check)


def test_split_init_matches_reference(gold):
    w0 = gold["w0"]
    hi, _ = O.split_init(w0, 17)
    assert np.array_equal(hi, gold["half16_v8_p0"])
    hi, tail = O.split_init(w0, 24)
    assert np.array_equal(hi, gold["split24_v8_p0"]) and np.array_equal(tail, gold["split24_v8_tail0"])
    hi, _ = O.split_init(w0, 16)
    assert np.array_equal(hi, gold["sr16_v8_p0"])


def test_plain_small_tensor_path_matches_reference(gold):
    p, g = gold["plain_p0"].copy(), gold["plain_g"]
    m, v = np.zeros_like(p), np.zeros_like(p)
    for t in (1, 2):
        amax = O.adam_update_plain(p, g, m, v, hyper_for(gold, t))
        for name, got in (("p", p), ("m", m), ("v", v)):
            assert np.array_equal(got.view(np.uint32), gold[f"plain_s{t}_{name}"].view(np.uint32)), (t, name)
        assert np.float32(amax) == gold[f"plain_s{t}_part"].max()


@pytest.fixture(scope="module")
def gold_fp8():
    return np.load(GOLDEN / "fp8_master_reference.npz")


def test_fp8_master_unit_growth_matches_reference(gold_fp8):
    """tests/test_fp8_master_range.py:36-46 on the reference's own update kernel: an update beyond 448 x unit grows the
    units of exactly the first and the last 512-block; every byte of the other blocks stays."""
    g = gold_fp8
    lr, b1, b2, eps, wd = (float(x) for x in g["hyper"])
    p, unit = g["p0"].reshape(-1).copy(), g["unit0"].copy()
    n = p.size
    m, ms, vs = np.zeros(n, dtype=np.uint8), np.zeros(-(-n // 64), dtype=np.float32), np.zeros(-(-n // 64), dtype=np.float32)
    for t in (1, 2):
        part = O.adam_update("float8_m4v4_sqrt", p, g["grads"][t - 1], m, None, ms, vs, step=t, key=int(g["key"][0]),
                             hyper=O.adam_hyper(lr, (b1, b2), eps, wd, t), unit=unit, grad_kind=0)
        for name, got in (("p", p), ("unit", unit), ("m", m), ("ms", ms), ("vs", vs), ("part", part)):
            want = g[f"s{t}_{name}"].reshape(-1)
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), f"step {t} {name}"
        if t == 1:
            assert np.nonzero(unit > g["unit0"])[0].tolist() == [0, len(unit) - 1]
            assert np.array_equal(p[512:-512], g["p0"].reshape(-1)[512:-512])
            vals = O.from_bf16_bits(O.fp8_decoded(p, unit))
            assert 0.22 < -vals[1] < 0.29 and 0.22 < vals[-1] < 0.29


def test_fp8_master_encode_matches_reference(gold_fp8):
    """master8.encode == pair(decoded weight): both NVFP4 orientations straight from E4M3 codes and per-block units."""
    g = gold_fp8
    for p, unit, dec, scale, outs in ((g["s2_p"], g["s2_unit"], g["decoded"], g["enc_scale"], ("enc_d", "enc_s", "enc_dt", "enc_st")),
                                      (g["b_p"], g["b_unit"], g["b_decoded"], g["b_scale"], ("b_d", "b_s", "b_dt", "b_st"))):
        assert np.array_equal(O.fp8_decoded(p, unit), dec)
        row, col = O.fp8_weight_pair(p, unit, float(scale[0]))
        assert np.array_equal(row[0], g[outs[0]]) and np.array_equal(row[1], g[outs[1]])
        assert np.array_equal(col[0], g[outs[2]]) and np.array_equal(col[1], g[outs[3]])
