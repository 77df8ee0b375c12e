"""Loss curve of NVFP4 full-parameter training against the same recipe in BF16 autocast with FP32 AdamW, over 200 steps
on the same seeded synthetic token stream.  Windowed means (20 steps) have to agree within 2 % wherever the curve is
flat enough for a vertical comparison (measured: 0.4 %, 0.2 %, 0.1 %, 0.3 % at steps 20, 100, 150, 200); through the
steep descent (loss 7.3 -> 1.8 between steps 20 and 100, where one step changes the loss by more than 2 %) the smoothed
NVFP4 curve has to stay within 2 % of the smoothed control curve shifted by at most four steps.

Two models: a small one (d 512), and two layers with the layer shapes, token count and learning rate of the 3.8 B benchmark
decoder (d 3072, 24 x 128 heads, SwiGLU 8192, 4 x 2048 tokens, lr 3e-4), where the rounding noise and the FP16 masters see
the magnitudes of the benchmark.  Measured there: 0.47 %, 0.38 %, 0.36 % at steps 100, 150, 200; its first 20-step window
lies in the initial collapse of the loss (10 -> 4) and is covered by the shifted-envelope criterion only."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

STEPS, WINDOW, TOLERANCE = 200, 20, 0.02
CFG = dict(layers=2, dim=512, heads=4, ffn=1536, vocab=2048, seq=256)
RECIPE = dict(lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)


def token_stream(steps, batch, seq, vocab, seed):
    """A first-order Markov source: next = (7 * token + 3 + small noise) mod vocab.  Learnable, not memorisable."""
    g = torch.Generator().manual_seed(seed)
    first = torch.randint(0, vocab, (steps, batch, 1), generator=g)
    noise = torch.randint(0, 4, (steps, batch, seq), generator=g)
    out = [first]
    for t in range(seq):
        out.append((out[-1] * 7 + 3 + noise[:, :, t:t + 1]) % vocab)
    return torch.cat(out, dim=2)


def windowed(losses, lo, hi):
    return sum(losses[lo:hi]) / (hi - lo)


# the layer shapes of the 3.8 B benchmark decoder (d 3072, 24 heads of 128, SwiGLU 8192) at its 4 x 2048 tokens per step
# and its learning rate; two layers and a small vocabulary keep the run to seconds
CFG_WIDE = dict(layers=2, dim=3072, heads=24, ffn=8192, vocab=2048, seq=2048)
RECIPE_WIDE = dict(lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)


@pytest.mark.parametrize("CFG,RECIPE,BATCH,FLAT_FROM", [(CFG, RECIPE, 8, 20), (CFG_WIDE, RECIPE_WIDE, 4, 100)],
                         ids=["d512", "benchmark_layer_shapes"])
def test_nvfp4_tracks_bf16_within_two_percent(CFG, RECIPE, BATCH, FLAT_FROM):
    import nvfp4_training as nv
    from nvfp4_training._workloads.llama import Decoder, token_loss, warm_attention
    from nvfp4_training._runtime import load_runtime
    device = torch.device("cuda")
    torch.manual_seed(0)
    with torch.device(device):
        base = Decoder(**CFG)
    ids = token_stream(STEPS, BATCH, CFG["seq"], CFG["vocab"], seed=0).to(device)

    # BF16 autocast control: FP32 master weights, torch.optim.AdamW (fused), same hyper-parameters
    control = copy.deepcopy(base)
    opt = torch.optim.AdamW(control.parameters(), fused=True, **RECIPE)
    ref = []
    for s in range(STEPS):
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = token_loss(control, ids[s, :, :-1].contiguous(), ids[s, :, 1:].contiguous())
        loss.backward()
        opt.step()
        ref.append(loss.item())

    load_runtime()[2].reset_stats(0)
    model = nv.enable_nvfp4(copy.deepcopy(base), profile="balanced", lr=RECIPE["lr"], betas=RECIPE["betas"],
                            weight_decay=RECIPE["weight_decay"], eps=RECIPE["eps"])
    warm_attention(model, BATCH, CFG["seq"], device)
    got = []
    with nv.capture_step(model, token_loss, ids[0, :, :-1], ids[0, :, 1:], steps=STEPS) as graph:
        for s in range(STEPS):
            got.append(graph.step(ids[s, :, :-1], ids[s, :, 1:]).item())
    nv.check_finite(model)

    assert ref[-1] < 0.7 * ref[0], "the control run has to learn for the comparison to mean anything"
    rows = [(hi, windowed(got, hi - WINDOW, hi), windowed(ref, hi - WINDOW, hi)) for hi in (20, 100, 150, 200)]
    print("window end, nvfp4, bf16:", rows)
    for hi, a, b in rows:
        assert hi < FLAT_FROM or abs(a - b) / b <= TOLERANCE, rows
    # whole curve: 5-step means of the NVFP4 run against the envelope of the control's 5-step means within +-4 steps
    # (measured worst deviation 0.75 %; the NVFP4 run trails the control by about two steps in the steep part)
    smooth = lambda xs: [sum(xs[i:i + 5]) / 5 for i in range(len(xs) - 4)]
    a, b = smooth(got), smooth(ref)
    outside = []
    for s in range(16, len(a)):
        near = b[max(0, s - 4): s + 5]
        if not min(near) * (1 - TOLERANCE) <= a[s] <= max(near) * (1 + TOLERANCE):
            outside.append((s, a[s], min(near), max(near)))
    assert not outside, outside
