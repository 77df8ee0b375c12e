"""Selection policy of pack_frozen_layers: every rejection happens before a module is touched and before any GPU work,
so these run without a device.  Cases follow the reference's tests/test_frozen.py:11-34."""
import pytest
from torch import nn

from nvfp4_training import pack_frozen_layers
from nvfp4_training import frozen


def test_reject_trainable_before_mutation():
    m = nn.Sequential(nn.Linear(8, 8).requires_grad_(False), nn.Linear(8, 8))
    with pytest.raises(ValueError):
        pack_frozen_layers(m, include=("*",))
    assert type(m[0]) is nn.Linear


def test_patterns_must_be_sequences():
    m = nn.Sequential(nn.Linear(8, 8).requires_grad_(False))
    with pytest.raises(ValueError):
        pack_frozen_layers(m, include="0")
    with pytest.raises(ValueError):
        pack_frozen_layers(m, include=("0",), keep="0")


def test_reject_unsupported_convolution():
    m = nn.Sequential(nn.Conv2d(8, 8, 3).requires_grad_(False))
    with pytest.raises(ValueError, match="unsupported selected layer"):
        pack_frozen_layers(m, include=("*",))


def test_reject_aliases():
    layer = nn.Linear(8, 8).requires_grad_(False)
    m = nn.ModuleDict({"first": layer, "second": layer})
    with pytest.raises(ValueError, match="aliases"):
        pack_frozen_layers(m, include=("*",))


def test_reject_shared_boundary_weight():
    m = nn.ModuleDict({"core": nn.Linear(8, 8), "boundary": nn.Linear(8, 8)}).requires_grad_(False)
    m["boundary"].weight = m["core"].weight
    with pytest.raises(ValueError, match="Shared parameters"):
        pack_frozen_layers(m, include=("core",))


def test_protected_attention_descendant():
    m = nn.MultiheadAttention(8, 2).requires_grad_(False)
    with pytest.raises(ValueError, match="No eligible"):
        pack_frozen_layers(m, include=("*",), keep=("out_proj",))


def test_pattern_matches_ancestors():
    assert frozen._matches("blocks.3.mlp.up", ("blocks.3",))
    assert frozen._matches("blocks.3.mlp.up", ("*.up",))
    assert not frozen._matches("blocks.3.mlp.up", ("blocks.4",))
    assert frozen._matches("", ("*",))


def test_plan_lists_kinds_and_skips():
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.stem = nn.Conv2d(4, 8, 1)
            self.attn = nn.MultiheadAttention(8, 2, batch_first=True)
            self.head = nn.Linear(8, 3)
    net = Net().requires_grad_(False)
    planned, skipped = frozen._plan(net, ("*",), ("head",))
    assert [(n, k) for n, _, k in planned] == [("stem", "pointwise"), ("attn", "mha")]
    assert skipped == [dict(name="head", reason="not selected or protected")]
