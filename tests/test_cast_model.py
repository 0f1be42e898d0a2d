"""``cast_model`` (modelled on the reference's ``test/test_optimizers.py:1052-1329``)."""

import pytest
import torch
import torch.nn as nn

from flashoptim_b200 import cast_model


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv = nn.Conv2d(3, 4, 3)
        self.bn = nn.BatchNorm2d(4)
        self.inorm = nn.InstanceNorm2d(4, affine=True, track_running_stats=True)
        self.gn = nn.GroupNorm(2, 4)
        self.ln = nn.LayerNorm(4)
        self.body = nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.Linear(8, 8))
        self.head = nn.Linear(8, 5)
        self.register_buffer("counter", torch.zeros(1, dtype=torch.long))
        self.register_buffer("scale", torch.ones(1))

    def forward(self, x):
        x = self.gn(self.inorm(self.bn(self.conv(x))))
        x = self.ln(x.mean((2, 3)))
        return self.head(self.body(x))


def test_default_cast_keeps_stateful_norms_fp32():
    m = Net()
    cast_model(m)
    assert m.conv.weight.dtype == torch.bfloat16 and m.head.bias.dtype == torch.bfloat16
    assert m.gn.weight.dtype == torch.bfloat16 and m.ln.weight.dtype == torch.bfloat16
    for mod in (m.bn, m.inorm):
        assert mod.weight.dtype == torch.float32 and mod.running_mean.dtype == torch.float32
    assert m.counter.dtype == torch.long and m.scale.dtype == torch.bfloat16


def test_non_selective_casts_everything():
    m = Net()
    cast_model(m, dtype=torch.float16, selective=False)
    assert m.bn.weight.dtype == torch.float16 and m.bn.running_var.dtype == torch.float16
    assert m.bn.num_batches_tracked.dtype == torch.long


@pytest.mark.parametrize("spec", ["head", "he*", "module"])
def test_full_precision_layer_keeps_fp32_output(spec):
    m = Net()
    cast_model(m, full_precision_layers=[m.head if spec == "module" else spec])
    assert m.head.weight.dtype == torch.float32 and m.body[0].weight.dtype == torch.bfloat16
    out = m(torch.randn(2, 3, 8, 8).bfloat16())
    assert out.dtype == torch.float32
    assert m.head._has_fp32_input_hook


def test_recast_layer_returns_to_narrow_dtype():
    m = Net()
    cast_model(m, full_precision_recast_layers=["body.0"])
    assert m.body[0].weight.dtype == torch.float32 and m.body[2].weight.dtype == torch.bfloat16
    seen = {}
    m.body[0].register_forward_hook(lambda mod, i, o: seen.update({"in": i[0].dtype}))
    out = m(torch.randn(2, 3, 8, 8).bfloat16())
    assert seen["in"] == torch.float32 and out.dtype == torch.bfloat16


def test_nested_names_need_a_wildcard():
    m = Net()
    cast_model(m, full_precision_layers=["0"])  # 'body.0' is not matched by '0'
    assert m.body[0].weight.dtype == torch.bfloat16
    m = Net()
    cast_model(m, full_precision_layers=["*.0"])
    assert m.body[0].weight.dtype == torch.float32


def test_hooks_are_registered_once():
    m = Net()
    cast_model(m, full_precision_layers=["head"])
    cast_model(m, full_precision_layers=["head"])
    assert len(m.head._forward_pre_hooks) == 1


def test_tied_parameters_stay_tied():
    emb = nn.Embedding(10, 4)
    head = nn.Linear(4, 10, bias=False)
    head.weight = emb.weight
    m = nn.ModuleDict({"emb": emb, "head": head})
    cast_model(m)
    assert m["emb"].weight is m["head"].weight and m["emb"].weight.dtype == torch.bfloat16
    # tied by storage only (two Parameter objects over one tensor)
    a, b = nn.Linear(4, 4, bias=False), nn.Linear(4, 4, bias=False)
    b.weight = nn.Parameter(a.weight.data)
    m2 = nn.Sequential(a, b)
    cast_model(m2)
    assert m2[0].weight.data_ptr() == m2[1].weight.data_ptr()


def test_tuple_outputs_are_recast():
    class Two(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(4, 4)

        def forward(self, x):
            return self.lin(x), 3, self.lin(x) * 2

    class Wrap(nn.Module):
        def __init__(self):
            super().__init__()
            self.two = Two()

        def forward(self, x):
            return self.two(x)

    m = Wrap()
    cast_model(m, full_precision_recast_layers=["two"])
    a, k, b = m(torch.randn(2, 4).bfloat16())
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and k == 3


def test_meta_device_parameters_are_not_merged():
    with torch.device("meta"):
        m = nn.Sequential(nn.Linear(4, 8), nn.Linear(8, 2))
    cast_model(m)
    assert m[0].weight.shape == (8, 4) and m[1].weight.shape == (2, 8)
    assert m[0].weight.dtype == torch.bfloat16 and m[0].weight.device.type == "meta"


def test_parameter_shared_by_two_modules_is_converted_once():
    """One Parameter object registered in two modules (how Hugging Face ties an output
    bias) is visited twice; the second visit must not pick up some other tensor that
    happens to live where a released fp32 tensor used to be."""

    class Owner(nn.Module):
        def __init__(self):
            super().__init__()
            self.bias = nn.Parameter(torch.randn(32))  # 64 bytes once narrowed ...

    class Head(nn.Module):
        def __init__(self, bias):
            super().__init__()
            self.decoder = nn.Linear(16, 32, bias=False)
            self.decoder.bias = bias  # same Parameter object as the owner's

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            # ... the size of the fp32 biases released just before it is converted
            self.body = nn.ModuleList([nn.Linear(16, 16) for _ in range(64)])
            self.owner = Owner()
            self.head = Head(self.owner.bias)

    for seed in range(5):
        torch.manual_seed(seed)
        m = Net()
        want = {n: p.detach().to(torch.bfloat16) for n, p in m.named_parameters(remove_duplicate=False)}
        cast_model(m, torch.bfloat16)
        assert m.head.decoder.bias is m.owner.bias
        for n, p in m.named_parameters(remove_duplicate=False):
            assert p.shape == want[n].shape and torch.equal(p, want[n]), n


def test_views_of_one_storage_with_different_shapes_are_cast_separately():
    m = nn.Module()
    base = torch.randn(4, 4)
    m.a = nn.Parameter(base)
    m.b = nn.Parameter(base.view(16))  # same address, other shape: not a tie cast_model can keep
    cast_model(m, torch.bfloat16)
    assert m.a.shape == (4, 4) and m.b.shape == (16,)
    assert torch.equal(m.a.view(16), m.b)
