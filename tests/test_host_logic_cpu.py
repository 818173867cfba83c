"""Host-side mirror of the reference's layer interface: constructor, state dict, dispatch.
Modelled on the reference's `tests/test_deconv_equivalence.py:244-254` (state-dict round
trip) and `tests/test_deconver.py` (shape/smoke), minus anything that needs a GPU."""

import contextlib

import pytest
import torch

import deconver_b200 as dcb
from conftest import load_golden
from deconver_b200._build import build_library


@pytest.fixture(scope="module", autouse=True)
def _built():
    build_library()


def test_constructor_defaults_and_derived_attributes():
    m = dcb.Deconv(64, (3, 3, 3), ratio=4)
    assert (m.groups, m.source_channels, m.filter_channels) == (64, 4, 1)
    assert (m.eps, m.num_iters, m.num_grad_iters) == (1e-16, 1, 1)
    assert m.init.h0.shape == (64, 4, 3, 3, 3)
    assert m.init.linear.linear.weight.shape == (256, 64, 1)
    m = dcb.NDC(12, (3, 3, 3), ratio=2, groups=3, num_iters=4, num_grad_iters=2)
    assert (m.groups, m.source_channels, m.filter_channels) == (3, 8, 4)
    assert m.init.h0.shape == (12, 8, 3, 3, 3)
    m = dcb.Deconv(8, (5,), source_channels=3)
    assert m.source_channels == 3
    with pytest.raises(AssertionError):
        dcb.Deconv(10, (3, 3), groups=4)


def test_state_dict_is_the_reference_layout():
    g = load_golden("layer_dw3d")
    m = dcb.Deconv(16, (3, 3, 3), ratio=4, groups=-1)
    assert list(m.state_dict().keys()) == [
        "init.h0", "init.linear.linear.weight", "init.linear.linear.bias"]
    state = {
        "init.h0": torch.from_numpy(g["h0"]),
        "init.linear.linear.weight": torch.from_numpy(g["weight"]),
        "init.linear.linear.bias": torch.from_numpy(g["bias"]),
    }
    m.load_state_dict(state, strict=True)  # a checkpoint of the reference loads as is
    for k, v in state.items():
        assert torch.equal(m.state_dict()[k], v)


def test_same_seed_same_initialisation_as_the_reference_fixture():
    # the fixture's parameters were drawn by the reference under seed 0 (bias shifted by +1)
    g = load_golden("layer_dw3d")
    torch.manual_seed(0)
    m = dcb.Deconv(16, (3, 3, 3), ratio=4, groups=-1, num_iters=1)
    assert torch.equal(m.init.h0.detach(), torch.from_numpy(g["h0"]))
    assert torch.equal(m.init.linear.linear.weight.detach(), torch.from_numpy(g["weight"]))
    assert torch.allclose(m.init.linear.linear.bias.detach() + 1.0, torch.from_numpy(g["bias"]))


def test_no_grad_window():
    m = dcb.Deconv(8, (3, 3, 3), ratio=2, num_iters=5, num_grad_iters=2)
    kinds = [type(m.context(it)) for it in range(1, 6)]
    assert kinds[:3] == [torch.no_grad] * 3
    assert kinds[3:] == [contextlib.nullcontext] * 2


@pytest.mark.parametrize("kwargs,fragment", [
    (dict(update_filter=True), "update_filter"),
    (dict(update_source=False), "update_source"),
    (dict(verbose=True), "verbose"),
    (dict(stride=1), "stride"),
])
def test_unsupported_configurations_raise(kwargs, fragment):
    m = dcb.Deconv(8, (3, 3, 3), ratio=2, **kwargs)
    assert not m.fast_path_applicable()
    assert fragment in m.unsupported_reason()
    with pytest.raises(NotImplementedError, match=fragment):
        m(torch.zeros(1, 8, 4, 4, 4))


def test_even_kernel_raises():
    m = dcb.Deconv(8, (4, 4), ratio=2)
    with pytest.raises(NotImplementedError, match="even"):
        m(torch.zeros(1, 8, 6, 6))


def test_cpu_tensors_are_refused_not_computed():
    m = dcb.Deconv(8, (3, 3, 3), ratio=4)
    with pytest.raises(NotImplementedError, match="CUDA only"):
        m(torch.rand(1, 8, 4, 4, 4))
    x, z = torch.rand(1, 8, 4, 4, 4), torch.rand(1, 32, 4, 4, 4)
    with pytest.raises(RuntimeError, match="no CPU path"):
        dcb.deconv_update(x, z, torch.rand(8, 4, 3, 3, 3), None, groups=8, m=1, sc=4,
                          eps=1e-16, relu_input=True)


def test_reconstruct_and_loss_shapes():
    m = dcb.Deconv(12, (3, 3, 3), ratio=2, groups=3)
    s = torch.rand(2, 24, 5, 4, 6)
    h = torch.rand(2, 12, 8, 3, 3, 3)
    x_hat = m.reconstruct(s, h)
    assert x_hat.shape == (2, 12, 5, 4, 6)
    loss = m.loss(m.split_channels(x_hat), m.split_channels(s), m.split_channels(h))
    assert loss.shape == (6,) and float(loss.max()) < 1e-6


def test_bench_reads_the_tracked_traffic_summary():
    """`roofline.traffic` comes from the tracked ncu summary, scaled by the batch; both arms of
    the benchmark print the same `config` object."""
    import re

    import bench

    traffic, source = bench.load_traffic(2)
    text = open(bench.TRAFFIC_FILE).read()
    rows = re.findall(r"^#\s+\w+_kernel\s+(\d+)\s+(\d+)\s*$", text, re.M)
    assert rows, "the summary lists the kernels it adds up"
    total_mb = sum(int(a) + int(b) for a, b in rows)
    assert traffic == 2 * total_mb * 1000 * 1000
    assert "profiles/" in source
    assert bench.config_of(4)["global_batch"] == 8
    assert bench.config_of(1) == bench.config_of(1)


def test_instance_norm_module_host_logic():
    """Constructor, state-dict keys and refusals of the instance-norm modules (no GPU needed)."""
    import deconver_b200 as dcb

    for mine, theirs in ((dcb.InstanceNorm3d(8), torch.nn.InstanceNorm3d(8)),
                         (dcb.InstanceNorm2d(8, affine=True), torch.nn.InstanceNorm2d(8, affine=True))):
        assert sorted(mine.state_dict()) == sorted(theirs.state_dict())
        mine.load_state_dict(theirs.state_dict())
    with pytest.raises(NotImplementedError):
        dcb.InstanceNorm3d(8, track_running_stats=True)
    with pytest.raises(RuntimeError, match="CUDA"):
        dcb.InstanceNorm1d(4)(torch.randn(2, 4, 10))          # there is no CPU path
    with pytest.raises(ValueError):
        dcb.InstanceNorm2d(4)(torch.randn(2, 4, 10))


def test_mlp_cpu_tensors_run_the_plain_sequence():
    m = dcb.MLP(4, out_channels=6, ratio=2, dropout=(0.0, 0.0))
    x = torch.randn(2, 4, 5, 5)
    ref = m.block(x)
    assert torch.equal(m(x), ref) and ref.shape == (2, 6, 5, 5)


def test_linear_and_mlp_keep_the_reference_state_dict_layout():
    """Against an installation of the reference where there is one (`baseline/_ref`): same
    state-dict keys and shapes for `Linear` (`layers/linear.py`) and `MLP` (`layers/mlp.py`),
    and weights move both ways."""
    import os
    import sys
    ref_root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "deconver")):
        pytest.skip("no reference installation under baseline/_ref")
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    from deconver.layers.linear import Linear as RefLinear
    from deconver.layers.mlp import MLP as RefMLP
    pairs = [(RefLinear(6, 10), dcb.Linear(6, 10)), (RefLinear(6, 10, bias=False), dcb.Linear(6, 10, bias=False)),
             (RefMLP(8, ratio=4), dcb.MLP(8, ratio=4)), (RefMLP(8, 5, hidden_channels=12), dcb.MLP(8, 5, hidden_channels=12))]
    x = {6: torch.randn(2, 6, 4, 5), 8: torch.randn(2, 8, 3, 3, 3)}
    for ref, mine in pairs:
        ref_sd, my_sd = ref.state_dict(), mine.state_dict()
        assert list(ref_sd) == list(my_sd)
        assert [tuple(v.shape) for v in ref_sd.values()] == [tuple(v.shape) for v in my_sd.values()]
        mine.load_state_dict(ref_sd, strict=True)
        ref.load_state_dict(mine.state_dict(), strict=True)
        inp = x[next(iter(ref_sd.values())).shape[1]]
        assert torch.allclose(ref(inp), mine(inp), atol=1e-6)     # CPU tensors: the plain sequence
