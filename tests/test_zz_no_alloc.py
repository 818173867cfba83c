"""`ndc_bwd_static`: the backward entry point for callers that cannot allocate.

Some hosts of the library (a plugin inside another framework's memory plan, a loop that
forbids cudaMalloc after start-up) have no allocator to take the backward pass's scratch
from, so this entry point keeps the scratch in a fixed array inside the library.  The test
calls it through the C ABI, twice in a row on different inputs, and checks every output
against the regular `ndc_bwd` entry point (same kernels, caller-provided workspace): the
results must be identical, and the second call must leave the device's free memory and
torch's allocator untouched.  It also checks that a geometry beyond the built-in array is
refused with a status, not run.

This file is named so that pytest collects it last.
"""

import pytest
import torch

from deconver_b200 import _lib

pytestmark = pytest.mark.gpu

CASES = [
    # batch, groups, m, sc, spatial, kernel   (depthwise tiled path, then the generic path)
    (2, 8, 1, 4, (10, 12, 16), (3, 3, 3)),
    (1, 6, 1, 4, (33, 40), (5, 5)),
    (2, 3, 2, 3, (6, 7, 5), (3, 3, 3)),
]


def _problem(case, seed, dev):
    B, G, m, sc, spatial, ks = case
    gen = torch.Generator(device=dev).manual_seed(seed)
    x = torch.rand(B, G * m, *spatial, device=dev, generator=gen)
    z = torch.randn(B, G * sc, *spatial, device=dev, generator=gen) * 0.5 + 0.3
    h = torch.rand(G * m, sc, *ks, device=dev, generator=gen) / 27
    bias = torch.randn(G * sc, device=dev, generator=gen) * 0.1
    gout = torch.randn(B, G * sc, *spatial, device=dev, generator=gen)
    desc = _lib.make_desc(B, G, m, sc, spatial, ks, 1e-16, True, _lib.NDC_F32)
    return desc, x, z, h, bias, gout


def _outputs(x, z, h, bias):
    return (torch.empty_like(x), torch.empty_like(z), torch.empty_like(h), torch.empty_like(bias))


@pytest.mark.parametrize("case", CASES, ids=["dw3d", "dw2d", "generic"])
def test_static_workspace_backward_matches_regular_backward(case):
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    for seed in (1, 2):  # two calls in a row: the second one finds the first one's leftovers
        desc, x, z, h, bias, gout = _problem(case, seed, dev)
        out, t1 = torch.empty_like(z), torch.empty_like(x)
        _lib.check(lib.ndc_fwd(desc, x.data_ptr(), z.data_ptr(), h.data_ptr(), bias.data_ptr(),
                               out.data_ptr(), t1.data_ptr(), st))
        need = lib.ndc_bwd_workspace_bytes(desc)
        assert 0 < need <= _lib.STATIC_WORKSPACE_BYTES
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        ref = _outputs(x, z, h, bias)
        _lib.check(lib.ndc_bwd(desc, x.data_ptr(), z.data_ptr(), t1.data_ptr(), h.data_ptr(),
                               bias.data_ptr(), gout.data_ptr(), *[t.data_ptr() for t in ref],
                               ws.data_ptr(), need, st))
        got = _outputs(x, z, h, bias)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(dev)
        held_before = torch.cuda.memory_allocated(dev)
        _lib.check(lib.ndc_bwd_static(desc, x.data_ptr(), z.data_ptr(), t1.data_ptr(),
                                      h.data_ptr(), bias.data_ptr(), gout.data_ptr(),
                                      *[t.data_ptr() for t in got], st))
        torch.cuda.synchronize()
        if seed == 2:
            # the array exists since the first call: this one takes no device memory at all,
            # neither from the driver nor from torch's allocator
            assert torch.cuda.mem_get_info(dev)[0] >= free_before
            assert torch.cuda.memory_allocated(dev) == held_before
        for name, a, b in zip(("gx", "gz", "gh", "gb"), got, ref):
            assert torch.isfinite(b).all(), name
            assert torch.equal(a, b), f"{name} differs between ndc_bwd_static and ndc_bwd (seed {seed})"


def test_static_workspace_refuses_what_does_not_fit():
    lib = _lib.load()
    desc = _lib.make_desc(2, 64, 1, 4, (64, 64, 64), (3, 3, 3), 1e-16, True, _lib.NDC_F32)
    assert lib.ndc_bwd_workspace_bytes(desc) > _lib.STATIC_WORKSPACE_BYTES
    dev = torch.device("cuda:0")
    t = torch.zeros(16, device=dev)
    p = t.data_ptr()
    status = lib.ndc_bwd_static(desc, p, p, p, p, None, p, p, p, None, None,
                                torch.cuda.current_stream().cuda_stream)
    assert status == 3
    assert b"ndc_bwd_static" in lib.ndc_last_error()
    torch.cuda.synchronize()
