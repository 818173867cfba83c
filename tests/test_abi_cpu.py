"""The C-ABI library loads without a GPU and exports every symbol the header declares.
No compute call is made here; only host-side queries."""

import ctypes
import os
import re

import pytest

from conftest import ROOT
from deconver_b200 import _lib
from deconver_b200._build import build_library


@pytest.fixture(scope="module")
def lib():
    build_library()
    return _lib.load()


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "ndc_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ndc_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    declared = _declared_functions()
    assert declared, "no declarations parsed from the header"
    assert sorted(_lib.SYMBOLS) == declared
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"


def test_descriptor_layout():
    # 10 int32 + float + 3 int32, no padding: the struct the header declares
    assert ctypes.sizeof(_lib.NdcDesc) == 56
    assert _lib.NdcDesc.eps.offset == 40 and _lib.NdcDesc.flags.offset == 52


def test_version_and_status_strings(lib):
    assert lib.ndc_version() == 1
    assert lib.ndc_status_string(0) == b"ok"
    for code in range(1, 6):
        assert lib.ndc_status_string(code) not in (b"ok", b"unknown status")
    assert lib.ndc_status_string(99) == b"unknown status"


def _desc(**kw):
    base = dict(batch=2, groups=8, m=1, sc=4, spatial=(6, 5, 7), kernel_size=(3, 3, 3),
                eps=1e-16, relu_input=True, dtype_code=_lib.NDC_F32)
    base.update(kw)
    return _lib.make_desc(**base)


def test_query_accepts_and_rejects(lib):
    path = ctypes.c_int32(-1)
    assert lib.ndc_query(_desc(), ctypes.byref(path)) == 0
    assert path.value == _lib.PATH_DEPTHWISE4
    # which family takes which geometry (host-side decision, no GPU needed)
    img = dict(groups=32, kernel_size=(5, 5))
    for spatial, want in [((256, 256), _lib.PATH_DEPTHWISE4_ROWS),    # the 2-D benchmark layer
                          ((128, 128), _lib.PATH_DEPTHWISE4_ROWS),
                          ((40, 65), _lib.PATH_DEPTHWISE4_ROWS),
                          ((64, 64), _lib.PATH_DEPTHWISE4_ROWS),      # two images side by side per CTA
                          ((6, 200), _lib.PATH_DEPTHWISE4),           # too few rows to march
                          ((64, 300), _lib.PATH_DEPTHWISE4_ROWS),     # one wide image per 128-thread CTA
                          ((64, 600), _lib.PATH_GENERIC)]:            # wider than a tile
        assert lib.ndc_query(_desc(spatial=spatial, **img), ctypes.byref(path)) == 0
        assert path.value == want, (spatial, path.value)
    # a single narrow image cannot fill a row CTA: band kernels
    assert lib.ndc_query(_desc(batch=1, spatial=(64, 64), **img), ctypes.byref(path)) == 0
    assert path.value == _lib.PATH_DEPTHWISE4
    assert lib.ndc_query(_desc(batch=16, groups=512, spatial=(32, 16), kernel_size=(5, 5)),
                         ctypes.byref(path)) == 0
    assert path.value == _lib.PATH_DEPTHWISE4_ROWS                    # sixteen images per CTA
    assert lib.ndc_query(_desc(groups=4, spatial=(128, 128), kernel_size=(3, 3)), ctypes.byref(path)) == 0
    assert path.value == _lib.PATH_DEPTHWISE4_ROWS
    assert lib.ndc_query(_desc(groups=4, spatial=(3, 40, 100), kernel_size=(1, 5, 5)),
                         ctypes.byref(path)) == 0
    assert path.value == _lib.PATH_DEPTHWISE4                         # a volume is not an image
    assert lib.ndc_query(_desc(groups=4, m=2), ctypes.byref(path)) == 0
    assert path.value == _lib.PATH_GENERIC                            # grouped, not depthwise
    assert lib.ndc_query(_desc(flags=_lib.FLAG_FORCE_GENERIC), ctypes.byref(path)) == 0
    assert path.value == _lib.PATH_GENERIC
    assert lib.ndc_query(_desc(kernel_size=(3, 4, 3)), None) == 1  # even kernel
    assert b"odd" in lib.ndc_last_error()
    assert lib.ndc_query(_desc(batch=0), None) == 1
    assert lib.ndc_query(_desc(dtype_code=7), None) == 1
    assert lib.ndc_query(_desc(flags=64), None) == 1
    assert lib.ndc_query(_desc(m=17), None) == 2  # beyond the kernels' channel limit
    assert lib.ndc_query(None, None) == 1


def test_workspace_query(lib):
    assert lib.ndc_bwd_workspace_bytes(_desc()) > 0
    assert lib.ndc_bwd_workspace_bytes(_desc(kernel_size=(2, 3, 3))) == 0
    big = lib.ndc_bwd_workspace_bytes(_desc(batch=32, groups=64, spatial=(128, 128, 128)))
    assert big > 0  # 64-bit size arithmetic: no overflow on >2^31-element tensors


def test_null_pointers_are_refused_without_touching_the_gpu(lib):
    d = _desc()
    assert lib.ndc_fwd(d, None, None, None, None, None, None, None) == 1
    assert b"NULL" in lib.ndc_last_error()
    assert lib.ndc_bwd(d, None, None, None, None, None, None, None, None, None, None, None, 0,
                       None) == 1
    assert lib.ndc_gconv(d, None, None, None, 0, None, None) == 1


def test_rank_padding():
    d = _lib.make_desc(1, 4, 1, 4, (11,), (5,), 1e-16, True, 0)
    assert (d.D, d.H, d.W, d.kD, d.kH, d.kW) == (1, 1, 11, 1, 1, 5)
    d = _lib.make_desc(1, 4, 1, 4, (9, 8), (3, 5), 1e-16, False, 1)
    assert (d.D, d.H, d.W, d.kD, d.kH, d.kW) == (1, 9, 8, 1, 3, 5)
    with pytest.raises(ValueError):
        _lib.make_desc(1, 4, 1, 4, (2, 2, 2, 2), (3, 3, 3, 3), 0.0, True, 0)
    with pytest.raises(ValueError):
        _lib.make_desc(1, 4, 1, 4, (9, 8), (3,), 0.0, True, 0)


def test_planner_on_random_geometries(lib):
    """Host-side planning (kernel family, tiling, workspace size) over a seeded sweep of
    geometries, including degenerate and very large ones: every query answers, the workspace
    is bounded by the scratch tensors the backward needs, and repeated queries agree."""
    import numpy as np

    rng = np.random.default_rng(7)
    path = ctypes.c_int32(-1)
    kernels = [(3, 3, 3), (5, 5), (3, 3), (1, 5, 5), (7,), (5, 5, 5), (3, 5)]
    for _ in range(400):
        ks = kernels[int(rng.integers(len(kernels)))]
        hi = {1: 5000, 2: 700, 3: 200}[len(ks)]
        spatial = tuple(int(rng.integers(1, hi)) for _ in ks)
        batch, groups = int(rng.integers(1, 33)), int(2 ** rng.integers(0, 10))
        m, sc = (1, 4) if rng.random() < 0.8 else (int(rng.integers(1, 5)), int(rng.integers(1, 9)))
        elems = batch * groups * int(np.prod(spatial))
        if elems * max(m, sc) >= 2 ** 40:
            continue
        d = _desc(batch=batch, groups=groups, m=m, sc=sc, spatial=spatial, kernel_size=ks)
        assert lib.ndc_query(d, ctypes.byref(path)) == 0, (batch, groups, m, sc, spatial, ks)
        assert path.value in (_lib.PATH_GENERIC, _lib.PATH_DEPTHWISE4, _lib.PATH_DEPTHWISE4_ROWS)
        if (m, sc) != (1, 4) or ks in [(7,), (5, 5, 5), (3, 5)]:
            assert path.value == _lib.PATH_GENERIC
        need = lib.ndc_bwd_workspace_bytes(d)
        assert need == lib.ndc_bwd_workspace_bytes(d)
        # gnum, gden (float32, source-sized), gt1 and a spare input-sized tensor, plus the
        # per-CTA records of the filter-gradient reduction (a few percent at most)
        bound = int(4 * elems * (2 * sc + 2 * m) * 1.05) + 64 * 1024 * 1024 + 4096 * batch * groups
        assert 0 < need <= bound, (need, bound, batch, groups, m, sc, spatial, ks)


def test_instance_norm_and_probe_entry_points_validate_without_a_gpu(lib):
    assert lib.ndc_inorm_workspace_bytes(2, 64) == 2 * 64 * 64 * 2 * 4
    assert lib.ndc_inorm_workspace_bytes(0, 64) == 0
    assert lib.ndc_inorm_fwd(2, 64, 4096, 0, None, None, None, 1e-5, None, None, None, 0, None) == 1
    assert b"NULL" in lib.ndc_inorm_last_error()
    assert lib.ndc_inorm_bwd(2, 64, 4096, 0, None, None, None, None, None, None, None, None, 0,
                             None) == 1
    assert lib.ndc_probe_fp32_fma(0, 0, None, 0, None, None) == 1
    assert b"iters" in lib.ndc_last_error()


def test_bias_entry_points_validate_without_a_gpu(lib):
    assert lib.ndc_bias_grad_workspace_bytes(2, 64) == 2 * 64 * 64 * 4
    assert lib.ndc_bias_add(2, 64, 4096, 0, None, None, None) == 1
    assert b"NULL" in lib.ndc_bias_last_error()
    assert lib.ndc_bias_grad(2, 64, 4096, 0, None, None, None, 0, None) == 1
    assert lib.ndc_bias_gelu_fwd(2, 64, 4096, 0, None, None, None, None) == 1
    assert b"NULL" in lib.ndc_bias_last_error()
    assert lib.ndc_bias_gelu_bwd(2, 64, 4096, 0, None, None, None, None, None, None, 0, None) == 1
    assert lib.ndc_bias_gelu_fwd(0, 64, 4096, 0, 16, None, 16, None) == 1
    assert b"positive" in lib.ndc_bias_last_error()
    assert lib.ndc_bias_gelu_fwd(2, 64, 4096, 7, 16, None, 16, None) == 1
    assert b"dtype" in lib.ndc_bias_last_error()
