"""Build and call the plain-C oracle (`ndc_oracle.c`).  TEST INFRASTRUCTURE.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this.
`build()` compiles the C file with gcc into `oracle/libndc_oracle.so`; the wrappers take and
return numpy arrays (float64 or float32, contiguous, channels-first).
"""

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libndc_oracle.so")
_SRC = [os.path.join(_HERE, "ndc_oracle.c"), os.path.join(_HERE, "ndc_oracle_body.inc")]


class _Dims(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in
                ("B", "G", "m", "sc", "D", "H", "W", "kD", "kH", "kW")]


def build(force: bool = False) -> str:
    """Compile the oracle if the shared object is missing or older than its sources."""
    stale = force or not os.path.exists(_SO) or any(
        os.path.getmtime(s) > os.path.getmtime(_SO) for s in _SRC
    )
    if stale:
        subprocess.check_call(
            ["gcc", "-O2", "-std=c99", "-fopenmp", "-shared", "-fPIC", "-o", _SO, _SRC[0]],
            cwd=_HERE,
        )
    return _SO


_lib = None


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _dims(x_shape, groups, m, sc, ks):
    spatial = list(x_shape[2:])
    lead = 3 - len(spatial)
    d, h, w = [1] * lead + spatial
    kd, kh, kw = [1] * lead + list(ks)
    return _Dims(x_shape[0], groups, m, sc, d, h, w, kd, kh, kw)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def forward(x, z, h, bias, *, groups, m, sc, eps, relu_input):
    """Returns ``(out, t1)`` as numpy arrays of ``x.dtype``."""
    dt = x.dtype
    assert dt in (np.float64, np.float32)
    x, z, h = (np.ascontiguousarray(a, dtype=dt) for a in (x, z, h))
    bias = None if bias is None else np.ascontiguousarray(bias, dtype=dt)
    out = np.empty_like(z)
    t1 = np.empty_like(x)
    fn = getattr(_load(), "ndc_oracle_fwd_f64" if dt == np.float64 else "ndc_oracle_fwd_f32")
    fn.restype = ctypes.c_int
    dm = _dims(x.shape, groups, m, sc, h.shape[2:])
    rc = fn(ctypes.byref(dm), _ptr(x), _ptr(z), _ptr(h), _ptr(bias), ctypes.c_double(eps),
            ctypes.c_int(int(relu_input)), _ptr(out), _ptr(t1))
    if rc:
        raise MemoryError("C oracle: allocation failed")
    return out, t1


def backward(x, z, h, bias, gout, *, groups, m, sc, eps, relu_input):
    """Returns ``(gx, gz, gh, gb)`` as numpy arrays of ``x.dtype``."""
    dt = x.dtype
    assert dt in (np.float64, np.float32)
    x, z, h, gout = (np.ascontiguousarray(a, dtype=dt) for a in (x, z, h, gout))
    bias = None if bias is None else np.ascontiguousarray(bias, dtype=dt)
    gx, gz, gh = np.empty_like(x), np.empty_like(z), np.empty_like(h)
    gb = np.empty(groups * sc, dtype=dt)
    fn = getattr(_load(), "ndc_oracle_bwd_f64" if dt == np.float64 else "ndc_oracle_bwd_f32")
    fn.restype = ctypes.c_int
    dm = _dims(x.shape, groups, m, sc, h.shape[2:])
    rc = fn(ctypes.byref(dm), _ptr(x), _ptr(z), _ptr(h), _ptr(bias), _ptr(gout),
            ctypes.c_double(eps), ctypes.c_int(int(relu_input)),
            _ptr(gx), _ptr(gz), _ptr(gh), _ptr(gb))
    if rc:
        raise MemoryError("C oracle: allocation failed")
    return gx, gz, gh, gb


if __name__ == "__main__":
    print(build(force=True))
