"""ctypes binding of `libndc_b200.so` (the C ABI declared in `include/ndc_b200.h`).

The library is the only compute path of this package.  If it has not been built the loader
raises; nothing falls back to PyTorch or to the CPU.
"""

import ctypes
import os

from ._build import LIB

NDC_F32, NDC_BF16 = 0, 1
NDC_OK = 0
PATH_GENERIC, PATH_DEPTHWISE4, PATH_DEPTHWISE4_ROWS = 0, 1, 2
STATIC_WORKSPACE_BYTES = 16 * 1024 * 1024
FLAG_FORCE_GENERIC = 1

# every symbol `include/ndc_b200.h` declares
SYMBOLS = (
    "ndc_version", "ndc_last_error", "ndc_status_string", "ndc_launch_count", "ndc_query",
    "ndc_fwd", "ndc_bwd_workspace_bytes", "ndc_bwd", "ndc_bwd_static", "ndc_gconv",
    "ndc_probe_fp32_fma", "ndc_inorm_workspace_bytes", "ndc_inorm_last_error", "ndc_inorm_fwd",
    "ndc_inorm_bwd", "ndc_bias_grad_workspace_bytes", "ndc_bias_last_error", "ndc_bias_add",
    "ndc_bias_grad", "ndc_bias_gelu_fwd", "ndc_bias_gelu_bwd",
)


class NdcDesc(ctypes.Structure):
    _fields_ = [
        ("batch", ctypes.c_int32), ("groups", ctypes.c_int32),
        ("m", ctypes.c_int32), ("sc", ctypes.c_int32),
        ("D", ctypes.c_int32), ("H", ctypes.c_int32), ("W", ctypes.c_int32),
        ("kD", ctypes.c_int32), ("kH", ctypes.c_int32), ("kW", ctypes.c_int32),
        ("eps", ctypes.c_float), ("relu_input", ctypes.c_int32),
        ("dtype", ctypes.c_int32), ("flags", ctypes.c_int32),
    ]


class NdcError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status, message):
        super().__init__(f"ndc_b200 status {status}: {message}")
        self.status = status


_lib = None


def load():
    """Load the shared library (once) and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB):
        raise RuntimeError(
            f"{LIB} has not been built; run `python -m deconver_b200._build`. "
            "This package has no other compute path."
        )
    lib = ctypes.CDLL(LIB)
    vp, fp = ctypes.c_void_p, ctypes.c_void_p
    dp = ctypes.POINTER(NdcDesc)
    lib.ndc_version.restype = ctypes.c_int
    lib.ndc_last_error.restype = ctypes.c_char_p
    lib.ndc_status_string.restype = ctypes.c_char_p
    lib.ndc_status_string.argtypes = [ctypes.c_int]
    lib.ndc_launch_count.restype = ctypes.c_uint64
    lib.ndc_query.restype = ctypes.c_int
    lib.ndc_query.argtypes = [dp, ctypes.POINTER(ctypes.c_int32)]
    lib.ndc_fwd.restype = ctypes.c_int
    lib.ndc_fwd.argtypes = [dp, vp, vp, fp, fp, vp, vp, vp]
    lib.ndc_bwd_workspace_bytes.restype = ctypes.c_size_t
    lib.ndc_bwd_workspace_bytes.argtypes = [dp]
    lib.ndc_bwd.restype = ctypes.c_int
    lib.ndc_bwd.argtypes = [dp, vp, vp, vp, fp, fp, vp, vp, vp, fp, fp, vp, ctypes.c_size_t, vp]
    lib.ndc_bwd_static.restype = ctypes.c_int
    lib.ndc_bwd_static.argtypes = [dp, vp, vp, vp, fp, fp, vp, vp, vp, fp, fp, vp]
    lib.ndc_gconv.restype = ctypes.c_int
    lib.ndc_gconv.argtypes = [dp, vp, fp, fp, ctypes.c_int32, vp, vp]
    lib.ndc_probe_fp32_fma.restype = ctypes.c_int
    lib.ndc_probe_fp32_fma.argtypes = [ctypes.c_int32, ctypes.c_int32, fp, ctypes.c_size_t,
                                       ctypes.POINTER(ctypes.c_uint64), vp]
    lib.ndc_inorm_workspace_bytes.restype = ctypes.c_size_t
    lib.ndc_inorm_workspace_bytes.argtypes = [ctypes.c_int32, ctypes.c_int32]
    lib.ndc_inorm_last_error.restype = ctypes.c_char_p
    lib.ndc_inorm_fwd.restype = ctypes.c_int
    lib.ndc_inorm_fwd.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, vp,
                                  fp, fp, ctypes.c_float, vp, fp, vp, ctypes.c_size_t, vp]
    lib.ndc_inorm_bwd.restype = ctypes.c_int
    lib.ndc_inorm_bwd.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, vp,
                                  vp, fp, fp, vp, fp, fp, vp, ctypes.c_size_t, vp]
    lib.ndc_bias_grad_workspace_bytes.restype = ctypes.c_size_t
    lib.ndc_bias_grad_workspace_bytes.argtypes = [ctypes.c_int32, ctypes.c_int32]
    lib.ndc_bias_last_error.restype = ctypes.c_char_p
    lib.ndc_bias_add.restype = ctypes.c_int
    lib.ndc_bias_add.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, vp, fp, vp]
    lib.ndc_bias_grad.restype = ctypes.c_int
    lib.ndc_bias_grad.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, vp, fp,
                                  vp, ctypes.c_size_t, vp]
    lib.ndc_bias_gelu_fwd.restype = ctypes.c_int
    lib.ndc_bias_gelu_fwd.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, vp,
                                      fp, vp, vp]
    lib.ndc_bias_gelu_bwd.restype = ctypes.c_int
    lib.ndc_bias_gelu_bwd.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, vp,
                                      vp, fp, vp, fp, vp, ctypes.c_size_t, vp]
    _lib = lib
    return lib


def check(status):
    if status != NDC_OK:
        raise NdcError(status, load().ndc_last_error().decode("utf-8", "replace"))


def make_desc(batch, groups, m, sc, spatial, kernel_size, eps, relu_input, dtype_code,
              flags=0):
    """Pad 1-D/2-D geometry to (D, H, W) with unit leading extents and unit taps, as the
    reference's launch helper does (deconver/deconvolution/kernels.py:713-725)."""
    if not 1 <= len(spatial) <= 3:
        raise ValueError("only 1-D, 2-D and 3-D inputs are supported")
    if len(kernel_size) != len(spatial):
        raise ValueError("kernel_size and the input's spatial rank differ")
    lead = 3 - len(spatial)
    d, h, w = [1] * lead + [int(v) for v in spatial]
    kd, kh, kw = [1] * lead + [int(v) for v in kernel_size]
    return NdcDesc(int(batch), int(groups), int(m), int(sc), d, h, w, kd, kh, kw, float(eps),
                   int(bool(relu_input)), int(dtype_code), int(flags))
