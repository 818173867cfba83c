"""deconver_b200: the NDC mixer update of Deconver on hand-written sm_100a CUDA kernels.

Public names follow the reference package (`deconver.deconvolution`): `Deconv` / `NDC`,
`Initializer`, `deconv_update`, `DeconvUpdate`.  The compute path is the shared library
`libndc_b200.so` (C ABI in `include/ndc_b200.h`); build it with
`python -m deconver_b200._build`.
"""

from ._build import build_library
from ._lib import NdcError, load as load_library
from .deconv import NDC, Deconv, Initializer
from .functional import DeconvUpdate, deconv_update, gconv, kernels_apply
from .linear import Linear
from .mlp import MLP, bias_gelu
from .norm import InstanceNorm1d, InstanceNorm2d, InstanceNorm3d, instance_norm

__all__ = [
    "Deconv", "NDC", "Initializer", "Linear", "MLP", "bias_gelu", "DeconvUpdate", "deconv_update", "gconv",
    "kernels_apply", "build_library", "load_library", "NdcError",
    "InstanceNorm1d", "InstanceNorm2d", "InstanceNorm3d", "instance_norm",
]
