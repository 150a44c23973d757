"""bitween_b200 -- the RTN quantize/pack and QuantizedLinear-forward path of the Bitween
library as hand-written sm_100a CUDA behind a C ABI, with the reference's Python surface.

    from bitween_b200 import Bitween, QuantizedLinear, quantize_rtn

`install_as_bitween()` registers the package under the name `bitween` so that code and pickles
written against the reference (`bitween.modules.QuantizedLinear`, `bitween.functional`,
`bitween.kernels.cuda_loader`, `bitween.gradual.base_wrapper.RTNWrapper`, `bitween.wrapper.WrapperLinear`) resolve to this implementation.
"""
import sys

from .functional import dequantize_rtn, quantize_rtn  # noqa: F401
from .modules import QuantizedLinear, QuantizedLinearFunction  # noqa: F401
from .quantizer.quantizer import Bitween  # noqa: F401

__version__ = "0.1.0"


def install_as_bitween():
    """Alias this package as `bitween` in sys.modules (drop-in for imports and unpickling)."""
    from . import functional, gradual, kernels, modules, quantizer, wrapper
    from .gradual import base_wrapper
    from .kernels import cuda_loader
    from .quantizer import func as qfunc, quantizer as qq
    me = sys.modules[__name__]
    sys.modules["bitween"] = me
    sys.modules["bitween.functional"] = functional
    sys.modules["bitween.modules"] = modules
    sys.modules["bitween.kernels"] = kernels
    sys.modules["bitween.kernels.cuda_loader"] = cuda_loader
    sys.modules["bitween.gradual"] = gradual
    sys.modules["bitween.gradual.base_wrapper"] = base_wrapper
    sys.modules["bitween.wrapper"] = wrapper
    sys.modules["bitween.quantizer"] = quantizer
    sys.modules["bitween.quantizer.quantizer"] = qq
    sys.modules["bitween.quantizer.func"] = qfunc
    return me
