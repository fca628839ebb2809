"""quarot_b200 -- B200-native kernels behind the ``quarot`` operator surface.

Mirrors the top-level API of the upstream package (quarot/__init__.py:1-71):
``matmul``, ``sym_quant``, ``sym_dequant`` and ``PackedQuantizedTensor`` plus the
``nn`` / ``functional`` / ``transformers`` sub-packages, and adds the fused entry
points the modules use (``hadamard``, ``hadamard_quant``, ``linear_i4``).  All
device work goes through the C-ABI library (include/quarot_b200.h); torch only
provides memory and streams.  Importing the package fails if the library has not
been built -- there is no fallback path.
"""
import sys

from . import _lib
from ._ops import (matmul, sym_quant, sym_dequant, PackedQuantizedTensor, hadamard, hadamard_quant,
                   linear_i4, linear_i4_outs, linear_i4_swiglu, interleave_gate_up, rmsnorm_quant, quant_linear_i4,
                   flatten_last_dim_and_return_shape)
from . import functional
from . import nn
from . import transformers

__all__ = ["matmul", "sym_quant", "sym_dequant", "PackedQuantizedTensor",
           "hadamard_quant", "hadamard", "linear_i4", "linear_i4_outs", "linear_i4_swiglu", "interleave_gate_up", "rmsnorm_quant", "quant_linear_i4", "install_as_quarot"]


def install_as_quarot():
    """Register this package under the name ``quarot`` so that code written against
    the upstream package (``import quarot``, ``from quarot.nn import Linear4bit``)
    runs on these kernels without modification."""
    me = sys.modules[__name__]
    sys.modules["quarot"] = me
    for sub in ("nn", "functional", "transformers"):
        sys.modules["quarot." + sub] = getattr(me, sub)
    sys.modules["quarot.functional.hadamard"] = functional.hadamard
    sys.modules["quarot.functional.quantization"] = functional.quantization
    sys.modules["quarot.nn.linear"] = nn.linear
    sys.modules["quarot.nn.quantization"] = nn.quantization
    sys.modules["quarot.nn.hadamard"] = nn.hadamard
    sys.modules["quarot.nn.normalization"] = nn.normalization
    return me
