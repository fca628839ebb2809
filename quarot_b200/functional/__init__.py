"""Functional surface of the upstream package (quarot/functional/__init__.py:1-5)."""
from . import hadamard
from . import quantization
from .quantization import pack_i4, unpack_i4, asym_quant_dequant, sym_quant_dequant
from .hadamard import (
    matmul_hadU_cuda,
    random_hadamard_matrix,
    apply_exact_had_to_linear)
