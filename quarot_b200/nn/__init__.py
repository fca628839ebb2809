"""Module surface of the upstream package (quarot/nn/__init__.py:1-4) plus the fused variants."""
from . import linear, normalization, quantization, hadamard
from .linear import Linear4bit
from .normalization import RMSNorm
from .quantization import Quantizer
from .hadamard import OnlineHadamard
from .fused import HadamardQuantizer, fuse_modules, HorizontalLinear4bit, fuse_qkv, fuse_gate_up
