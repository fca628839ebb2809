"""Host-side quantisation helpers: int4 nibble packing and the fake-quant formulas.

Same names, arguments and results as the upstream module
(quarot/functional/quantization.py:1-74).  Plain torch, device-agnostic; used at
initialisation time (weight packing) and by callers outside the hot path.  The
hot-path equivalents are the CUDA kernels behind ``quarot_b200.sym_quant`` and
``quarot_b200.hadamard_quant``.
"""
import torch


def get_minq_maxq(bits: int, sym: bool):
    """Integer range of a `bits`-wide code as 0-dim tensors: signed if sym, else unsigned."""
    hi = 2 ** (bits - 1) - 1 if sym else 2 ** bits - 1
    lo = -hi - 1 if sym else 0
    return torch.tensor(lo), torch.tensor(hi)


def two_compl(x, bits: int):
    """Map negative values to their two's-complement representation in `bits` bits."""
    return torch.where(x < 0, x + (1 << bits), x)


def _codes(x, scale, offset, lo, hi):
    return torch.clamp(torch.round(x / scale) + offset, lo, hi)


def asym_quant(x, scale, zero, maxq):
    scale, zero = scale.to(x.device), zero.to(x.device)
    return _codes(x, scale, zero, 0, maxq), scale, zero


def asym_dequant(q, scale, zero):
    return (q - zero) * scale


def asym_quant_dequant(x, scale, zero, maxq):
    q, scale, zero = asym_quant(x, scale, zero, maxq)
    return asym_dequant(q, scale, zero)


def sym_quant(x, scale, maxq):
    scale = scale.to(x.device)
    return _codes(x, scale, 0, -(maxq + 1), maxq), scale


def sym_dequant(q, scale):
    return q * scale


def sym_quant_dequant(x, scale, maxq):
    q, scale = sym_quant(x, scale, maxq)
    return sym_dequant(q, scale)


def pack_i4(q):
    """Two signed 4-bit values per byte: element 2j -> low nibble, 2j+1 -> high nibble."""
    assert torch.is_signed(q), 'The tensor to be packed should be signed int'
    lo, hi = get_minq_maxq(4, True)
    assert bool(((q >= lo) & (q <= hi)).all()), 'int4 values must lie in [-8, 7]'
    nib = (q.to(torch.int16) & 0xF).to(torch.uint8)
    return nib[..., 0::2] | (nib[..., 1::2] << 4)


def unpack_i4(x: torch.Tensor):
    """Inverse of pack_i4; returns sign-extended int32 with twice the last dimension."""
    assert x.dtype == torch.uint8, 'The tensor to be unpacked should be stored in uint8'
    both = torch.stack((x & 0x0F, x >> 4), dim=-1).to(torch.int32)
    both = both - ((both & 8) << 1)
    return both.reshape(*x.shape[:-1], x.shape[-1] * 2)
