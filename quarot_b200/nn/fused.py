"""Fusion of OnlineHadamard -> Quantizer into one kernel launch.

The callers (e.g. the down_proj of a rotated LLaMA MLP) build
``Sequential(OnlineHadamard, Quantizer, Linear4bit)``.  `fuse_modules` rewrites such
sequences in place to ``Sequential(HadamardQuantizer, Identity, Linear4bit)``: same
indices, so state-dict keys like ``down_proj.2.weight`` stay valid, but the
transform, the absmax, the scale and the int4 packing happen in a single pass over
the activations.
"""
import torch

from .. import _ops
from ..functional import hadamard as F_had
from .hadamard import OnlineHadamard
from .quantization import Quantizer


class HadamardQuantizer(torch.nn.Module):
    """OnlineHadamard(hadamard_dim) followed by Quantizer(input_clip_ratio), fused."""

    def __init__(self, hadamard_dim, input_clip_ratio=1.0, had_rem_dim=None):
        super().__init__()
        self.hadamard_dim = hadamard_dim
        self.input_clip_ratio = input_clip_ratio
        table, self.rem_dim = F_had.get_hadK(hadamard_dim)
        # same buffer (and state-dict key) as OnlineHadamard, so checkpoints of fused and unfused models interchange
        if table is not None:
            self.register_buffer("had_rem_dim", had_rem_dim if had_rem_dim is not None else table.to(torch.float16))
        else:
            self.had_rem_dim = None

    def forward(self, x):
        table = F_had.device_table(self.rem_dim, x.device) if self.rem_dim > 1 else None
        q, s, _ = _ops.hadamard_quant(x, table, self.rem_dim, self.input_clip_ratio)
        return _ops.PackedQuantizedTensor(q, s.view(x.shape[:-1]).unsqueeze(1))


def fuse_modules(model):
    """Replace every adjacent (OnlineHadamard, Quantizer) pair inside a Sequential by the fused module."""
    count = 0
    for mod in model.modules():
        if isinstance(mod, torch.nn.Sequential):
            for i in range(len(mod) - 1):
                a, b = mod[i], mod[i + 1]
                if isinstance(a, OnlineHadamard) and isinstance(b, Quantizer):
                    n = getattr(a, "hadamard_dim", None)
                    if n is None:
                        continue
                    mod[i] = HadamardQuantizer(n, b.input_clip_ratio, a.had_rem_dim)
                    mod[i + 1] = torch.nn.Identity()
                    count += 1
    return count


class SwiGLULinear4bit(torch.nn.Module):
    """gate_proj and up_proj of a LLaMA MLP (two Linear4bit modules without bias) as one module that returns
    act_fn(gate_proj(x)) * up_proj(x) for a PackedQuantizedTensor x: one GEMM over the row-interleaved weights with
    the SiLU product in its epilogue, so neither projection is written to memory.  The interleaved copy is built
    once here from the modules' canonical [N, K/2] buffers (the checkpoint layout is not changed)."""

    def __init__(self, gate_proj, up_proj):
        super().__init__()
        if gate_proj.bias is not None or up_proj.bias is not None:
            raise ValueError("SwiGLULinear4bit: projections with bias are not supported")
        self.intermediate_size = gate_proj.weight.shape[0]
        self.register_buffer("weight_gu", _ops.interleave_gate_up(gate_proj.weight, up_proj.weight))
        self.register_buffer("scales_gu", _ops.interleave_gate_up(gate_proj.weight_scales.view(-1),
                                                                 up_proj.weight_scales.view(-1)))

    def forward(self, x):
        assert type(x) == _ops.PackedQuantizedTensor
        rows = x.quantized_x.numel() // x.quantized_x.shape[-1]
        if rows > 128:
            return _ops.linear_i4_swiglu(x.quantized_x, x.scales_x, self.weight_gu, self.scales_gu)
        # few token rows: one GEMM over the interleaved weights, the product as separate elementwise kernels
        both = _ops.linear_i4(x.quantized_x, x.scales_x, self.weight_gu, self.scales_gu)
        both = both.view(*both.shape[:-1], -1, 2, 128)
        gate, up = both[..., 0, :], both[..., 1, :]
        out = torch.nn.functional.silu(gate) * up
        return out.reshape(*out.shape[:-2], self.intermediate_size)


class RMSNormQuantizer(torch.nn.Module):
    """RMSNorm(mean_dim, eps) followed by Quantizer(input_clip_ratio), fused: what stands in front of the q/k/v and
    gate/up projections of a rotated LLaMA layer (the residual stream keeps the un-normalised x, so the normalised
    fp16 tensor is never needed on its own)."""

    def __init__(self, mean_dim, eps=1e-5, input_clip_ratio=1.0):
        super().__init__()
        self.mean_dim, self.eps, self.input_clip_ratio = mean_dim, eps, input_clip_ratio

    def forward(self, x):
        q, s, _ = _ops.rmsnorm_quant(x, self.mean_dim, self.eps, self.input_clip_ratio)
        return _ops.PackedQuantizedTensor(q, s.view(x.shape[:-1]).unsqueeze(1))


class QuantLinear4bit(torch.nn.Module):
    """Sequential(Quantizer, Linear4bit) as one module: with one or two token rows (single-sequence decode) the
    quantiser runs inside the weight-streaming CUDA-core kernel, otherwise the two modules run one after the other
    (every CTA of the fused kernel quantises all rows itself, which stops paying off at four rows: measured)."""

    FUSED_MAX_ROWS = 2     # measured cross-over between one launch and two

    def __init__(self, quantizer, linear):
        super().__init__()
        self.quantizer, self.linear = quantizer, linear

    def forward(self, x):
        rows = x.numel() // x.shape[-1]
        if rows <= self.FUSED_MAX_ROWS and x.dtype == torch.float16:
            return _ops.quant_linear_i4(x, self.linear.weight, self.linear.weight_scales, self.linear.bias,
                                        self.quantizer.input_clip_ratio)
        return self.linear(self.quantizer(x))

