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

    FUSED_MAX_ROWS = 1     # measured cross-over between one launch and two (two rows: 36 us against 33 us per 7B layer)

    def __init__(self, quantizer, linear):
        super().__init__()
        self.quantizer, self.linear = quantizer, linear

    def forward(self, x):
        rows = x.numel() // x.shape[-1]
        if rows <= self.FUSED_MAX_ROWS and x.dtype == torch.float16:
            return _ops.quant_linear_i4(x, self.linear.weight, self.linear.weight_scales, self.linear.bias,
                                        self.quantizer.input_clip_ratio)
        return self.linear(self.quantizer(x))



class HorizontalLinear4bit(torch.nn.Module):
    """Several Linear4bit modules that read the same quantised input -- q/k/v of an attention block, gate/up of an
    MLP (e2e/quantized_llama/modeling_llama.py:40-44,108-110: one Quantizer feeds all of them) -- as ONE GEMM.

    The modules' `weight`, `weight_scales` and `bias` are concatenated along the output channels; the modules then
    hold VIEWS of the concatenated buffers, so nothing is stored twice, `state_dict()` / `load_state_dict()` of the
    model keep their per-projection keys (`q_proj.weight`, ...) and loading a checkpoint writes straight into the
    fused operand.  The concatenated buffers are not part of the state dict.  forward returns one tensor per module
    (column slices of the single [..., sum N] result).  Moving the model to another device afterwards breaks the
    sharing (torch moves every buffer on its own): fuse after `.to(device)`, or call `refresh()`.
    """

    def __init__(self, *linears):
        super().__init__()
        if len(linears) < 2:
            raise ValueError("HorizontalLinear4bit: at least two modules")
        k = linears[0].weight.shape[1]
        with_bias = [lin.bias is not None for lin in linears]
        if any(lin.weight.shape[1] != k for lin in linears) or (any(with_bias) and not all(with_bias)):
            raise ValueError("HorizontalLinear4bit: modules must share in_features and either all or none have a bias")
        self._linears = list(linears)           # a plain list: the modules stay where they are in the model
        self.splits = [lin.weight.shape[0] for lin in linears]
        self.refresh()

    def refresh(self):
        lins = self._linears
        self.register_buffer("weight", torch.cat([lin.weight for lin in lins], dim=0), persistent=False)
        self.register_buffer("weight_scales", torch.cat([lin.weight_scales.view(-1, 1) for lin in lins], dim=0),
                             persistent=False)
        if lins[0].bias is not None:
            self.register_buffer("bias", torch.cat([lin.bias for lin in lins], dim=0), persistent=False)
        else:
            self.bias = None
        start = 0
        for lin, n in zip(lins, self.splits):
            lin.weight = self.weight[start:start + n]
            lin.weight_scales = self.weight_scales[start:start + n]
            if self.bias is not None:
                lin.bias = self.bias[start:start + n]
            start += n

    def forward(self, x):
        assert type(x) == _ops.PackedQuantizedTensor
        out = _ops.linear_i4(x.quantized_x, x.scales_x, self.weight, self.weight_scales, self.bias)
        return out.split(self.splits, dim=-1)


def fuse_qkv(attention):
    """`attention.q_proj / k_proj / v_proj` (Linear4bit) as one GEMM: returns the HorizontalLinear4bit, whose forward
    gives (q, k, v) for the PackedQuantizedTensor that `attention.quantizer` produced.  State-dict keys are unchanged."""
    return HorizontalLinear4bit(attention.q_proj, attention.k_proj, attention.v_proj)


def fuse_gate_up(mlp, swiglu=False):
    """`mlp.gate_proj / up_proj` as one GEMM: (gate, up) = fused(x), or, with swiglu=True, a SwiGLULinear4bit whose
    forward returns act_fn(gate) * up with the product inside the GEMM epilogue.  State-dict keys are unchanged."""
    if swiglu:
        return SwiGLULinear4bit(mlp.gate_proj, mlp.up_proj)
    return HorizontalLinear4bit(mlp.gate_proj, mlp.up_proj)
