import torch

from .. import _ops
from ..functional.quantization import pack_i4


class Linear4bit(torch.nn.Module):
    """Symmetric 4-bit linear layer (quarot/nn/linear.py:24-79).

    Buffers (the checkpoint contract): `weight` uint8 [out, in/2] (int4 packed),
    `weight_scales` [out, 1], optional `bias` [out].  forward takes a
    PackedQuantizedTensor and returns fp16: int4 x int4 -> int32 GEMM on the tensor
    cores with the per-token x per-channel dequantisation (and bias) fused into
    the epilogue -- one kernel instead of upstream's matmul + sym_dequant pair.
    """

    def __init__(self, in_features, out_features, bias=False, dtype=torch.float16):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.register_buffer('weight_scales', torch.zeros((self.out_features, 1), requires_grad=False))
        self.register_buffer('weight', torch.randint(1, 7, (self.out_features, self.in_features // 2),
                                                     dtype=torch.uint8, requires_grad=False))
        if bias:
            self.register_buffer('bias', torch.zeros((self.out_features), dtype=dtype))
        else:
            self.bias = None

    def forward(self, x):
        assert type(x) == _ops.PackedQuantizedTensor  # quantised input is required
        return _ops.linear_i4(x.quantized_x, x.scales_x, self.weight, self.weight_scales, self.bias)

    @staticmethod
    def from_float(module: torch.nn.Linear, weight_scales=None):
        """Linear4bit with the shapes, bias flag and float dtype of `module` (quarot/nn/linear.py:58-79).

        With `weight_scales` ([out_features, 1]) the float weights -- expected to lie on the int4 grid times those
        scales already -- are divided by the scales, rounded with torch.round, packed two codes per byte and stored
        together with the scales and the bias.  Without scales nothing is converted: the result keeps the random
        codes and zero scales of the constructor (the upstream benchmarks build their layers this way and then
        overwrite the scales).  The division runs on the GPU; the buffers of the result stay on the CPU.
        """
        w = module.weight.data
        has_bias = module.bias is not None
        q = Linear4bit(module.in_features, module.out_features, bias=has_bias, dtype=w.dtype).to(w.dtype)
        if weight_scales is None:
            return q
        assert weight_scales.shape == (module.out_features, 1), 'weight_scales should have shape (out_features, 1)'
        codes = torch.round(w.cuda() / weight_scales.cuda()).to(torch.int8)
        q.weight.copy_(pack_i4(codes).cpu())
        q.weight_scales.copy_(weight_scales.to(w.dtype))
        if has_bias:
            q.bias.copy_(module.bias)
        return q
