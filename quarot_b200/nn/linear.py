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
        """Build a Linear4bit from a float Linear whose weights are already on the int4
        grid times `weight_scales` ([out, 1]); without scales the module keeps its
        random initial buffers (what the upstream benchmarks rely on)."""
        weight_matrix = module.weight.data
        int_module = Linear4bit(module.in_features, module.out_features,
                                bias=module.bias is not None, dtype=weight_matrix.dtype).to(weight_matrix.dtype)
        if weight_scales is not None:
            assert weight_scales.shape == (module.out_features, 1), 'weight_scales should have shape (out_features, 1)'
            weight_matrix = weight_matrix.cuda()
            int_module.weight_scales.copy_(weight_scales.to(weight_matrix.dtype))
            int_rounded_weight = (weight_matrix / weight_scales.cuda()).round()
            int_module.weight.copy_(pack_i4(int_rounded_weight.to(torch.int8)).cpu())
            if module.bias is not None:
                int_module.bias.copy_(module.bias)
        return int_module
