import torch

from .. import _ops


class Quantizer(torch.nn.Module):
    """Per-token symmetric INT4 activation quantiser (quarot/nn/quantization.py:4-13).

    scale = fp16(max|x| / 7) * input_clip_ratio per token, codes
    clamp(round(x / scale), -8, 7) packed two per byte.  Absmax, scale, quantise and
    pack run in ONE kernel (upstream: ~5 torch kernels + sym_quant).  The scale tensor
    keeps upstream's shape quirk: the token axes with a singleton inserted at dim 1
    ([M, 1] for 2-D input, [B, 1, S] for 3-D input).
    """

    def __init__(self, input_clip_ratio=1.0):
        super().__init__()
        self.input_clip_ratio = input_clip_ratio

    def forward(self, x):
        q, s, _ = _ops.hadamard_quant(x, None, 0, self.input_clip_ratio)
        scales_x = s.view(x.shape[:-1]).unsqueeze(1)
        return _ops.PackedQuantizedTensor(q, scales_x)
