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

    def __init__(self, hadamard_dim, input_clip_ratio=1.0):
        super().__init__()
        self.hadamard_dim = hadamard_dim
        self.input_clip_ratio = input_clip_ratio
        self.rem_dim = F_had.get_hadK(hadamard_dim)[1]

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
                    mod[i] = HadamardQuantizer(n, b.input_clip_ratio)
                    mod[i + 1] = torch.nn.Identity()
                    count += 1
    return count
