"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

Real LLaMA-2 activations and checkpoints are not available offline; these
generators stand in for them: outlier-Gaussian fp16 activations (N(0,1) with 8
seeded channels scaled x50), uniform int4 weight codes in [-8, 7] packed two per
byte, per-channel fp16 weight scales ~ U(0.005, 0.02).
"""
import torch

from .functional.quantization import pack_i4

# (name, K, N, online Hadamard on K?) for one decoder layer
LLAMA2_7B = (("qkv", 4096, 12288, False), ("o_proj", 4096, 4096, False),
             ("gate_up", 4096, 22016, False), ("down", 11008, 4096, True))
LLAMA2_70B = (("qkv", 8192, 10240, False), ("o_proj", 8192, 8192, False),
              ("gate_up", 8192, 57344, False), ("down", 28672, 8192, True))
LLAMA2_70B_MLP = (("gate_up", 8192, 57344, False), ("down", 28672, 8192, True))
LLAMA2_7B_MLP = (("gate_up", 4096, 22016, False), ("down", 11008, 4096, True))
CONFIG0 = (("cfg0", 4096, 4096, True),)


def activations(M, K, seed=1234, outlier_channels=8, outlier_scale=50.0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g, dtype=torch.float32)
    idx = torch.randperm(K, generator=g)[: min(outlier_channels, K)]
    x[:, idx] *= outlier_scale
    return x.to(torch.float16).to(device)


def weights(N, K, seed=4321, device="cpu"):
    """(packed uint8 [N, K/2], scales fp16 [N, 1])."""
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(-8, 8, (N, K), generator=g, dtype=torch.int8)
    scales = (torch.rand(N, 1, generator=g) * 0.015 + 0.005).to(torch.float16)
    return pack_i4(codes).to(device), scales.to(device)


def weights_device(N, K, seed=4321, device="cuda"):
    """Same distribution generated directly on the device (for large shapes); not bit-identical to weights()."""
    g = torch.Generator(device=device).manual_seed(seed)
    packed = torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.uint8, device=device)
    scales = (torch.rand(N, 1, generator=g, device=device) * 0.015 + 0.005).to(torch.float16)
    return packed, scales


def activations_device(M, K, seed=1234, outlier_channels=8, outlier_scale=50.0, device="cuda"):
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(M, K, generator=g, dtype=torch.float32, device=device)
    idx = torch.randperm(K, generator=g, device=device)[: min(outlier_channels, K)]
    x[:, idx] *= outlier_scale
    return x.to(torch.float16)
