"""Generate kv_cache.npz: outputs of the upstream KV-cache quantisation helpers on small seeded inputs.

The upstream module quarot/transformers/kv_cache.py imports the project's CUDA extension and the
fast_hadamard_transform package at import time; neither is needed by the two pure-torch helpers that define the 4-bit
cache format (asym_quantize_and_pack_i4, unpack_i4_and_asym_dequantize), so the module is loaded by file path with
empty stand-ins for those imports and the helpers are run on the CPU.

Usage:  python tests/golden/make_golden_kv.py /path/to/upstream/checkout
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_kv_module(root):
    pkg = types.ModuleType("quarot")
    pkg.__path__ = [os.path.join(root, "quarot")]
    pkg._CUDA = types.ModuleType("quarot._CUDA")
    sys.modules["quarot"] = pkg
    sys.modules["quarot._CUDA"] = pkg._CUDA
    fht = types.ModuleType("fast_hadamard_transform")
    fht.hadamard_transform = None
    sys.modules["fast_hadamard_transform"] = fht
    for name, rel in (("quarot.functional", "quarot/functional/__init__.py"),):
        m = types.ModuleType(name)
        m.__path__ = [os.path.join(root, "quarot", "functional")]
        sys.modules[name] = m
    spec = importlib.util.spec_from_file_location("quarot.functional.quantization",
                                                  os.path.join(root, "quarot/functional/quantization.py"))
    q = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(q)
    sys.modules["quarot.functional.quantization"] = q
    tr = types.ModuleType("quarot.transformers")
    tr.__path__ = [os.path.join(root, "quarot", "transformers")]
    sys.modules["quarot.transformers"] = tr
    spec = importlib.util.spec_from_file_location("quarot.transformers.kv_cache",
                                                  os.path.join(root, "quarot/transformers/kv_cache.py"))
    kv = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(kv)
    return kv


def main():
    kv = load_kv_module(sys.argv[1])
    g = torch.Generator().manual_seed(77)
    out = {}
    cases = {
        "gauss": torch.randn(3, 5, 4, 128, generator=g) * 2.0,
        "outlier": torch.randn(2, 3, 2, 128, generator=g) * torch.where(torch.rand(2, 3, 2, 128, generator=g) > 0.97, 30.0, 1.0),
        "tiny": torch.randn(1, 4, 2, 128, generator=g) * 1e-4,
        "const": torch.full((1, 2, 1, 128), 0.75),
        "ties": (torch.randint(0, 31, (1, 6, 2, 128), generator=g).float() * 0.5 - 3.0),
    }
    for name, x in cases.items():
        x = x.to(torch.float16)
        q, scale, zero = kv.asym_quantize_and_pack_i4(x)
        out[name + "_x"] = x.numpy()
        out[name + "_q"] = q.numpy()
        out[name + "_scale"] = scale.numpy()
        out[name + "_zero"] = zero.numpy()
        out[name + "_deq"] = kv.unpack_i4_and_asym_dequantize(q, scale, zero).numpy()
    np.savez_compressed(os.path.join(HERE, "kv_cache.npz"), **out)
    print("wrote kv_cache.npz with", len(out), "arrays")


if __name__ == "__main__":
    main()
