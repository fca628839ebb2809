"""Generate the golden fixtures in this directory from an upstream QuaRot checkout.

Runs the upstream project's own CPU-capable torch functions
(quarot/functional/hadamard.py: get_hadK, matmul_hadU, matmul_hadUt;
quarot/functional/quantization.py: sym_quant, pack_i4, unpack_i4;
quarot/nn/normalization.py: RMSNorm;
the scale formula of quarot/nn/quantization.py:10 evaluated inline) on small
seeded inputs and stores inputs and outputs.  The upstream modules are loaded
by file path with an empty stand-in for the CUDA-only ``fast_hadamard_transform``
import, which these functions never call.

Usage:  python tests/golden/make_golden.py /path/to/upstream/checkout
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load(root, name, rel):
    sys.modules.setdefault("fast_hadamard_transform", types.ModuleType("fast_hadamard_transform"))
    spec = importlib.util.spec_from_file_location(name, os.path.join(root, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def outlier_rows(gen, rows, cols, n_out=8, factor=50.0):
    x = torch.randn(rows, cols, generator=gen, dtype=torch.float32)
    idx = torch.randperm(cols, generator=gen)[: min(n_out, cols)]
    x[:, idx] *= factor
    return x.to(torch.float16)


def main():
    root = sys.argv[1]
    H = load(root, "_up_hadamard", "quarot/functional/hadamard.py")
    Q = load(root, "_up_quant", "quarot/functional/quantization.py")
    gen = torch.Generator().manual_seed(20240406)

    # ---- Hadamard: every table family, pure powers of two, and the three model sizes
    had = {}
    sizes = [(2, 3), (8, 3), (32, 3), (64, 3), (128, 2), (1024, 2), (4096, 1), (8192, 1),
             (12 * 8, 3), (20 * 4, 3), (28 * 4, 3), (36 * 2, 3), (40 * 4, 3), (52 * 2, 3),
             (60 * 2, 3), (108 * 2, 2), (140 * 2, 2), (156 * 2, 2), (172 * 2, 2),
             (13824, 1), (11008, 1), (28672, 1)]
    for n, rows in sizes:
        x16 = outlier_rows(gen, rows, n, n_out=2, factor=20.0)
        hk, k = H.get_hadK(n)
        had["n%d_k" % n] = np.int64(k)
        had["n%d_x" % n] = x16.numpy()
        had["n%d_y32" % n] = H.matmul_hadU(x16.float()).numpy()
        had["n%d_y16" % n] = H.matmul_hadU(x16).numpy()
        if n <= 512:
            had["n%d_yt32" % n] = H.matmul_hadUt(x16.float()).numpy()
    np.savez_compressed(os.path.join(HERE, "hadamard.npz"), **had)

    # ---- Quantizer: scales, codes, packed bytes; includes exact .5 ties, +-max ties, odd width
    qz = {}
    cases = {"a": outlier_rows(gen, 16, 256), "b": outlier_rows(gen, 5, 4096), "c": outlier_rows(gen, 3, 11008)}
    tie = torch.zeros(4, 64, dtype=torch.float16)
    tie[0] = torch.linspace(-7, 7, 64).to(torch.float16)            # scale exactly 1
    tie[1, :29] = torch.arange(-7, 7.5, 0.5).to(torch.float16)      # x.5 ties at scale 1
    tie[1, 63] = 7.0
    tie[2, 0], tie[2, 1], tie[2, 2] = 3.5, -3.5, 3.5                # +max and -max equal magnitude
    tie[3] = (torch.arange(64) % 15 - 7).to(torch.float16) * 0.37
    cases["tie"] = tie
    cases["odd"] = outlier_rows(gen, 6, 34)[:, :33].contiguous()    # odd column count
    for name, x in cases.items():
        for clip in (1.0, 0.9):
            s = (torch.max(torch.abs(x), dim=-1)[0].unsqueeze(1) / 7).to(torch.float16) * clip
            q, _ = Q.sym_quant(x, s, torch.tensor(7))
            tag = "%s_clip%d" % (name, int(clip * 100))
            qz[tag + "_x"] = x.numpy()
            qz[tag + "_s"] = s.numpy()
            qz[tag + "_q"] = q.to(torch.int8).numpy()
            if x.shape[1] % 2 == 0:
                p = Q.pack_i4(q.to(torch.int8))
                qz[tag + "_p"] = p.numpy()
                qz[tag + "_u"] = Q.unpack_i4(p).numpy()
    np.savez_compressed(os.path.join(HERE, "quantizer.npz"), **qz)

    # ---- int4 matmul identity: unpack both sides, int32 matmul
    mm = {}
    for tag, (m, n, k) in {"s": (5, 7, 64), "m": (33, 48, 256), "l": (130, 272, 1024)}.items():
        a = torch.randint(-8, 8, (m, k), generator=gen, dtype=torch.int8)
        b = torch.randint(-8, 8, (n, k), generator=gen, dtype=torch.int8)
        ap, bp = Q.pack_i4(a), Q.pack_i4(b)
        c = Q.unpack_i4(ap) @ Q.unpack_i4(bp).T
        mm[tag + "_a"], mm[tag + "_b"], mm[tag + "_c"] = ap.numpy(), bp.numpy(), c.numpy()
    np.savez_compressed(os.path.join(HERE, "matmul.npz"), **mm)
    # ---- weight-less RMSNorm (the module in front of the quantiser of the q/k/v and gate/up inputs)
    N = load(root, "_up_norm", "quarot/nn/normalization.py")
    gen2 = torch.Generator().manual_seed(20240407)
    rn = {}
    for tag, (rows, n) in {"a": (9, 64), "b": (7, 4096), "c": (3, 11008), "d": (4, 8192)}.items():
        x = outlier_rows(gen2, rows, n)
        x[0] = 0
        rn[tag + "_x"] = x.numpy()
        rn[tag + "_y"] = N.RMSNorm(n, eps=1e-5)(x).numpy()
    np.savez_compressed(os.path.join(HERE, "rmsnorm.npz"), **rn)
    for f in ("hadamard.npz", "quantizer.npz", "matmul.npz", "rmsnorm.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
