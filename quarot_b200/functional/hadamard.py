"""Hadamard helpers behind the upstream names (quarot/functional/hadamard.py:5-147).

``get_hadK`` serves the fixed +-1 tables (stored bit-packed in ``_had_tables``),
``matmul_hadU`` / ``matmul_hadUt`` are device-agnostic torch implementations used
offline (random orthogonal matrices in fp64, weight rotation), and
``matmul_hadU_cuda`` runs the transform in one CUDA kernel through the C-ABI.
"""
import math

import numpy as np
import torch

from . import _had_tables

_TABLE_ORDERS = (172, 156, 140, 108, 60, 52, 36, 28, 40, 20, 12)  # divisibility is tested in this order
_TABLE_CACHE = {}
_DEVICE_TABLE_CACHE = {}


def is_pow2(n):
    return (n & (n - 1) == 0) and (n > 0)


def _table(k):
    t = _TABLE_CACHE.get(k)
    if t is None:
        bits = np.unpackbits(np.frombuffer(bytes.fromhex(_had_tables.PACKED[k]), dtype=np.uint8))[: k * k]
        t = torch.from_numpy(1.0 - 2.0 * bits.astype(np.float32)).reshape(k, k)
        _TABLE_CACHE[k] = t
    return t


def get_hadK(n, transpose=False):
    """(float32 K x K table or None, K) for a transform of length n; n / K must be a power of two."""
    for k in _TABLE_ORDERS:
        if n % k == 0:
            assert (is_pow2(n // k))
            h = _table(k)
            return (h.T if transpose else h).clone(), k
    assert (is_pow2(n))
    return None, 1


def device_table(k, device, transpose=False):
    """fp16 copy of table k on `device`, cached (what the CUDA kernels take as had_k)."""
    key = (k, str(device), transpose)
    t = _DEVICE_TABLE_CACHE.get(key)
    if t is None:
        h = _table(k)
        t = (h.T if transpose else h).contiguous().to(device=device, dtype=torch.float16)
        _DEVICE_TABLE_CACHE[key] = t
    return t


def matmul_hadU(X, transpose=False):
    """X (hadK (x) H)^T / sqrt(n) over the last axis, in X's dtype, on X's device."""
    n = X.shape[-1]
    hadK, K = get_hadK(n, transpose)
    m = n // K
    v = X.reshape(-1, K, m).clone()
    rows = v.shape[0]
    h = 1
    while h < m:
        w = v.view(rows, K, m // (2 * h), 2, h)
        v = torch.stack((w[..., 0, :] + w[..., 1, :], w[..., 0, :] - w[..., 1, :]), dim=3).reshape(rows, K, m)
        h *= 2
    if K > 1:
        v = hadK.view(1, K, K).to(v) @ v
    return v.reshape(X.shape) / torch.tensor(n).sqrt()


def matmul_hadUt(X):
    return matmul_hadU(X, transpose=True)


def random_hadamard_matrix(size, device):
    """Randomised Hadamard matrix H diag(+-1) / sqrt(size) in fp64 (used for offline rotation)."""
    Q = torch.randint(low=0, high=2, size=(size,)).to(torch.float64)
    Q = Q * 2 - 1
    Q = torch.diag(Q)
    return matmul_hadU(Q).to(device)


def matmul_hadU_cuda(X, hadK, K):
    """Online Hadamard on a CUDA tensor.  hadK is the K x K table (any float dtype /
    device; None when K == 1).  fp16 and fp32 inputs run in one CUDA kernel with fp32
    internal arithmetic; other dtypes are transformed in fp32 and cast back."""
    from .. import _ops
    if not X.is_cuda:
        raise RuntimeError("matmul_hadU_cuda: X must be a CUDA tensor")
    table = None
    if K > 1:
        table = hadK
        if not (table.is_cuda and table.device == X.device and table.dtype == torch.float16 and table.is_contiguous()):
            table = table.to(device=X.device, dtype=torch.float16).contiguous()
    if X.dtype in (torch.float16, torch.float32):
        return _ops.hadamard(X, table, K)
    return _ops.hadamard(X.float(), table, K).to(X.dtype)


def matmul_hadUt_cuda(X, hadK, K):
    """Transform with the transposed table (upstream's version raises a TypeError,
    quarot/functional/hadamard.py:105-106; this one works)."""
    return matmul_hadU_cuda(X, hadK.T.contiguous() if hadK is not None else None, K)


def apply_exact_had_to_linear(module, had_dim=-1, output=False):
    """Rotate the weights of a torch.nn.Linear in place (offline preparation)."""
    assert isinstance(module, torch.nn.Linear)
    in_features, out_features = module.in_features, module.out_features
    if had_dim != -1:
        assert is_pow2(had_dim), "Hadamard dimension must be a power of 2!"
    W_ = module.weight.data
    dtype, dev = W_.dtype, W_.device
    W_ = W_.float().cuda()
    if had_dim == -1:
        if output:
            had_K, K = get_hadK(out_features)
            W_ = matmul_hadU_cuda(W_.t().contiguous(), had_K, K).t()
        else:
            had_K, K = get_hadK(in_features)
            W_ = matmul_hadU_cuda(W_, had_K, K)
    else:
        if output:
            Wt = W_.t().contiguous()
            shape = Wt.shape
            Wt = matmul_hadU_cuda(Wt.reshape(-1, shape[-1] // had_dim, had_dim), None, 1)
            W_ = Wt.reshape(shape).t()
        else:
            raise NotImplementedError("Not implemented (or tested) yet!")
    module.weight.data = W_.to(device=dev, dtype=dtype)
