import torch

from .. import _ops
from ..functional import hadamard as F_had


class OnlineHadamard(torch.nn.Module):
    """Online Hadamard transform over the last axis (quarot/nn/hadamard.py:5-23).

    `hadamard_dim` selects the factorisation had_K (x) Walsh (get_hadK).  The CUDA
    kernel always accumulates in fp32 and rounds once to the input dtype, so
    `force_fp32` changes nothing numerically for fp16 inputs; the flag and the
    `had_rem_dim` buffer are kept for state-dict and constructor compatibility.
    """

    def __init__(self, hadamard_dim, force_fp32=False):
        super().__init__()
        self.fp32_had = force_fp32
        self.hadamard_dim = hadamard_dim
        had_rem_dim, self.rem_dim = F_had.get_hadK(hadamard_dim)
        if had_rem_dim is not None:
            self.register_buffer("had_rem_dim", had_rem_dim)
            if not self.fp32_had:
                self.had_rem_dim = self.had_rem_dim.to(torch.float16)
        else:
            self.had_rem_dim = None

    def _table(self, device):
        if self.rem_dim == 1:
            return None
        return F_had.device_table(self.rem_dim, device)

    def forward(self, x):
        if x.dtype == torch.float16 or x.dtype == torch.float32:
            return _ops.hadamard(x, self._table(x.device), self.rem_dim)
        x_dtype = x.dtype
        return _ops.hadamard(x.float(), self._table(x.device), self.rem_dim).to(x_dtype)
