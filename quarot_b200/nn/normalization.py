import torch


class RMSNorm(torch.nn.Module):
    """Weight-less RMS normalisation computed in fp32 (quarot/nn/normalization.py:3-21).

    The learned scale of the original LLaMA norm is folded into the following
    linear layers offline, so only x / sqrt(mean(x^2) + eps) remains.
    """

    def __init__(self, mean_dim: int, eps=1e-5):
        super().__init__()
        self.eps = eps
        self.mean_dim = mean_dim

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out_dtype = x.dtype
        xf = x.float() if x.dtype == torch.float16 else x
        ms = xf.pow(2).sum(-1, keepdim=True) / self.mean_dim
        return (xf * torch.rsqrt(ms + self.eps)).to(out_dtype)
