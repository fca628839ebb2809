"""Multi-GPU forms of the quantized-linear path (one process per GPU, torch.distributed).

Two partitionings, both from the fact that token rows and output channels are independent:

* row sharding -- every rank holds the full weights and runs the unchanged modules on its own
  contiguous block of token rows; there is no collective on the data path (`shard_rows`,
  `gather_rows` exists only to verify equality with the single-GPU result);
* column split -- rank r holds output channels [r N/G, (r+1) N/G) of one Linear4bit (weights,
  scales, bias), every rank sees all token rows, and the fp16 result slabs are all-gathered over
  NVLink (`ColumnSplitLinear4bit`).

The upstream project has no multi-GPU code on this path; the upstream Linear4bit launches on the
legacy default stream without a device guard (quarot/nn/linear.py:43-44, quarot/kernels/gemm.cu:41).
"""
import torch
import torch.distributed as dist

from . import _ops


def shard_rows(num_rows, world_size, rank):
    """[start, end) of the contiguous block of token rows owned by `rank` (sizes differ by at most 1)."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError("bad rank %d / world size %d" % (rank, world_size))
    base, extra = divmod(num_rows, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def gather_rows(local, num_rows, group=None):
    """Concatenate the row shards of all ranks (verification helper; not on the data path)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    spans = [shard_rows(num_rows, world, r) for r in range(world)]
    mine = spans[rank][1] - spans[rank][0]
    if local.shape[0] != mine:
        raise RuntimeError("gather_rows: this rank holds %d rows, expected %d" % (local.shape[0], mine))
    # shards differ by at most one row; collectives want equal sizes, so pad to the largest
    most = max(e - s for (s, e) in spans)
    padded = torch.zeros((most,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[:mine] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([parts[r][: spans[r][1] - spans[r][0]] for r in range(world)], dim=0)


def split_columns(weight, weight_scales, bias, world_size, rank):
    """The slice of a Linear4bit's buffers (weight [N, K/2], weight_scales [N, 1], bias [N] or None)
    that rank `rank` owns under a column split.  N must be divisible by the world size."""
    n = weight.shape[0]
    if n % world_size:
        raise ValueError("out_features %d is not divisible by %d ranks" % (n, world_size))
    per = n // world_size
    sl = slice(rank * per, (rank + 1) * per)
    return (weight[sl].contiguous(), weight_scales[sl].contiguous(),
            None if bias is None else bias[sl].contiguous())


class ColumnSplitLinear4bit(torch.nn.Module):
    """Linear4bit whose output channels are split over the ranks of a process group.

    forward(PackedQuantizedTensor with ALL token rows) -> fp16 [..., N] on every rank: the local
    int4 GEMM (with fused dequantisation) produces the slab [M, N/G]; the slabs are all-gathered
    ([G, M, N/G]) and interleaved into row-major [M, N].  `compute` is the function that evaluates
    the local slab (default: the CUDA kernel); tests on CPU ranks inject a reference.
    """

    def __init__(self, weight, weight_scales, bias=None, group=None, compute=None):
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        w, s, b = split_columns(weight, weight_scales, bias, self.world, self.rank)
        self.register_buffer("weight", w)
        self.register_buffer("weight_scales", s)
        if b is not None:
            self.register_buffer("bias", b)
        else:
            self.bias = None
        self.out_features = weight.shape[0]
        self._compute = compute if compute is not None else _ops.linear_i4

    def local_forward(self, x):
        assert type(x) == _ops.PackedQuantizedTensor
        return self._compute(x.quantized_x, x.scales_x, self.weight, self.weight_scales, self.bias)

    def forward(self, x, gathered_out=None):
        local = self.local_forward(x)
        lead = local.shape[:-1]
        local2 = local.reshape(-1, local.shape[-1]).contiguous()
        m, n_loc = local2.shape
        if self.world == 1:
            if gathered_out is None:
                return local
            gathered_out.view(m, n_loc).copy_(local2)
            return gathered_out.view(*lead, self.out_features)
        slabs = torch.empty((self.world, m, n_loc), dtype=local2.dtype, device=local2.device)
        dist.all_gather_into_tensor(slabs.view(self.world * m, n_loc), local2, group=self.group)
        out = gathered_out if gathered_out is not None else torch.empty((m, self.out_features), dtype=local2.dtype,
                                                                        device=local2.device)
        out.view(m, self.world, n_loc).copy_(slabs.permute(1, 0, 2))
        return out.view(*lead, self.out_features)


class SymmetricOutput:
    """An fp16 [rows, cols] matrix that exists at the same place in a symmetric allocation on every rank of the
    group, together with the device addresses under which THIS process can write every rank's copy over NVLink
    (torch.distributed symmetric memory).  `barrier()` is a device-side barrier over the ranks on the current
    stream: one before the copies are overwritten, one before they are read."""

    def __init__(self, rows, cols, device, group=None):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only, no multicast objects
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.local = symm_mem.empty((rows, cols), dtype=torch.float16, device=device)
        self.handle = symm_mem.rendezvous(self.local, self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.rows, self.cols = rows, cols

    def barrier(self):
        self.handle.barrier()


class FusedColumnSplitLinear4bit(ColumnSplitLinear4bit):
    """Column split without the all-gather: the epilogue of the local GEMM stores every tile of its [M, N/G] slab
    straight into the column block [r N/G, (r+1) N/G) of EVERY rank's full [M, N] matrix (one tiled store per
    rank, the remote ones cross NVLink while the tensor cores work on the next tile)."""

    def forward(self, x, target):
        """x: PackedQuantizedTensor with all token rows; target: SymmetricOutput of shape [M, N].  Returns the
        local [M, N] matrix after all ranks' slabs have landed."""
        assert type(x) == _ops.PackedQuantizedTensor
        n_loc = self.weight.shape[0]
        if target.cols != self.out_features or n_loc * self.world != self.out_features:
            raise RuntimeError("FusedColumnSplitLinear4bit: target has %d columns, expected %d" % (target.cols, self.out_features))
        col_bytes = 2 * n_loc * self.rank
        rows = x.quantized_x.numel() // x.quantized_x.shape[-1]
        target.barrier()          # nobody still reads the previous contents
        if rows > 128:
            # destinations start with this rank's own copy and go round the ring: the kernel visits them in an order that
            # depends on the tile and the warp only, so at any moment the ranks write to different peers
            ptrs = target.ptrs[self.rank:] + target.ptrs[:self.rank]
            _ops.linear_i4_outs(x.quantized_x, x.scales_x, self.weight, self.weight_scales, self.bias,
                                [p + col_bytes for p in ptrs], target.cols)
        else:
            # few token rows (served by the decode kernels): the slab is computed locally and copied into the
            # column block of every rank's matrix
            local = self.local_forward(x).reshape(rows, n_loc)
            for g in range(self.world):
                peer = target.handle.get_buffer(g, (target.rows, target.cols), torch.float16)
                peer[:rows, self.rank * n_loc:(self.rank + 1) * n_loc].copy_(local)
        target.barrier()          # every rank's slab is in every copy
        return target.local

