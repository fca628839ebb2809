"""Thin torch wrappers over the C-ABI entry points (shape handling, checks, output allocation).

Mirrors the top-level functions of the upstream package (quarot/__init__.py:31-71)
and the argument checks of its bindings (quarot/kernels/bindings.cpp:9-87).
"""
import torch

from . import _lib

_lib_c = _lib.lib


def flatten_last_dim_and_return_shape(x: torch.Tensor):
    shape_excl_last = x.shape[:-1]
    return x.view(-1, x.shape[-1]), shape_excl_last


def _check_cuda_contig(op, **tensors):
    """The checks of the upstream bindings (quarot/kernels/bindings.cpp:11-16,29-34,52-64)."""
    dev = None
    for name, t in tensors.items():
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("%s: %s must be a CUDA tensor" % (op, name))
        if not t.is_contiguous():
            raise RuntimeError("%s: %s must be contiguous" % (op, name))
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("%s: %s is on %s, expected %s" % (op, name, t.device, dev))
    return dev


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def matmul(A, B):
    """int32 C[..., N] = unpack(A)[..., K] @ unpack(B)[N, K]^T  (quarot/__init__.py:37-41)."""
    assert A.shape[-1] % 32 == 0, "A.shape[-1]: {} must be multiplication of 32".format(A.shape[-1])
    A, A_shape_excl_last = flatten_last_dim_and_return_shape(A)
    B, B_shape_excl_last = flatten_last_dim_and_return_shape(B)
    dev = _check_cuda_contig("matmul", A=A, B=B)
    if A.dtype != torch.uint8 or B.dtype != torch.uint8:
        raise RuntimeError("matmul: packed int4 operands must be uint8")
    if A.shape[1] != B.shape[1]:
        raise RuntimeError("matmul: inner dimensions differ (%d vs %d packed bytes)" % (A.shape[1], B.shape[1]))
    M, N, K = A.shape[0], B.shape[0], A.shape[1] * 2
    with torch.cuda.device(dev):
        C = torch.empty((M, N), dtype=torch.int32, device=dev)
        _lib.check(_lib_c.qr_matmul_i4_i32(A.data_ptr(), B.data_ptr(), M, N, K, C.data_ptr(), _stream(dev)),
                   "matmul")
    return C.view(*A_shape_excl_last, *B_shape_excl_last)


def sym_quant(x, scale):
    """uint8 q[..., ceil(K/2)] = pack(clamp(round(x / scale), -8, 7))  (quarot/__init__.py:43-46)."""
    assert x.dtype == scale.dtype == torch.float16
    x, x_shape_excl_last = flatten_last_dim_and_return_shape(x)
    scale = scale.view(-1)
    dev = _check_cuda_contig("sym_quant", x=x, scale=scale)
    if scale.shape[0] != x.shape[0]:
        raise RuntimeError("sym_quant: scale has %d entries, x has %d rows" % (scale.shape[0], x.shape[0]))
    rows, cols = x.shape
    with torch.cuda.device(dev):
        q = torch.empty((rows, (cols + 1) // 2), dtype=torch.uint8, device=dev)
        _lib.check(_lib_c.qr_sym_quant_i4(x.data_ptr(), scale.data_ptr(), rows, cols, q.data_ptr(), _stream(dev)),
                   "sym_quant")
    return q.view(*x_shape_excl_last, -1)


def sym_dequant(q, scale_row, scale_col, bits=32):
    """fp16 out = scale_row * scale_col * half(q)  (quarot/__init__.py:48-52)."""
    assert q.dtype == torch.int32
    assert scale_row.dtype == scale_col.dtype == torch.float16
    q, q_shape_excl_last = flatten_last_dim_and_return_shape(q)
    scale_row = scale_row.view(-1)
    dev = _check_cuda_contig("sym_dequant", q=q, scale_row=scale_row, scale_col=scale_col)
    rows, cols = q.shape
    if scale_row.shape[0] != rows:
        raise RuntimeError("sym_dequant: scale_row has %d entries, q has %d rows" % (scale_row.shape[0], rows))
    if scale_col.shape[0] != cols:
        raise RuntimeError("sym_dequant: scale_col has %d entries, q has %d columns" % (scale_col.shape[0], cols))
    if bits != 32:
        raise RuntimeError("Unsupported data type")
    with torch.cuda.device(dev):
        out = torch.empty((rows, cols), dtype=torch.float16, device=dev)
        _lib.check(_lib_c.qr_sym_dequant_i32_f16(q.data_ptr(), scale_row.data_ptr(), scale_col.data_ptr(),
                                                 rows, cols, out.data_ptr(), _stream(dev)), "sym_dequant")
    return out.view(*q_shape_excl_last, -1)


class PackedQuantizedTensor:
    """Packed int4 activations plus their per-token scales (quarot/__init__.py:55-71)."""

    def __init__(self, quantized_x: torch.Tensor, scales_x: torch.Tensor):
        self.quantized_x = quantized_x
        self.scales_x = scales_x

    def size(self):
        return self.quantized_x.size()

    @property
    def device(self):
        return self.quantized_x.device

    @property
    def dtype(self):
        return self.quantized_x.dtype


# ------------------------------------------------------------------ fused entry points
def _heads_axis_view(x, K):
    """(base, heads, head_dim) when x is the transposed view [..., head_dim, heads] of a contiguous fp16 tensor
    [..., heads, head_dim] that the heads-axis kernel serves (what the attention block hands to its Hadamard in front
    of o_proj), else None."""
    if K != 1 or x.dim() < 2 or x.dtype != torch.float16 or x.is_contiguous():
        return None
    base = x.transpose(-1, -2)
    heads, hd = base.shape[-2], base.shape[-1]
    n = heads * hd
    if not base.is_contiguous() or heads & (heads - 1) or hd & (hd - 1) or hd < 32 or not 256 <= n <= 4096:
        return None
    return base, heads, hd


def hadamard(x, had_k=None, K=1):
    """Online Hadamard over the last axis of an fp16/fp32 CUDA tensor (one kernel)."""
    tv = _heads_axis_view(x, K) if x.is_cuda else None
    if tv is not None:
        base, heads, hd = tv
        with torch.cuda.device(base.device):
            y = torch.empty_like(base)
            rows = base.numel() // (heads * hd)
            _lib.check(_lib_c.qr_hadamard_heads_f16(base.data_ptr(), y.data_ptr(), rows, heads, hd, _stream(base.device)),
                       "hadamard (heads axis)")
        return y.transpose(-1, -2)
    x2, shape_excl_last = flatten_last_dim_and_return_shape(x.contiguous())
    dev = _check_cuda_contig("hadamard", x=x2, had_k=had_k)
    rows, n = x2.shape
    with torch.cuda.device(dev):
        y = torch.empty_like(x2)
        hk = had_k.data_ptr() if had_k is not None else None
        if x2.dtype == torch.float16:
            rc = _lib_c.qr_hadamard_f16(x2.data_ptr(), y.data_ptr(), rows, n, hk, K, _stream(dev))
        elif x2.dtype == torch.float32:
            rc = _lib_c.qr_hadamard_f32(x2.data_ptr(), y.data_ptr(), rows, n, hk, K, _stream(dev))
        else:
            raise RuntimeError("hadamard: dtype %s not supported (fp16 or fp32)" % x2.dtype)
        _lib.check(rc, "hadamard")
    return y.view(*shape_excl_last, n)


def hadamard_quant(x, had_k=None, K=0, clip=1.0, return_y=False, out_q=None, out_s=None):
    """Fused [Hadamard ->] per-token scale -> int4 quantise-and-pack.

    x fp16 [..., n].  K = 0 skips the transform.  Returns (q uint8 [..., n/2],
    scales fp16 [rows], y fp16 [..., n] or None).  out_q / out_s may supply
    preallocated contiguous outputs of those shapes.
    """
    assert x.dtype == torch.float16
    x2, shape_excl_last = flatten_last_dim_and_return_shape(x)
    dev = _check_cuda_contig("hadamard_quant", x=x2, had_k=had_k)
    rows, n = x2.shape
    if n % 2:
        raise RuntimeError("hadamard_quant: last dimension must be even")
    with torch.cuda.device(dev):
        q = out_q if out_q is not None else torch.empty((rows, n // 2), dtype=torch.uint8, device=dev)
        s = out_s if out_s is not None else torch.empty((rows,), dtype=torch.float16, device=dev)
        if q.numel() != rows * (n // 2) or s.numel() != rows or not q.is_contiguous() or not s.is_contiguous():
            raise RuntimeError("hadamard_quant: preallocated outputs have the wrong size")
        y = torch.empty((rows, n), dtype=torch.float16, device=dev) if return_y else None
        _lib.check(_lib_c.qr_hadamard_quant_i4(
            x2.data_ptr(), rows, n, n, had_k.data_ptr() if had_k is not None else None, K, float(clip),
            q.data_ptr(), s.data_ptr(), y.data_ptr() if y is not None else None, _stream(dev)), "hadamard_quant")
    return (q.view(*shape_excl_last, n // 2), s.view(-1), y.view(*shape_excl_last, n) if y is not None else None)


_WORKSPACES = {}


def reset_workspaces():
    """Forget the cached scratch buffers.  A kernel that gave up on a bounded wait (non-zero
    `_lib.kernel_status()`) may leave counters or sums behind in its scratch; fresh zeroed buffers are
    allocated on the next use."""
    _WORKSPACES.clear()


def _workspace(dev, nbytes):
    """Per-(device, stream) zero-initialised scratch for narrow layers at decode sizes, grown on demand.
    Launches on one stream are ordered, so they can share it; different streams get their own."""
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
        _WORKSPACES[key] = ws
    return ws


def linear_i4(q_x, scales_x, weight, weight_scales, bias=None, out=None, use_workspace=True):
    """Fused Linear4bit forward: int4 GEMM with the dequantisation in the epilogue.

    q_x uint8 [..., K/2], scales_x fp16 (any shape with one entry per row),
    weight uint8 [N, K/2], weight_scales fp16 [N] or [N, 1].  Returns fp16 [..., N].
    For decode-sized inputs (at most 64 rows) on narrow layers the work is dealt out to all SMs through a
    cached scratch buffer (`use_workspace=False` runs without scratch; results are identical).
    """
    assert q_x.shape[-1] % 32 == 0, "A.shape[-1]: {} must be multiplication of 32".format(q_x.shape[-1])
    assert scales_x.dtype == weight_scales.dtype == torch.float16
    A, A_shape_excl_last = flatten_last_dim_and_return_shape(q_x)
    sx = scales_x.view(-1)
    sw = weight_scales.view(-1)
    dev = _check_cuda_contig("linear_i4", q_x=A, scales_x=sx, weight=weight, weight_scales=sw, bias=bias)
    if A.dtype != torch.uint8 or weight.dtype != torch.uint8:
        raise RuntimeError("linear_i4: packed int4 operands must be uint8")
    M, N, K = A.shape[0], weight.shape[0], A.shape[1] * 2
    if weight.shape[1] != A.shape[1]:
        raise RuntimeError("linear_i4: inner dimensions differ")
    if sx.shape[0] != M or sw.shape[0] != N:
        raise RuntimeError("linear_i4: scale sizes do not match the operands")
    if bias is not None and (bias.dtype != torch.float16 or bias.numel() != N):
        raise RuntimeError("linear_i4: bias must be fp16 with one entry per output channel")
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty((M, N), dtype=torch.float16, device=dev)
        ldo = out.stride(0) if M > 1 else max(out.stride(0), N)
        ws_bytes = _lib_c.qr_linear_workspace_bytes(M, N, K) if use_workspace else 0
        if ws_bytes:
            ws = _workspace(dev, ws_bytes)
            rc = _lib_c.qr_linear_i4_f16_ws(A.data_ptr(), sx.data_ptr(), weight.data_ptr(), sw.data_ptr(),
                                            bias.data_ptr() if bias is not None else None, M, N, K,
                                            out.data_ptr(), ldo, ws.data_ptr(), ws.numel(), _stream(dev))
        else:
            rc = _lib_c.qr_linear_i4_f16(A.data_ptr(), sx.data_ptr(), weight.data_ptr(), sw.data_ptr(),
                                         bias.data_ptr() if bias is not None else None, M, N, K,
                                         out.data_ptr(), ldo, _stream(dev))
        _lib.check(rc, "linear_i4")
    return out.view(*A_shape_excl_last, N) if out.is_contiguous() else out


def linear_i4_outs(q_x, scales_x, weight, weight_scales, bias, out_ptrs, ldo):
    """Fused Linear4bit forward whose [M, N] result is written to several places at once: `out_ptrs` are device
    addresses (ints) of [M, N] blocks with row pitch `ldo`, on this GPU or on peers this process can address.
    One tiled store per destination leaves the epilogue; see qr_linear_i4_f16_outs.  Returns nothing."""
    assert q_x.shape[-1] % 32 == 0, "A.shape[-1]: {} must be multiplication of 32".format(q_x.shape[-1])
    A, _ = flatten_last_dim_and_return_shape(q_x)
    sx = scales_x.view(-1)
    sw = weight_scales.view(-1)
    dev = _check_cuda_contig("linear_i4_outs", q_x=A, scales_x=sx, weight=weight, weight_scales=sw, bias=bias)
    M, N, K = A.shape[0], weight.shape[0], A.shape[1] * 2
    if weight.shape[1] != A.shape[1] or sx.shape[0] != M or sw.shape[0] != N:
        raise RuntimeError("linear_i4_outs: operand sizes do not match")
    import ctypes
    arr = (ctypes.c_void_p * len(out_ptrs))(*[int(p) for p in out_ptrs])
    with torch.cuda.device(dev):
        rc = _lib_c.qr_linear_i4_f16_outs(A.data_ptr(), sx.data_ptr(), weight.data_ptr(), sw.data_ptr(),
                                          bias.data_ptr() if bias is not None else None, M, N, K,
                                          arr, len(out_ptrs), int(ldo), _stream(dev))
        _lib.check(rc, "linear_i4_outs")


def linear_i4_swiglu(q_x, scales_x, weight_gu, scales_gu, out=None):
    """silu(gate_proj(x)) * up_proj(x) as one GEMM with the product in the epilogue.

    weight_gu uint8 [2 I, K/2] and scales_gu fp16 [2 I] hold the gate and up weights interleaved in groups of 128
    output channels (see `interleave_gate_up`).  Returns fp16 [..., I].  Needs more than 128 token rows."""
    assert q_x.shape[-1] % 32 == 0, "A.shape[-1]: {} must be multiplication of 32".format(q_x.shape[-1])
    A, A_shape_excl_last = flatten_last_dim_and_return_shape(q_x)
    sx = scales_x.view(-1)
    sw = scales_gu.view(-1)
    dev = _check_cuda_contig("linear_i4_swiglu", q_x=A, scales_x=sx, weight=weight_gu, weight_scales=sw)
    M, N2, K = A.shape[0], weight_gu.shape[0], A.shape[1] * 2
    if weight_gu.shape[1] != A.shape[1] or sx.shape[0] != M or sw.shape[0] != N2:
        raise RuntimeError("linear_i4_swiglu: operand sizes do not match")
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty((M, N2 // 2), dtype=torch.float16, device=dev)
        rc = _lib_c.qr_linear_i4_swiglu_f16(A.data_ptr(), sx.data_ptr(), weight_gu.data_ptr(), sw.data_ptr(),
                                            M, N2, K, out.data_ptr(), out.stride(0), _stream(dev))
        _lib.check(rc, "linear_i4_swiglu")
    return out.view(*A_shape_excl_last, N2 // 2) if out.is_contiguous() else out


def interleave_gate_up(gate, up, group=128):
    """Rows of `gate` and `up` ([I, ...], same shape) interleaved in groups of `group` rows:
    [gate[0:g]; up[0:g]; gate[g:2g]; up[g:2g]; ...] -- the operand layout of linear_i4_swiglu."""
    if gate.shape != up.shape or gate.shape[0] % group:
        raise ValueError("interleave_gate_up: shapes %s / %s, rows must be a multiple of %d" % (tuple(gate.shape), tuple(up.shape), group))
    t = gate.shape[0] // group
    rest = tuple(gate.shape[1:])
    both = torch.stack((gate.reshape(t, group, *rest), up.reshape(t, group, *rest)), dim=1)
    return both.reshape(2 * gate.shape[0], *rest).contiguous()


def rmsnorm_quant(x, mean_dim, eps=1e-5, clip=1.0, return_y=False):
    """Weight-less RMSNorm followed by the per-token quantiser, in one pass over x.

    x fp16 [..., n].  Returns (q uint8 [..., n/2], scales fp16 [rows], y fp16 [..., n] or None)."""
    assert x.dtype == torch.float16
    x2, shape_excl_last = flatten_last_dim_and_return_shape(x)
    dev = _check_cuda_contig("rmsnorm_quant", x=x2)
    rows, n = x2.shape
    with torch.cuda.device(dev):
        q = torch.empty((rows, n // 2), dtype=torch.uint8, device=dev)
        s = torch.empty((rows,), dtype=torch.float16, device=dev)
        y = torch.empty((rows, n), dtype=torch.float16, device=dev) if return_y else None
        rc = _lib_c.qr_rmsnorm_quant_i4(x2.data_ptr(), rows, n, x2.stride(0), int(mean_dim), float(eps), float(clip),
                                        q.data_ptr(), s.data_ptr(), y.data_ptr() if return_y else None, _stream(dev))
        _lib.check(rc, "rmsnorm_quant")
    return (q.view(*shape_excl_last, n // 2), s, y.view(*shape_excl_last, n) if return_y else None)


def quant_linear_i4(x, weight, weight_scales, bias=None, clip=1.0, out=None):
    """Quantizer + Linear4bit in one launch for at most 8 token rows (x fp16 [..., K] -> fp16 [..., N])."""
    assert x.dtype == torch.float16
    x2, shape_excl_last = flatten_last_dim_and_return_shape(x)
    sw = weight_scales.view(-1)
    dev = _check_cuda_contig("quant_linear_i4", x=x2, weight=weight, weight_scales=sw, bias=bias)
    M, K = x2.shape
    N = weight.shape[0]
    if weight.shape[1] * 2 != K or sw.shape[0] != N:
        raise RuntimeError("quant_linear_i4: operand sizes do not match")
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty((M, N), dtype=torch.float16, device=dev)
        ldo = out.stride(0) if M > 1 else max(out.stride(0), N)
        rc = _lib_c.qr_quant_linear_i4_f16(x2.data_ptr(), x2.stride(0) if M > 1 else max(x2.stride(0), K), float(clip),
                                           weight.data_ptr(), sw.data_ptr(), bias.data_ptr() if bias is not None else None,
                                           M, N, K, out.data_ptr(), ldo, _stream(dev))
        _lib.check(rc, "quant_linear_i4")
    return out.view(*shape_excl_last, N) if out.is_contiguous() else out

