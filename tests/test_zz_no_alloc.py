"""The allocation-free entry point qr_linear_i4_f16_static, called through the C ABI.

Some hosts of this library cannot allocate device memory in the decode loop: the process handed
its whole HBM budget to one arena at start-up, so there is nothing left for a cudaMalloc to take
the split-K workspace from (and a cudaMalloc that does succeed stalls every stream of the device
while it runs).  For them the kernel's scratch is a fixed array inside the library.  The check:
the same inputs through the ordinary entry point and through the static one give identical bits,
twice in a row (the second call finds the first call's leftovers in the shared array), and a shape
whose scratch would not fit is refused with a message instead of being run.

Collected last on purpose (file name), so that a run that stops at the first failure has already
executed every other test; it also passes on its own in a fresh process.
"""
import ctypes

import pytest
import torch

from quarot_b200 import _lib
from quarot_b200.functional.quantization import pack_i4

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LIMIT = (1 << 20) + (64 << 10)      # size of the scratch array inside the library


def _inputs(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    a = pack_i4(torch.randint(-8, 8, (M, K), generator=g, dtype=torch.int8)).to(DEV)
    w = pack_i4(torch.randint(-8, 8, (N, K), generator=g, dtype=torch.int8)).to(DEV)
    sa = (torch.rand(M, generator=g) * 0.5 + 0.05).half().to(DEV)
    sw = (torch.rand(N, generator=g) * 0.015 + 0.005).half().to(DEV)
    bias = (torch.randn(N, generator=g) * 0.5).half().to(DEV)
    return a, sa, w, sw, bias


def _call(fn, a, sa, w, sw, bias, M, N, K):
    out = torch.full((M, N), float("nan"), dtype=torch.float16, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(a.data_ptr(), sa.data_ptr(), w.data_ptr(), sw.data_ptr(), bias.data_ptr(), M, N, K,
            out.data_ptr(), N, stream)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("M,N,K", [(40, 4096, 11008), (48, 4096, 16384), (64, 4096, 11008), (24, 4096, 28672)])
def test_static_scratch_entry_matches_ordinary_entry_twice(M, N, K):
    lib = _lib.lib
    # these shapes do use the array: 33 .. 64 token rows on a narrow layer, or rows too long for the kernel that serves
    # fewer token rows without scratch
    assert 0 < lib.qr_linear_workspace_bytes(M, N, K) <= LIMIT
    first = _inputs(M, N, K, seed=1)
    second = _inputs(M, N, K, seed=2)
    for args in (first, second):                                        # two calls in a row share the array
        want = _call(lib.qr_linear_i4_f16, *args, M, N, K)
        got = _call(lib.qr_linear_i4_f16_static, *args, M, N, K)
        assert torch.equal(got, want)
    assert _lib.kernel_status() == 0


def test_static_scratch_entry_calls_of_different_shapes_share_the_array_and_allocate_nothing():
    lib = _lib.lib
    shapes = [(64, 4096, 11008), (40, 1000, 9216), (16, 4096, 4096), (48, 4096, 11008), (40, 1000, 9216), (64, 4096, 11008),
              (48, 4096, 4096)]      # the last one: two passes of the scratch-free kernel between calls that use the array
    cases = [(_inputs(M, N, K, seed=5 + i), (M, N, K)) for i, (M, N, K) in enumerate(shapes)]
    wants = [_call(lib.qr_linear_i4_f16, *args, *shape) for (args, shape) in cases]
    _call(lib.qr_linear_i4_f16_static, *cases[0][0], *cases[0][1])       # first call on the device: address look-up
    outs = [torch.full((M, N), float("nan"), dtype=torch.float16, device=DEV) for (M, N, K) in shapes]
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    stream = torch.cuda.current_stream().cuda_stream
    for (args, (M, N, K)), out in zip(cases, outs):                      # back to back on one stream, no host sync between
        a, sa, w, sw, bias = args
        rc = lib.qr_linear_i4_f16_static(a.data_ptr(), sa.data_ptr(), w.data_ptr(), sw.data_ptr(), bias.data_ptr(), M, N, K,
                                         out.data_ptr(), N, stream)
        assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before                   # the calls took no device memory
    for out, want in zip(outs, wants):
        assert torch.equal(out, want)
    assert _lib.kernel_status() == 0


def test_static_scratch_entry_refuses_what_does_not_fit():
    lib = _lib.lib
    # 40 tiles of 128 output channels x (128 x 64 int32 sums) = 1.25 MiB: more than the array holds
    M, N, K = 64, 5120, 10240
    assert lib.qr_linear_workspace_bytes(M, N, K) > LIMIT
    dummy = torch.zeros(16, dtype=torch.uint8, device=DEV)
    p = dummy.data_ptr()
    rc = lib.qr_linear_i4_f16_static(p, p, p, p, None, M, N, K, p, N, None)
    assert rc == -3 and "built-in scratch" in _lib.last_error()
    # a shape that needs no scratch at all (a wide layer: the weight rows are dealt out to the SMs) is simply run
    a, sa, w, sw, bias = _inputs(16, 24576, 1024, seed=3)
    assert lib.qr_linear_workspace_bytes(16, 24576, 1024) == 0
    want = _call(lib.qr_linear_i4_f16, a, sa, w, sw, bias, 16, 24576, 1024)
    got = _call(lib.qr_linear_i4_f16_static, a, sa, w, sw, bias, 16, 24576, 1024)
    assert torch.equal(got, want)
