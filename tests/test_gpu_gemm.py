"""CUDA kernels of family (b) -- int4 GEMM (tcgen05) and the fused dequant epilogue --
against the CPU oracle and the upstream-generated fixtures, through the C-ABI."""
import numpy as np
import pytest
import torch

import quarot_b200 as qb
from quarot_b200 import _lib, synth
from quarot_b200.functional.quantization import pack_i4
from oracle import quarot_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rand_packed(rows, k, seed):
    g = torch.Generator().manual_seed(seed)
    return pack_i4(torch.randint(-8, 8, (rows, k), generator=g, dtype=torch.int8))


def test_matmul_matches_upstream_fixtures(golden):
    g = golden["matmul"]
    for t in ("s", "m", "l"):
        a, b = torch.from_numpy(g[t + "_a"]).to(DEV), torch.from_numpy(g[t + "_b"]).to(DEV)
        c = qb.matmul(a, b).cpu()
        assert c.dtype == torch.int32 and np.array_equal(c.numpy(), g[t + "_c"]), t
    assert _lib.kernel_status() == 0


@pytest.mark.parametrize("M,N,K", [(1, 16, 64), (3, 7, 64), (8, 4096, 4096), (16, 128, 192), (17, 130, 256),
                                   (32, 272, 1024), (33, 48, 320), (64, 256, 4096), (65, 256, 128),
                                   (128, 256, 128), (129, 257, 448), (130, 272, 1024), (256, 512, 11008),
                                   (300, 1000, 2048), (512, 384, 28672)])
def test_matmul_bit_exact_random_shapes(M, N, K):
    a, b = _rand_packed(M, K, M * 3 + K), _rand_packed(N, K, N * 5 + K)
    c = qb.matmul(a.to(DEV), b.to(DEV)).cpu()
    assert torch.equal(c, O.matmul_i4(a, b))
    assert _lib.kernel_status() == 0


def test_matmul_extreme_codes_no_overflow():
    # all -8 x all -8 is the largest accumulator: 64 K (x256 inside the kernel)
    K = 28672
    a = torch.full((130, K // 2), 0x88, dtype=torch.uint8)
    b = torch.full((40, K // 2), 0x88, dtype=torch.uint8)
    c = qb.matmul(a.to(DEV), b.to(DEV)).cpu()
    assert int(c.min()) == int(c.max()) == 64 * K
    b7 = torch.full((40, K // 2), 0x77, dtype=torch.uint8)
    c = qb.matmul(a.to(DEV), b7.to(DEV)).cpu()
    assert int(c.min()) == int(c.max()) == -56 * K


def test_matmul_leading_dims_and_errors():
    a, b = _rand_packed(2 * 3, 128, 1).view(2, 3, 64), _rand_packed(5, 128, 2)
    c = qb.matmul(a.to(DEV), b.to(DEV))
    assert c.shape == (2, 3, 5)
    assert torch.equal(c.cpu().view(6, 5), O.matmul_i4(a.view(6, 64), b))
    with pytest.raises(AssertionError):
        qb.matmul(torch.zeros(2, 24, dtype=torch.uint8, device=DEV), b.to(DEV))
    with pytest.raises(RuntimeError):
        qb.matmul(a.to(DEV), torch.zeros(5, 32, dtype=torch.uint8, device=DEV))
    with pytest.raises(RuntimeError):
        qb.matmul(a.to(DEV).transpose(0, 1), b.to(DEV))


TILE_CONFIGS = {
    "2sm_ss_grid3": {"gemm_grid": 3},
    "2sm_bn256": {"gemm_bn2": 256},
    "2sm_bn240": {"gemm_bn2": 240},
    "2sm_bn224_grid3": {"gemm_bn2": 224, "gemm_grid": 3},
    "2sm_bn192": {"gemm_bn2": 192},
    "2sm_ss_elementwise_stores": {"gemm_tma_out": 0},
    "1sm_bn256": {"gemm_2sm": 0},
    "1sm_bn128": {"gemm_2sm": 0, "gemm_bn": 128},
    "1sm_bn64": {"gemm_2sm": 0, "gemm_bn": 64},
    "1sm_pst3": {"gemm_2sm": 0, "gemm_pst": 3},
    "1sm_grid3": {"gemm_2sm": 0, "gemm_grid": 3},
}
TILE_DEFAULTS = {"gemm_2sm": 1, "gemm_bn2": 0, "gemm_bn": 256, "gemm_pst": 4, "gemm_grid": 0, "gemm_tma_out": 1}


@pytest.mark.parametrize("tiles", sorted(TILE_CONFIGS))
def test_matmul_other_tile_configs_agree(tiles):
    a, b = _rand_packed(300, 2048, 1), _rand_packed(1000, 2048, 2)
    want = O.matmul_i4(a, b)
    sx = (torch.rand(300) * 0.5 + 0.05).half()
    sw = (torch.rand(1000) * 0.015 + 0.005).half()
    bias = (torch.randn(1000) * 0.5).half()
    for k, v in TILE_CONFIGS[tiles].items():
        _lib.set_tuning(k, v)
    try:
        c = qb.matmul(a.to(DEV), b.to(DEV)).cpu()
        o = qb.linear_i4(a.to(DEV), sx.to(DEV), b.to(DEV), sw.to(DEV)).cpu()
        ob = qb.linear_i4(a.to(DEV), sx.to(DEV), b.to(DEV), sw.to(DEV), bias.to(DEV)).cpu()
    finally:
        for k, v in TILE_DEFAULTS.items():
            _lib.set_tuning(k, v)
    assert torch.equal(c, want)
    assert torch.equal(o, O.sym_dequant_fp32(want, sx, sw).half())
    assert torch.equal(ob, O.sym_dequant_fp32(want, sx, sw).half() + bias)
    assert _lib.kernel_status() == 0


@pytest.mark.parametrize("M,N,K,pitch", [(300, 1000, 512, 2048), (520, 264, 256, 272), (257, 72, 128, 84)])
def test_linear_into_a_strided_output(M, N, K, pitch):
    """The result may land in a column block of a wider matrix (row pitch > N): everything outside the
    block stays untouched, for the tiled-store epilogue (pitch a multiple of 8) and the element-wise one."""
    a, w = _rand_packed(M, K, 5), _rand_packed(N, K, 6)
    sx = (torch.rand(M) * 0.5 + 0.05).half()
    sw = (torch.rand(N) * 0.015 + 0.005).half()
    bias = torch.randn(N).half()
    want = O.sym_dequant_fp32(O.matmul_i4(a, w), sx, sw).half() + bias
    off = 8
    buf = torch.full((M, pitch), 7.0, dtype=torch.float16, device=DEV)
    view = buf[:, off:off + N]
    qb.linear_i4(a.to(DEV), sx.to(DEV), w.to(DEV), sw.to(DEV), bias.to(DEV), out=view)
    got = buf.cpu()
    assert torch.equal(got[:, off:off + N], want)
    assert bool((got[:, :off] == 7.0).all()) and bool((got[:, off + N:] == 7.0).all())
    assert _lib.kernel_status() == 0


def _linear_close(out, ref):
    err = (out.double() - ref.double()).abs()
    tol = 1e-2 * ref.double().abs() + 1e-2 * float(ref.abs().max()) * 2.0 ** -10
    return bool((err <= tol).all()), float((err / (ref.double().abs() + 1e-6)).max())


@pytest.mark.parametrize("M,N,K,bias", [(1, 4096, 4096, False), (8, 256, 4096, True), (32, 272, 1024, False),
                                        (64, 512, 11008, True), (129, 257, 448, True), (256, 4096, 4096, False),
                                        (300, 1000, 2048, True)])
def test_linear_fused_dequant_vs_fp32_oracle(M, N, K, bias):
    g = torch.Generator().manual_seed(M + N)
    a, w = _rand_packed(M, K, 3), _rand_packed(N, K, 4)
    sx = (torch.rand(M, generator=g) * 0.5 + 0.05).half()
    sw = (torch.rand(N, 1, generator=g) * 0.015 + 0.005).half()
    bvec = (torch.randn(N, generator=g) * 0.5).half() if bias else None
    out = qb.linear_i4(a.to(DEV), sx.to(DEV), w.to(DEV), sw.to(DEV), bvec.to(DEV) if bias else None).cpu()
    ref = O.sym_dequant_fp32(O.matmul_i4(a, w), sx, sw)
    if bias:
        # upstream adds the bias in fp16 after rounding the product
        assert torch.equal(out, ref.half() + bvec)
    else:
        ok, worst = _linear_close(out, ref)
        assert ok, worst
        # one fp32 product rounded once: identical to the fp32 oracle rounded to fp16
        assert torch.equal(out, ref.half())
    assert _lib.kernel_status() == 0


def test_module_graph_config0_slice():
    """Sequential(OnlineHadamard, Quantizer, Linear4bit) as the callers build it, 256 token rows of config 0."""
    M, K, N = 256, 4096, 4096
    x = synth.activations(M, K, seed=1234)
    w, sw = synth.weights(N, K, seed=4321)
    lin = qb.nn.Linear4bit(K, N).to(DEV)
    lin.weight.copy_(w)
    lin.weight_scales = sw.to(DEV)
    seq = torch.nn.Sequential(qb.nn.OnlineHadamard(K), qb.nn.Quantizer(), lin).to(DEV)
    out = seq(x.to(DEV).view(2, 128, K))
    assert out.shape == (2, 128, N) and out.dtype == torch.float16
    # oracle fed with the kernel's own Hadamard output
    y = seq[0](x.to(DEV)).cpu()
    s = O.quantizer_scales(y)
    acc = O.matmul_i4(O.pack_i4(O.sym_quant_codes(y, s)), w)
    ref = O.sym_dequant_fp32(acc, s, sw)
    assert torch.equal(out.cpu().view(M, N), ref.half())
    # int32 path of the unfused operators agrees bit for bit
    p = seq[1](seq[0](x.to(DEV)))
    assert torch.equal(qb.matmul(p.quantized_x, lin.weight).cpu(), acc)
    # and the whole thing is within 1e-2 of the fp32 reference built from the fp32 Hadamard
    full = O.linear4bit_forward(x, w, sw, hadamard_dim=K)
    rel = (out.cpu().view(M, N).float() - full["out"]).norm() / full["out"].norm()
    assert float(rel) < 1e-2
    # fused module rewrite gives the same output
    assert qb.nn.fuse_modules(seq) == 1
    assert torch.equal(seq(x.to(DEV).view(2, 128, K)), out)
    assert _lib.kernel_status() == 0


def test_from_float_roundtrip():
    g = torch.Generator().manual_seed(2)
    lin = torch.nn.Linear(256, 64, bias=True).half()
    codes = torch.randint(-8, 8, (64, 256), generator=g).half()
    s_w = (torch.rand(64, 1, generator=g) * 0.01 + 0.005).half()
    lin.weight.data = codes * s_w
    q = qb.nn.Linear4bit.from_float(lin, weight_scales=s_w).to(DEV)
    assert torch.equal(O.unpack_i4(q.weight.cpu()).half(), codes)
    x = synth.activations(9, 256, seed=1).to(DEV)
    out = torch.nn.Sequential(qb.nn.Quantizer(), q)(x)
    ref = O.linear4bit_forward(x.cpu(), q.weight.cpu(), s_w, bias=lin.bias.data)
    assert torch.allclose(out.cpu().float(), ref["out"], rtol=4e-3, atol=4e-3)
    rnd = qb.nn.Linear4bit.from_float(torch.nn.Linear(64, 8, bias=False).half())
    assert float(rnd.weight_scales.abs().max()) == 0.0


def test_full_size_config0_properties():
    """The single-linear configuration (M 2048, K 4096, N 4096) at full size: checksum identity over all 8.4 M accumulators plus sampled rows."""
    M, K, N = 2048, 4096, 4096
    x = synth.activations(M, K, seed=1234).to(DEV)
    w, sw = synth.weights(N, K, seed=4321)
    q, s, y = qb.hadamard_quant(x, None, 1, 1.0, return_y=True)
    acc = qb.matmul(q, w.to(DEV))
    # sum_mn C[m,n] == sum_k (sum_m A[m,k]) (sum_n B[n,k])
    ua, ub = O.unpack_i4(q.cpu()).long(), O.unpack_i4(w).long()
    assert int(acc.long().sum()) == int((ua.sum(0) * ub.sum(0)).sum())
    rows = torch.arange(0, M, 37)
    assert torch.equal(acc.cpu()[rows], O.matmul_i4(q.cpu()[rows], w))
    # codes bit-exact for the sampled rows given the kernel's Hadamard output
    s_ref = O.quantizer_scales(y.cpu()[rows])
    assert torch.equal(s.cpu()[rows], s_ref)
    assert torch.equal(q.cpu()[rows], O.pack_i4(O.sym_quant_codes(y.cpu()[rows], s_ref)))
    out = qb.linear_i4(q, s, w.to(DEV), sw.to(DEV))
    ref = O.sym_dequant_fp32(acc.cpu()[rows], s_ref, sw)
    assert torch.equal(out.cpu()[rows], ref.half())
    # determinism: a second run is bitwise identical
    assert torch.equal(qb.linear_i4(q, s, w.to(DEV), sw.to(DEV)), out)
    assert _lib.kernel_status() == 0


@pytest.fixture
def tcgen05_decode_kernel():
    """At most 32 token rows go to the mma.sync weight-streaming kernel by default; these tests are about the tcgen05
    decode kernel behind it (33 .. 64 rows, or rows of more values than fit into shared memory), so they switch the
    other one off."""
    _lib.set_tuning("gemv_mma_max_m", 0)
    _lib.set_tuning("gemm_splitk", 2)          # narrow layers through scratch memory whatever K (default: K > 8192 only)
    yield
    _lib.set_tuning("gemv_mma_max_m", 32)
    _lib.set_tuning("gemm_splitk", 1)


@pytest.mark.usefixtures("tcgen05_decode_kernel")
@pytest.mark.parametrize("M,N,K", [(5, 4096, 4096), (8, 4096, 4096), (32, 4096, 11008), (24, 4096, 4096),
                                   (17, 1000, 2048), (32, 512, 28672), (64, 7000, 1024)])
def test_decode_unit_split_matches_row_split(M, N, K):
    """Decode-sized M on a narrow layer: with scratch memory the (tile, stage) units are dealt out to the SMs and pieces
    of a tile are summed with integer atomics; without it the weight rows are dealt out.  Same bits, also over repeated
    launches (the kernel leaves counters and sums at zero) and against the kernel that puts the tokens on the MMA rows."""
    g = torch.Generator().manual_seed(M + K)
    a, w = _rand_packed(M, K, 11), _rand_packed(N, K, 12)
    sx = (torch.rand(M, generator=g) * 0.5 + 0.05).half()
    sw = (torch.rand(N, generator=g) * 0.015 + 0.005).half()
    bias = (torch.randn(N, generator=g) * 0.5).half()
    assert _lib.lib.qr_linear_workspace_bytes(M, N, K) > 0
    ad, wd, sxd, swd, bd = a.to(DEV), w.to(DEV), sx.to(DEV), sw.to(DEV), bias.to(DEV)
    ref = O.sym_dequant_fp32(O.matmul_i4(a, w), sx, sw).half() + bias
    one = qb.linear_i4(ad, sxd, wd, swd, bd, use_workspace=False)
    for _ in range(3):
        assert torch.equal(qb.linear_i4(ad, sxd, wd, swd, bd), one)
    assert torch.equal(one.cpu(), ref)
    _lib.set_tuning("gemm_decode", 0)
    _lib.set_tuning("gemv_max_m", 0)
    try:
        assert _lib.lib.qr_linear_workspace_bytes(M, N, K) == 0
        assert torch.equal(qb.linear_i4(ad, sxd, wd, swd, bd), one)
    finally:
        _lib.set_tuning("gemm_decode", 1)
        _lib.set_tuning("gemv_max_m", 0)
    assert _lib.kernel_status() == 0


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (2, 1000, 2048), (3, 12288, 4096), (5, 4096, 11008), (8, 22016, 4096),
                                   (7, 33, 64), (8, 8192, 28672), (1, 1, 64)])
def test_weight_streaming_kernel_for_a_few_rows(M, N, K):
    """M <= 8 on the CUDA-core kernel (by default it serves only the quantiser-fused call; gemv_max_m = 8 sends all of
    these shapes to it): one pass over the packed weights with dp4a; exact accumulators and the same dequantisation arithmetic as
    the tensor-core kernels."""
    _lib.set_tuning("gemv_max_m", 8)
    try:
        _weight_streaming_case(M, N, K)
    finally:
        _lib.set_tuning("gemv_max_m", 0)


def _weight_streaming_case(M, N, K):
    g = torch.Generator().manual_seed(M * 7 + N)
    a, w = _rand_packed(M, K, 61), _rand_packed(N, K, 62)
    sx = (torch.rand(M, generator=g) * 0.5 + 0.05).half()
    sw = (torch.rand(N, generator=g) * 0.015 + 0.005).half()
    bias = (torch.randn(N, generator=g) * 0.5).half()
    acc = O.matmul_i4(a, w)
    ad, wd = a.to(DEV), w.to(DEV)
    assert torch.equal(qb.matmul(ad, wd).cpu(), acc)
    out = qb.linear_i4(ad, sx.to(DEV), wd, sw.to(DEV), bias.to(DEV))
    assert torch.equal(out.cpu(), O.sym_dequant_fp32(acc, sx, sw).half() + bias)
    out2 = qb.linear_i4(ad, sx.to(DEV), wd, sw.to(DEV))
    assert torch.equal(out2.cpu(), O.sym_dequant_fp32(acc, sx, sw).half())
    assert _lib.kernel_status() == 0


@pytest.mark.usefixtures("tcgen05_decode_kernel")
def test_workspace_argument_errors():
    a, w = _rand_packed(16, 4096, 1).to(DEV), _rand_packed(4096, 4096, 2).to(DEV)
    sx, sw = torch.ones(16, device=DEV).half(), torch.ones(4096, device=DEV).half()
    out = torch.empty(16, 4096, device=DEV, dtype=torch.float16)
    need = _lib.lib.qr_linear_workspace_bytes(16, 4096, 4096)
    small = torch.zeros(256, dtype=torch.uint8, device=DEV)
    rc = _lib.lib.qr_linear_i4_f16_ws(a.data_ptr(), sx.data_ptr(), w.data_ptr(), sw.data_ptr(), None, 16, 4096, 4096,
                                      out.data_ptr(), 4096, small.data_ptr(), small.numel(), None)
    assert rc == -1 and "workspace" in _lib.last_error() and need > 256
    assert _lib.lib.qr_linear_workspace_bytes(2048, 4096, 4096) == 0     # prefill shapes need no scratch
    assert _lib.lib.qr_linear_workspace_bytes(16, 12288, 4096) == 0      # nor do wide layers at decode sizes
    _lib.set_tuning("gemv_mma_max_m", 32)                                 # the default: up to 32 rows without scratch
    assert _lib.lib.qr_linear_workspace_bytes(2, 4096, 4096) == 0
    assert _lib.lib.qr_linear_workspace_bytes(32, 4096, 4096) == 0
    assert _lib.lib.qr_linear_workspace_bytes(33, 4096, 4096) == 0       # a small layer: two passes of that kernel
    assert _lib.lib.qr_linear_workspace_bytes(33, 4096, 8192) > 0
    _lib.set_tuning("gemm_splitk", 1)                                     # the default: scratch only for long rows
    assert _lib.lib.qr_linear_workspace_bytes(33, 4096, 8192) == 0
    assert _lib.lib.qr_linear_workspace_bytes(33, 4096, 11008) > 0
    _lib.set_tuning("gemm_splitk", 2)
    assert _lib.lib.qr_linear_workspace_bytes(32, 4096, 28672) > 0       # rows too long for that kernel's shared memory


@pytest.mark.usefixtures("tcgen05_decode_kernel")
def test_one_workspace_serves_calls_of_different_shapes():
    """Decode calls of different shapes share the cached workspace; every call leaves its counters at zero and
    partial tiles never land in the counter region, whatever the order of the shapes (more tiles after fewer)."""
    shapes = [(8, 4096, 4096), (64, 512, 28672), (64, 12288, 4096), (300, 1000, 2048), (32, 1000, 2048),
              (8, 4096, 4096), (64, 22016, 4096), (16, 4096, 11008), (64, 12288, 4096)]
    cases = {}
    for (M, N, K) in set(shapes):
        a, w = _rand_packed(M, K, M).to(DEV), _rand_packed(N, K, N).to(DEV)
        sx = (torch.rand(M) * 0.5 + 0.05).half().to(DEV)
        sw = (torch.rand(N) * 0.015 + 0.005).half().to(DEV)
        cases[(M, N, K)] = (a, sx, w, sw, qb.linear_i4(a, sx, w, sw, use_workspace=False))
    for shape in shapes:
        a, sx, w, sw, want = cases[shape]
        assert torch.equal(qb.linear_i4(a, sx, w, sw), want), shape
    assert _lib.kernel_status() == 0


def test_linear_into_several_outputs_at_once():
    """qr_linear_i4_f16_outs: the epilogue stores every block to each destination (here three column blocks of
    local matrices standing in for the ranks of a column split); bits equal the single-output call."""
    M, N, K = 520, 1000, 1024
    a, w = _rand_packed(M, K, 31).to(DEV), _rand_packed(N, K, 32).to(DEV)
    sx = (torch.rand(M) * 0.5 + 0.05).half().to(DEV)
    sw = (torch.rand(N) * 0.015 + 0.005).half().to(DEV)
    bias = torch.randn(N).half().to(DEV)
    want = qb.linear_i4(a, sx, w, sw, bias)
    pitch, off = 3 * N + 8, N + 8          # column block [off, off + N) of three wider matrices
    bufs = [torch.full((M, pitch), 3.0, dtype=torch.float16, device=DEV) for _ in range(3)]
    qb.linear_i4_outs(a, sx, w, sw, bias, [b.data_ptr() + 2 * off for b in bufs], pitch)
    torch.cuda.synchronize()
    for b in bufs:
        assert torch.equal(b[:, off:off + N], want)
        assert bool((b[:, :off] == 3.0).all()) and bool((b[:, off + N:] == 3.0).all())
    with pytest.raises(RuntimeError):      # decode-sized calls are not served by this entry point
        qb.linear_i4_outs(a[:8], sx[:8], w, sw, bias, [bufs[0].data_ptr(), bufs[1].data_ptr()], pitch)
    assert _lib.kernel_status() == 0


@pytest.mark.parametrize("M,I,K", [(300, 256, 512), (2048, 1024, 4096), (129, 11008, 256)])
def test_gate_up_gemm_with_swiglu_epilogue(M, I, K):
    """silu(gate_proj(x)) * up_proj(x) from one GEMM over interleaved weights: equal to the two Linear4bit calls
    followed by the fp16 elementwise product (bit for bit against torch's CUDA kernels, and against the CPU
    oracle up to the last fp16 bit of the exponential)."""
    a = _rand_packed(M, K, 41)
    wg, wu = _rand_packed(I, K, 42), _rand_packed(I, K, 43)
    sx = (torch.rand(M) * 0.05 + 0.005).half()
    sg = (torch.rand(I) * 0.015 + 0.005).half()
    su = (torch.rand(I) * 0.015 + 0.005).half()
    ad, sxd = a.to(DEV), sx.to(DEV)
    g = qb.linear_i4(ad, sxd, wg.to(DEV), sg.to(DEV))
    u = qb.linear_i4(ad, sxd, wu.to(DEV), su.to(DEV))
    w_gu = qb.interleave_gate_up(wg.to(DEV), wu.to(DEV))
    s_gu = qb.interleave_gate_up(sg.to(DEV), su.to(DEV))
    got = qb.linear_i4_swiglu(ad, sxd, w_gu, s_gu)
    unfused = torch.nn.functional.silu(g) * u
    assert got.shape == (M, I)
    assert torch.equal(got, unfused)
    want = O.swiglu_fp16(g.cpu(), u.cpu())
    diff = (got.cpu().float() - want.float()).abs()
    assert bool((diff <= want.float().abs() * 2.0 ** -9 + 1e-7).all())
    assert float((got.cpu() == want).float().mean()) > 0.999
    assert _lib.kernel_status() == 0


def test_swiglu_module_and_small_batches():
    from quarot_b200.nn.fused import SwiGLULinear4bit
    I, K = 512, 1024
    gate, up = qb.nn.Linear4bit(K, I).to(DEV), qb.nn.Linear4bit(K, I).to(DEV)
    for lin, seed in ((gate, 51), (up, 52)):
        lin.weight = _rand_packed(I, K, seed).to(DEV)
        lin.weight_scales = (torch.rand(I, 1) * 0.015 + 0.005).half().to(DEV)
    fused = SwiGLULinear4bit(gate, up)
    quant = qb.nn.Quantizer()
    for rows in (7, 128, 400):
        x = synth.activations(rows, K, seed=rows).to(DEV)
        xq = quant(x)
        want = torch.nn.functional.silu(gate(xq)) * up(xq)
        assert torch.equal(fused(xq), want), rows
    assert _lib.kernel_status() == 0


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (3, 1000, 2048), (8, 12288, 4096), (5, 512, 11008)])
@pytest.mark.parametrize("clip", [1.0, 0.9])
def test_quantizer_inside_the_weight_streaming_kernel(M, N, K, clip):
    """Quantizer + Linear4bit in one launch (M <= 8): the same bits as the two modules."""
    from quarot_b200.nn.fused import QuantLinear4bit
    x = synth.activations(M, K, seed=M + K).to(DEV)
    x[0, :7] = 0
    lin = qb.nn.Linear4bit(K, N, bias=True).to(DEV)
    lin.weight = _rand_packed(N, K, 71).to(DEV)
    lin.weight_scales = (torch.rand(N, 1) * 0.015 + 0.005).half().to(DEV)
    lin.bias = torch.randn(N).half().to(DEV)
    quant = qb.nn.Quantizer(clip)
    want = lin(quant(x))
    got = qb.quant_linear_i4(x, lin.weight, lin.weight_scales, lin.bias, clip)
    assert torch.equal(got, want)
    assert torch.equal(QuantLinear4bit(quant, lin)(x), want)
    xq = quant(x)
    ref = O.sym_dequant_fp32(O.matmul_i4(xq.quantized_x.cpu(), lin.weight.cpu()), xq.scales_x.cpu().view(-1),
                             lin.weight_scales.cpu()).half() + lin.bias.cpu()
    assert torch.equal(got.cpu(), ref)
    # more rows than the fused kernel takes: the module falls back to the two calls
    xb = synth.activations(9, K, seed=9).to(DEV)
    assert torch.equal(QuantLinear4bit(quant, lin)(xb), lin(quant(xb)))
    assert _lib.kernel_status() == 0



@pytest.mark.parametrize("halves", [0, 1, 2])
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (5, 12288, 4096), (8, 4096, 11008), (16, 22016, 4096), (13, 1000, 2048),
                                   (9, 33, 1024), (16, 7, 4096), (12, 300, 1088), (7, 4096, 64), (16, 130, 320),
                                   (11, 5000, 1152), (16, 17, 192), (2, 64, 20480),
                                   (32, 4096, 4096), (24, 1000, 11008), (32, 33, 1024), (17, 300, 1088), (16, 520, 8192),
                                   (8, 1000, 8192), (32, 260, 8192), (3, 77, 16384), (29, 2500, 4096)])
def test_weight_streaming_kernel_with_warp_level_mmas(M, N, K, halves):
    """1 .. 32 token rows: weights straight from global memory into the A fragments of mma.sync.m16n8k32.s8, K split
    over the warps of a CTA.  Exact int32 accumulators, the epilogue arithmetic of the other kernels, ragged N and K,
    an output pitch that is not a multiple of anything, repeated launches, with and without programmatic dependent
    launch; four and eight pieces per row in flight (K = 8192, 16384 take eight); two CTAs of eight warps per SM, one
    of sixteen (forced, and where the token rows leave no choice: 24 rows of K = 11008 run with a single reduction
    area per half)."""
    g = torch.Generator().manual_seed(M * 41 + N)
    a, w = _rand_packed(M, K, 91), _rand_packed(N, K, 92)
    sx = (torch.rand(M, generator=g) * 0.5 + 0.05).half()
    sw = (torch.rand(N, generator=g) * 0.015 + 0.005).half()
    bias = (torch.randn(N, generator=g) * 0.5).half()
    acc = O.matmul_i4(a, w)
    ref = O.sym_dequant_fp32(acc, sx, sw).half()
    ad, wd = a.to(DEV), w.to(DEV)
    _lib.set_tuning("gemv_max_m", 0)
    _lib.set_tuning("gemv_mma_halves", halves)
    try:
        for pdl in (0, 1):
            _lib.set_tuning("pdl", pdl)
            assert torch.equal(qb.matmul(ad, wd).cpu(), acc)
            out = qb.linear_i4(ad, sx.to(DEV), wd, sw.to(DEV), bias.to(DEV))
            assert torch.equal(out.cpu(), ref + bias)
            wide = torch.full((M, N + 3), 7.0, dtype=torch.float16, device=DEV)
            for _ in range(2):
                qb.linear_i4(ad, sx.to(DEV), wd, sw.to(DEV), out=wide[:, :N])
                assert torch.equal(wide[:, :N].cpu(), ref)
            assert bool((wide[:, N:] == 7.0).all())
        # the tcgen05 decode kernel gives the same bits
        _lib.set_tuning("gemv_mma_max_m", 0)
        assert torch.equal(qb.linear_i4(ad, sx.to(DEV), wd, sw.to(DEV)).cpu(), ref)
    finally:
        _lib.set_tuning("gemv_max_m", 0)
        _lib.set_tuning("gemv_mma_max_m", 32)
        _lib.set_tuning("gemv_mma_halves", 0)
        _lib.set_tuning("pdl", 2)
    assert _lib.kernel_status() == 0


@pytest.mark.usefixtures("tcgen05_decode_kernel")
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (3, 12288, 4096), (5, 4096, 11008), (8, 22016, 4096), (16, 4096, 4096),
                                   (13, 1000, 2048), (16, 8192, 28672), (9, 33, 1024), (16, 7, 4096), (12, 300, 1088), (32, 4096, 4096), (64, 22016, 4096), (40, 4096, 11008), (33, 1000, 256), (64, 130, 320),
                                   (16, 20000, 1024)])
def test_weight_streaming_tensor_core_kernel(M, N, K):
    """Decode-sized M on the tensor cores: (tile, stage) units dealt out evenly to the SMs, pieces of a tile summed in
    scratch memory with integer atomics.  gemv_max_m = 0 routes the shapes the CUDA-core kernel would otherwise take
    through it as well.  Exact accumulators, the epilogue arithmetic of the other kernels; the same bits with and
    without scratch memory, with programmatic dependent launch switched on, and over repeated launches (the kernel
    leaves its scratch at zero)."""
    g = torch.Generator().manual_seed(M * 31 + N)
    a, w = _rand_packed(M, K, 71), _rand_packed(N, K, 72)
    sx = (torch.rand(M, generator=g) * 0.5 + 0.05).half()
    sw = (torch.rand(N, generator=g) * 0.015 + 0.005).half()
    bias = (torch.randn(N, generator=g) * 0.5).half()
    acc = O.matmul_i4(a, w)
    ad, wd = a.to(DEV), w.to(DEV)
    _lib.set_tuning("gemv_max_m", 0)
    try:
        for pdl in (0, 1):
            _lib.set_tuning("pdl", pdl)
            assert torch.equal(qb.matmul(ad, wd).cpu(), acc)
            out = qb.linear_i4(ad, sx.to(DEV), wd, sw.to(DEV), bias.to(DEV))
            assert torch.equal(out.cpu(), O.sym_dequant_fp32(acc, sx, sw).half() + bias)
            for _ in range(2):
                out2 = qb.linear_i4(ad, sx.to(DEV), wd, sw.to(DEV))
                assert torch.equal(out2.cpu(), O.sym_dequant_fp32(acc, sx, sw).half())
            out3 = qb.linear_i4(ad, sx.to(DEV), wd, sw.to(DEV), use_workspace=False)
            assert torch.equal(out3.cpu(), O.sym_dequant_fp32(acc, sx, sw).half())
    finally:
        _lib.set_tuning("gemv_max_m", 0)
        _lib.set_tuning("pdl", 2)
    assert _lib.kernel_status() == 0


@pytest.mark.parametrize("M,N,K", [(64, 4096, 4096), (40, 1000, 2048), (33, 130, 320), (48, 260, 11008), (64, 7, 64)])
def test_two_passes_of_the_weight_streaming_kernel(M, N, K):
    """33 .. 64 token rows of a small layer run as two launches of the mma.sync kernel (32 rows, then the rest): exact
    accumulators, the epilogue of the other kernels, an output pitch of its own; the same bits with the knob off
    (the tcgen05 decode kernel)."""
    g = torch.Generator().manual_seed(M * 7 + N)
    a, w = _rand_packed(M, K, 11), _rand_packed(N, K, 12)
    sx = (torch.rand(M, generator=g) * 0.5 + 0.05).half()
    sw = (torch.rand(N, generator=g) * 0.015 + 0.005).half()
    bias = (torch.randn(N, generator=g) * 0.5).half()
    acc = O.matmul_i4(a, w)
    ref = O.sym_dequant_fp32(acc, sx, sw).half()
    ad, wd = a.to(DEV), w.to(DEV)
    assert _lib.lib.qr_linear_workspace_bytes(M, N, K) == 0
    try:
        for knob in (1, 0):
            _lib.set_tuning("gemv_mma_two_pass", knob)
            assert torch.equal(qb.matmul(ad, wd).cpu(), acc)
            assert torch.equal(qb.linear_i4(ad, sx.to(DEV), wd, sw.to(DEV), bias.to(DEV)).cpu(), ref + bias)
            wide = torch.full((M, N + 5), 7.0, dtype=torch.float16, device=DEV)
            qb.linear_i4(ad, sx.to(DEV), wd, sw.to(DEV), out=wide[:, :N])
            assert torch.equal(wide[:, :N].cpu(), ref) and bool((wide[:, N:] == 7.0).all())
    finally:
        _lib.set_tuning("gemv_mma_two_pass", 1)
    assert _lib.kernel_status() == 0
