"""CUDA kernels of family (a) against the CPU oracle and the upstream-generated fixtures.
Every call goes through the C-ABI library (ctypes) -- see quarot_b200/_ops.py."""
import numpy as np
import pytest
import torch

import quarot_b200 as qb
from quarot_b200 import _lib, synth
from quarot_b200.functional import hadamard as FH
from oracle import quarot_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.int16)


@pytest.fixture(params=["auto", "tcgen05"], autouse=True)
def kronecker_kernel_choice(request):
    """Shapes n = 64 K go to the per-row kernel up to 128 rows and to the persistent tcgen05 kernel above; the small,
    ragged row counts of this module run once with that rule and once with the tcgen05 kernel forced."""
    _lib.set_tuning("hadq_tc", 2 if request.param == "tcgen05" else 1)
    yield
    _lib.set_tuning("hadq_tc", 1)


def test_sym_quant_matches_upstream_fixtures(golden):
    g = golden["quantizer"]
    for t in sorted(k[:-2] for k in g.files if k.endswith("_x")):
        x = torch.from_numpy(g[t + "_x"]).to(DEV)
        s = torch.from_numpy(g[t + "_s"]).to(DEV)
        q = qb.sym_quant(x, s).cpu()
        want = O.pack_i4(torch.from_numpy(g[t + "_q"]))
        assert q.shape == want.shape and torch.equal(q, want), t


def test_sym_quant_all_fp16_values_times_many_scales():
    # every finite fp16 value as x, 192 assorted scales: exercises the division + double rounding exhaustively
    allv = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16).view(torch.float16)
    allv = allv[torch.isfinite(allv)]
    allv = allv[: (allv.numel() // 8) * 8]
    g = torch.Generator().manual_seed(5)
    scales = torch.cat((torch.rand(96, generator=g) * 4 + 1e-3, torch.rand(64, generator=g) * 1e-3 + 1e-6,
                        torch.tensor([1.0, 0.5, 1 / 7, 3.0, 6e-8, 1e-4, 2.0, 65504.0 / 7]),
                        torch.rand(24, generator=g) * 9000 + 10)).to(torch.float16)
    x = allv.unsqueeze(0).repeat(scales.numel(), 1).contiguous()
    q = qb.sym_quant(x.to(DEV), scales.to(DEV)).cpu()
    want = O.pack_i4(O.sym_quant_codes(x, scales))
    bad = (q != want).sum().item()
    assert bad == 0, "%d of %d bytes differ" % (bad, want.numel())


def test_sym_quant_zero_scale_and_shapes():
    x = torch.randn(2, 3, 64, device=DEV).half()
    s = torch.zeros(2, 3, device=DEV).half()
    q = qb.sym_quant(x, s)
    # x / 0 = +-inf saturates to 7 / -8, exactly like torch
    assert q.shape == (2, 3, 32)
    assert torch.equal(q.cpu().view(6, 32), O.pack_i4(O.sym_quant_codes(x.cpu().view(6, 64), s.cpu().view(6))))
    z = qb.sym_quant(torch.zeros_like(x), s)
    assert int(z.max()) == 0
    with pytest.raises(RuntimeError):
        qb.sym_quant(x, torch.zeros(5, device=DEV).half())
    with pytest.raises(RuntimeError):
        qb.sym_quant(x.transpose(0, 1), s.view(-1))


def test_sym_dequant_matches_upstream_arithmetic():
    g = torch.Generator().manual_seed(11)
    for rows, cols in ((1, 4), (7, 13), (33, 128), (130, 272)):
        acc = torch.randint(-70000, 70000, (rows, cols), generator=g, dtype=torch.int32)
        sr = (torch.rand(rows, generator=g) * 0.5 + 0.01).half()
        sc = (torch.rand(cols, generator=g) * 0.02 + 0.005).half()
        out = qb.sym_dequant(acc.to(DEV), sr.to(DEV), sc.to(DEV)).cpu()
        want = O.sym_dequant_fp16(acc, sr, sc)
        assert torch.equal(_bits(out), _bits(want)), (rows, cols)
    with pytest.raises(RuntimeError):
        qb.sym_dequant(acc.to(DEV), sr.to(DEV), sc.to(DEV), bits=16)


def _had_close(y, ref32):
    """fp16 kernel output vs the fp32 operator: 1e-3 of the row's largest magnitude, plus half an fp16 ulp."""
    ref = ref32.double()
    err = (y.double() - ref).abs()
    tol = 1e-3 * ref.abs().amax(dim=-1, keepdim=True) + ref.abs() * 2.0 ** -11 + 1e-7
    return bool((err <= tol).all()), float((err / (ref.abs().amax(dim=-1, keepdim=True) + 1e-30)).max())


def test_hadamard_f16_matches_upstream_fixtures(golden):
    g = golden["hadamard"]
    for key in sorted(k for k in g.files if k.endswith("_k")):
        n = int(key[1:-2])
        k = int(g[key])
        x = torch.from_numpy(g["n%d_x" % n]).to(DEV)
        table = FH.device_table(k, DEV) if k > 1 else None
        y = qb.hadamard(x, table, k).cpu()
        ok, worst = _had_close(y, torch.from_numpy(g["n%d_y32" % n]))
        assert ok, (n, worst)


def test_hadamard_f32_and_functional_entry(golden):
    g = golden["hadamard"]
    for n in (64, 96, 112, 344, 1024, 11008):
        k = int(g["n%d_k" % n])
        x = torch.from_numpy(g["n%d_x" % n]).float().to(DEV)
        hk, kk = FH.get_hadK(n)
        y = qb.functional.matmul_hadU_cuda(x, hk, kk).cpu()
        ref = torch.from_numpy(g["n%d_y32" % n])
        assert y.dtype == torch.float32 and kk == k
        assert torch.allclose(y, ref, rtol=1e-5, atol=1e-5 * float(ref.abs().max())), n
    # transposed table entry point works (upstream's raises)
    x = torch.from_numpy(g["n96_x"]).float().to(DEV)
    hk, kk = FH.get_hadK(96)
    yt = FH.matmul_hadUt_cuda(x, hk, kk).cpu()
    assert torch.allclose(yt, torch.from_numpy(g["n96_yt32"]), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("n,rows", [(32, 64), (64, 32), (128, 24), (512, 6), (1024, 5), (2048, 3), (4096, 17),
                                    (8192, 3), (11008, 9), (28672, 3), (13824, 2), (17920, 2), (19968, 2),
                                    (5120, 4), (160, 8), (344, 4), (36 * 64, 3), (52 * 128, 2), (60 * 64, 2),
                                    (12 * 256, 3), (20 * 64, 3)])
def test_hadamard_random_vs_oracle_all_families(n, rows):
    x = synth.activations(rows, n, seed=100 + n, outlier_channels=4, outlier_scale=30.0)
    k = O.get_hadK(n)[1]
    table = FH.device_table(k, DEV) if k > 1 else None
    y = qb.hadamard(x.to(DEV), table, k).cpu()
    ok, worst = _had_close(y, O.hadamard(x.float()))
    assert ok, (n, worst)
    # the A/B switch to the generic kernel gives the same answer within the same tolerance
    _lib.set_tuning("hadq_path", 1)
    try:
        y2 = qb.hadamard(x.to(DEV), table, k).cpu()
    finally:
        _lib.set_tuning("hadq_path", 0)
    ok2, worst2 = _had_close(y2, O.hadamard(x.float()))
    assert ok2, (n, worst2)


@pytest.mark.parametrize("n,K,rows", [(256, 0, 5), (4096, 0, 17), (11008, 0, 3), (22016 // 2, 0, 2), (96, 0, 3),
                                      (4096, 1, 17), (1024, 1, 4), (8192, 1, 2), (64, 1, 9), (256, 1, 5),
                                      (11008, 172, 9), (28672, 28, 3), (13824, 108, 2), (344, 172, 3),
                                      (112, 28, 4), (6912, 108, 5), (8960, 140, 3), (9984, 156, 7), (11008, 172, 32),
                                      (11008, 172, 1), (11008, 172, 40)])
@pytest.mark.parametrize("clip", [1.0, 0.9])
def test_fused_hadamard_quant_bit_exact_given_own_hadamard(n, K, rows, clip):
    x = synth.activations(rows, n, seed=7 * n + K)
    table = FH.device_table(K, DEV) if K > 1 else None
    q, s, y = qb.hadamard_quant(x.to(DEV), table, K, clip, return_y=True)
    q, s, y = q.cpu(), s.cpu(), y.cpu()
    if K == 0:
        assert torch.equal(_bits(y), _bits(x))
    else:
        ok, worst = _had_close(y, O.hadamard(x.float()))
        assert ok, worst
    s_ref = O.quantizer_scales(y, clip)
    assert torch.equal(_bits(s), _bits(s_ref))
    want = O.pack_i4(O.sym_quant_codes(y, s_ref))
    assert torch.equal(q, want)
    # without the side output the codes are the same
    q2, s2, none = qb.hadamard_quant(x.to(DEV), table, K, clip)
    assert none is None and torch.equal(q2.cpu(), q) and torch.equal(_bits(s2), _bits(s))


@pytest.mark.parametrize("n,K,rows", [(11008, 172, 1), (11008, 172, 8), (11008, 172, 32), (6912, 108, 6), (8960, 140, 2),
                                      (9984, 156, 11)])
def test_few_rows_shared_by_a_cluster_give_the_bits_of_one_cta_per_row(n, K, rows):
    """Up to 32 rows of n = 64 K are transformed by clusters of four CTAs that share a row (each a quarter of the dense
    factor's output rows, the absmax exchanged through distributed shared memory): the same Hadamard output, scales
    and codes as with one CTA per row, also over repeated launches."""
    x = synth.activations(rows, n, seed=n + rows).to(DEV)
    x[0, :5] = 0
    table = FH.device_table(K, DEV)
    try:
        _lib.set_tuning("hadq_tc", 1)          # the reference form is the mma.sync kernel with one CTA per row
        _lib.set_tuning("hadq_split", 0)
        q0, s0, y0 = qb.hadamard_quant(x, table, K, 0.9, return_y=True)
        _lib.set_tuning("hadq_split", 1)
        for _ in range(2):
            q1, s1, y1 = qb.hadamard_quant(x, table, K, 0.9, return_y=True)
            assert torch.equal(_bits(y1), _bits(y0)) and torch.equal(_bits(s1), _bits(s0)) and torch.equal(q1, q0)
        q2, s2, _ = qb.hadamard_quant(x, table, K, 0.9)
        assert torch.equal(q2, q0) and torch.equal(_bits(s2), _bits(s0))
    finally:
        _lib.set_tuning("hadq_split", 1)
    assert _lib.kernel_status() == 0


def test_division_by_reciprocal_gives_ieee_codes_for_every_fp16_pair():
    """The quantisers multiply by RN(1/s) instead of dividing; the library checks all finite fp16 x against
    all finite non-zero fp16 s on the device and reports how many int4 codes differ from IEEE division."""
    import ctypes
    bad = ctypes.c_uint64(123)
    _lib.check(_lib.lib.qr_debug_division_check(ctypes.byref(bad)), "qr_debug_division_check")
    assert bad.value == 0


@pytest.mark.parametrize("n,K", [(4096, 0), (4096, 1), (11008, 0), (11008, 172), (28672, 28)])
@pytest.mark.parametrize("magnitude", [2.0 ** -22, 2.0 ** -15, 1.0, 3000.0])
def test_fused_quant_ties_and_tiny_scales(n, K, magnitude):
    """Rows built from half-integer multiples of a power of two hit round-half-even ties; tiny magnitudes push
    the scale into the subnormal fp16 range, where the code clamp matters; clip < 1 saturates."""
    g = torch.Generator().manual_seed(n + K)
    x = (torch.randint(-14, 15, (6, n), generator=g).float() * 0.5 * magnitude).half()
    table = FH.device_table(K, DEV) if K > 1 else None
    for clip in (1.0, 0.7):
        q, s, y = qb.hadamard_quant(x.to(DEV), table, K, clip, return_y=True)
        q, s, y = q.cpu(), s.cpu(), y.cpu()
        s_ref = O.quantizer_scales(y, clip)
        assert torch.equal(_bits(s), _bits(s_ref))
        assert torch.equal(q, O.pack_i4(O.sym_quant_codes(y, s_ref)))


def test_fused_quant_edge_rows():
    x = torch.zeros(4, 4096, dtype=torch.float16)
    x[1, 5] = 7.0            # scale exactly 1
    x[1, 6] = 2.5            # tie -> 2
    x[1, 7] = -3.5           # tie -> -4
    x[2] = 6e-8              # all fp16 subnormal
    x[3, 0], x[3, 1] = 65504.0, -65504.0
    q, s, _ = qb.hadamard_quant(x.to(DEV), None, 0, 1.0)
    q, s = q.cpu(), s.cpu()
    assert float(s[0]) == 0.0 and int(q[0].max()) == 0          # zero row: scale 0, zero codes
    assert float(s[2]) == 0.0 and int(q[2].min()) == 0x77       # scale underflows to 0: x / 0 = +inf -> 7
    s_ref = O.quantizer_scales(x)
    assert torch.equal(_bits(s), _bits(s_ref))
    want = O.pack_i4(O.sym_quant_codes(x, s_ref))
    assert torch.equal(q, want)
    u = O.unpack_i4(q)
    assert int(u[1, 6]) == 2 and int(u[1, 7]) == -4 and int(u[3, 0]) == 7 and int(u[3, 1]) == -7


def test_quantizer_module_shapes_and_parity():
    x = synth.activations(6 * 5, 512, seed=3).view(6, 5, 512)
    qz = qb.nn.Quantizer(0.95)
    out = qz(x.to(DEV))
    assert isinstance(out, qb.PackedQuantizedTensor)
    assert out.quantized_x.shape == (6, 5, 256) and out.scales_x.shape == (6, 1, 5)
    assert out.size() == out.quantized_x.size() and out.dtype == torch.uint8 and out.device.type == "cuda"
    s_ref = O.quantizer_scales(x, 0.95)
    assert torch.equal(_bits(out.scales_x.view(-1)), _bits(s_ref))
    assert torch.equal(out.quantized_x.cpu().view(30, 256), O.pack_i4(O.sym_quant_codes(x.view(30, 512), s_ref)))
    out2 = qz(x.view(30, 512).to(DEV))
    assert out2.scales_x.shape == (30, 1)


def test_online_hadamard_module_and_fusion_agree():
    for n in (4096, 11008):
        x = synth.activations(12, n, seed=n).to(DEV)
        had, had32 = qb.nn.OnlineHadamard(n).to(DEV), qb.nn.OnlineHadamard(n, force_fp32=True).to(DEV)
        y = had(x)
        assert y.dtype == torch.float16 and torch.equal(y, had32(x))
        ok, worst = _had_close(y.cpu(), O.hadamard(x.cpu().float()))
        assert ok, worst
        p1 = qb.nn.Quantizer()(y)
        p2 = qb.nn.HadamardQuantizer(n)(x)
        assert torch.equal(p1.quantized_x, p2.quantized_x) and torch.equal(p1.scales_x, p2.scales_x)
    # heads-axis use: a transposed (non-contiguous) view with a short last dim
    a = synth.activations(4 * 128, 32, seed=9).view(4, 128, 32).transpose(1, 2).to(DEV)  # [4, 32, 128] non-contig
    y = qb.nn.OnlineHadamard(128).to(DEV)(a)
    ok, worst = _had_close(y.cpu(), O.hadamard(a.cpu().float()))
    assert ok, worst


@pytest.mark.parametrize("n,rows", [(4096, 33), (8192, 5), (11008, 3), (64, 9), (5120, 4)])
@pytest.mark.parametrize("clip", [1.0, 0.9])
def test_rmsnorm_quant_fused(n, rows, clip):
    """RMSNorm + Quantizer in one pass: the normalised row within fp16 rounding of the fp32 operator (the order of
    the sum of squares and the rsqrt differ in the last bits), scales and codes bit-exact given that row."""
    x = synth.activations(rows, n, seed=3 * n + rows)
    x[0] = 0                                    # zero row: rsqrt(eps) * 0 = 0, scale 0, zero codes
    q, s, y = qb.rmsnorm_quant(x.to(DEV), n, 1e-5, clip, return_y=True)
    q, s, y = q.cpu(), s.cpu(), y.cpu()
    ref = O.rmsnorm_fp16(x, n, 1e-5)
    err = (y.double() - ref.double()).abs()
    assert bool((err <= ref.double().abs() * 2.0 ** -10 + 1e-7).all())
    assert float((y == ref).float().mean()) > 0.99
    s_ref = O.quantizer_scales(y, clip)
    assert torch.equal(_bits(s), _bits(s_ref))
    assert torch.equal(q, O.pack_i4(O.sym_quant_codes(y, s_ref)))
    # module form, and equality with the unfused modules on the device (same kernels for the quantiser)
    from quarot_b200.nn.fused import RMSNormQuantizer
    fused = RMSNormQuantizer(n, 1e-5, clip)(x.to(DEV))
    q2, s2, _ = qb.rmsnorm_quant(x.to(DEV), n, 1e-5, clip)
    assert torch.equal(fused.quantized_x.cpu(), q) and torch.equal(q2.cpu(), q)
    assert fused.scales_x.shape == (rows, 1)



@pytest.mark.parametrize("heads,head_dim", [(32, 128), (8, 128), (16, 64), (64, 64), (64, 128), (2, 128)])
def test_heads_axis_hadamard_on_the_transposed_view(heads, head_dim):
    """OnlineHadamard(num_heads) on attn_output.transpose(-1, -2), as the attention block calls it in front of o_proj:
    transform over the heads axis without a transposed copy where the strided kernel serves the shape (up to 4096
    values per token), through a contiguous copy otherwise; the result has the strides of the input view."""
    g = torch.Generator().manual_seed(heads * head_dim)
    attn = (torch.randn(2, 37, heads, head_dim, generator=g) * 3).half().to(DEV)
    view = attn.transpose(-1, -2)                      # [2, 37, head_dim, heads], last axis strided
    y = qb.nn.OnlineHadamard(heads).to(DEV)(view)
    assert y.shape == view.shape and y.dtype == torch.float16
    ref = O.hadamard(view.cpu().float().contiguous())
    ok, worst = _had_close(y.cpu().contiguous(), ref)
    assert ok, worst
    back = y.transpose(-1, -2).reshape(2, 37, heads * head_dim)
    assert back.shape == (2, 37, heads * head_dim)
    if 256 <= heads * head_dim <= 4096 and head_dim >= 32:
        assert y.transpose(-1, -2).is_contiguous()      # no copy on the way back either
        # the C entry point in place (y may alias x): the same bits; the other heads-axis kernel: the same values within
        # the rounding of the transform
        inplace = attn.clone()
        _lib.check(_lib.lib.qr_hadamard_heads_f16(inplace.data_ptr(), inplace.data_ptr(), 2 * 37, heads, head_dim, None), "heads")
        assert torch.equal(inplace, y.transpose(-1, -2))
        _lib.set_tuning("hadq_heads", 0)
        try:
            other = qb.nn.OnlineHadamard(heads).to(DEV)(view)
        finally:
            _lib.set_tuning("hadq_heads", 1)
        ok, worst = _had_close(other.cpu().contiguous(), ref)
        assert ok, worst


@pytest.mark.parametrize("n,rows", [(256, 7), (512, 3), (1024, 50), (2048, 13), (4096, 29)])
def test_warp_per_row_walsh_kernel(n, rows):
    """The register-resident Walsh kernel (tensor-core stage on bits 0, 1, 3, 4, shuffles on bits 5..7) serves whole-row
    transforms when switched on: Hadamard within 1e-3 of the fp32 operator, scales and codes bit-exact given it."""
    x = synth.activations(rows, n, seed=n + rows).to(DEV)
    _lib.set_tuning("hadq_walsh", 1)
    try:
        q, s, y = qb.hadamard_quant(x, None, 1, 1.0, return_y=True)
        y2 = qb.hadamard(x, None, 1)
    finally:
        _lib.set_tuning("hadq_walsh", 0)
    ok, worst = _had_close(y.cpu(), O.hadamard(x.cpu().float()))
    assert ok, worst
    assert torch.equal(y, y2)
    s_ref = O.quantizer_scales(y.cpu())
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.cpu(), O.pack_i4(O.sym_quant_codes(y.cpu(), s_ref)))
