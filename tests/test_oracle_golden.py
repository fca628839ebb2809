"""The CPU oracle against fixtures produced by the upstream torch functions."""
import numpy as np
import torch

from oracle import quarot_oracle as O


def _sizes(g):
    return sorted(int(k[1:-2]) for k in g.files if k.endswith("_k"))


def test_tables_are_hadamard_and_pinned():
    import hashlib
    from quarot_b200.functional import _had_tables as T
    d = hashlib.sha256()
    for k in (12, 20, 28, 36, 40, 52, 60, 108, 140, 156, 172):
        d.update(T.PACKED[k].encode())
        h = O._tables()[k]
        assert torch.equal(h @ h.T, k * torch.eye(k))
    assert d.hexdigest() == T.SHA256


def test_get_hadK_dispatch(golden):
    g = golden["hadamard"]
    for n in _sizes(g):
        _, k = O.get_hadK(n)
        assert k == int(g["n%d_k" % n]), n
    assert O.get_hadK(4096)[1] == 1 and O.get_hadK(11008)[1] == 172 and O.get_hadK(28672)[1] == 28
    assert O.get_hadK(13824)[1] == 108 and O.get_hadK(40)[1] == 40 and O.get_hadK(32)[1] == 1


def test_hadamard_bit_exact_vs_upstream(golden):
    g = golden["hadamard"]
    for n in _sizes(g):
        x = torch.from_numpy(g["n%d_x" % n])
        assert np.array_equal(O.hadamard(x.float()).numpy(), g["n%d_y32" % n]), n
        assert np.array_equal(O.hadamard(x).numpy(), g["n%d_y16" % n]), n
        if "n%d_yt32" % n in g.files:
            assert np.array_equal(O.hadamard(x.float(), transpose=True).numpy(), g["n%d_yt32" % n]), n


def test_hadamard_is_kron_operator():
    # y = x (hadK (x) H)^T / sqrt(n): explicit Kronecker matrix for a non-symmetric table
    n, k = 96, 12
    hk, kk = O.get_hadK(n)
    assert kk == k and not torch.equal(hk, hk.T)
    h = torch.tensor([[1.0]])
    for _ in range(3):
        h = torch.cat((torch.cat((h, h), 1), torch.cat((h, -h), 1)), 0)
    full = torch.kron(hk, h)
    x = torch.randn(5, n, dtype=torch.float64)
    ref = x @ full.double().T / np.sqrt(n)
    assert torch.allclose(O.hadamard(x), ref, atol=1e-12)
    # round trip with the transpose
    assert torch.allclose(O.hadamard(O.hadamard(x), transpose=True), x, atol=1e-12)


def test_quantizer_bit_exact_vs_upstream(golden):
    g = golden["quantizer"]
    tags = sorted(k[:-2] for k in g.files if k.endswith("_x"))
    assert len(tags) == 10
    for t in tags:
        x = torch.from_numpy(g[t + "_x"])
        clip = int(t.split("clip")[1]) / 100
        s = O.quantizer_scales(x, clip)
        assert np.array_equal(s.numpy().view(np.uint16), g[t + "_s"].reshape(-1).view(np.uint16)), t
        q = O.sym_quant_codes(x, s)
        assert np.array_equal(q.numpy(), g[t + "_q"]), t
        if t + "_p" in g.files:
            p = O.pack_i4(q)
            assert np.array_equal(p.numpy(), g[t + "_p"]), t
            assert np.array_equal(O.unpack_i4(p).numpy(), g[t + "_u"]), t


def test_pack_odd_width_and_roundtrip():
    q = torch.randint(-8, 8, (7, 33), dtype=torch.int8)
    p = O.pack_i4(q)
    assert p.shape == (7, 17)
    u = O.unpack_i4(p)
    assert torch.equal(u[:, :33], q.to(torch.int32)) and torch.all(u[:, 33] == 0)


def test_zero_row_defined_as_zero_codes():
    x = torch.zeros(2, 64, dtype=torch.float16)
    s = O.quantizer_scales(x)
    assert torch.all(s == 0)
    assert torch.all(O.sym_quant_codes(x, s) == 0)


def test_matmul_bit_exact_vs_upstream(golden):
    g = golden["matmul"]
    for t in ("s", "m", "l"):
        c = O.matmul_i4(torch.from_numpy(g[t + "_a"]), torch.from_numpy(g[t + "_b"]))
        assert c.dtype == torch.int32 and np.array_equal(c.numpy(), g[t + "_c"]), t


def test_dequant_forms_agree():
    acc = torch.randint(-3000, 3000, (9, 13), dtype=torch.int32)
    sr = torch.rand(9).half() * 0.1 + 0.01
    sc = torch.rand(13).half() * 0.02 + 0.005
    a = O.sym_dequant_fp16(acc, sr, sc).float()
    b = O.sym_dequant_fp32(acc, sr, sc)
    assert torch.allclose(a, b, rtol=4e-3, atol=1e-4)


def test_linear_forward_shapes():
    x = torch.randn(6, 128).half()
    w = O.pack_i4(torch.randint(-8, 8, (24, 128), dtype=torch.int8))
    ws = torch.rand(24, 1).half() * 0.01 + 0.005
    r = O.linear4bit_forward(x, w, ws, hadamard_dim=128)
    assert r["out"].shape == (6, 24) and r["packed"].shape == (6, 64) and r["acc"].dtype == torch.int32


def test_rmsnorm_bit_exact_vs_upstream(golden):
    g = golden["rmsnorm"]
    for tag in ("a", "b", "c", "d"):
        x = torch.from_numpy(g[tag + "_x"])
        y = O.rmsnorm_fp16(x, x.shape[-1], 1e-5)
        assert torch.equal(y.view(torch.int16), torch.from_numpy(g[tag + "_y"]).view(torch.int16)), tag


def test_swiglu_is_the_fp16_product_of_torch():
    gen = torch.Generator().manual_seed(3)
    g = (torch.randn(64, 256, generator=gen) * 3).half()
    u = (torch.randn(64, 256, generator=gen) * 3).half()
    assert torch.equal(O.swiglu_fp16(g, u), torch.nn.functional.silu(g) * u)



def test_kv_cache_quantisation_bit_exact_vs_upstream():
    """The 4-bit KV-cache format: the oracle's restatement of asym_quantize_and_pack_i4 / unpack_i4_and_asym_dequantize
    against outputs of the upstream helpers (tests/golden/make_golden_kv.py)."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "kv_cache.npz"))
    for name in ("gauss", "outlier", "tiny", "const", "ties"):
        x = torch.from_numpy(g[name + "_x"])
        q, scale, zero = O.kv_asym_quant_pack(x)
        assert np.array_equal(q.numpy(), g[name + "_q"]), name
        assert np.array_equal(scale.numpy().view(np.uint16), g[name + "_scale"].view(np.uint16)), name
        assert np.array_equal(zero.numpy().view(np.uint16), g[name + "_zero"].view(np.uint16)), name
        deq = O.kv_unpack_dequant(q, scale, zero)
        assert np.array_equal(deq.numpy().view(np.uint16), g[name + "_deq"].view(np.uint16)), name
