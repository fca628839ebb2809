"""Host-side logic that needs no GPU: packing helpers, table dispatch, module surface, C-ABI exports."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import quarot_b200
from quarot_b200 import _lib
from quarot_b200.functional import hadamard as FH
from quarot_b200.functional import quantization as FQ
from oracle import quarot_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cabi_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "quarot_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(qr_[a-z0-9_]+)\s*\(", header))
    assert declared and declared == set(_lib.SIGNATURES)
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert _lib.lib.qr_version() == 100
    assert _lib.last_error() == ""


def test_cabi_argument_errors_without_gpu():
    # argument validation happens before any CUDA call
    rc = _lib.lib.qr_matmul_i4_i32(None, None, 4, 4, 64, None, None)
    assert rc == -1 and "null" in _lib.last_error()
    rc = _lib.lib.qr_set_tuning(b"no_such_key", 1)
    assert rc == -1
    assert _lib.lib.qr_matmul_i4_i32(None, None, 0, 4, 64, None, None) == 0  # empty problem is a no-op
    assert _lib.lib.qr_sym_quant_i4(None, None, 0, 16, None, None) == 0
    assert _lib.lib.qr_hadamard_quant_i4(None, 0, 64, 64, None, 1, 1.0, None, None, None, None) == 0
    with pytest.raises(RuntimeError):
        _lib.check(_lib.lib.qr_hadamard_f16(None, None, 2, 48, None, 1, None), "hadamard")


def test_pack_unpack_match_golden(golden):
    g = golden["quantizer"]
    for t in sorted(k[:-2] for k in g.files if k.endswith("_p")):
        q = torch.from_numpy(g[t + "_q"])
        p = FQ.pack_i4(q)
        assert np.array_equal(p.numpy(), g[t + "_p"])
        assert np.array_equal(FQ.unpack_i4(p).numpy(), g[t + "_u"])
    with pytest.raises(AssertionError):
        FQ.pack_i4(torch.tensor([[9, 0]], dtype=torch.int8))
    with pytest.raises(AssertionError):
        FQ.pack_i4(torch.tensor([[1, 0]], dtype=torch.uint8))
    with pytest.raises(AssertionError):
        FQ.unpack_i4(torch.zeros(2, 2, dtype=torch.int8))


def test_fake_quant_formulas():
    x = torch.randn(4, 16)
    s = x.abs().amax(dim=-1, keepdim=True) / 7
    q, _ = FQ.sym_quant(x, s, torch.tensor(7))
    assert q.min() >= -8 and q.max() <= 7
    assert torch.allclose(FQ.sym_quant_dequant(x, s, torch.tensor(7)), q * s)
    lo, hi = FQ.get_minq_maxq(4, True)
    assert (int(lo), int(hi)) == (-8, 7)
    lo, hi = FQ.get_minq_maxq(4, False)
    assert (int(lo), int(hi)) == (0, 15)
    z = torch.full((4, 1), 8.0)
    y = FQ.asym_quant_dequant(x, s, z, torch.tensor(15))
    assert y.shape == x.shape


def test_tables_and_host_hadamard_match_golden(golden):
    g = golden["hadamard"]
    for key in (k for k in g.files if k.endswith("_k")):
        n = int(key[1:-2])
        hk, k = FH.get_hadK(n)
        assert k == int(g[key])
        if hk is not None:
            assert torch.equal(hk, O.get_hadK(n)[0])
        x = torch.from_numpy(g["n%d_x" % n])
        assert np.array_equal(FH.matmul_hadU(x.float()).numpy(), g["n%d_y32" % n]), n
    with pytest.raises(AssertionError):
        FH.get_hadK(100)     # 100 = 20 * 5
    with pytest.raises(AssertionError):
        FH.get_hadK(1000)    # 1000 = 40 * 25
    q = FH.random_hadamard_matrix(64, "cpu")
    assert q.dtype == torch.float64 and torch.allclose(q @ q.T, torch.eye(64, dtype=torch.float64), atol=1e-12)


def test_module_surface_and_state_dict_contract():
    lin = quarot_b200.nn.Linear4bit(64, 16, bias=True)
    sd = lin.state_dict()
    assert set(sd) == {"weight", "weight_scales", "bias"}
    assert sd["weight"].shape == (16, 32) and sd["weight"].dtype == torch.uint8
    assert sd["weight_scales"].shape == (16, 1) and sd["bias"].shape == (16,)
    assert int(sd["weight"].min()) >= 1 and int(sd["weight"].max()) <= 6
    had = quarot_b200.nn.OnlineHadamard(11008)
    assert had.rem_dim == 172 and had.had_rem_dim.dtype == torch.float16 and had.had_rem_dim.shape == (172, 172)
    assert quarot_b200.nn.OnlineHadamard(11008, force_fp32=True).had_rem_dim.dtype == torch.float32
    assert quarot_b200.nn.OnlineHadamard(4096).had_rem_dim is None
    seq = torch.nn.Sequential(quarot_b200.nn.OnlineHadamard(256), quarot_b200.nn.Quantizer(0.9),
                              quarot_b200.nn.Linear4bit(256, 8))
    keys_before = set(seq.state_dict())
    assert quarot_b200.nn.fuse_modules(seq) == 1
    assert isinstance(seq[0], quarot_b200.nn.HadamardQuantizer) and seq[0].input_clip_ratio == 0.9
    assert set(seq.state_dict()) == keys_before
    rms = quarot_b200.nn.RMSNorm(8)
    x = torch.randn(3, 8).half()
    ref = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)).half()
    assert torch.equal(rms(x), ref)
    with pytest.raises(NotImplementedError):
        quarot_b200.transformers.MultiLayerPagedKVCache4Bit(1, 16, 64, "cpu", 1, 2, 128, disable_quant=True)
    cache = quarot_b200.transformers.MultiLayerPagedKVCache4Bit(2, 16, 100, "cpu", 3, 4, 128)
    assert cache.pages.shape == (14, 3, 2, 4, 16, 64) and cache.pages.dtype == torch.uint8
    assert cache.scales.shape == (14, 3, 2, 4, 16, 2) and cache.get_seq_length() == 0 and cache.to_legacy_cache() is cache
    cache.length = 33
    specs = cache.get_cache_specs_for_flash_infer(None)
    assert specs["kv_indptr"].tolist() == [0, 3, 6] and specs["kv_indices"].tolist() == [0, 2, 4, 1, 3, 5]
    assert specs["last_page_offset"].tolist() == [1, 1]


def test_ops_reject_cpu_tensors():
    a = torch.zeros(2, 32, dtype=torch.uint8)
    with pytest.raises(RuntimeError):
        quarot_b200.matmul(a, a)
    with pytest.raises(AssertionError):
        quarot_b200.matmul(torch.zeros(2, 24, dtype=torch.uint8), a)
    with pytest.raises(AssertionError):
        quarot_b200.sym_quant(torch.zeros(2, 8), torch.zeros(2))
    with pytest.raises(AssertionError):
        quarot_b200.sym_dequant(torch.zeros(2, 8), torch.zeros(2).half(), torch.zeros(8).half())
    with pytest.raises(RuntimeError):
        quarot_b200.sym_quant(torch.zeros(2, 8).half(), torch.zeros(2).half())


def test_install_as_quarot_alias():
    quarot_b200.install_as_quarot()
    import quarot
    from quarot.nn import Linear4bit, Quantizer, OnlineHadamard  # noqa: F401
    import quarot.functional.hadamard as h
    assert quarot is quarot_b200 and h.get_hadK(28672)[1] == 28
    assert quarot.functional.quantization.get_minq_maxq is FQ.get_minq_maxq


def test_synth_distributions():
    from quarot_b200 import synth
    x = synth.activations(64, 512, seed=7)
    assert x.dtype == torch.float16 and x.shape == (64, 512)
    big = (x.float().abs().mean(0) > 10).sum()
    assert int(big) == 8
    w, s = synth.weights(32, 128, seed=3)
    assert w.shape == (32, 64) and s.shape == (32, 1) and s.dtype == torch.float16
    assert float(s.min()) >= 0.005 - 1e-4 and float(s.max()) <= 0.02 + 1e-4
    u = FQ.unpack_i4(w)
    assert int(u.min()) == -8 and int(u.max()) == 7
    assert torch.equal(synth.activations(64, 512, seed=7), x)


def test_gate_up_interleave_layout():
    """Operand layout of the SwiGLU GEMM: groups of 128 gate rows alternate with the same 128 up rows."""
    I = 384
    gate = torch.arange(I).view(I, 1).repeat(1, 3)
    up = gate + 10000
    both = quarot_b200.interleave_gate_up(gate, up)
    assert both.shape == (2 * I, 3)
    for t in range(I // 128):
        assert torch.equal(both[256 * t:256 * t + 128], gate[128 * t:128 * (t + 1)])
        assert torch.equal(both[256 * t + 128:256 * t + 256], up[128 * t:128 * (t + 1)])
    with pytest.raises(ValueError):
        quarot_b200.interleave_gate_up(gate[:100], up[:100])


def test_new_entry_points_validate_arguments_without_gpu():
    lib = _lib.lib
    assert lib.qr_rmsnorm_quant_i4(None, 0, 4096, 4096, 4096, 1e-5, 1.0, None, None, None, None) == 0
    assert lib.qr_rmsnorm_quant_i4(None, 4, 4096, 4096, 4096, 1e-5, 1.0, None, None, None, None) == -1
    assert lib.qr_linear_i4_f16_outs(None, None, None, None, None, 256, 256, 256, None, 1, 256, None) == -1
    assert "outputs" in _lib.last_error()



def test_bench_tables_and_cpu_generators_match_synth():
    """bench.py repeats the layer tables and the CPU generators of quarot_b200/synth.py so that its reference arm
    runs without importing the product package; they must stay identical."""
    import importlib.util
    from quarot_b200 import synth
    spec = importlib.util.spec_from_file_location("_bench_for_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    for name, table in bench.LAYERS.items():
        assert table == getattr(synth, name), name
    assert torch.equal(bench._cpu_activations(O, 5, 256, 1234), synth.activations(5, 256, seed=1234))
    w, s = bench._cpu_weights(O, 7, 64, 4321)
    w2, s2 = synth.weights(7, 64, seed=4321)
    assert torch.equal(w, w2) and torch.equal(s, s2)
    src = open(os.path.join(ROOT, "bench.py")).read()
    ref_arm = src[src.index("def cpu_reference_run"):src.index("# ------------------------------------------------------------------ device arm")]
    assert "quarot_b200" not in ref_arm.replace("quarot_b200/synth.py", "")
