"""The module graphs that the upstream benchmark builds (benchmarks/qlinear_benchmark.py:56-84), on the GPU:
Sequential(Quantizer, Linear4bit.from_float(linear, s_w)) and the two Sequential(OnlineHadamard(in, force_fp32),
Quantizer, Linear4bit.from_float(...)) variants, built through the `quarot` alias with integer weights in [-8, 6],
unit scales and uniform activations, at the script's sizes.  The int4 output must equal the oracle's."""
import importlib.util
import os

import pytest
import torch

import quarot_b200
from quarot_b200 import _lib
from oracle import quarot_oracle as O

pytestmark = pytest.mark.gpu
UPSTREAM = os.environ.get("QUAROT_UPSTREAM", "/root/reference")


@pytest.mark.parametrize("fin,fout,rows", [(4096, 4096, 2048), (4096, 11008, 2048), (8192, 28672, 512)])
def test_benchmark_module_graphs_match_oracle(fin, fout, rows):
    quarot_b200.install_as_quarot()
    from quarot.nn import Linear4bit, Quantizer, OnlineHadamard
    g = torch.Generator(device="cuda").manual_seed(fin + fout)
    x = torch.rand((1, rows, fin), generator=g, device="cuda").to(torch.float16)
    base = torch.nn.Linear(fin, fout, bias=False).cuda().to(torch.float16)
    base.weight.data = torch.randint(-8, 7, base.weight.shape, generator=g, device="cuda").to(torch.float16)
    s_w = torch.ones((fout, 1), dtype=torch.float16, device="cuda")
    plain = torch.nn.Sequential(Quantizer(input_clip_ratio=1.0), Linear4bit.from_float(base, weight_scales=s_w)).cuda()
    had32 = torch.nn.Sequential(OnlineHadamard(fin, force_fp32=True), Quantizer(input_clip_ratio=1.0),
                                Linear4bit.from_float(base, weight_scales=s_w)).cuda()
    had16 = torch.nn.Sequential(OnlineHadamard(fin, force_fp32=False), Quantizer(input_clip_ratio=1.0),
                                Linear4bit.from_float(base, weight_scales=s_w)).cuda()
    w_packed = plain[1].weight.cpu()
    assert torch.equal(O.unpack_i4(w_packed), base.weight.data.cpu().to(torch.int32))
    sample = torch.arange(0, rows, 29)

    def check(out, y):
        assert out.shape == (1, rows, fout) and out.dtype == torch.float16
        y = y.reshape(rows, fin).cpu()[sample]
        s = O.quantizer_scales(y)
        acc = torch.cat([O.matmul_i4(O.pack_i4(O.sym_quant_codes(y, s)), w_packed[r:r + 8192])
                         for r in range(0, fout, 8192)], dim=1)
        assert torch.equal(out.reshape(rows, fout).cpu()[sample], O.sym_dequant_fp32(acc, s, s_w.cpu()).half())

    check(plain(x), x)
    y32 = had32[0](x)
    y_ref = O.hadamard(x.reshape(rows, fin).cpu()[sample].float())
    assert float((y32.reshape(rows, fin).cpu()[sample].float() - y_ref).abs().max() / y_ref.abs().max()) < 1e-3
    check(had32(x), y32)
    check(had16(x), had16[0](x))
    assert _lib.kernel_status() == 0


@pytest.mark.skipif(not os.path.exists(os.path.join(UPSTREAM, "benchmarks", "qlinear_benchmark.py")),
                    reason="needs an upstream checkout (QUAROT_UPSTREAM) next to the GPU")
def test_upstream_benchmark_script_runs_unmodified(capsys):
    """benchmarks/qlinear_benchmark.py loaded by path and run as it is (fewer timing repetitions, set from outside)."""
    quarot_b200.install_as_quarot()
    path = os.path.join(UPSTREAM, "benchmarks", "qlinear_benchmark.py")
    spec = importlib.util.spec_from_file_location("_upstream_qlinear_benchmark", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.num_bench_steps, mod.num_warmup_steps = 3, 1
    import argparse
    for layer_type in ("v_proj", "down_proj"):
        mod.linear4bit_benchmark(argparse.Namespace(bsz=1, seq_len=2048, layer_type=layer_type))
    assert "Int4 time" in capsys.readouterr().out
    assert _lib.kernel_status() == 0


def test_fused_qkv_and_gate_up_equal_the_separate_projections():
    from quarot_b200 import synth
    hidden, kv, inter, rows = 1024, 256, 2816, 300
    dev = "cuda:0"

    def lin(i, o, seed):
        m = quarot_b200.nn.Linear4bit(i, o).to(dev)
        w, s = synth.weights(o, i, seed=seed)
        m.weight, m.weight_scales = w.to(dev), s.to(dev)
        return m

    class Block(torch.nn.Module):
        pass
    attn, mlp = Block(), Block()
    attn.q_proj, attn.k_proj, attn.v_proj = lin(hidden, hidden, 1), lin(hidden, kv, 2), lin(hidden, kv, 3)
    mlp.gate_proj, mlp.up_proj = lin(hidden, inter, 4), lin(hidden, inter, 5)
    x = quarot_b200.nn.Quantizer()(synth.activations(rows, hidden, seed=6).to(dev))
    want = [m(x) for m in (attn.q_proj, attn.k_proj, attn.v_proj, mlp.gate_proj, mlp.up_proj)]
    q, k, v = quarot_b200.nn.fuse_qkv(attn)(x)
    g, u = quarot_b200.nn.fuse_gate_up(mlp)(x)
    for got, ref in zip((q, k, v, g, u), want):
        assert torch.equal(got, ref)
    act = quarot_b200.nn.fuse_gate_up(mlp, swiglu=True)(x)
    assert torch.equal(act, torch.nn.functional.silu(want[3]) * want[4])
    assert _lib.kernel_status() == 0
