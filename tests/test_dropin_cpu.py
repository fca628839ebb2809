"""Drop-in checks that need no GPU: upstream caller code resolves against this package, and the checkpoint key
contract of the upstream converter (e2e/checkpoint_utils/quantize_llama_checkpoint.py:29-66) loads into modules
built the way the upstream model builds them (e2e/quantized_llama/modeling_llama.py:95-119)."""
import importlib.util
import os

import pytest
import torch

import quarot_b200
from quarot_b200.functional.quantization import pack_i4, unpack_i4

UPSTREAM = os.environ.get("QUAROT_UPSTREAM", "/root/reference")


@pytest.mark.skipif(not os.path.exists(os.path.join(UPSTREAM, "benchmarks", "qlinear_benchmark.py")),
                    reason="needs an upstream checkout (QUAROT_UPSTREAM)")
def test_upstream_benchmark_script_imports_against_this_package():
    """benchmarks/qlinear_benchmark.py, loaded unmodified by path after install_as_quarot(): its
    `from quarot.nn import Linear4bit, Quantizer, OnlineHadamard` must bind to these modules."""
    quarot_b200.install_as_quarot()
    path = os.path.join(UPSTREAM, "benchmarks", "qlinear_benchmark.py")
    spec = importlib.util.spec_from_file_location("_upstream_qlinear_benchmark", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.Linear4bit is quarot_b200.nn.Linear4bit
    assert mod.Quantizer is quarot_b200.nn.Quantizer
    assert mod.OnlineHadamard is quarot_b200.nn.OnlineHadamard
    assert callable(mod.linear4bit_benchmark) and callable(mod.module_benchmark)
    assert (4096, 11008) in mod.mlp_sizes and (8192, 8192) in mod.model_sizes


class _Attention(torch.nn.Module):
    """The quantised sub-modules of the upstream attention block, same attribute names and nesting."""

    def __init__(self, hidden, heads, kv_hidden):
        super().__init__()
        lin = lambda i, o: quarot_b200.nn.Linear4bit.from_float(torch.nn.Linear(i, o, bias=False).half())
        self.quantizer = quarot_b200.nn.Quantizer()
        self.q_proj, self.k_proj, self.v_proj = lin(hidden, hidden), lin(hidden, kv_hidden), lin(hidden, kv_hidden)
        self.o_proj_hadamard = quarot_b200.nn.OnlineHadamard(heads)
        self.o_proj = torch.nn.Sequential(quarot_b200.nn.Quantizer(), lin(hidden, hidden))


class _MLP(torch.nn.Module):
    def __init__(self, hidden, inter):
        super().__init__()
        lin = lambda i, o: quarot_b200.nn.Linear4bit.from_float(torch.nn.Linear(i, o, bias=False).half())
        self.quantizer = quarot_b200.nn.Quantizer()
        self.up_proj, self.gate_proj = lin(hidden, inter), lin(hidden, inter)
        self.down_proj = torch.nn.Sequential(quarot_b200.nn.OnlineHadamard(inter), quarot_b200.nn.Quantizer(),
                                             lin(inter, hidden))


class _Layer(torch.nn.Module):
    def __init__(self, hidden, heads, kv_hidden, inter):
        super().__init__()
        self.self_attn = _Attention(hidden, heads, kv_hidden)
        self.mlp = _MLP(hidden, inter)


def test_converter_state_dict_loads_with_its_key_renames():
    hidden, heads, kv_hidden, inter = 128, 4, 64, 344          # 344 = 172 * 2: the MLP Hadamard has a table factor
    # what the converter holds before renaming: float weights on the int4 grid times per-channel scales
    g = torch.Generator().manual_seed(5)
    shapes = {"self_attn.q_proj": (hidden, hidden), "self_attn.k_proj": (kv_hidden, hidden),
              "self_attn.v_proj": (kv_hidden, hidden), "self_attn.o_proj": (hidden, hidden),
              "mlp.up_proj": (inter, hidden), "mlp.gate_proj": (inter, hidden), "mlp.down_proj": (hidden, inter)}
    renames = {"mlp.down_proj": "mlp.down_proj.2", "self_attn.o_proj": "self_attn.o_proj.1"}
    new_dict, codes = {}, {}
    for name, (n, k) in shapes.items():
        c = torch.randint(-8, 8, (n, k), generator=g)
        s = (torch.rand(n, 1, generator=g) * 0.01 + 0.005).half()
        key = name
        for old, new in renames.items():
            key = key.replace(old, new)
        float_w = c.half() * s
        new_dict[key + ".weight_scales"] = s
        new_dict[key + ".weight"] = pack_i4((float_w / s).round().to(torch.int8))
        codes[key] = c
    layer = _Layer(hidden, heads, kv_hidden, inter)
    result = layer.load_state_dict(new_dict, strict=False)
    # the converter's own acceptance test (quantize_llama_checkpoint.py:65-66)
    assert all("had_rem_dim" in k for k in result.missing_keys), result
    assert result.missing_keys == ["mlp.down_proj.0.had_rem_dim"]
    assert len(result.unexpected_keys) == 0, result
    for key, c in codes.items():
        mod = layer.get_submodule(key)
        assert torch.equal(unpack_i4(mod.weight), c.to(torch.int32))
        assert mod.weight_scales.dtype == torch.float16 and mod.weight_scales.shape == (c.shape[0], 1)
    # the fused rewrite keeps every key in place
    before = set(layer.state_dict())
    assert quarot_b200.nn.fuse_modules(layer) == 1
    assert set(layer.state_dict()) == before


def test_horizontal_fusion_keeps_the_checkpoint_keys_and_shares_storage():
    """fuse_qkv / fuse_gate_up: one concatenated operand, the projections hold views of it, state-dict keys unchanged,
    and a checkpoint loaded afterwards lands in the fused operand."""
    layer = _Layer(128, 4, 64, 344)
    keys = set(layer.state_dict())
    qkv = quarot_b200.nn.fuse_qkv(layer.self_attn)
    gu = quarot_b200.nn.fuse_gate_up(layer.mlp)
    assert set(layer.state_dict()) == keys
    assert qkv.splits == [128, 64, 64] and qkv.weight.shape == (256, 64) and gu.weight.shape == (688, 64)
    assert layer.self_attn.k_proj.weight.data_ptr() == qkv.weight[128:192].data_ptr()
    new = {k: (torch.randint(0, 255, v.shape, dtype=torch.uint8) if v.dtype == torch.uint8 else torch.rand_like(v))
           for k, v in layer.state_dict().items()}
    layer.load_state_dict(new)
    assert torch.equal(qkv.weight, torch.cat([new["self_attn.q_proj.weight"], new["self_attn.k_proj.weight"],
                                              new["self_attn.v_proj.weight"]]))
    assert torch.equal(gu.weight_scales, torch.cat([new["mlp.gate_proj.weight_scales"], new["mlp.up_proj.weight_scales"]]))
    with pytest.raises(ValueError):
        quarot_b200.nn.HorizontalLinear4bit(layer.self_attn.q_proj)
