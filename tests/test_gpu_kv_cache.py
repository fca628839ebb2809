"""Paged 4-bit KV cache on the GPU against the CPU oracle: the append kernel's bytes and (scale, zero) pairs are
bit-exact given the kernel's own fp16 Hadamard output (and bit-exact outright without the transform), the page layout
is the upstream one, and the decode attention is within 2e-3 of the fp32 oracle computed from the cached codes."""
import numpy as np
import pytest
import torch

import quarot_b200 as qb
from quarot_b200.transformers import MultiLayerPagedKVCache4Bit
from quarot_b200.transformers import kv_cache as KV
from oracle import quarot_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _states(b, s, h, seed, scale=2.0):
    g = torch.Generator().manual_seed(seed)
    k = (torch.randn(b, s, h, 128, generator=g) * scale).half()
    v = (torch.randn(b, s, h, 128, generator=g) * scale).half()
    return k, v


def test_torch_helpers_match_upstream_fixture():
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "kv_cache.npz"))
    for name in ("gauss", "outlier", "tiny", "const", "ties"):
        x = torch.from_numpy(g[name + "_x"]).to(DEV)
        q, scale, zero = KV.asym_quantize_and_pack_i4(x)
        assert np.array_equal(q.cpu().numpy(), g[name + "_q"]), name
        assert np.array_equal(scale.cpu().numpy().view(np.uint16), g[name + "_scale"].view(np.uint16)), name
        deq = KV.unpack_i4_and_asym_dequantize(q, scale, zero)
        assert np.array_equal(deq.cpu().numpy().view(np.uint16), g[name + "_deq"].view(np.uint16)), name


@pytest.mark.parametrize("hadamard", [False, True])
def test_append_kernel_writes_the_upstream_bytes(hadamard):
    """Prompt of 37 tokens, then three single-token appends, two layers; every page slot holds what the oracle's
    quantiser gives for the corresponding (token, head) row, keys Hadamard-transformed first when asked for."""
    B, H, L, P = 2, 3, 2, 16
    cache = MultiLayerPagedKVCache4Bit(B, P, 64, DEV, L, H, 128, hadamard_dtype=torch.float16 if hadamard else None)
    cache.pages.fill_(0xEE)
    cache.scales.fill_(-1.0)
    steps = [_states(B, 37, H, seed=1)] + [_states(B, 1, H, seed=2 + i) for i in range(3)]
    for (k, v) in steps:
        for layer in range(L):
            r = cache.update((k + layer).half().to(DEV), v.to(DEV), layer, {})
    assert callable(r) and cache.get_seq_length() == 40
    allk = torch.cat([k for (k, _) in steps], dim=1)
    allv = torch.cat([v for (_, v) in steps], dim=1)
    specs = cache.get_cache_specs_for_flash_infer(None)
    pages, params = cache.pages.cpu(), cache.scales.cpu()
    for layer in range(L):
        kk = (allk + layer).half()
        if hadamard:
            y = qb.hadamard(kk.to(DEV), None, 1).cpu()                        # the kernel family's own fp16 Hadamard
            ref = O.kv_hadamard(kk)
            assert float((y.float() - ref).abs().max() / ref.abs().max()) < 1e-3
            kk = y
        for which, x in ((0, kk), (1, allv)):
            q, scale, zero = O.kv_asym_quant_pack(x)                            # [B, T, H, 64], [B, T, H, 1]
            for b in range(B):
                for t in range(40):
                    pg = int(specs["kv_indices"][int(specs["kv_indptr"][b]) + t // P])
                    got = pages[pg, layer, which, :, t % P]
                    par = params[pg, layer, which, :, t % P]
                    assert torch.equal(got, q[b, t]), (layer, which, b, t)
                    assert torch.equal(par[:, 0], scale[b, t, :, 0]) and torch.equal(par[:, 1], zero[b, t, :, 0])
    # slots beyond the sequence were never touched
    last_page = int(specs["kv_indices"][int(specs["kv_indptr"][0]) + 2])
    assert int(pages[last_page, 0, 0, 0, 8:].min()) == 0xEE


@pytest.mark.parametrize("B,H,P,T,hadamard", [(1, 4, 16, 45, True), (3, 2, 8, 129, True), (2, 32, 16, 700, False),
                                              (1, 1, 1, 5, True), (2, 3, 64, 64, False)])
def test_decode_attention_matches_the_oracle(B, H, P, T, hadamard):
    L = 2
    cache = MultiLayerPagedKVCache4Bit(B, P, T + 3, DEV, L, H, 128, hadamard_dtype=torch.float16 if hadamard else None)
    k, v = _states(B, T, H, seed=T)
    for layer in range(L):
        out = cache.update(k.to(DEV), (v * (layer + 1)).half().to(DEV), layer, {})
        assert out[0].shape == k.shape                                       # the prompt comes back unchanged
    for step in range(2):
        k1, v1 = _states(B, 1, H, seed=1000 + step)
        g = torch.Generator().manual_seed(2000 + step)
        q = (torch.randn(B, 1, H, 128, generator=g) * 1.5).half()
        for layer in range(L):
            attend = cache.update(k1.to(DEV), v1.to(DEV), layer, {})
            got = attend(q.to(DEV))
            assert got.shape == (B, 1, H, 128) and got.dtype == torch.float16
            specs = cache.get_cache_specs_for_flash_infer(None)
            qq = q.view(B, H, 128)
            if hadamard:
                qq = O.kv_hadamard(qq).half()
            ref = O.paged_decode_attention(qq, cache.pages.cpu(), cache.scales.cpu(), layer, specs["kv_indptr"].cpu(),
                                           specs["kv_indices"].cpu(), specs["last_page_offset"].cpu())
            err = (got.view(B, H, 128).cpu().float() - ref).abs().max() / ref.abs().max()
            assert float(err) < 2e-3, (step, layer, float(err))
    # the attention the cache computes is the attention over the quantised tensors, close to the unquantised one
    assert cache.get_seq_length() == T + 2


def test_first_update_with_an_attention_mask_packs_only_real_tokens():
    B, H, P, S = 2, 2, 16, 24
    cache = MultiLayerPagedKVCache4Bit(B, P, 32, DEV, 1, H, 128, hadamard_dtype=None)
    k, v = _states(B, S, H, seed=9)
    mask = torch.ones(B, S, dtype=torch.int64)
    mask[0, :4] = 0                                   # left padding: sequence 0 has 20 tokens, sequence 1 has 24
    cache.update(k.to(DEV), v.to(DEV), 0, {"attention_mask": mask.to(DEV)})
    specs = cache.get_cache_specs_for_flash_infer(mask.to(DEV))
    assert specs["last_page_offset"].tolist() == [4, 8]
    qk, sk, zk = O.kv_asym_quant_pack(k)
    pages = cache.pages.cpu()
    for b, offset in ((0, 4), (1, 0)):
        for t in range(int(mask[b].sum())):
            pg = int(specs["kv_indices"][int(specs["kv_indptr"][b]) + t // P])
            assert torch.equal(pages[pg, 0, 0, :, t % P], qk[b, t + offset])
