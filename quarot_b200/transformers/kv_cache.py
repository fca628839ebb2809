"""Paged 4-bit KV cache behind the upstream name (quarot/transformers/kv_cache.py:130-289).

Same constructor, same `update()` contract and the same memory layout as upstream -- pages
[pages, layers, 2, heads, page_size, head_dim / 2] uint8 with per-(token, head) fp16 (scale, zero) pairs beside them
-- so a model written against `quarot.transformers.MultiLayerPagedKVCache4Bit` runs unchanged.  Underneath, two fused
CUDA kernels replace upstream's chain: `qr_kv_append_i4` (Hadamard of the keys over the head dimension, asymmetric
int4 quantisation, packing and the write into the page slot, for prompt and single-token appends alike) and
`qr_kv_decode_i4` (Hadamard of the query, then single-token attention straight from the packed pages).

Not built: `disable_quant=True` (the fp16 variant of the cache) raises NotImplementedError.
"""
import functools
import math

import torch

from .. import _lib, _ops
from ..functional.quantization import get_minq_maxq

_lib_c = _lib.lib


def asym_quantize_and_pack_i4(x: torch.Tensor):
    """Per-(token, head) asymmetric int4 codes of x over its last axis, two per byte, with (scale, zero) -- the format of
    the cache, in torch (quarot/transformers/kv_cache.py:10-24).  The CUDA append kernel produces the same bytes."""
    _, maxq = get_minq_maxq(bits=4, sym=False)
    xmax = torch.amax(x, dim=-1, keepdim=True)
    xmin = torch.amin(x, dim=-1, keepdim=True)
    scale = (xmax - xmin).clamp(min=1e-5) / maxq
    zero = -xmin
    q = torch.clamp(torch.round((x + zero) / scale), 0, maxq).to(dtype=torch.uint8)
    return q[..., 0::2] | (q[..., 1::2] << 4), scale, zero


def unpack_i4_and_asym_dequantize(q, scale, zero):
    """Inverse of the above: code * scale - zero (quarot/transformers/kv_cache.py:26-30)."""
    assert q.dtype == torch.uint8
    codes = torch.stack((q & 0x0f, (q >> 4) & 0x0f), dim=-1).view(*q.shape[:-1], q.shape[-1] * 2)
    return codes * scale - zero


def matmul_had_cuda(X, dtype):
    """Walsh-Hadamard transform over the last axis with scale 1/sqrt(n), computed in `dtype` and returned in X's dtype
    (quarot/transformers/kv_cache.py:32-35); one kernel with fp32 arithmetic inside."""
    return _ops.hadamard(X.to(dtype).contiguous(), None, 1).to(X.dtype).view(X.shape)


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def append_kv_i4(kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, k, v, layer_idx, seqlen_indptr=None,
                 hadamard_k=True):
    """Quantise the new keys / values k, v (fp16 [tokens, heads, head_dim]) and write them into their page slots.  The
    page table must already describe the sequences WITH the new tokens.  seqlen_indptr [batch + 1] gives the new tokens
    per sequence (a prompt); without it every sequence appends one token.  Stands in for upstream's
    asym_quantize_and_pack_i4 + init_kv_i4 / append_kv_i4 (quarot/transformers/kv_cache.py:38-62)."""
    tokens, heads, head_dim = k.shape
    assert v.shape == k.shape and k.dtype == v.dtype == torch.float16
    assert k.is_contiguous() and v.is_contiguous() and kv_data.is_contiguous() and kv_param.is_contiguous()
    dev = kv_data.device
    with torch.cuda.device(dev):
        _lib.check(_lib_c.qr_kv_append_i4(
            kv_data.data_ptr(), kv_param.data_ptr(), kv_indptr.data_ptr(), kv_indices.data_ptr(), last_page_offset.data_ptr(),
            k.data_ptr(), v.data_ptr(), seqlen_indptr.data_ptr() if seqlen_indptr is not None else None,
            tokens, last_page_offset.shape[0], kv_data.shape[1], int(layer_idx), heads, kv_data.shape[4], head_dim,
            1 if hadamard_k else 0, _stream(dev)), "append_kv_i4")


def batch_decode_i4(o, q, kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, layer_idx, hadamard_q=False):
    """o[b, h] = softmax(q[b, h] K^T / sqrt(d)) V over the packed pages, one new token per sequence
    (quarot/transformers/kv_cache.py:64-72); with hadamard_q the query is Hadamard-transformed first."""
    batch, heads, head_dim = q.shape
    assert o.shape == q.shape and q.dtype == o.dtype == torch.float16 and q.is_contiguous() and o.is_contiguous()
    dev = kv_data.device
    with torch.cuda.device(dev):
        _lib.check(_lib_c.qr_kv_decode_i4(
            o.data_ptr(), q.data_ptr(), kv_data.data_ptr(), kv_param.data_ptr(), kv_indptr.data_ptr(), kv_indices.data_ptr(),
            last_page_offset.data_ptr(), batch, kv_data.shape[1], int(layer_idx), heads, kv_data.shape[4], head_dim,
            1 if hadamard_q else 0, _stream(dev)), "batch_decode_i4")


class _AttentionStub(object):
    """What `update()` hands back once the prompt is cached: attention of one new token against the cache."""

    def __init__(self, cache_page_size, device, n_layers, disable_quant, hadamard_dtype):
        self.cache_page_size = cache_page_size
        self.n_layers = n_layers
        self.disable_quant = disable_quant
        self.hadamard_dtype = hadamard_dtype

    def forward(self, q, num_kv_heads, attention_kwargs, layer_idx):
        batch_size, q_len, num_qo_heads, head_dim = q.shape
        assert q_len == 1
        q = q.reshape(batch_size, num_qo_heads, head_dim).contiguous()
        attn_output = torch.empty_like(q)
        batch_decode_i4(attn_output, q, **attention_kwargs, layer_idx=layer_idx,
                        hadamard_q=self.hadamard_dtype is not None)
        return attn_output.unsqueeze(1)


class MultiLayerPagedKVCache4Bit:
    def __init__(self, batch_size, page_size, max_seq_len, device, n_layers, num_heads, head_dim,
                 disable_quant=False, hadamard_dtype=torch.float16):
        if disable_quant:
            raise NotImplementedError("MultiLayerPagedKVCache4Bit(disable_quant=True): the fp16 variant of the cache is not built")
        if head_dim != 128:
            raise NotImplementedError("MultiLayerPagedKVCache4Bit: head_dim must be 128 (as in the upstream kernels)")
        self.page_size = page_size
        self.batch_size = batch_size
        max_page_cnt = self.page_cnt_from_length(max_seq_len)
        self.disable_quant = disable_quant
        self.pages = torch.empty((max_page_cnt * batch_size, n_layers, 2, num_heads, page_size, head_dim // 2),
                                 dtype=torch.uint8, device=device)
        self.scales = torch.empty((max_page_cnt * batch_size, n_layers, 2, num_heads, page_size, 2),
                                  dtype=torch.float16, device=device)
        self.max_seq_len = max_seq_len
        self._needs_init = [True] * n_layers
        self.length = 0
        self.device = device
        self.hadamard_dtype = hadamard_dtype
        self._stub = _AttentionStub(self.page_size, device, n_layers, disable_quant=self.disable_quant,
                                    hadamard_dtype=self.hadamard_dtype)

    def page_cnt_from_length(self, length):
        return (length + self.page_size - 1) // self.page_size

    def _ensure_page_cnt_per_batch(self, expected_page_cnt_per_batch):
        if expected_page_cnt_per_batch * self.batch_size <= self.pages.shape[0]:
            return
        raise NotImplementedError

    @property
    def seen_tokens(self):
        return self.length

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        """First call per layer (the prompt): caches the keys / values and returns them unchanged, for the caller's own
        prefill attention.  Later calls (one token per sequence): caches the token and returns a callable that maps the
        query [batch, 1, heads, head_dim] to the attention output against the cache."""
        b_sz, added_length, num_heads, head_dim = key_states.shape
        assert b_sz == self.batch_size
        attention_mask = (cache_kwargs or {}).get("attention_mask")
        if layer_idx == 0:
            new_length = self.length + added_length
            self._ensure_page_cnt_per_batch(self.page_cnt_from_length(new_length))
            self.length = new_length
        specs = self.get_cache_specs_for_flash_infer(attention_mask)
        had = self.hadamard_dtype is not None
        k = key_states.reshape(b_sz * added_length, num_heads, head_dim)
        v = value_states.reshape(b_sz * added_length, num_heads, head_dim)
        if self._needs_init[layer_idx]:
            self._needs_init[layer_idx] = False
            if attention_mask is not None:
                keep = attention_mask.flatten().bool()
                k, v = k[keep], v[keep]
                seqlens = torch.nn.functional.pad(
                    torch.cumsum(attention_mask.sum(dim=-1, dtype=torch.int32), dim=0, dtype=torch.int32), (1, 0))
            else:
                seqlens = torch.arange(self.batch_size + 1, device=self.device, dtype=torch.int) * added_length
            append_kv_i4(specs["kv_data"], specs["kv_param"], specs["kv_indptr"], specs["kv_indices"],
                         specs["last_page_offset"], k.contiguous(), v.contiguous(), layer_idx,
                         seqlen_indptr=seqlens.to(torch.int32).contiguous(), hadamard_k=had)
            return key_states, value_states
        assert added_length == 1
        append_kv_i4(specs["kv_data"], specs["kv_param"], specs["kv_indptr"], specs["kv_indices"],
                     specs["last_page_offset"], k.contiguous(), v.contiguous(), layer_idx, hadamard_k=had)
        return functools.partial(self._stub.forward, num_kv_heads=num_heads, attention_kwargs=specs, layer_idx=layer_idx)

    def get_cache_specs_for_flash_infer(self, attention_mask):
        """Page table of the cache as the kernels take it: sequence b owns pages b, b + batch, b + 2 batch, ..."""
        if attention_mask is not None:
            seqlens = attention_mask.sum(dim=-1, dtype=torch.int32)
        else:
            seqlens = torch.tensor([self.length], dtype=torch.int32, device=self.device).expand(self.batch_size)
        page_cnt = self.page_cnt_from_length(seqlens)
        if (page_cnt[0] != page_cnt).any():
            raise NotImplementedError("Current implementation does not support the case where batches have different number of pages")
        page_cnt = page_cnt[0]
        page_ptr = seqlens % self.page_size
        page_ptr = torch.where((seqlens != 0) & (page_ptr == 0), self.page_size, page_ptr)
        ar = functools.partial(torch.arange, device=self.device, dtype=torch.int)
        return {
            "kv_data": self.pages,
            "kv_indptr": (ar(0, self.batch_size + 1) * page_cnt).to(torch.int32).contiguous(),
            "kv_indices": ((ar(page_cnt) * self.batch_size).unsqueeze(0) + ar(self.batch_size).unsqueeze(1)).view(-1).to(torch.int32).contiguous(),
            "last_page_offset": page_ptr.to(torch.int32).contiguous(),
            "kv_param": self.scales,
        }

    def get_seq_length(self, layer_idx=0):
        return self.length

    def get_max_length(self):
        return None

    def to_legacy_cache(self):
        return self
