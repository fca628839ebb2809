"""Placeholder for the upstream ``quarot.transformers`` sub-package.

The paged 4-bit KV cache (quarot/transformers/kv_cache.py:130-289) and its
attention kernels are outside the quantized-linear path this package implements.
The sub-package exists so that ``import quarot.transformers`` succeeds; using the
cache raises.
"""


class MultiLayerPagedKVCache4Bit:
    def __init__(self, *args, **kwargs):
        raise NotImplementedError(
            "MultiLayerPagedKVCache4Bit (4-bit paged KV cache) is not part of quarot_b200; "
            "only the OnlineHadamard / Quantizer / Linear4bit path is implemented")
