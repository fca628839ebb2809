"""The upstream ``quarot.transformers`` sub-package: the paged 4-bit KV cache (quarot/transformers/__init__.py)."""
from .kv_cache import MultiLayerPagedKVCache4Bit
