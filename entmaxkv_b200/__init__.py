"""entmaxkv_b200: the sparse entmax decode step of deep-spin/entmaxkv as hand-written
sm_100a CUDA behind the reference's Python API (entmaxkv/__init__.py:1-15)."""

from .kv_cache import PagedKVCache
from .attention_topk import sparse_attention_decode_paged
from .attention_gaussian import sparse_attention_decode_gaussian_aware_entmax

__version__ = "0.1.0"

__all__ = [
    "PagedKVCache",
    "sparse_attention_decode_paged",
    "sparse_attention_decode_gaussian_aware_entmax",
]
