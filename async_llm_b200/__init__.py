"""B200-native cache-view attention and Gated DeltaNet kernels behind the AsyncLLM seams."""

from .attention_backend import B200AttnBackend
from .block_ops import BlockOps
from .blocks import AsyncContext, CacheBlock, CacheView, SharedBlock, WorkerGroup
from .kvpool import BaseKVCachePool, MHAKVCache, PageAllocator
from .view_attention import (PrefillSpec, SharedCacheAttention, SharedCacheAttnMetadata,
                             SharedDecodeAttentionBuffers, SharedPrefillAttentionBuffers)

__all__ = [
    "B200AttnBackend", "BlockOps", "AsyncContext", "CacheBlock", "CacheView", "SharedBlock", "WorkerGroup",
    "BaseKVCachePool", "MHAKVCache", "PageAllocator",
    "PrefillSpec", "SharedCacheAttention", "SharedCacheAttnMetadata", "SharedDecodeAttentionBuffers", "SharedPrefillAttentionBuffers",
]
