"""B200-native paged-KV attention path with the call surface of lite_llama's
``kv_engine`` / paged-attention modules.

* :mod:`.kernels` — ``update_kv_buffer``, ``flash_decoding``,
  ``paged_chunk_flash_attention``, ``flash_attention2_no_pad`` (CUDA, via libb200kv.so)
* :mod:`.paged_attention` — ``PagedKVCacheManager``, ``PagedReqTokensManager``
* :mod:`.kv_engine` — refcounts, prefix cache, prefill packer and chunk planner
"""

from .kv_engine import (  # noqa: F401
    ChunkedPrefillPlanner,
    KVBlockRefCounter,
    MixedLengthPrefillPacker,
    PackedPrefillPlan,
    PackedPrefillRequest,
    PrefillChunk,
    PrefixCache,
    PrefixCacheMatch,
)
from .paged_attention import PagedKVCacheManager, PagedReqTokensManager  # noqa: F401
from .kernels import (  # noqa: F401
    flash_attention2_no_pad,
    flash_decoding,
    paged_chunk_flash_attention,
    update_kv_buffer,
    update_kv_buffer_split,
)

__version__ = "0.1.0"
