"""B200 (sm_100a) attention + Gated-DeltaNet operators behind TinyTitan's operator interface.

Everything here forwards to libtinytitan_cuda.so through its C ABI (include/tinytitan_cuda.h);
there is no PyTorch, Triton or CPU implementation behind these classes.
"""
from ._lib import (TT_BF16, TT_F16, InvalidArgument, TinyTitanError, UnsupportedShape, lib)
from .managers import FULL, LINEAR, SWA, ArchConfig, GDNStateManager, KVCacheManager, KVView, KVWindow
from .operators import (GDN, Attention, AttentionSplitGeometry, Context, DecodeSession, GDNSession, KVFormat,
                        LinearAttentionConfig, PeerExchange, PrefillAttention, PrefillAttentionParams, QSAIndexer,
                        SparseIndexerConfig, quantize_kv_rows)

__all__ = [
    "TT_F16", "TT_BF16", "TinyTitanError", "InvalidArgument", "UnsupportedShape", "lib", "Context", "Attention",
    "AttentionSplitGeometry", "DecodeSession", "KVFormat", "PrefillAttention", "PrefillAttentionParams", "GDN",
    "GDNSession", "quantize_kv_rows", "QSAIndexer", "SparseIndexerConfig", "PeerExchange", "LinearAttentionConfig", "ArchConfig", "KVCacheManager", "KVView", "KVWindow", "GDNStateManager", "SWA",
    "FULL", "LINEAR",
]
