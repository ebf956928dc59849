"""Python face of the sm_100a kernels."""
from .attention import PagedAttention, PrefillAttention, paged_attn_reference, prefill_attn_reference
from .flow import CreditPage, LocalPacer, new_status, read_status
from .gemm import gemm, pick_config, pick_splits
from .kv_cache import BLOCK_TOKENS, BlockAllocator, KVGeometry, PagedKVPool
from .kv_transfer import FanoutTarget, KvTransferFlow, MulticastPools, RemotePool, link_bytes, reference_transfer
from .memhog import Memhog
from .small import argmax, embedding, rmsnorm, rope_append, rope_inv_freq, sample, sample_reference, silu_mul

__all__ = [
    "PagedAttention", "PrefillAttention", "paged_attn_reference", "prefill_attn_reference", "CreditPage", "LocalPacer", "new_status", "read_status", "gemm", "pick_config", "pick_splits",
    "BLOCK_TOKENS", "BlockAllocator", "KVGeometry", "PagedKVPool", "FanoutTarget", "KvTransferFlow", "MulticastPools", "RemotePool", "link_bytes", "reference_transfer",
    "Memhog", "argmax", "embedding", "rmsnorm", "rope_append", "rope_inv_freq", "sample", "sample_reference", "silu_mul",
]
