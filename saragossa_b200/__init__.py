"""saragossa_b200: the B200-native KV-cache hot path behind the reference's
resident-cache API (C ABI in include/sgk.h, CUDA kernels in csrc/)."""
from .resident import (KV_BF16, KV_F32, KV_U8G32, PAGE_TOKENS, Batch, DecodeResidentState, DeviceBuffer,
                       FullAttentionState, InferError, LinearAttentionState, PagePool, Rope, Sequence, Step,
                       encode_gated_delta_step_batch, make_rope)
from .prefix import (BlockAwarePrefixCache, BlockHash, DecoderPrefixCache, MemoryGuard, PrefixBlockHit,
                     longest_prefix_entry_index)

__all__ = [
    "KV_F32", "KV_BF16", "KV_U8G32", "PAGE_TOKENS", "Batch", "DecodeResidentState", "DeviceBuffer",
    "FullAttentionState", "InferError", "LinearAttentionState", "PagePool", "Rope", "Sequence", "Step", "make_rope",
    "encode_gated_delta_step_batch",
    "BlockAwarePrefixCache", "BlockHash", "DecoderPrefixCache", "MemoryGuard", "PrefixBlockHit", "longest_prefix_entry_index",
]
