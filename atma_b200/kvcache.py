"""Paged KV-cache scatter with the reference's signature (inference/layers/attention.py:30-56)."""

import torch

from . import _lib


@torch.no_grad()
def store_kvcache(key, value, k_cache, v_cache, slot_mapping):
    """Write (N, num_heads, head_dim) key/value rows into flat paged-cache slots; a slot of
    -1 skips the row.  The caches are updated in place."""
    _lib.require_cuda(key, "store_kvcache")
    lib = _lib.load()
    N, num_heads, head_dim = key.shape
    D = num_heads * head_dim
    assert slot_mapping.numel() == N
    assert key.stride(-1) == 1 and value.stride(-1) == 1
    assert key.stride(1) == head_dim and value.stride(1) == head_dim
    assert k_cache.stride(1) == D and v_cache.stride(1) == D
    assert k_cache.dtype == key.dtype and v_cache.dtype == value.dtype
    if slot_mapping.dtype != torch.int32 or not slot_mapping.is_contiguous():
        slot_mapping = slot_mapping.to(torch.int32).contiguous()
    _lib.check(lib.atma_store_kvcache(_lib.ptr(key), key.stride(0), _lib.ptr(value), value.stride(0),
                                      _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(slot_mapping),
                                      N, D, key.element_size(), _lib.stream_ptr()))
