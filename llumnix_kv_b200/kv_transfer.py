"""Import guard around the native extension plus small shape helpers.

Role of ``blade_kvt/kv_transfer.py``: ``IS_AVAILABLE`` tells callers whether the engine can be
used, and ``get_kv_transfer_token_bytes`` computes the per-token byte size of one layer's
cache on one TP rank (blade_kvt/kv_transfer.py:96-109).
"""
from __future__ import annotations

try:
    from llumnix_kv_b200 import load_ops as _load_ops

    _load_ops()
    from llumnix_kv_b200.kv_transfer_impl import (  # noqa: F401
        KVTransferClient,
        KVTransferProtocolType,
        KVTransferServer,
        ReqMeta,
        alloc_kv_cache_peer_mappable,
        alloc_phy_cont_mem,
        connect_naming,
        current_worker_info,
        support_transfers_protocols,
    )

    IS_AVAILABLE = True
    IMPORT_ERROR = None
except Exception as ex:  # pragma: no cover - exercised only on broken installs
    IS_AVAILABLE = False
    IMPORT_ERROR = ex

    class _Unavailable:
        def __init__(self, *a, **kw):
            raise RuntimeError(f"llumnix_kv_b200 native extension is not available: {IMPORT_ERROR}")

    KVTransferClient = KVTransferServer = ReqMeta = _Unavailable  # type: ignore


def get_kv_transfer_token_bytes(itemsize: int, head_dim: int, num_attention_heads: int, tp_size: int,
                                kv_lora_rank: int = 0, qk_rope_head_dim: int = 0, num_query_group: int = 0,
                                is_MLA: bool = False) -> int:
    """Bytes one token occupies in one layer's cache on one TP rank."""
    if is_MLA:
        # latent + rope, replicated on every rank
        return itemsize * (kv_lora_rank + qk_rope_head_dim)
    kv_heads = num_query_group if num_query_group > 0 else num_attention_heads
    heads_per_rank = max(1, kv_heads // tp_size)
    return 2 * itemsize * head_dim * heads_per_rank
