""""kvt+kvs": a prefill engine whose prompts' KV goes both to the decode engine and to the
node's host-DRAM store, and whose repeated prefixes come back from that store
(blade_kvt/hybrid_connector/kvsp.py:32-118).  ``kvs_backend`` in the extra config names the
store flavour; the reference's "vineyard" and "mooncake" values select the in-repo store here,
because those services are replaced by it.
"""
from __future__ import annotations

from .engine_proxy import KVConnectorRole, VllmConfig
from .filekvtbackend import PairMeta, StorePlusKVT

KVSPMeta = PairMeta


class KVSP(StorePlusKVT):
    def __init__(self, vllm_config: VllmConfig, role: KVConnectorRole, kv_cache_config=None, **kw):
        flavour = vllm_config.kv_transfer_config.get_from_extra_config("kvs_backend", "pinned")
        if flavour not in ("pinned", "vineyard", "mooncake", "v6d_object"):
            raise ValueError(f"unknown kvs_backend {flavour!r} for the 'kvs+kvt' backend")
        from .kvsbackend import KVSBackend

        super().__init__(vllm_config, role, kv_cache_config, KVSBackend, **kw)
