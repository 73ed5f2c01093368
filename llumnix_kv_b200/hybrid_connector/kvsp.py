""""kvt+kvs": a prefill engine whose prompts' KV goes both to the decode engine and to the
node's host-DRAM store, and whose repeated prefixes come back from that store
(blade_kvt/hybrid_connector/kvsp.py:32-118).  ``kvs_backend`` in the extra config names the
store flavour ("vineyard", "mooncake", "v6d_object": kvs_flavours.py); every flavour runs over the
in-repo store, which replaces those services.
"""
from __future__ import annotations

from .engine_proxy import KVConnectorRole, VllmConfig
from .filekvtbackend import PairMeta, StorePlusKVT

KVSPMeta = PairMeta


class KVSP(StorePlusKVT):
    def __init__(self, vllm_config: VllmConfig, role: KVConnectorRole, kv_cache_config=None, **kw):
        from .kvs_flavours import flavour_class

        flavour = vllm_config.kv_transfer_config.get_from_extra_config("kvs_backend", "pinned")
        super().__init__(vllm_config, role, kv_cache_config, flavour_class(flavour), **kw)


class V6dObjectKVTBackend(StorePlusKVT):
    """"v6d_object+kvt": the object-store flavour owns the request's loads and its save-done, the KVT prefill
    sender rides along as a sidecar that only transfers (blade_kvt/hybrid_connector/v6d_object_kvt_backend.py:61-185).
    The KVT half sees the request first, so a hybrid model's prompt is shortened once for both: what is stored
    is what is transferred.  Producer roles only."""

    def __init__(self, vllm_config: VllmConfig, role: KVConnectorRole, kv_cache_config=None, **kw):
        kcfg = vllm_config.kv_transfer_config
        if kcfg is None or not kcfg.is_kv_producer:
            raise ValueError("v6d_object+kvt backend requires a producer-capable kv_role (kv_producer or kv_both)")
        from .kvs_flavours import V6dObjectBackend

        super().__init__(vllm_config, role, kv_cache_config, V6dObjectBackend, **kw)
