"""``kv_both`` with the "kvt" backend: a prefill engine that also keeps a file store.

Loads come from the file store, saves go to both the file store and the decode engine
(blade_kvt/hybrid_connector/filekvtbackend.py:35-115).  It is the smallest example of a
composite: two backends behind one HybridBackend, their operation plans merged, their step
metadata carried side by side.
"""
from __future__ import annotations

import dataclasses
from collections.abc import AsyncGenerator
from typing import Optional

from .backend import BackendMeta, HybridBackend, OperationPlan, merge_operation_plans
from .engine_proxy import KVCacheBlocks, KVConnectorRole, Request, SchedulerOutput, VllmConfig
from .utils import IoRet


@dataclasses.dataclass
class PairMeta(BackendMeta):
    s: BackendMeta = dataclasses.field(default_factory=BackendMeta)   # store half
    p: BackendMeta = dataclasses.field(default_factory=BackendMeta)   # prefill-sender half

    def __bool__(self):
        return bool(self.s) or bool(self.p)

    def wants_nan_flag(self) -> bool:
        return self.s.wants_nan_flag() or self.p.wants_nan_flag()

    def set_nan_flag(self, flag) -> None:
        self.s.set_nan_flag(flag)
        self.p.set_nan_flag(flag)


class StorePlusKVT(HybridBackend):
    """A store backend (loads and saves) combined with the KVT prefill sender (saves only)."""

    def __init__(self, vllm_config: VllmConfig, role: KVConnectorRole, kv_cache_config, store_cls, **kw):
        super().__init__(vllm_config, role, kv_cache_config, **kw)
        from .kvtbackend import PBackend

        self._s = store_cls(vllm_config, role, kv_cache_config, **kw)
        self._p = PBackend(vllm_config, role, kv_cache_config, **kw)

    # ---- worker half ------------------------------------------------------------------------------
    def register_kv_caches(self, kv_caches: dict) -> None:
        self._s.register_kv_caches(kv_caches)
        self._p.register_kv_caches(kv_caches)

    def bind_backend_metadata(self, meta: BackendMeta) -> None:
        self._s.bind_backend_metadata(meta.s)
        self._p.bind_backend_metadata(meta.p)

    def clear_backend_metadata(self) -> None:
        self._s.clear_backend_metadata()
        self._p.clear_backend_metadata()

    def bypass_bind(self, meta: BackendMeta) -> None:
        self._s.bypass_bind(meta.s)
        self._p.bypass_bind(meta.p)

    def bypass_clear(self) -> None:
        self._s.bypass_clear()
        self._p.bypass_clear()

    async def async_load_kv(self, m: BackendMeta) -> AsyncGenerator:
        assert isinstance(m, PairMeta)
        async for ret in self._s.async_load_kv(m.s):
            yield ret

    def async_save_kv_layer(self, layer_name: str, kv_layer, m: BackendMeta) -> Optional[AsyncGenerator]:
        assert isinstance(m, PairMeta)
        self._p.async_save_kv_layer(layer_name, kv_layer, m.p)    # records the layer event; completion comes by RPC
        return self._s.async_save_kv_layer(layer_name, kv_layer, m.s)

    def save_done_source(self) -> Optional[str]:
        return self._s.save_done_source()

    def stop(self) -> None:
        for b in (self._s, self._p):
            if hasattr(b, "stop"):
                b.stop()

    # ---- scheduler half ---------------------------------------------------------------------------
    async def async_get_num_new_matched_tokens(self, req: Request, num_computed_tokens: int) -> int:
        return await self._s.async_get_num_new_matched_tokens(req, num_computed_tokens)

    async def async_update_state_after_alloc(self, request: Request, blocks: KVCacheBlocks,
                                             num_external_tokens: int) -> Optional[IoRet]:
        return await self._s.async_update_state_after_alloc(request, blocks, num_external_tokens)

    async def async_cleanup(self, req: Request) -> None:
        await self._s.async_cleanup(req)
        await self._p.async_cleanup(req)

    def get_operations(self, req: Request) -> OperationPlan:
        # the KVT half goes first: it may shorten a hybrid model's prompt
        p_ops = self._p.get_operations(req)
        s_ops = self._s.get_operations(req)
        return merge_operation_plans(s_ops, p_ops)

    def build_backend_meta(self, sout: SchedulerOutput) -> BackendMeta:
        return PairMeta(s=self._s.build_backend_meta(sout), p=self._p.build_backend_meta(sout))

    # what the engine core and tests reach through the composite
    def wait_workers_registered(self, timeout=None) -> bool:
        return True


class FilePBackend(StorePlusKVT):
    def __init__(self, vllm_config: VllmConfig, role: KVConnectorRole, kv_cache_config=None, **kw):
        from .file_backend import FileBackend

        super().__init__(vllm_config, role, kv_cache_config, FileBackend, **kw)
