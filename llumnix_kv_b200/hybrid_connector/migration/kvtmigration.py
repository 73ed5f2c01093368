""""kvt+migration": one role-free engine that can be prefill sender, decode receiver and
migration source / destination at once (blade_kvt/hybrid_connector/migration/kvtmigration.py:
48-170).  Which half handles a request is decided per request from its parameters.
"""
from __future__ import annotations

import logging
from collections.abc import AsyncGenerator
from typing import Optional

import msgspec

from ..backend import BackendMeta, HybridBackend, OperationPlan, merge_operation_plans
from ..engine_proxy import KVCacheBlocks, KVConnectorRole, Request, SchedulerOutput, VllmConfig, get_param
from ..kvtbackend import (CODE_OK, CODE_REQNOTFOUND, P_KVT_STATE, P_REMOTE_DECODE, PREFILL_RESP, DBackend, PBackend,
                          RKVTDInfo)
from ..utils import IoRet
from . import KVT_SUSPEND_REQ, SRC_INFO, SuspendReq
from .backend import MigrationBackend, pack_msg, read_body

logger = logging.getLogger("llumnix_kv_b200.hybrid_connector")


class KVTMigration(HybridBackend):
    def __init__(self, vllm_config: VllmConfig, role: KVConnectorRole, kv_cache_config=None, **kw):
        super().__init__(vllm_config, role, kv_cache_config, **kw)
        self._p = PBackend(vllm_config, role, kv_cache_config, **kw)
        self._d = DBackend(vllm_config, role, kv_cache_config, **kw)
        self._m = MigrationBackend(vllm_config, role, kv_cache_config, dbackend=self._d, **kw)
        if role == KVConnectorRole.SCHEDULER:
            self._engine.sched_rpc_server().register_method(KVT_SUSPEND_REQ, self._on_transfer_suspend_kv)
            self._kvtreqdec = msgspec.msgpack.Decoder(RKVTDInfo)

    # ---- worker half: this engine both sends (client) and receives (server) ------------------------------
    def register_kv_caches(self, kv_caches: dict) -> None:
        self._p.register_kv_caches(kv_caches)
        self._d.register_kv_caches(kv_caches)

    def bind_backend_metadata(self, meta: BackendMeta) -> None:
        self._p.bind_backend_metadata(meta)

    def clear_backend_metadata(self) -> None:
        self._p.clear_backend_metadata()

    def bypass_bind(self, meta: BackendMeta) -> None:
        self._p.bypass_bind(meta)

    def bypass_clear(self) -> None:
        self._p.bypass_clear()

    async_load_kv = None  # type: ignore[assignment]

    def async_save_kv_layer(self, layer_name: str, kv_layer, m: BackendMeta) -> Optional[AsyncGenerator]:
        r = self._p.async_save_kv_layer(layer_name, kv_layer, m)
        assert r is None
        return None

    def stop(self) -> None:
        for b in (self._p, self._d):
            if hasattr(b, "stop"):
                b.stop()

    # ---- scheduler half ---------------------------------------------------------------------------------
    def wait_workers_registered(self, timeout=None) -> bool:
        return self._d.wait_workers_registered(timeout)

    def migration_status(self) -> dict:
        return self._m.migration_status()

    def on_outputs(self, outputs: dict) -> None:
        self._m.on_outputs(outputs)

    async def async_get_num_new_matched_tokens(self, req: Request, num_computed_tokens: int) -> int:
        if get_param(req, SRC_INFO):
            return 0
        return await self._d.async_get_num_new_matched_tokens(req, num_computed_tokens)

    async def async_update_state_after_alloc(self, request: Request, blocks: KVCacheBlocks,
                                             num_external_tokens: int) -> Optional[IoRet]:
        if get_param(request, SRC_INFO):
            return await self._m.async_update_state_after_alloc(request, blocks, num_external_tokens)
        return await self._d.async_update_state_after_alloc(request, blocks, num_external_tokens)

    def get_operations(self, req: Request) -> OperationPlan:
        m_ops = self._m.get_operations(req)
        if m_ops[0] > 0:
            return m_ops     # arriving by migration: that is its one load
        if get_param(req, P_KVT_STATE) is not None or get_param(req, P_REMOTE_DECODE) is not None:
            kvt_ops = self._p.get_operations(req)
        else:
            kvt_ops = self._d.get_operations(req)
        return merge_operation_plans(m_ops, kvt_ops)

    def build_backend_meta(self, sout: SchedulerOutput) -> BackendMeta:
        self._d.build_backend_meta(sout)
        self._m.build_backend_meta(sout)
        return self._p.build_backend_meta(sout)

    async def _on_transfer_suspend_kv(self, reader, writer):
        """Source side of a migration with KV: push the KV, then let go of the request."""
        req: RKVTDInfo = self._kvtreqdec.decode(await read_body(reader))
        resp = await self._p.submit_transfer_kv(req)
        if resp.computed == -1:
            resp.code = CODE_REQNOTFOUND
        if resp.code == CODE_OK:
            sus = await self._m.do_suspend(SuspendReq(reqid=req.reqid))
            if sus.code != CODE_OK:
                resp.code = sus.code
            resp.output_token_ids = sus.output_token_ids
        writer.write(pack_msg(PREFILL_RESP, resp))
        await writer.drain()
