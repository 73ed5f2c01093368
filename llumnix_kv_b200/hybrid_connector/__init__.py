"""HybridConnector: the vLLM-style KV connector facade.

One class, two halves selected by role: in the engine-core process it is the
``HybridScheduler`` (request lifecycle, RPC endpoint), in each worker process the
``HybridWorker`` (``start_load_kv`` / ``save_kv_layer`` entry points).  Entry points and their
semantics follow blade_kvt/hybrid_connector/__init__.py:1776-1937.
"""
from __future__ import annotations

from typing import Any, Optional

from .backend import (PD_CLIENT_INDEX, PD_FINISH_REASON, PD_SAVED, PD_STOP_REASON, AbortReq, BackendMeta,  # noqa: F401
                      HCSchedOutput, HybridBackend, HybridMetadata, IoDoneReqs, OperationPlan, get_backend_cls,
                      has_setup_save, merge_operation_plans, req_aborted, set_operation_sources)
from .engine_proxy import (EngineProxy, FinishReason, KVCacheBlocks, KVConnectorMetadata, KVConnectorRole, Request,  # noqa: F401
                           SchedulerOutput, VllmConfig, WorkerProxy, current_engine, current_worker, get_param,
                           set_param)
from .scheduler import HybridConnectorStats, HybridScheduler  # noqa: F401
from .utils import IoRet, IoState, try_advance  # noqa: F401
from .worker import HybridWorker

P_REMOTE_DECODE = "do_remote_decode"
P_IGNORE_OUTPUTS = "ignore_output"


class HybridConnector:
    def __init__(self, vllm_config: VllmConfig, role: KVConnectorRole, kv_cache_config=None,
                 engine: Optional[EngineProxy] = None, worker: Optional[WorkerProxy] = None):
        self._role = role
        self._sched: Optional[HybridScheduler] = None
        self._worker: Optional[HybridWorker] = None
        global _g_scheduler, _g_worker
        if role == KVConnectorRole.SCHEDULER:
            self._sched = HybridScheduler(vllm_config, kv_cache_config, engine or current_engine())
            _g_scheduler = self._sched
        else:
            self._worker = HybridWorker(vllm_config, kv_cache_config, worker or current_worker())
            _g_worker = self._worker

    # ---- scheduler side -------------------------------------------------------------------------
    def get_num_new_matched_tokens(self, request: Request, num_computed_tokens: int) -> tuple:
        assert self._sched is not None
        return self._sched.get_num_new_matched_tokens(request, num_computed_tokens)

    def update_state_after_alloc(self, request: Request, blocks: KVCacheBlocks, num_external_tokens: int, **kw):
        assert self._sched is not None
        return self._sched.update_state_after_alloc(request, blocks, num_external_tokens, **kw)

    def build_connector_meta(self, scheduler_output: SchedulerOutput) -> KVConnectorMetadata:
        assert self._sched is not None
        return self._sched.build_connector_meta(scheduler_output)

    def step(self) -> Optional[dict]:
        assert self._sched is not None
        return self._sched.step()

    def has_requests(self) -> bool:
        assert self._sched is not None
        return self._sched.has_requests()

    @property
    def pending_requests(self) -> list:
        assert self._sched is not None
        return self._sched.pending_requests

    def on_add_req(self, req: Request) -> bool:
        assert self._sched is not None
        return self._sched.on_add_req(req)

    def on_abort_req(self, reqid: str, reason: str = "", output: bool = True, iscore: bool = True) -> None:
        assert self._sched is not None
        self._sched.on_abort_req(AbortReq(reqid=reqid, output=output, reason=reason), iscore)

    def request_finished_all_groups(self, request: Request, block_ids: tuple) -> tuple:
        """Called when the engine frees a finished request.  Never delays the free: a save in
        flight holds its own block references.  The returned params tell a dual-request frontend
        whether the KV has already left (``kv_transfer_done``) or is still leaving
        (``kv_transfer_pending`` now, ``kv_transfer_done`` in a later empty output)."""
        assert self._sched is not None
        self._sched.mark_post_scheduler_save_extra(request.request_id)
        if get_param(request, P_REMOTE_DECODE) and not get_param(request, P_IGNORE_OUTPUTS):
            reason = request.get_finished_reason()
            if reason == FinishReason.ABORT:
                return (False, None)
            if get_param(request, PD_SAVED):
                return (False, {"kv_transfer_done": True})
            set_param(request, PD_FINISH_REASON, reason)
            set_param(request, PD_STOP_REASON, request.stop_reason)
            set_param(request, PD_CLIENT_INDEX, request.client_index)
            return (False, {"kv_transfer_pending": True})
        return (False, None)

    def get_hybrid_connector_stats(self, num_gpu_blocks: int) -> HybridConnectorStats:
        assert self._sched is not None
        return self._sched.get_hybrid_connector_stats(num_gpu_blocks)

    # ---- worker side ----------------------------------------------------------------------------
    def bind_connector_metadata(self, m: KVConnectorMetadata) -> None:
        assert isinstance(m, HybridMetadata) and self._worker is not None
        self._worker.bind_connector_metadata(m)

    def has_connector_metadata(self) -> bool:
        assert self._worker is not None
        return self._worker.has_connector_metadata()

    def clear_connector_metadata(self) -> None:
        assert self._worker is not None
        self._worker.clear_connector_metadata()

    def register_kv_caches(self, kv_caches: dict) -> None:
        assert self._worker is not None
        self._worker.register_kv_caches(kv_caches)

    def start_load_kv(self, forward_context: Any = None, **kwargs) -> None:
        assert self._worker is not None
        self._worker.start_load_kv(**kwargs)

    def wait_for_layer_load(self, layer_name: str) -> None:
        return  # loads complete before the request is scheduled; nothing to wait for per layer

    def save_kv_layer(self, layer_name: str, kv_layer, attn_metadata: Any = None, **kwargs) -> None:
        assert self._worker is not None
        self._worker.save_kv_layer(layer_name, kv_layer, **kwargs)

    def wait_for_save(self) -> None:
        return  # saves are asynchronous; completion reaches the scheduler as SAVE_DONE

    def wants_nan_flag(self) -> bool:
        assert self._worker is not None
        return self._worker.wants_nan_flag()

    def set_nan_flag(self, flag) -> None:
        assert self._worker is not None
        self._worker.set_nan_flag(flag)


_g_scheduler: Optional[HybridScheduler] = None
_g_worker: Optional[HybridWorker] = None


def hybridsched() -> HybridScheduler:
    assert _g_scheduler is not None
    return _g_scheduler


def hybridworker() -> HybridWorker:
    assert _g_worker is not None
    return _g_worker


def wakeup_scheduler() -> None:
    hybridsched().wakeup_scheduler()


def send_bypass_task(kv_connector_metadata) -> None:
    hybridsched().send_bypass_task(kv_connector_metadata)


def try_setup_save(req: Request, source: str) -> bool:
    return hybridsched().try_setup_save(req, source)


def mark_backend_save_done(req: Request, source: str) -> None:
    hybridsched().mark_backend_save_done(req, source)
