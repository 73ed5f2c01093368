"""The only seam between the connector and the engine it plugs into.

Everything the control plane needs from an engine goes through an ``EngineProxy`` (scheduler
side) or a ``WorkerProxy`` (worker side): block allocation with reference counting, the
request table, adding / finishing / aborting requests, waking the engine loop, the event loops
of the connector's own threads and the scheduler's RPC server.  Function names follow
blade_kvt/hybrid_connector/engine_proxy.py (sched_allocate_slots :168-206, sched_get_blocks /
acquire / free :231-253, sched_add_req / finish_req / get_req :255-294, core_add_req /
abort_req :319-343, get/set/pop_param :346-369, wakeup_core :533-540, core_init / worker_init
:543-565).  The reference binds these to one process-global forked-vLLM engine; here they are
methods of an object so that several engines can live in one process, with module-level
``core_init`` / ``worker_init`` keeping the one-engine-per-process style available.
"""
from __future__ import annotations

import logging
import os
from typing import Any, Iterable, Optional

from llumnix_kv_b200 import envs
from llumnix_kv_b200.engine.config import VllmConfig
from llumnix_kv_b200.engine.types import (EngineCoreOutput, EngineCoreRequest, EngineCoreRequestType, FinishReason,
                                          KVCacheBlocks, KVConnectorMetadata, KVConnectorRole, Request,
                                          RequestStatus, SamplingParams, SchedulerOutput)

from .utils import RpcServer, start_asyncio_thread

__all__ = [
    "EngineProxy", "WorkerProxy", "core_init", "worker_init", "current_engine", "current_worker", "get_param",
    "set_param", "pop_param", "update_params", "core_get_param", "core_update_params", "get_logger",
    "EngineCoreOutput", "EngineCoreRequest", "FinishReason", "KVCacheBlocks", "KVConnectorMetadata",
    "KVConnectorRole", "Request", "SchedulerOutput", "VllmConfig", "get_p_node_pop_len", "sched_rpc_server_port",
    "scheduler_rpc_host",
]


def get_logger(name: str):
    return logging.getLogger(name)


# ---- per-request parameter dict ("kv_transfer_params") -------------------------------------------
def get_param(req: Request, key: str, defval: Any = None):
    if req.kv_transfer_params is None:
        return defval
    return req.kv_transfer_params.get(key, defval)


def set_param(req: Request, key: str, val: Any) -> None:
    if req.kv_transfer_params is None:
        req.kv_transfer_params = {}
    req.kv_transfer_params[key] = val


def pop_param(req: Request, key: str, defval: Any = None):
    if req.kv_transfer_params is None:
        return defval
    return req.kv_transfer_params.pop(key, defval)


def update_params(req: Request, newval: dict) -> None:
    if req.kv_transfer_params is None:
        req.kv_transfer_params = {}
    req.kv_transfer_params.update(newval)


def core_get_param(req: EngineCoreRequest, key: str, defval: Any = None):
    if req.sampling_params is None or req.sampling_params.extra_args is None:
        return defval
    params = req.sampling_params.extra_args.get("kv_transfer_params")
    return defval if params is None else params.get(key, defval)


def core_update_params(req: EngineCoreRequest, newval: dict) -> None:
    if req.sampling_params is None:
        req.sampling_params = SamplingParams()
    if req.sampling_params.extra_args is None:
        req.sampling_params.extra_args = {}
    params = req.sampling_params.extra_args.get("kv_transfer_params")
    if params is None:
        req.sampling_params.extra_args["kv_transfer_params"] = dict(newval)
    else:
        params.update(newval)


def get_p_node_pop_len(cfg: VllmConfig) -> int:
    """Tokens a prefill node holds back from a hybrid model's prompt: 1 + speculative tokens."""
    n = 1
    if cfg.model_config.is_hybrid and cfg.speculative_config and cfg.speculative_config.num_speculative_tokens:
        n += cfg.speculative_config.num_speculative_tokens
    return n


def sched_rpc_server_port(cfg: VllmConfig) -> int:
    dp_master = int(os.environ.get("VLLM_DP_MASTER_PORT", "0") or 0)
    if dp_master > 0 and (os.getenv("AQUILA_RPC_PROTOCOL") or os.getenv("MASTER_ADDRESS")):
        return dp_master + 10 + cfg.parallel_config.data_parallel_rank + 256
    assert cfg.kv_transfer_config is not None
    port = cfg.kv_transfer_config.get_from_extra_config("rpc_port", None)
    if port is not None:
        return int(port)
    return int(cfg.kv_transfer_config.engine_available_port)


def scheduler_rpc_host(cfg: VllmConfig) -> str:
    return os.getenv("MASTER_ADDRESS") or "127.0.0.1"


class EngineProxy:
    """Scheduler-side seam of one engine."""

    def __init__(self, core, cfg: VllmConfig):
        self.core = core
        self.cfg = cfg
        self.sched_loop = start_asyncio_thread("hybridsched")
        self.rpc_server = RpcServer(sched_rpc_server_port(cfg), "hybridsched")
        self.rpc_server.start(self.sched_loop)
        if cfg.kv_transfer_config is not None:
            # an ephemeral port (0) is resolved once and published to everything that reads the config
            cfg.kv_transfer_config.engine_available_port = self.rpc_server.port()
            if "rpc_port" in cfg.kv_transfer_config.kv_connector_extra_config:
                cfg.kv_transfer_config.kv_connector_extra_config["rpc_port"] = self.rpc_server.port()

    # ---- loops / rpc -----------------------------------------------------------------------
    def get_hybrid_sched_loop(self):
        return self.sched_loop

    def sched_rpc_server(self) -> RpcServer:
        return self.rpc_server

    def rpc_port(self) -> int:
        return self.rpc_server.port()

    # ---- scheduler -------------------------------------------------------------------------
    def _sched(self):
        return self.core.scheduler

    def sched_allocate_slots(self, req: Request, load: bool, save: bool, prealloc: int = 0, gamma: int = 0
                             ) -> Optional[KVCacheBlocks]:
        """Reserve every block the request's prompt needs before the engine sees the request.
        A loading (decode-side) request must not have its fresh blocks zeroed: the transfer
        may land before the engine would zero them."""
        sched = self._sched()
        n = req.num_tokens + prealloc
        if save:
            n += gamma + 1
        # VLLM_ZERO_HYBRID_KV_CACHE=0 turns the zeroing of fresh blocks off altogether (engine_proxy.py:183-199
        # of the reference: skip_zero_for_kvt_recv or not envs.VLLM_ZERO_HYBRID_KV_CACHE)
        new = sched.kv_cache_manager.allocate_slots(req, n, skip_new_block_zeroing=load or not envs.VLLM_ZERO_HYBRID_KV_CACHE)
        if new is None:
            return None
        req.num_computed_tokens = 0
        req.skip_reading_prefix_cache = True
        return KVCacheBlocks(sched.kv_cache_manager.get_blocks(req.request_id))

    def sched_discard_zero_block_ids(self, block_ids: Iterable[int]) -> None:
        self._sched().kv_cache_manager.discard_new_block_ids(block_ids)

    def sched_cache_blocks(self, req: Request, num_computed_tokens: int) -> None:
        return  # the minimal engine has no prefix cache to publish into

    def sched_get_blocks(self, reqid: str) -> KVCacheBlocks:
        return KVCacheBlocks(self._sched().kv_cache_manager.get_blocks(reqid))

    def sched_free_blocks(self, blks: KVCacheBlocks) -> None:
        pool = self._sched().kv_cache_manager.block_pool
        for grp in blks.blocks:
            pool.free_blocks(reversed(grp))

    @staticmethod
    def sched_acquire_blocks(blks: KVCacheBlocks) -> None:
        for grp in blks.blocks:
            for b in grp:
                if not b.is_null:
                    b.ref_cnt += 1

    def sched_finish_req(self, request_ids) -> None:
        self._sched().finish_requests(request_ids, RequestStatus.FINISHED_ABORTED)

    def sched_get_finished_req_ids(self) -> set:
        return self._sched().finished_req_ids

    def sched_get_req(self, reqid: str) -> Optional[Request]:
        return self._sched().requests.get(reqid)

    def sched_get_kvblk_ids(self, reqid: str) -> list:
        return self._sched().kv_cache_manager.get_block_ids(reqid)

    def sched_add_req(self, req: Request) -> None:
        self._sched().add_request(req)

    # ---- engine core -----------------------------------------------------------------------
    @staticmethod
    def req2corereq(req: Request) -> EngineCoreRequest:
        sp = SamplingParams(max_tokens=req.sampling_params.max_tokens, min_tokens=req.sampling_params.min_tokens,
                            extra_args={"kv_transfer_params": None})
        return EngineCoreRequest(request_id=req.request_id, prompt_token_ids=list(req.prompt_token_ids),
                                 sampling_params=sp, eos_token_id=req.eos_token_id, arrival_time=req.arrival_time,
                                 client_index=req.client_index, trace_headers=req.trace_headers,
                                 queue_server_address=req.queue_server_address)

    def core_abort_req(self, reqid: str, reason: str, output: bool) -> None:
        conn = self._sched().get_kv_connector()
        assert conn is not None
        conn.on_abort_req(reqid, reason, output, iscore=False)

    def core_add_req(self, request: EngineCoreRequest) -> None:
        self.core.input_queue.put_nowait((EngineCoreRequestType.ADD, request))

    def wakeup_core(self) -> None:
        self.core.input_queue.put_nowait((EngineCoreRequestType.WAKEUP, None))


class WorkerProxy:
    """Worker-side seam: which TP rank this is, where its cache lives, its connector loop."""

    def __init__(self, cfg: VllmConfig, tp_rank: int, device: str):
        self.cfg = cfg
        self.tp_rank = tp_rank
        self.device = device
        self.worker_loop = start_asyncio_thread(f"hybridworker{tp_rank}", device)

    def get_hybrid_worker_loop(self):
        return self.worker_loop

    def get_tensor_model_parallel_rank(self) -> int:
        return self.tp_rank

    def get_tensor_model_parallel_world_size(self) -> int:
        return self.cfg.parallel_config.tensor_parallel_size


_g_engine: Optional[EngineProxy] = None
_g_worker: Optional[WorkerProxy] = None


def core_init(core, cfg: VllmConfig) -> EngineProxy:
    global _g_engine
    _g_engine = EngineProxy(core, cfg)
    return _g_engine


def worker_init(cfg: VllmConfig, tp_rank: int, device: str) -> WorkerProxy:
    global _g_worker
    _g_worker = WorkerProxy(cfg, tp_rank, device)
    return _g_worker


def current_engine() -> EngineProxy:
    assert _g_engine is not None, "core_init() has not been called in this process"
    return _g_engine


def current_worker() -> WorkerProxy:
    assert _g_worker is not None, "worker_init() has not been called in this process"
    return _g_worker


# ---- which cache shape does this engine's attention backend use --------------------------------------
def attention_backend() -> str:
    return os.environ.get("VLLM_ATTENTION_BACKEND", "")


def use_mla() -> bool:
    return "mla" in attention_backend().lower()


def use_sparse_mla() -> bool:
    return use_mla() and "sparse" in attention_backend().lower()


def use_flashinfer() -> bool:
    return "flashinfer" in attention_backend().lower()


def use_turboquant(cfg: VllmConfig) -> bool:
    if os.environ.get("VLLM_FLASH_ATTN_USE_FAST_TURBOQUANT") or os.environ.get("VLLM_FLASH_ATTN_USE_FAKE_TURBOQUANT"):
        return True
    dt = cfg.cache_config.cache_dtype
    return bool(dt and "tq" in dt.lower())


def is_kvt_consumer_backend(cfg: VllmConfig) -> bool:
    """A decode engine whose KV arrives by transfer (engine_proxy.py:86-90 of the reference)."""
    kv = cfg.kv_transfer_config
    return kv is not None and kv.kv_role == "kv_consumer" and kv.get_from_extra_config("backend", None) == "kvt"


def is_statemodel(cfg: VllmConfig) -> bool:
    """Whether any cache group of the model holds recurrent state (GDN / KDA layers) rather than attention KV
    (engine_proxy.py:579-592 of the reference walks the KV cache groups' specs)."""
    return cfg.model_config.num_gdn_groups > 0


def use_kvt_decode_prefix_cache(cfg: VllmConfig) -> bool:
    """Prefix reuse on a decode engine that receives KV is only worked out for hybrid models with state
    layers and prefix caching on (engine_proxy.py:93-102 of the reference); ``align_seen_tokens_for_kvt``
    then trims what is reused to whole blocks of every attention group."""
    return bool(getattr(cfg.cache_config, "enable_prefix_caching", False)) and is_statemodel(cfg)


def kvt_protocol() -> str:
    from llumnix_kv_b200 import envs

    return envs.VLLM_KV_TRANS_PROTOCOL


def kvt_cache_shape(cfg: VllmConfig, sm_major: Optional[int] = None) -> int:
    """Cache-shape id of this engine's paged cache, from the attention backend and the GPU
    generation (blade_kvt/hybrid_connector/kvtbackend.py:524-563, engine_proxy.py:477-507):
    FlashInfer keeps HND pages on SM 10.x (shapes 5 / 7 for hybrid models) and NHD on SM 12.x
    (hybrid only, shape 3); sparse MLA registers two tensors per layer (4); TurboQuant is 6; Kimi-K3
    style KDA models are 8; FlashAttention is NHD (2, or 3 for hybrid models)."""
    hybrid = cfg.model_config.is_hybrid
    if use_turboquant(cfg):
        return 6
    if use_sparse_mla():
        return 4
    if cfg.model_config.use_mla and hybrid:
        return 8
    if use_flashinfer():
        if sm_major is None:
            import torch

            sm_major = torch.cuda.get_device_capability()[0] if torch.cuda.is_available() else 10
        if sm_major == 10:
            return 7 if hybrid else 5
        if sm_major == 12:
            if hybrid:
                return 3
            raise ValueError("non-hybrid FlashInfer pages are HND only; SM 12.x keeps NHD")
        raise ValueError(f"the FlashInfer path needs SM 10.x or 12.x, got SM {sm_major}.x")
    return 3 if hybrid else 2


def align_seen_tokens_for_kvt(per_group_hits: list, token_group_block_sizes: list, dcp_world_size: int = 1,
                              replicated: Optional[list] = None) -> int:
    """Prefix a decode engine may reuse before asking a prefill engine for the rest: the shortest
    hit among the token-indexed (attention / indexer) cache groups, rounded down to a common
    multiple of their block sizes; ordinary attention groups are striped over the decode context
    parallel ranks, replicated ones (MLA latent, indexer) are not (engine_proxy.py:105-165).
    Recurrent-state groups are not part of the boundary: their state always travels whole."""
    import math

    if not per_group_hits:
        return 0
    replicated = replicated or [False] * len(per_group_hits)
    sizes = [b if r else b * dcp_world_size for b, r in zip(token_group_block_sizes, replicated)]
    align = math.lcm(*sizes)
    return min(per_group_hits) // align * align
