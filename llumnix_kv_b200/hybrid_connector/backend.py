"""Backend contract of the HybridConnector, RPC heads of the done / abort protocol and the
per-request parameter keys shared by the scheduler half, the worker half and the backends.

A backend is one way of moving KV (PD transfer, KVStore, migration, file demo ...).  It has
a scheduler half (decides per request what to load / save, talks to peers) and a worker half
(touches the cache tensors).  Contract: blade_kvt/hybrid_connector/__init__.py:170-470.
"""
from __future__ import annotations

import dataclasses
from collections.abc import AsyncGenerator
from typing import Optional

import msgspec

from .engine_proxy import (EngineProxy, KVCacheBlocks, KVConnectorMetadata, KVConnectorRole, Request,
                           SchedulerOutput, VllmConfig, WorkerProxy, get_param, set_param)
from .utils import IoRet

# ---- RPC heads (4-byte little-endian, first bytes of every message) --------------------------------
SAVE_DONE_REQ = 0x20181221       # worker -> scheduler: msgpack IoDoneReqs
LOAD_DONE_REQ = 0x20181222
SAVE_DONE2_REQ = 0x20181223      # native engine's send-done body under a save-done head
SAVE_DONE_RESP = 0x91218102
LOAD_DONE_RESP = SAVE_DONE_RESP
GET_BYPASS_HANDLE = 0x20181226
GET_BYPASS_HANDLE_RESP = 0x20181227

# ---- per-request parameter keys --------------------------------------------------------------------
HB_IORET = "_HybridBackend_IORET"
HB_SAVE_IORET = "_HybridBackend_SAVE_IORET"      # save outcome, read by async_cleanup (seal vs discard)
HB_LOAD_SOURCES = "_HybridBackend_LOAD_SOURCES"
HB_SAVE_SOURCES = "_HybridBackend_SAVE_SOURCES"
PREALLOC_KEY = "_hbprealloc"
CLEANUP_RC_KEY = "_HybridBackend_cleanup_rc"
ADD_REQ_LOGGED_KEY = "_hb_add_req_logged"
SAVE_PREPARED = "hbsaveprepared"
ABORTED = "hbreqisaborted"
SAVE_ABORTED = "hbreqsaveaborted"
PD_FINISH_REASON = "_pd_finish_reason"
PD_STOP_REASON = "_pd_stop_reason"
PD_CLIENT_INDEX = "_pd_client_index"
PD_SAVED = "_pd_saved"

OperationPlan = tuple  # (load_count, save_count, load_sources, save_sources)


class BackendMeta:
    """What a backend's scheduler half hands to its worker half for one step.  Falsy = nothing to do."""

    def __bool__(self):
        return False

    def wants_nan_flag(self) -> bool:
        """True when this step stores KV whose validity depends on the forward pass being NaN-free
        (blade_kvt/hybrid_connector/v6d_object_backend.py:78-90)."""
        return False

    def set_nan_flag(self, flag) -> None:
        """The model runner's ``isnan(hidden_states).any()`` tensor of this step."""


@dataclasses.dataclass
class HybridMetadata(KVConnectorMetadata):
    reqs: BackendMeta
    stepid: int = 0       # starts at 1024, +1 per engine step
    substepid: int = 0    # 0 = main step, >= 1 = bypass substeps of that step


@dataclasses.dataclass
class HCSchedOutput(SchedulerOutput):
    """SchedulerOutput plus what the connector decided since the previous step."""

    hc_aborted_load: list = dataclasses.field(default_factory=list)
    hc_aborted_save: list = dataclasses.field(default_factory=list)
    hc_stop0: list = dataclasses.field(default_factory=list)
    hc_parent: Optional[SchedulerOutput] = None
    hc_stepid: int = 0
    hc_substepid: int = 0


@dataclasses.dataclass
class AbortReq:
    reqid: str
    output: bool
    reason: str


class IoDoneReqs(msgspec.Struct, array_like=True, omit_defaults=True, gc=False):
    worker_tprank: int
    reqids: list[IoRet]


def set_operation_sources(req: Request, load_sources: tuple = (), save_sources: tuple = ()) -> None:
    if load_sources:
        set_param(req, HB_LOAD_SOURCES, tuple(load_sources))
    if save_sources:
        set_param(req, HB_SAVE_SOURCES, tuple(save_sources))


def merge_operation_plans(*plans: OperationPlan) -> OperationPlan:
    return (sum(p[0] for p in plans), sum(p[1] for p in plans),
            tuple(s for p in plans for s in p[2]), tuple(s for p in plans for s in p[3]))


def inc_cleanup_rc(req: Request) -> int:
    rc = get_param(req, CLEANUP_RC_KEY, 0) + 1
    set_param(req, CLEANUP_RC_KEY, rc)
    return rc


def dec_cleanup_rc(req: Request) -> int:
    rc = get_param(req, CLEANUP_RC_KEY, 0)
    assert rc > 0
    set_param(req, CLEANUP_RC_KEY, rc - 1)
    return rc - 1


def req_aborted(req: Request) -> bool:
    return bool(get_param(req, ABORTED, False))


def has_setup_save(req: Request) -> bool:
    return bool(get_param(req, SAVE_PREPARED))


class HybridBackend:
    SOURCE_LABEL: Optional[str] = None

    def __init__(self, vllm_config: VllmConfig, role: KVConnectorRole, kv_cache_config=None,
                 engine: Optional[EngineProxy] = None, worker: Optional[WorkerProxy] = None, connector=None):
        self._vllm_config = vllm_config
        self._role = role
        self._kv_cache_config = kv_cache_config
        self._engine = engine      # scheduler role
        self._worker = worker      # worker role
        self._connector = connector  # the HybridScheduler / HybridWorker that owns this backend
        self.is_hybrid = vllm_config.model_config.is_hybrid
        self._enable_prefix_caching = vllm_config.cache_config.enable_prefix_caching
        self.hybrid_model_send_layer: list = []
        self._num_gdn_layers = 0
        self._num_ple_layers = 0
        self._ple_group_index: Optional[int] = None
        self._has_indexer_cache = False
        self._num_kv_cache_groups = 0
        self._group_types: list = []
        if kv_cache_config is not None and self.is_hybrid:
            self._parse_kv_cache_config(kv_cache_config)

    def _parse_kv_cache_config(self, kv_cache_config) -> None:
        """Hybrid models order their block groups [gdn ... gdn, indexer?, attn, ple?]; the order is
        what the native planner relies on, so it is validated here."""
        groups = kv_cache_config.kv_cache_groups or []
        self._num_kv_cache_groups = len(groups)
        self._group_types = []
        for grp in groups:
            names = grp.layer_names
            if any("linear_attn" in n for n in names):
                self._group_types.append("gdn")
            elif any("indexer" in n for n in names):
                self._group_types.append("indexer")
            elif any(".ple" in n for n in names):
                self._group_types.append("ple")
            else:
                self._group_types.append("attn")
        t = self._group_types
        self._num_gdn_layers = t.count("gdn")
        self._num_ple_layers = t.count("ple")
        self._ple_group_index = t.index("ple") if self._num_ple_layers else None
        self._has_indexer_cache = "indexer" in t
        n = self._num_gdn_layers
        expect = ["gdn"] * n + (["indexer"] if self._has_indexer_cache else []) + ["attn"] + \
                 (["ple"] if self._num_ple_layers else [])
        assert t == expect, f"KV cache groups must be ordered [gdn.., indexer?, attn, ple?]; got {t}"

    def get_request(self, request_id: str) -> Optional[Request]:
        assert self._engine is not None
        return self._engine.sched_get_req(request_id)

    # ---- worker side (worker thread unless noted) ----------------------------------------------
    def register_kv_caches(self, kv_caches: dict) -> None:
        return

    def bind_backend_metadata(self, meta: BackendMeta) -> None:
        return

    def clear_backend_metadata(self) -> None:
        return

    def bypass_bind(self, meta: BackendMeta) -> None:     # bypass loop thread
        self.bind_backend_metadata(meta)

    def bypass_clear(self) -> None:
        self.clear_backend_metadata()

    # Set to None in subclasses that never load (the worker then skips the call entirely).
    async def async_load_kv(self, m: BackendMeta) -> AsyncGenerator:
        raise NotImplementedError()
        yield IoRet()  # pragma: no cover

    def async_save_kv_layer(self, layer_name: str, kv_layer, m: BackendMeta) -> Optional[AsyncGenerator]:
        return None

    def source_label(self) -> str:
        assert self.SOURCE_LABEL is not None, f"{type(self).__name__} must declare SOURCE_LABEL"
        return self.SOURCE_LABEL

    def save_done_source(self) -> Optional[str]:
        return self.source_label()

    # ---- scheduler side ---------------------------------------------------------------------
    # disagg thread.  Returns how many tokens [num_computed, num_computed + n) this backend will load.
    async def async_get_num_new_matched_tokens(self, req: Request, num_computed_tokens: int) -> int:
        return 0

    async def async_update_state_after_alloc(self, request: Request, blocks: KVCacheBlocks,
                                             num_external_tokens: int) -> Optional[IoRet]:
        return None

    async def async_cleanup(self, req: Request) -> None:
        return

    # core thread
    def on_queued_req_aborted(self, req: Request) -> None:
        """The scheduler dropped a request that was still queued in the connector: no block was allocated, no load
        or save was set up, so none of the abort paths that go through those will ever run for it.  A backend that
        holds something on the request's behalf from before (a peer waiting for an answer) settles it here.
        Composites pass the call on to their parts."""
        for part in vars(self).values():
            if isinstance(part, HybridBackend):
                part.on_queued_req_aborted(req)

    # core thread.  (load_count, save_count, load_sources, save_sources)
    def get_operations(self, req: Request) -> OperationPlan:
        return 0, 0, (), ()

    # core thread
    def build_backend_meta(self, sout: SchedulerOutput) -> BackendMeta:
        return BackendMeta()


def get_backend_cls(cfg: VllmConfig) -> type:
    """Backend selection table (blade_kvt/hybrid_connector/__init__.py:599-678)."""
    assert cfg.kv_transfer_config is not None, "kv_transfer_config must be set for HybridConnector"
    kcfg = cfg.kv_transfer_config
    backend = kcfg.get_from_extra_config("backend", None)
    assert backend is not None, "kv_connector_extra_config['backend'] must be set"
    if backend == "migration":
        from .migration.backend import MigrationBackend
        return MigrationBackend
    if backend in ("kvt+migration", "migration+kvt"):
        from .migration.kvtmigration import KVTMigration
        return KVTMigration
    if backend in ("kvt+kvs", "kvs+kvt"):
        from .kvsp import KVSP
        return KVSP
    if backend == "local_file":
        from .file_backend import FileBackend
        return FileBackend
    if backend == "kvt":
        if kcfg.kv_role == "kv_both":
            from .filekvtbackend import FilePBackend
            return FilePBackend
        if kcfg.is_kv_consumer:
            from .kvtbackend import DBackend
            return DBackend
        if kcfg.is_kv_producer:
            from .kvtbackend import PBackend
            return PBackend
        raise ValueError("kv_role must be kv_producer or kv_consumer for the 'kvt' backend")
    if backend in ("kvs", "mooncake", "v6d_object"):
        assert kcfg.kv_role == "kv_both", f"kv_role must be 'kv_both' for the {backend} backend"
        from .kvs_flavours import flavour_class
        # "kvs" is the Vineyard-style adapter unless kvs_backend names another flavour (kvsbackend.py:158 of the reference)
        return flavour_class(kcfg.get_from_extra_config("kvs_backend", backend) if backend == "kvs" else backend)
    if backend in ("v6d_object+kvt", "kvt+v6d_object"):
        if not kcfg.is_kv_producer:
            raise ValueError("the KVT half of this composite is producer-only: kv_role must be kv_producer or kv_both")
        from .kvsp import V6dObjectKVTBackend
        return V6dObjectKVTBackend
    raise ValueError(f"Unknown backend: {backend}")
