"""Scheduler half of the HybridConnector: the request lifecycle around asynchronous KV loads
and saves.

Two threads touch it.  The engine's *core thread* calls ``on_add_req`` / ``step`` /
``build_connector_meta`` / ``on_abort_req``; the connector's *disagg thread* (an asyncio loop)
runs RPC handlers and backend coroutines.  Hand-off between them is through deques (append and
popleft are atomic in CPython) plus ``wakeup_core``.

Lifecycle (blade_kvt/hybrid_connector/__init__.py:699-1538):
  on_add_req      ask the backend what to load / save; park the request in ``_waiting``
  _step_waiting   reserve blocks; for a save take an extra reference on them so they outlive the
                  request until the save completes; for a load start the backend coroutine
  _step_loaded    fold the loaded token count into the request, hand it to the engine scheduler,
                  or abort it if the load failed
  _step_saved     emit ``kv_transfer_done`` (or remember that the save finished first) and drop
                  the extra block references
  _step_aborting  classify an abort by where the request currently is
"""
from __future__ import annotations

import asyncio
import json
import logging
import struct
import time
from collections import Counter, defaultdict, deque
from dataclasses import dataclass, field
from typing import Any, Optional

import msgspec

from .backend import (ABORTED, ADD_REQ_LOGGED_KEY, HB_IORET, HB_LOAD_SOURCES, HB_SAVE_IORET, HB_SAVE_SOURCES,
                      LOAD_DONE_REQ, LOAD_DONE_RESP, PD_CLIENT_INDEX, PD_FINISH_REASON, PD_SAVED, PD_STOP_REASON,
                      PREALLOC_KEY, SAVE_ABORTED, SAVE_DONE2_REQ, SAVE_DONE_REQ, SAVE_DONE_RESP, SAVE_PREPARED,
                      GET_BYPASS_HANDLE, GET_BYPASS_HANDLE_RESP, AbortReq, BackendMeta, HCSchedOutput, HybridMetadata,
                      IoDoneReqs, dec_cleanup_rc, get_backend_cls, has_setup_save, inc_cleanup_rc, req_aborted,
                      set_operation_sources)
from .engine_proxy import (EngineCoreOutput, EngineProxy, FinishReason, KVCacheBlocks, Request, SchedulerOutput,
                           VllmConfig, get_p_node_pop_len, get_param, set_param)
from .utils import IoRet, IoState, handle_done_req, kill_me_if_exception, try_advance

logger = logging.getLogger("llumnix_kv_b200.hybrid_connector")

FAKE_REQID = "__FAKE_REQID_FOR_HYBRID_CONNECTOR__"
_ALREADY_ABORTED = object()      # an abort that found its request aborted before: no second answer


@dataclass
class HybridConnectorStats:
    kv_cache_usage: float
    pre_scheduler_load_kv_cache_usage: float
    post_scheduler_save_kv_cache_usage: float
    saving_status: str
    loading_status: str
    saving_ready_to_teardown_count: int
    load_done_count: int
    load_failed_count: int
    load_latency_ms_sum: float
    load_latency_ms_max: float
    save_done_count: int
    save_failed_count: int
    save_latency_ms_sum: float
    save_latency_ms_max: float
    save_done_count_by_source: dict = field(default_factory=dict)
    save_failed_count_by_source: dict = field(default_factory=dict)
    save_latency_ms_sum_by_source: dict = field(default_factory=dict)
    save_latency_ms_max_by_source: dict = field(default_factory=dict)


class _LoadingReq(IoState):
    def __init__(self, req: Request):
        super().__init__()
        self._req = req
        self.start_time = time.monotonic()


class _SavingReq(IoState):
    def __init__(self, req: Request, kvblks: KVCacheBlocks, save_count: int = 1, expected_sources: tuple = ()):
        super().__init__(signals_per_worker=save_count)
        self.expected_sources = expected_sources
        self._req = req
        self.kvblks = kvblks
        self.start_time = time.monotonic()
        self.source_done_times: dict = {}
        self.source_failed: dict = {}


def _put_abort_resp(out: dict, req: Request) -> None:
    out[req.client_index].append(EngineCoreOutput(
        request_id=req.request_id, new_token_ids=[req.eos_token_id or 0], finish_reason=FinishReason.ABORT,
        queue_server_address=req.queue_server_address))


def combine_outputs(*outs: Optional[dict]) -> Optional[dict]:
    merged: dict = {}
    for o in outs:
        if not o:
            continue
        for k, v in o.items():
            if v:
                merged.setdefault(k, []).extend(v)
    return merged or None


class HybridScheduler:
    def __init__(self, vllm_config: VllmConfig, kv_cache_config, engine: EngineProxy):
        self._cfg = vllm_config
        self._kv_cache_config = kv_cache_config
        self._engine = engine
        self.loop: asyncio.AbstractEventLoop = engine.get_hybrid_sched_loop()
        self._packenc = msgspec.msgpack.Encoder()
        self._iodonedec = msgspec.msgpack.Decoder(IoDoneReqs)
        # ---- shared by core and disagg threads (deques only) ----
        self._waiting: deque = deque()      # (req, load_count, save_count)
        self._loaded: deque = deque()       # Request
        self._saved: deque = deque()        # reqid
        self._prepared: deque = deque()     # reqid (a step is wanted)
        self._aborting: deque = deque()     # AbortReq
        # ---- core thread only ----
        self._abortmeta_load: list = []
        self._abortmeta_save: list = []
        self._stop0: list = []
        self._stepid = 1024
        self._substepid = 1
        # ---- written by the core thread, read by the disagg thread ----
        self._saving: dict[str, _SavingReq] = {}
        self._loading: dict[str, _LoadingReq] = {}
        self._extra_kv_block_ids: dict = {}
        self._extra_kv_block_refcounts: Counter = Counter()
        self._extra_kv_block_refcounts_by_kind: dict = defaultdict(Counter)
        self._reset_lifecycle_stats()
        self._reqs_ts: dict = {}
        self.bypass_remote_subscribe_addr: Optional[str] = None
        self._bypass_socket = None
        self._start_rpc_server()
        BackendCls = get_backend_cls(vllm_config)
        self._backend = BackendCls(vllm_config, _scheduler_role(), kv_cache_config, engine=engine, connector=self)

    # ---- rpc -----------------------------------------------------------------------------------
    def _start_rpc_server(self) -> None:
        from llumnix_kv_b200 import envs

        if envs.VLLM_ENABLE_BYPASS_TASK:
            self._start_bypass_publisher()
        srv = self._engine.sched_rpc_server()
        srv.register_method(SAVE_DONE_REQ, self._on_save_done)
        srv.register_method(SAVE_DONE2_REQ, self._on_save_done2)
        srv.register_method(LOAD_DONE_REQ, self._on_load_done)
        srv.register_method(GET_BYPASS_HANDLE, self._get_bypass_handle)

    def _start_bypass_publisher(self) -> None:
        """XPUB socket over which step metadata produced between engine steps reaches the workers."""
        import zmq
        import zmq.asyncio

        # the context is kept: one that is only reachable through its socket is torn down by the garbage
        # collector, and a teardown waits for unsent messages unless the socket says not to (LINGER 0)
        self._bypass_ctx = zmq.asyncio.Context()
        self._bypass_socket = self._bypass_ctx.socket(zmq.XPUB)
        self._bypass_socket.setsockopt(zmq.LINGER, 0)
        self._bypass_socket.setsockopt(zmq.XPUB_VERBOSE, True)
        port = self._bypass_socket.bind_to_random_port("tcp://127.0.0.1")
        self.bypass_remote_subscribe_addr = f"tcp://127.0.0.1:{port}"
        logger.info("bypass server socket started at: %s", self.bypass_remote_subscribe_addr)

    def close_bypass(self) -> None:
        """Engine shutdown: closes the publisher on its own loop; unsent metadata is dropped."""
        sock, self._bypass_socket = self._bypass_socket, None
        if sock is None:
            return

        async def _close():
            sock.close(linger=0)

        try:
            asyncio.run_coroutine_threadsafe(_close(), self.loop).result(5)
        except Exception:       # the loop is gone already: the socket dies with the process
            logger.debug("bypass publisher not closed cleanly", exc_info=True)

    @kill_me_if_exception
    async def _send_bypass_task(self, meta: HybridMetadata):
        import pickle

        sock = self._bypass_socket
        if sock is not None:
            await sock.send(pickle.dumps(meta))

    def send_bypass_task(self, meta: HybridMetadata) -> None:
        if meta.reqs and self._bypass_socket is not None:
            asyncio.run_coroutine_threadsafe(self._send_bypass_task(meta), self.loop)

    async def _get_bypass_handle(self, reader, writer):
        body = self._packenc.encode(self.bypass_remote_subscribe_addr or "")
        writer.write(struct.pack("=II", GET_BYPASS_HANDLE_RESP, len(body)) + body)
        await writer.drain()

    # ---- small helpers -------------------------------------------------------------------------
    def _tp_size(self) -> int:
        return self._cfg.parallel_config.tensor_parallel_size

    @property
    def pending_requests(self) -> list:
        """Requests the connector holds that the engine scheduler cannot see yet."""
        reqs = [r for r, _, _ in self._waiting]
        reqs.extend(s._req for s in self._loading.values())
        return reqs

    def _add_ts(self, req: Request, tag: str) -> None:
        cid = get_param(req, "correlation_id")
        if cid is None:
            return
        if tag == "on_add_req":
            self._reqs_ts[cid] = {}
        ts = self._reqs_ts.get(cid)
        if ts is None:
            return
        ts[tag] = time.monotonic() * 1000
        if tag == "done":
            keys = list(ts)
            intervals = {f"{a} -> {b}": ts[b] - ts[a] for a, b in zip(keys, keys[1:])}
            logger.info("HybridScheduler time stats: correlation_id=%s, num_prompt_tokens=%s, "
                        "num_computed_tokens=%s, num_external_computed_tokens=%s, intervals=%s", cid,
                        req.num_prompt_tokens, req.num_computed_tokens, req.num_external_computed_tokens, intervals)
            self._reqs_ts.pop(cid, None)

    @staticmethod
    def _kv_block_ids(kvblks: KVCacheBlocks) -> set:
        return {b.block_id for grp in kvblks.blocks for b in grp if not b.is_null}

    def _track_extra_kv_blocks(self, kind: str, reqid: str, kvblks: KVCacheBlocks) -> None:
        self._untrack_extra_kv_blocks(kind, reqid)
        ids = self._kv_block_ids(kvblks)
        if not ids:
            return
        self._extra_kv_block_ids[(kind, reqid)] = ids
        self._extra_kv_block_refcounts.update(ids)
        self._extra_kv_block_refcounts_by_kind[kind].update(ids)

    def _untrack_extra_kv_blocks(self, kind: str, reqid: str) -> None:
        ids = self._extra_kv_block_ids.pop((kind, reqid), None)
        if not ids:
            return
        for counts in (self._extra_kv_block_refcounts, self._extra_kv_block_refcounts_by_kind[kind]):
            for b in ids:
                counts[b] -= 1
                if counts[b] <= 0:
                    del counts[b]

    # ---- stats ---------------------------------------------------------------------------------
    def _reset_lifecycle_stats(self) -> None:
        self._lc = dict(load_done=0, load_failed=0, load_ms_sum=0.0, load_ms_max=0.0, save_done=0, save_failed=0,
                        save_ms_sum=0.0, save_ms_max=0.0)
        self._lc_src_done: dict = defaultdict(int)
        self._lc_src_failed: dict = defaultdict(int)
        self._lc_src_ms_sum: dict = defaultdict(float)
        self._lc_src_ms_max: dict = defaultdict(float)

    def _record_lifecycle_done(self, kind: str, start_time: float, failed: bool) -> None:
        ms = max(0.0, (time.monotonic() - start_time) * 1000)
        assert kind in ("load", "save")
        self._lc[f"{kind}_done"] += 1
        self._lc[f"{kind}_ms_sum"] += ms
        self._lc[f"{kind}_ms_max"] = max(self._lc[f"{kind}_ms_max"], ms)
        if failed:
            self._lc[f"{kind}_failed"] += 1

    def get_hybrid_connector_stats(self, num_gpu_blocks: int) -> HybridConnectorStats:
        total = num_gpu_blocks - 1

        def usage(counter) -> float:
            return len(counter) / total if total > 0 and counter is not None else 0.0

        saving_status, ready = self._saving_req_status()
        lc = self._lc
        stats = HybridConnectorStats(
            kv_cache_usage=usage(self._extra_kv_block_refcounts),
            pre_scheduler_load_kv_cache_usage=usage(self._extra_kv_block_refcounts_by_kind.get("load")),
            post_scheduler_save_kv_cache_usage=usage(self._extra_kv_block_refcounts_by_kind.get("save")),
            saving_status=saving_status, loading_status=self._loading_req_status(),
            saving_ready_to_teardown_count=ready, load_done_count=lc["load_done"],
            load_failed_count=lc["load_failed"], load_latency_ms_sum=lc["load_ms_sum"],
            load_latency_ms_max=lc["load_ms_max"], save_done_count=lc["save_done"],
            save_failed_count=lc["save_failed"], save_latency_ms_sum=lc["save_ms_sum"],
            save_latency_ms_max=lc["save_ms_max"], save_done_count_by_source=dict(self._lc_src_done),
            save_failed_count_by_source=dict(self._lc_src_failed),
            save_latency_ms_sum_by_source=dict(self._lc_src_ms_sum),
            save_latency_ms_max_by_source=dict(self._lc_src_ms_max))
        self._reset_lifecycle_stats()
        return stats

    def mark_post_scheduler_save_extra(self, reqid: str) -> None:
        state = self._saving.get(reqid)
        if state is not None:
            self._track_extra_kv_blocks("save", reqid, state.kvblks)

    def _mark_save_source_done_time(self, state: _SavingReq, ioret: IoRet) -> None:
        """Runs under the ledger's lock after each accepted signal: stamps a backend's save as done
        once every rank has reported it."""
        src = ioret.source
        if src is None or src in state.source_done_times or state.ranks_reporting(src) < self._tp_size():
            return
        state.source_done_times[src] = time.monotonic()
        state.source_failed[src] = state.source_moved_nothing(src)

    def _saving_req_status(self) -> tuple:
        counts: dict = defaultdict(int)
        ready = 0
        for state in tuple(self._saving.values()):
            sources = tuple(get_param(state._req, HB_SAVE_SOURCES, ()))
            with state.lock:
                if sources:
                    pending = tuple(s for s in sources if state.ranks_reporting(s) < self._tp_size())
                    if not pending:
                        ready += 1
                        continue
                    label = "+".join(pending)
                else:
                    label = "unknown"
            counts[label] += 1
        return json.dumps(dict(sorted(counts.items()))), ready

    def _loading_req_status(self) -> str:
        counts: dict = defaultdict(int)
        for state in tuple(self._loading.values()):
            counts["+".join(get_param(state._req, HB_LOAD_SOURCES, ()) or ("unknown",))] += 1
        return json.dumps(dict(sorted(counts.items())))

    # ---- core thread: step ---------------------------------------------------------------------
    def step(self) -> Optional[dict]:
        kvt_done = self._step_saved()
        self._step_waiting()
        self._step_loaded()
        return combine_outputs(kvt_done, self._step_aborting())

    def _step_saved(self) -> dict:
        kvt_done: dict = {}
        while self._saved:
            reqid = self._saved.popleft()
            state = self._saving.get(reqid)
            if state is not None:
                req = state._req
                save_ioret: Optional[IoRet] = get_param(req, HB_SAVE_IORET, None)
                save_failed = save_ioret is not None and save_ioret.n is not None and save_ioret.n == 0
                self._record_lifecycle_done("save", state.start_time, save_failed or req_aborted(req))
                with state.lock:
                    done_times, failed = dict(state.source_done_times), dict(state.source_failed)
                for src, t_done in done_times.items():
                    ms = max(0.0, (t_done - state.start_time) * 1000)
                    self._lc_src_done[src] += 1
                    self._lc_src_ms_sum[src] += ms
                    self._lc_src_ms_max[src] = max(self._lc_src_ms_max[src], ms)
                    if failed.get(src, False) or req_aborted(req):
                        self._lc_src_failed[src] += 1
                finish_reason = get_param(req, PD_FINISH_REASON)
                if finish_reason is not None:
                    # the request finished before its save did: announce the transfer now
                    kvt_done.setdefault(get_param(req, PD_CLIENT_INDEX), []).append(EngineCoreOutput(
                        request_id=reqid, new_token_ids=[], finish_reason=finish_reason,
                        stop_reason=get_param(req, PD_STOP_REASON), num_cached_tokens=max(req.num_cached_tokens, 0),
                        kv_transfer_params={"kv_transfer_done": True}))
                else:
                    # the save finished first: request_finished_all_groups will announce it
                    set_param(req, PD_SAVED, True)
            self._release_save(reqid)
        return kvt_done

    def _setup_save(self, req: Request, kvblks: KVCacheBlocks, save_count: int = 1) -> None:
        assert not has_setup_save(req)
        inc_cleanup_rc(req)
        assert req.request_id not in self._saving
        sources = tuple(get_param(req, HB_SAVE_SOURCES, ()))
        assert sources, f"missing save sources for reqid={req.request_id}"
        assert len(sources) == save_count, f"save sources {sources} vs save_count {save_count}"
        self._saving[req.request_id] = _SavingReq(req, kvblks, save_count, sources)
        self._engine.sched_acquire_blocks(kvblks)   # the blocks now outlive the request
        set_param(req, SAVE_PREPARED, True)

    def _release_save(self, reqid: str) -> None:
        """Undoes _setup_save once the save has ended and the request has finished: the blocks go back
        to the engine.  Idempotent: whichever of the two events comes second finds nothing left."""
        state = self._saving.pop(reqid, None)
        if state is None:
            logger.info("save of %s was already released", reqid)
            return
        assert has_setup_save(state._req)
        set_param(state._req, SAVE_PREPARED, False)
        self._untrack_extra_kv_blocks("save", reqid)
        self._engine.sched_free_blocks(state.kvblks)

    async def _cleanup(self, req: Request) -> None:
        if dec_cleanup_rc(req) <= 0:
            await self._backend.async_cleanup(req)

    def _step_waiting(self) -> None:
        gamma = get_p_node_pop_len(self._cfg) - 1
        while self._waiting:
            req, load_count, save_count = self._waiting[0]
            prealloc = get_param(req, PREALLOC_KEY, 0)
            kvblks = self._engine.sched_allocate_slots(req, load_count > 0, save_count > 0, prealloc, gamma)
            if kvblks is not None or not get_param(req, ADD_REQ_LOGGED_KEY, False):
                logger.info("add req. reqid=%s promptlen=%s computed=%s maxcomputed=%s load=%s save=%s nokvblks=%s",
                            req.request_id, req.num_prompt_tokens, req.num_computed_tokens, req.max_computed_tokens(),
                            load_count, save_count, kvblks is None)
                set_param(req, ADD_REQ_LOGGED_KEY, True)
            if kvblks is None:
                break  # out of blocks: retry next step, keep FIFO order
            self._waiting.popleft()
            if save_count > 0:
                self._setup_save(req, kvblks, save_count)
            if load_count > 0:
                inc_cleanup_rc(req)
                assert req.request_id not in self._loading
                self._loading[req.request_id] = _LoadingReq(req)
                self._track_extra_kv_blocks("load", req.request_id, kvblks)
                self._add_ts(req, "load_enqueue")
                asyncio.run_coroutine_threadsafe(self._resolve_load(req, kvblks), self.loop)
            else:
                self._loaded.append(req)   # nothing to load: visible to the engine right away

    def _step_loaded(self) -> None:
        while self._loaded:
            req: Request = self._loaded.popleft()
            ioret: Optional[IoRet] = get_param(req, HB_IORET, None)
            if ioret is None:
                ioret = IoRet(ex=None, n=0)
            load_state = self._loading.pop(req.request_id, None)
            loaded = ioret.n or 0
            req.num_computed_tokens += loaded
            req.num_external_computed_tokens += loaded
            max_computed = req.max_computed_tokens()
            # stop0: the load already reached the boundary up to which this engine would compute
            will_stop0 = False
            if max_computed is not None:
                assert max_computed < req.num_prompt_tokens
                will_stop0 = max_computed <= req.num_computed_tokens
            if (load_state is not None and ioret.ex is None and not req_aborted(req) and loaded > 0
                    and self._cfg.cache_config.enable_prefix_caching and will_stop0):
                self._engine.sched_cache_blocks(req, req.num_computed_tokens)
            if will_stop0:
                req.set_max_computed_tokens(req.num_computed_tokens)
                self._stop0.append(req)
            load_failed = ioret.ex is not None or req_aborted(req)
            if load_state is not None:
                self._record_lifecycle_done("load", load_state.start_time, load_failed)
            self._untrack_extra_kv_blocks("load", req.request_id)
            self._engine.sched_add_req(req)
            self._add_ts(req, "done")
            if load_failed:
                # a load that the other side declined leaves the request alive where it was: no word to the client
                declined = getattr(ioret.ex, "silent", False)
                self.on_abort_req(AbortReq(req.request_id, output=not req_aborted(req) and not declined, reason="load fail"),
                                  iscore=True)

    def on_add_req(self, req: Request) -> bool:
        load_count, save_count, load_sources, save_sources = self._backend.get_operations(req)
        set_operation_sources(req, load_sources, save_sources)
        req.trace_wrapper.on_req_kv_start("load")
        req.trace_wrapper.on_req_kv_start("save")
        if load_count > 0 or save_count > 0:
            self._add_ts(req, "on_add_req")
            self._waiting.append((req, load_count, save_count))
            return True
        return False

    def _step_aborting(self) -> Optional[dict]:
        """Serves the queued aborts.  Where a request is decides what an abort means: still queued
        here (never reached the engine), loading (the backend must be told, the engine does not know
        it yet), known to the engine (finish it there), and - independently - saving."""
        replies: dict = defaultdict(list)
        while self._aborting:
            areq: AbortReq = self._aborting.popleft()
            victim = self._abort_queued(areq)
            if victim is None:
                victim = self._abort_loading(areq)
            if victim is None:
                victim = self._abort_in_engine(areq)
                self._abort_saving(areq)
            if victim is not None and victim is not _ALREADY_ABORTED and areq.output:
                _put_abort_resp(replies, victim)
        return replies

    def _abort_queued(self, areq: AbortReq) -> Optional[Request]:
        pos = next((i for i, entry in enumerate(self._waiting) if entry[0].request_id == areq.reqid), None)
        if pos is None:
            return None
        req = self._waiting[pos][0]
        del self._waiting[pos]
        logger.info("abort of a queued request: %s", areq)
        self._backend.on_queued_req_aborted(req)
        # the engine frees what it knows: hand the request over and finish it at once
        self._engine.sched_add_req(req)
        self._engine.sched_finish_req(areq.reqid)
        return req

    def _abort_loading(self, areq: AbortReq):
        state = self._loading.get(areq.reqid)
        if state is None:
            return None
        req = state._req
        if get_param(req, ABORTED, False):
            return _ALREADY_ABORTED      # the backend has been told; nothing is answered twice
        logger.info("abort of a loading request: %s", areq)
        assert self._engine.sched_get_req(areq.reqid) is None
        set_param(req, ABORTED, True)
        self._abortmeta_load.append(req)
        return req

    def _abort_in_engine(self, areq: AbortReq) -> Optional[Request]:
        req = self._engine.sched_get_req(areq.reqid)
        if req is None:
            return None
        logger.info("abort of a scheduled request: %s status=%s tokens=%s", areq, req.status, req.num_tokens)
        self._engine.sched_finish_req(areq.reqid)
        if req in self._stop0:
            self._stop0.remove(req)
        return req

    def _abort_saving(self, areq: AbortReq) -> None:
        state = self._saving.get(areq.reqid)
        if state is None or get_param(state._req, SAVE_ABORTED, False):
            return
        logger.info("abort of a saving request: %s", areq)
        assert has_setup_save(state._req)
        set_param(state._req, SAVE_ABORTED, True)
        self._abortmeta_save.append(state._req)

    # thread safe
    def on_abort_req(self, areq: AbortReq, iscore: bool) -> None:
        if iscore:
            self._aborting.append(areq)
        else:
            self._q_append(self._aborting, areq)

    # ---- disagg thread ---------------------------------------------------------------------------
    def _q_append(self, q: deque, item: Any) -> None:
        q.append(item)
        if len(q) == 1:
            self._engine.wakeup_core()

    @kill_me_if_exception
    async def _resolve_load(self, req: Request, kvblks: KVCacheBlocks):
        """Asks the backend how many tokens it can bring and binds them to the allocated blocks.
        Three outcomes: nothing to bring, or the backend finished (or failed) on the spot - the
        request is loaded now; otherwise the workers will report, and a step must run to hand them
        the metadata."""
        promised = await self._backend.async_get_num_new_matched_tokens(req, req.num_computed_tokens)
        outcome = await self._backend.async_update_state_after_alloc(req, kvblks, promised)
        self._add_ts(req, "after_alloc")
        if outcome is None and promised > 0:
            set_param(req, "_hb_promised_tokens", promised)
            self._q_append(self._prepared, req.request_id)
            return
        if outcome is not None and outcome.n is None:
            outcome.n = promised      # an immediate answer without a count covers the whole promise
        await self.mark_loaded(req, outcome)

    async def mark_loaded(self, req: Request, ioret: Optional[IoRet] = None) -> None:
        set_param(req, HB_IORET, ioret)
        self._q_append(self._loaded, req)
        self._add_ts(req, "mark_loaded")
        await self._cleanup(req)

    async def _do_save_done(self, worker_tprank: int, ioret: IoRet) -> None:
        state: Optional[_SavingReq] = try_advance(self._saving, ioret, worker_tprank, self._tp_size(),
                                                  on_signal_advanced=self._mark_save_source_done_time)
        if state is None:
            return
        with state.lock:
            failed = any(state.source_failed.values())
        if failed:
            set_param(state._req, HB_SAVE_IORET, IoRet(n=0))
        logger.info("mark saved. reqid=%s", ioret.reqid)
        state._req.trace_wrapper.on_req_kv_end("save")
        self._q_append(self._saved, ioret.reqid)
        await self._cleanup(state._req)

    async def _do_save_done2(self, worker_tprank: int, ioret: IoRet) -> None:
        if ioret.source is None:
            ioret.source = "kvt"   # the native engine's message carries no source
        await self._do_save_done(worker_tprank, ioret)

    async def _on_save_done2(self, reader, writer):
        await handle_done_req(reader, writer, self._do_save_done2, SAVE_DONE_RESP)

    async def _read_iodone(self, reader) -> IoDoneReqs:
        (n,) = struct.unpack("=I", await reader.readexactly(4))
        reqs = self._iodonedec.decode(await reader.readexactly(n))
        for r in reqs.reqids:
            if r.ex is not None and not isinstance(r.ex, BaseException):
                r.ex = RuntimeError(f"worker {reqs.worker_tprank}: {r.ex}")      # a worker's failure travels as text
        return reqs

    async def _on_save_done(self, reader, writer):
        reqs = await self._read_iodone(reader)
        writer.write(struct.pack("=I", SAVE_DONE_RESP))
        await asyncio.gather(*(self._do_save_done(reqs.worker_tprank, r) for r in reqs.reqids))
        await writer.drain()

    async def _do_load_done(self, worker_tprank: int, ioret: IoRet) -> None:
        state: Optional[_LoadingReq] = try_advance(self._loading, ioret, worker_tprank, self._tp_size())
        if state is None:
            return
        merged = state.merge()
        if merged.n is None and merged.ex is None:
            # a worker that reports no count loaded everything the backend promised
            merged.n = get_param(state._req, "_hb_promised_tokens", 0)
        logger.info("mark loaded. reqid=%s ioret=%s", state._req.request_id, merged)
        state._req.trace_wrapper.on_req_kv_end("load")
        self._add_ts(state._req, "load_done")
        await self.mark_loaded(state._req, merged)

    async def _on_load_done(self, reader, writer):
        reqs = await self._read_iodone(reader)
        writer.write(struct.pack("=I", LOAD_DONE_RESP))
        await asyncio.gather(*(self._do_load_done(reqs.worker_tprank, r) for r in reqs.reqids))
        await writer.drain()

    # ---- core thread: connector API ------------------------------------------------------------
    def get_num_new_matched_tokens(self, request: Request, num_computed_tokens: int) -> tuple:
        return 0, False   # loads happen before the engine sees the request, never through this hook

    def update_state_after_alloc(self, request: Request, blocks: KVCacheBlocks, num_external_tokens: int, **kw):
        assert num_external_tokens == 0

    def build_connector_meta(self, sout: SchedulerOutput) -> HybridMetadata:
        self._prepared.clear()
        data = dict(sout.__dict__)
        hc_parent: Optional[SchedulerOutput] = data.get("hc_parent")
        if hc_parent is None:
            stepid, substepid = self._stepid, 0
            self._stepid += 1
            self._substepid = 1
        else:
            # a bypass substep rides on its parent step's id
            if hc_parent.kv_connector_metadata is None:
                hc_parent.kv_connector_metadata = HybridMetadata(reqs=BackendMeta(), stepid=self._stepid, substepid=0)
                self._stepid += 1
                self._substepid = 1
            parent_meta = hc_parent.kv_connector_metadata
            assert isinstance(parent_meta, HybridMetadata)
            stepid, substepid = parent_meta.stepid, self._substepid
            self._substepid += 1
        data.update(hc_aborted_load=self._abortmeta_load, hc_aborted_save=self._abortmeta_save,
                    hc_stop0=self._stop0, hc_parent=hc_parent, hc_stepid=stepid, hc_substepid=substepid)
        hcsout = HCSchedOutput(**data)
        self._abortmeta_load, self._abortmeta_save, self._stop0 = [], [], []
        reqs = self._backend.build_backend_meta(hcsout)
        return HybridMetadata(reqs=reqs, stepid=stepid, substepid=substepid)

    def has_requests(self) -> bool:
        return bool(self._waiting or self._loaded or self._saved or self._aborting or self._abortmeta_load
                    or self._abortmeta_save or self._stop0 or self._prepared)

    def wakeup_scheduler(self) -> None:
        """Make sure the engine runs a step (and with it build_connector_meta) soon."""
        self._q_append(self._prepared, FAKE_REQID)

    # ---- helpers used by backends (core thread) --------------------------------------------------
    def try_setup_save(self, req: Request, source: str) -> bool:
        if has_setup_save(req):
            return False
        set_operation_sources(req, save_sources=(source,))
        self._setup_save(req, self._engine.sched_get_blocks(req.request_id))
        return True

    def mark_backend_save_done(self, req: Request, source: str) -> None:
        """A backend declares the save of ``req`` finished on every rank (nothing was sent, or it
        was aborted) so that the extra block references unwind."""
        assert source is not None
        for rank in range(self._tp_size()):
            asyncio.run_coroutine_threadsafe(self._do_save_done(rank, IoRet(reqid=req.request_id, source=source)),
                                             self.loop)


def _scheduler_role():
    from .engine_proxy import KVConnectorRole

    return KVConnectorRole.SCHEDULER
