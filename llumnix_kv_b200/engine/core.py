"""Engine core of the minimal engine: the loop that owns the scheduler, talks to the
scheduler half of the connector and drives the workers.

One iteration is what the reference's forked engine does around its connector
(call order in blade_kvt/hybrid_connector/__init__.py: on_add_req at admission, ``step()``
before scheduling, ``build_connector_meta`` on the scheduler output, the workers' forward
pass with the metadata bound, then output processing).  The loop sleeps on its input queue;
the connector wakes it through ``EngineProxy.wakeup_core`` when something it waits for
(a finished load, a finished save, an abort) has happened on another thread.
"""
from __future__ import annotations

import logging
import queue
import threading
import time
from typing import Callable, Optional

from llumnix_kv_b200.hybrid_connector import HybridConnector
from llumnix_kv_b200.hybrid_connector.engine_proxy import EngineProxy, KVConnectorRole

from .config import VllmConfig
from .scheduler import MiniScheduler
from .types import EngineCoreOutput, EngineCoreRequest, EngineCoreRequestType, Request
from .worker import MiniWorker, make_kv_cache_config

logger = logging.getLogger("llumnix_kv_b200.engine")


class MiniEngineCore:
    def __init__(self, cfg: VllmConfig, devices: Optional[list] = None, start: bool = True,
                 output_cb: Optional[Callable[[int, list], None]] = None):
        self.cfg = cfg
        self.input_queue: "queue.Queue" = queue.Queue()
        self.outputs: "queue.Queue" = queue.Queue()
        self._output_cb = output_cb
        self.scheduler = MiniScheduler(cfg, cfg.model_config.group_types())
        self.proxy: Optional[EngineProxy] = None
        self.connector: Optional[HybridConnector] = None
        tp = cfg.parallel_config.tensor_parallel_size
        devices = devices or [cfg.device] * tp
        kv_cache_config = make_kv_cache_config(cfg)
        if cfg.kv_transfer_config is not None:
            # the scheduler half opens the RPC port the workers report to, so it comes first
            self.proxy = EngineProxy(self, cfg)
            self._sched_conn_pending = kv_cache_config
        self.workers = []
        if cfg.kv_transfer_config is not None:
            # worker halves register with the scheduler half while it is being constructed
            # (decode side without naming blocks until every rank has registered)
            t = threading.Thread(target=self._make_workers, args=(devices,), daemon=True)
            t.start()
            self.connector = HybridConnector(cfg, KVConnectorRole.SCHEDULER, kv_cache_config, engine=self.proxy)
            self.scheduler.connector = self.connector
            t.join()
            backend = self.connector._sched._backend
            if hasattr(backend, "wait_workers_registered"):
                assert backend.wait_workers_registered(60), "workers did not register with the scheduler"
        else:
            self._make_workers(devices)
        self._stop = False
        self._thread: Optional[threading.Thread] = None
        self._finished: dict[str, EngineCoreOutput] = {}
        self._tokens: dict[str, list] = {}
        self._cv = threading.Condition()
        self.steps = 0
        self.bypass_substeps = 0
        self._last_sout = None
        from llumnix_kv_b200 import envs as _envs

        self._bypass = bool(_envs.VLLM_ENABLE_BYPASS_TASK)
        if start:
            self.start()

    def _make_workers(self, devices: list) -> None:
        self.workers = [MiniWorker(self.cfg, r, devices[r]) for r in range(len(devices))]

    # ---- public API ---------------------------------------------------------------------------
    def add_request(self, req: EngineCoreRequest) -> None:
        self.input_queue.put_nowait((EngineCoreRequestType.ADD, req))

    def abort_requests(self, request_ids: list) -> None:
        self.input_queue.put_nowait((EngineCoreRequestType.ABORT, list(request_ids)))

    def wait_finished(self, reqid: str, timeout: float = 30.0) -> Optional[EngineCoreOutput]:
        with self._cv:
            self._cv.wait_for(lambda: reqid in self._finished, timeout)
            return self._finished.get(reqid)

    def output_tokens(self, reqid: str) -> list:
        return list(self._tokens.get(reqid, []))

    def start(self) -> None:
        self._thread = threading.Thread(target=self.run_loop, name="enginecore", daemon=True)
        self._thread.start()

    def shutdown(self) -> None:
        self._stop = True
        self.input_queue.put_nowait((EngineCoreRequestType.WAKEUP, None))
        if self._thread is not None:
            self._thread.join(10)
        for w in self.workers:
            if w.connector is not None:
                w.connector._worker.closing = True
        if self.connector is not None and self.proxy is not None:
            self.connector._sched.close_bypass()
            self.proxy.rpc_server.close(self.proxy.sched_loop)
        for w in self.workers:
            if w.connector is not None:
                b = w.connector._worker._backend
                if hasattr(b, "stop"):
                    b.stop()

    # ---- loop ---------------------------------------------------------------------------------
    def _handle_input(self, kind, payload) -> None:
        if kind == EngineCoreRequestType.ADD:
            req = Request.from_engine_core_request(payload)
            if self.connector is not None and self.connector.on_add_req(req):
                return   # the connector holds it until its load / block reservation is done
            self.scheduler.add_request(req)
        elif kind == EngineCoreRequestType.ABORT:
            for rid in payload:
                if self.connector is not None:
                    self.connector.on_abort_req(rid, "client abort", True, iscore=True)
                else:
                    from .types import RequestStatus

                    self.scheduler.finish_requests(rid, RequestStatus.FINISHED_ABORTED)

    def _publish(self, outputs: Optional[dict]) -> None:
        if not outputs:
            return
        if self.connector is not None:
            # outputs of requests that belong to a migration-aware frontend leave through the backend
            hook = getattr(self.connector._sched._backend, "on_outputs", None)
            if hook is not None:
                hook(outputs)
        with self._cv:
            for client, outs in outputs.items():
                for o in outs:
                    self._tokens.setdefault(o.request_id, []).extend(o.new_token_ids)
                    if o.finished and not (o.kv_transfer_params or {}).get("kv_transfer_pending"):
                        self._finished[o.request_id] = o
                    elif o.finished:
                        self._finished.setdefault(o.request_id + "#pending", o)
                    self.outputs.put_nowait((client, o))
                if self._output_cb is not None:
                    self._output_cb(client, outs)
            self._cv.notify_all()

    def has_work(self) -> bool:
        return self.scheduler.has_unfinished_requests() or \
            (self.connector is not None and self.connector.has_requests()) or bool(self.scheduler.finished_req_ids)

    def step(self) -> None:
        self.steps += 1
        if self.connector is not None:
            self._publish(self.connector.step())
        if not (self.scheduler.has_unfinished_requests() or self.scheduler.finished_req_ids
                or (self.connector is not None and self.connector.has_requests())):
            return
        sout = self.scheduler.schedule()
        if self.connector is not None and self._bypass and sout.total_num_scheduled_tokens == 0 \
                and not sout.finished_req_ids and self._last_sout is not None:
            # Nothing to compute, but the connector has work for the workers (a decode engine asked
            # for KV that is already complete): hand it to them as a substep of the last step
            # through the bypass channel instead of running an empty forward pass.
            sout.hc_parent = self._last_sout
            meta = self.connector.build_connector_meta(sout)
            if meta.reqs:
                self.bypass_substeps += 1
                self.connector._sched.send_bypass_task(meta)
            return
        if self.connector is not None:
            sout.kv_connector_metadata = self.connector.build_connector_meta(sout)
            self._last_sout = sout
        if sout.total_num_scheduled_tokens == 0 and not sout.kv_connector_metadata and not sout.finished_req_ids:
            return
        sampled: dict = {}
        for w in self.workers:
            sampled = w.execute_model(sout)
        outputs = self.scheduler.update_from_output(sout, sampled)
        for outs in outputs.values():
            for o in outs:
                for tok in o.new_token_ids:
                    for w in self.workers:
                        w.append_token(o.request_id, tok)
        self._publish(outputs)

    def run_loop(self) -> None:
        while not self._stop:
            try:
                block = not self.has_work()
                kind, payload = self.input_queue.get(block=block, timeout=0.5 if block else None)
                self._handle_input(kind, payload)
                while True:
                    kind, payload = self.input_queue.get_nowait()
                    self._handle_input(kind, payload)
            except queue.Empty:
                pass
            try:
                before = self.steps
                self.step()
                if self.has_work() and self.steps == before + 1 and not self.scheduler.running \
                        and not self.scheduler.waiting:
                    time.sleep(0.0005)   # only connector work pending: do not spin hot
            except Exception:
                logger.exception("engine core step failed")
                raise
