"""A small continuous-batching scheduler with chunked prefill.

It offers what the connector's engine seam needs from vLLM's v1 scheduler: request table,
add / finish, per-step SchedulerOutput with new vs. cached requests and their block ids, the
prefill boundary ``max_computed_tokens`` of requests whose decode happens elsewhere, and the
finish hook where the connector decides what the request's last output says about its KV.
"""
from __future__ import annotations

from collections import deque
from typing import Iterable, Optional, Union

from .config import VllmConfig
from .kv_cache import KVCacheManager
from .types import (CachedRequestData, EngineCoreOutput, FinishReason, NewRequestData, Request, RequestStatus,
                    SchedulerOutput)


class MiniScheduler:
    def __init__(self, cfg: VllmConfig, group_types: Optional[list] = None):
        self.vllm_config = cfg
        self.block_size = cfg.cache_config.block_size
        self.kv_cache_manager = KVCacheManager(cfg.cache_config.num_gpu_blocks, self.block_size, group_types)
        self.requests: dict[str, Request] = {}
        self.waiting: deque = deque()
        self.running: list = []
        self.finished_req_ids: set = set()
        self._scheduled_before: set = set()
        self.connector = None  # scheduler-role HybridConnector, set by the engine core

    # ---- request table ---------------------------------------------------------------------
    def add_request(self, req: Request) -> None:
        self.requests[req.request_id] = req
        req.status = RequestStatus.WAITING
        self.waiting.append(req)

    def get_kv_connector(self):
        return self.connector

    def finish_requests(self, request_ids: Union[str, Iterable[str]], status: RequestStatus) -> None:
        if isinstance(request_ids, str):
            request_ids = [request_ids]
        for rid in request_ids:
            req = self.requests.get(rid)
            if req is None or req.is_finished():
                continue
            if req in self.running:
                self.running.remove(req)
            else:
                try:
                    self.waiting.remove(req)
                except ValueError:
                    pass
            req.status = status
            self._free_request(req)

    def _free_request(self, req: Request) -> Optional[dict]:
        params = None
        if self.connector is not None:
            _delay, params = self.connector.request_finished_all_groups(
                req, tuple(self.kv_cache_manager.get_block_ids(req.request_id)))
        self.kv_cache_manager.free(req)
        self.finished_req_ids.add(req.request_id)
        self.requests.pop(req.request_id, None)
        self._scheduled_before.discard(req.request_id)
        return params

    def has_unfinished_requests(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- scheduling ------------------------------------------------------------------------
    def _target_tokens(self, req: Request) -> int:
        """How far this request may be computed right now (prompt, or prompt + generated so far)."""
        limit = req.num_tokens
        mx = req.max_computed_tokens()
        if mx is not None:
            limit = min(limit, mx)
        return limit

    def schedule(self) -> SchedulerOutput:
        sout = SchedulerOutput()
        budget = self.vllm_config.scheduler_config.max_num_batched_tokens
        cached = CachedRequestData()
        for req in list(self.running):
            if budget <= 0:
                break
            n = min(self._target_tokens(req) - req.num_computed_tokens, budget)
            if n <= 0:
                continue
            new = self.kv_cache_manager.allocate_slots(req, req.num_computed_tokens + n)
            if new is None:
                continue
            cached.req_ids.append(req.request_id)
            cached.new_block_ids.append(new.get_block_ids())
            cached.num_computed_tokens.append(req.num_computed_tokens)
            sout.num_scheduled_tokens[req.request_id] = n
            budget -= n
        while self.waiting and budget > 0 and len(self.running) < self.vllm_config.scheduler_config.max_num_seqs:
            req = self.waiting[0]
            n = min(self._target_tokens(req) - req.num_computed_tokens, budget)
            if n <= 0:
                # nothing to compute (a decode-side request fully loaded up to its boundary):
                # it still becomes running so that it can finish / be handed over
                self.waiting.popleft()
                req.status = RequestStatus.RUNNING
                self.running.append(req)
                continue
            new = self.kv_cache_manager.allocate_slots(req, req.num_computed_tokens + n)
            if new is None:
                break
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            sout.scheduled_new_reqs.append(NewRequestData(
                req.request_id, list(req.all_token_ids), self.kv_cache_manager.get_block_ids(req.request_id),
                req.num_computed_tokens))
            self._scheduled_before.add(req.request_id)
            sout.num_scheduled_tokens[req.request_id] = n
            budget -= n
        sout.scheduled_cached_reqs = cached
        sout.total_num_scheduled_tokens = sum(sout.num_scheduled_tokens.values())
        sout.finished_req_ids = self.finished_req_ids
        self.finished_req_ids = set()
        return sout

    def update_from_output(self, sout: SchedulerOutput, sampled: dict) -> dict:
        """Advance the scheduled requests; returns {client_index: [EngineCoreOutput]}."""
        outputs: dict = {}
        for rid, n in sout.num_scheduled_tokens.items():
            req = self.requests.get(rid)
            if req is None:
                continue
            req.num_computed_tokens += n
            new_tokens = []
            if req.num_computed_tokens >= req.num_tokens and rid in sampled:
                tok = sampled[rid]
                req.append_output_token_ids(tok)
                new_tokens = [tok]
            finish: Optional[FinishReason] = None
            mx = req.max_computed_tokens()
            if new_tokens and req.eos_token_id is not None and new_tokens[0] == req.eos_token_id and \
                    len(req.output_token_ids) >= req.sampling_params.min_tokens:
                req.status, finish = RequestStatus.FINISHED_STOPPED, FinishReason.STOP
            elif len(req.output_token_ids) >= req.max_tokens:
                req.status, finish = RequestStatus.FINISHED_LENGTH, FinishReason.LENGTH
            elif mx is not None and req.num_computed_tokens >= mx and not new_tokens:
                # prefill-only request that stops at its KV boundary without sampling
                req.status, finish = RequestStatus.FINISHED_LENGTH, FinishReason.LENGTH
            params = None
            if finish is not None:
                self.running.remove(req)
                params = self._free_request(req)
            if new_tokens or finish is not None:
                outputs.setdefault(req.client_index, []).append(EngineCoreOutput(
                    rid, new_tokens, finish, req.stop_reason, params, req.num_cached_tokens,
                    req.queue_server_address))
        return outputs
