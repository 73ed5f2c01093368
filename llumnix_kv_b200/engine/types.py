"""Request / output / scheduler-output records of the minimal engine.

Field names follow the vLLM v1 objects the reference connector touches (Request,
EngineCoreRequest, EngineCoreOutput, SchedulerOutput, NewRequestData, CachedRequestData,
KVCacheBlocks; see the imports of blade_kvt/hybrid_connector/engine_proxy.py) so that the
control-plane code reads the same.
"""
from __future__ import annotations

import dataclasses
import enum
import time
from typing import Any, Optional

import msgspec


class FinishReason(enum.IntEnum):
    STOP = 0
    LENGTH = 1
    ABORT = 2


class RequestStatus(enum.IntEnum):
    WAITING = 0
    RUNNING = 1
    FINISHED_STOPPED = 2
    FINISHED_LENGTH = 3
    FINISHED_ABORTED = 4

    @staticmethod
    def is_finished(s: "RequestStatus") -> bool:
        return s >= RequestStatus.FINISHED_STOPPED


class EngineCoreRequestType(enum.Enum):
    ADD = b"\x00"
    ABORT = b"\x01"
    WAKEUP = b"\x02"


class SamplingParams(msgspec.Struct, omit_defaults=True):
    max_tokens: int = 16
    min_tokens: int = 0
    extra_args: Optional[dict] = None


class EngineCoreRequest(msgspec.Struct, omit_defaults=True):
    """What travels between engines (PREFILL_REQ pushes a whole request to a prefill engine)."""

    request_id: str
    prompt_token_ids: list[int]
    sampling_params: Optional[SamplingParams] = None
    eos_token_id: Optional[int] = None
    arrival_time: float = 0.0
    client_index: int = 0
    priority: int = 0
    trace_headers: Optional[dict] = None
    queue_server_address: Optional[str] = None


class RequestTrace:
    """Per-request KV timing marks and W3C trace context.

    The scheduler half calls ``on_req_kv_start/end("load" | "save")`` around a request's KV I/O
    (blade_kvt/hybrid_connector/__init__.py:1185-1186,1304,1345); backends that talk to a store ask
    ``traceparent(op)`` for the header they hand over as request context
    (blade_kvt/hybrid_connector/kvsbackend.py:403,481), so that the store's spans hang under the
    request's trace.  Without an incoming ``traceparent`` header there is no context to propagate."""

    def __init__(self, trace_headers: Optional[dict] = None):
        self.headers = dict(trace_headers) if trace_headers else {}
        self.marks: dict = {}          # "load" / "save" -> [start, end] (time.monotonic)

    def on_req_kv_start(self, kind: str) -> None:
        self.marks[kind] = [time.monotonic(), None]

    def on_req_kv_end(self, kind: str) -> None:
        m = self.marks.get(kind)
        if m is not None and m[1] is None:
            m[1] = time.monotonic()

    def elapsed(self, kind: str) -> Optional[float]:
        m = self.marks.get(kind)
        return None if m is None or m[1] is None else m[1] - m[0]

    def traceparent(self, op: str) -> Optional[str]:
        """A child of the request's span, named by ``op``: same trace id, span id derived from (parent, op)."""
        parent = self.headers.get("traceparent")
        if not parent:
            return None
        parts = parent.split("-")
        if len(parts) != 4 or len(parts[1]) != 32 or len(parts[2]) != 16:
            return None
        import hashlib

        span = hashlib.blake2b(f"{parts[2]}/{op}".encode(), digest_size=8).hexdigest()
        return f"{parts[0]}-{parts[1]}-{span}-{parts[3]}"


class Request:
    def __init__(self, request_id: str, prompt_token_ids: list, sampling_params: Optional[SamplingParams] = None,
                 eos_token_id: Optional[int] = None, client_index: int = 0, arrival_time: float = 0.0,
                 kv_transfer_params: Optional[dict] = None, trace_headers: Optional[dict] = None,
                 queue_server_address: Optional[str] = None):
        self.request_id = request_id
        self.prompt_token_ids = list(prompt_token_ids)
        self.sampling_params = sampling_params or SamplingParams()
        self.eos_token_id = eos_token_id
        self.client_index = client_index
        self.arrival_time = arrival_time or time.time()
        self.kv_transfer_params: Optional[dict] = kv_transfer_params
        self.trace_headers = trace_headers
        self.queue_server_address = queue_server_address
        self.num_prompt_tokens = len(self.prompt_token_ids)
        self.output_token_ids: list[int] = []
        self._all_token_ids = list(self.prompt_token_ids)
        self.num_computed_tokens = 0
        self.num_external_computed_tokens = 0
        self.num_cached_tokens = 0
        self.num_preemptions = 0
        self.status = RequestStatus.WAITING
        self.stop_reason: Any = None
        self._max_computed_tokens: Optional[int] = None
        self.skip_reading_prefix_cache = False
        self.trace_wrapper = RequestTrace(trace_headers)
        self.block_hashes: list = []

    def compute_block_hashes(self, block_size: int) -> list:
        """Chained hashes of the prompt's full blocks (32 bytes each): hash_i covers every token up to the end
        of block i, the property the engine's prefix cache and the store backends key on.  Cached per request."""
        n = self.num_prompt_tokens // block_size
        if len(self.block_hashes) < n or getattr(self, "_block_hash_size", block_size) != block_size:
            import hashlib
            import struct

            self._block_hash_size = block_size
            out, prev = [], b""
            for i in range(n):
                h = hashlib.sha256(prev)
                h.update(struct.pack(f"<{block_size}q", *self.prompt_token_ids[i * block_size:(i + 1) * block_size]))
                prev = h.digest()
                out.append(prev)
            self.block_hashes = out
        return self.block_hashes

    @classmethod
    def from_engine_core_request(cls, r: EngineCoreRequest) -> "Request":
        params = None
        if r.sampling_params is not None and r.sampling_params.extra_args:
            params = r.sampling_params.extra_args.get("kv_transfer_params")
        return cls(r.request_id, r.prompt_token_ids, r.sampling_params, r.eos_token_id, r.client_index,
                   r.arrival_time, dict(params) if params else None, r.trace_headers, r.queue_server_address)

    @property
    def all_token_ids(self) -> list:
        return self._all_token_ids

    @property
    def num_tokens(self) -> int:
        return len(self._all_token_ids)

    @property
    def max_tokens(self) -> int:
        return self.sampling_params.max_tokens

    def append_output_token_ids(self, tok: int) -> None:
        self.output_token_ids.append(tok)
        self._all_token_ids.append(tok)

    # Prefill boundary of a request whose KV leaves for another engine: the scheduler never
    # computes past it (None = no boundary).
    def max_computed_tokens(self) -> Optional[int]:
        return self._max_computed_tokens

    def set_max_computed_tokens(self, n: Optional[int]) -> None:
        self._max_computed_tokens = n

    def is_finished(self) -> bool:
        return RequestStatus.is_finished(self.status)

    def get_finished_reason(self) -> Optional[FinishReason]:
        return {RequestStatus.FINISHED_STOPPED: FinishReason.STOP, RequestStatus.FINISHED_LENGTH: FinishReason.LENGTH,
                RequestStatus.FINISHED_ABORTED: FinishReason.ABORT}.get(self.status)


@dataclasses.dataclass
class EngineCoreOutput:
    request_id: str
    new_token_ids: list
    finish_reason: Optional[FinishReason] = None
    stop_reason: Any = None
    kv_transfer_params: Optional[dict] = None
    num_cached_tokens: int = 0
    queue_server_address: Optional[str] = None

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None


@dataclasses.dataclass
class KVCacheBlock:
    block_id: int
    ref_cnt: int = 0
    is_null: bool = False


@dataclasses.dataclass
class KVCacheBlocks:
    """Per KV-cache group, the blocks of one request."""

    blocks: tuple

    def get_block_ids(self) -> list:
        return [[b.block_id for b in grp] for grp in self.blocks]

    def __add__(self, other: "KVCacheBlocks") -> "KVCacheBlocks":
        return KVCacheBlocks(tuple(list(a) + list(b) for a, b in zip(self.blocks, other.blocks)))


@dataclasses.dataclass
class NewRequestData:
    req_id: str
    prompt_token_ids: list
    block_ids: list           # [[ids of group 0], ...]
    num_computed_tokens: int


@dataclasses.dataclass
class CachedRequestData:
    req_ids: list = dataclasses.field(default_factory=list)
    new_block_ids: list = dataclasses.field(default_factory=list)
    num_computed_tokens: list = dataclasses.field(default_factory=list)


@dataclasses.dataclass
class SchedulerOutput:
    scheduled_new_reqs: list = dataclasses.field(default_factory=list)
    scheduled_cached_reqs: CachedRequestData = dataclasses.field(default_factory=CachedRequestData)
    num_scheduled_tokens: dict = dataclasses.field(default_factory=dict)
    total_num_scheduled_tokens: int = 0
    finished_req_ids: set = dataclasses.field(default_factory=set)
    kv_connector_metadata: Any = None


class KVConnectorRole(enum.Enum):
    SCHEDULER = 0
    WORKER = 1


class KVConnectorMetadata:
    pass
