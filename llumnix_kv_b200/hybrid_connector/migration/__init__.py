"""Live migration of requests between engines: wire constants and small helpers.

Every RPC is ``head:u32`` followed, where it has a body, by ``len:u32`` and a msgpack body
(blade_kvt/hybrid_connector/migration/__init__.py:11-47, migration/backend.py:142-143,181-185).
A frontend that takes part in migration identifies itself to the engines by a client index
above 0xFFFF that encodes where its output server listens: ``ipv4 << 16 | port``
(:66-91).
"""
from __future__ import annotations

from typing import Optional

import msgspec

NEW_OUTPUT_REQ, NEW_OUTPUT_RESP = 20080808, 80808002      # body: EngineCoreOutputs (engine -> frontend)
NEW_REQ_REQ, NEW_REQ_RESP = 20080818, 81808002            # body: EngineCoreRequest (frontend -> engine)
ABORT_REQS_REQ, ABORT_REQS_RESP = 20080828, 82808002      # body: list[str]
MIGRATE_TO_REQ, MIGRATE_TO_RESP = 20080901, 10908002      # body: EngineCoreRequest / MigrateResp
SUSPEND_REQ, SUSPEND_RESP = 20080903, 30908002            # body: SuspendReq / SuspendResp
KVT_SUSPEND_REQ = 0x20240912                              # body: RKVTDInfo; answered like TRANSFER_KV_REQ

OUTPUT_TOKENS_N = "_hbmigrateoutputtokensn"               # output tokens the request had when it was sent away
SRC_INFO = "__HybridConnector_Migration_Src_Info__"       # (addr, port) of the engine the request comes from
SUSPEND_EVT = "__HybridConnector_Migration_Suspend_Event__"


class MigrateResp(msgspec.Struct, array_like=True, omit_defaults=True, gc=False):
    code: int


class SuspendReq(msgspec.Struct, array_like=True, omit_defaults=True, gc=False):
    reqid: str


class SuspendResp(msgspec.Struct, array_like=True, omit_defaults=True, gc=False):
    code: int
    output_token_ids: list[int] = []


class WireOutput(msgspec.Struct, array_like=True, omit_defaults=True, gc=False):
    request_id: str
    new_token_ids: list[int]
    finish_reason: Optional[int] = None
    kv_transfer_params: Optional[dict] = None
    num_cached_tokens: int = 0


class EngineCoreOutputs(msgspec.Struct, array_like=True, omit_defaults=True, gc=False):
    engine_index: int
    outputs: list[WireOutput]


def is_migration(idx: int) -> bool:
    return idx > 0xFFFF


def ipport2int(ip: str, port: int) -> int:
    a, b, c, d = (int(x) for x in ip.split("."))
    return ((a << 24 | b << 16 | c << 8 | d) << 16) | port


def int2ipport(val: int) -> tuple:
    ip = val >> 16
    return ".".join(str((ip >> s) & 0xFF) for s in (24, 16, 8, 0)), val & 0xFFFF
