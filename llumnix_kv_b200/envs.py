"""Environment knobs of the Python control plane.

The reference reads these through a forked ``vllm.envs`` (VLLM_KV_TRANS_PROTOCOL, VLLM_ENABLE_BYPASS_TASK/SUBSTEP, VLLM_KVT_MAX_DELAY_MS,
VLLM_KVT_GONE_REQ_TTL_S, VLLM_PD_TRY_CONNECT_TIMEOUT_SECONDS, VLLM_PD_CONNMANAGER_CAP,
VLLM_KVS_*, LLUMNIX_MAX_*_MIG_IN ...).  Values are read at attribute access so tests can
change them with ``os.environ``.
"""
from __future__ import annotations

import os
from typing import Any, Callable

_DEFS: dict[str, tuple[Callable[[str], Any], Any]] = {
    "VLLM_KV_TRANS_PROTOCOL": (str, ""),             # "", "tcp", "shm", "nvlink"
    "VLLM_ENABLE_BYPASS_TASK": (lambda v: v not in ("0", "", "false"), False),
    "VLLM_ENABLE_BYPASS_SUBSTEP": (lambda v: v not in ("0", "", "false"), False),
    "VLLM_KVT_MAX_DELAY_MS": (float, 3000.0),
    "VLLM_KVT_GONE_REQ_TTL_S": (int, 60),
    "VLLM_KVT_NVLS_FANOUT": (lambda v: v not in ("0", "", "false"), True),   # relay replicated caches through a decode group's multicast
    "VLLM_PD_TRY_CONNECT_TIMEOUT_SECONDS": (float, 120.0),
    "VLLM_PD_CONNMANAGER_CAP": (int, 512),
    "VLLM_KVS_IO_TIMEOUT_SECONDS": (float, 30.0),
    "VLLM_KVS_ON_MIN_LENGTH": (int, 0),
    "VLLM_KVS_TTL_SECONDS": (float, 300.0),
    "VLLM_KVS_CAPACITY_BYTES": (int, 1 << 30),
    "VLLM_KVS_STORE_NAN_CHECK": (int, 0),
    "VLLM_KVS_USE_REQUEST_HASH": (lambda v: v not in ("0", "", "false"), False),
    "VLLM_ZERO_HYBRID_KV_CACHE": (lambda v: v not in ("0", "", "false"), True),
    "VLLM_LOG_STATS_INTERVAL": (float, 10.0),
    "VLLM_HOST_IP": (str, ""),
    "LLUMNIX_MAX_REQ_MIG_IN": (int, 64),
    "LLUMNIX_MAX_TOKEN_MIG_IN": (int, 1 << 20),
    "LLUMNIX_DETAILED_MIG_STATUS": (lambda v: v not in ("0", "", "false"), False),
}


def __getattr__(name: str):
    if name not in _DEFS:
        raise AttributeError(name)
    conv, default = _DEFS[name]
    raw = os.environ.get(name)
    if raw is None:
        return default
    try:
        return conv(raw)
    except ValueError:
        return default


def get_ip() -> str:
    ip = os.environ.get("VLLM_HOST_IP")
    return ip if ip else "127.0.0.1"
