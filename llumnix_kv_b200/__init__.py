"""llumnix_kv_b200: a Blackwell-native KV-cache transfer and storage framework.

Public surface (names follow the reference package ``blade_kvt``):

* ``llumnix_kv_b200.hybrid_connector`` - HybridConnector control plane (scheduler / worker
  halves, backends, RPC protocol).
* ``llumnix_kv_b200.kv_transfer`` / ``kv_transfer_impl`` - ``KVTransferClient`` /
  ``KVTransferServer`` over the native engine.
* ``llumnix_kv_b200.kvtransfer_ops`` - the native extension (C++ engine + sm_100a kernels).
* ``llumnix_kv_b200.ops`` - kernel-level Python wrappers and their PyTorch oracles.
"""
from __future__ import annotations

import importlib
import os

__version__ = "0.1.0"


def load_ops(build_if_missing: bool = True):
    """Import the native extension, compiling it in-tree first when it is absent.

    Raises if it cannot be loaded: nothing in this package silently falls back to PyTorch.
    """
    try:
        return _loaded(importlib.import_module("llumnix_kv_b200.kvtransfer_ops"))
    except ImportError:
        if not build_if_missing or os.environ.get("LLUMNIX_KV_NO_AUTOBUILD") == "1":
            raise
    from . import _build

    _build.build()
    importlib.invalidate_caches()
    return _loaded(importlib.import_module("llumnix_kv_b200.kvtransfer_ops"))


_atexit_registered = False


def _loaded(mod):
    """The process-global client / server of the reference-named functions own threads; stop them while the
    interpreter is still whole instead of leaving that to the C++ runtime's exit handlers."""
    global _atexit_registered
    if not _atexit_registered:
        import atexit

        atexit.register(mod.shutdown_kv_transfer)
        _atexit_registered = True
    return mod


def set_envs() -> None:
    """Default environment of the native engine (role of blade_kvt/__init__.py:42-61; the ACCL_* settings
    of the reference configure its RDMA library and have no reader here).  The backends call this before
    they create a transfer client or server (kvtbackend.py:524-525 of the reference)."""
    os.environ.setdefault("BLLM_KVTRANS_FSNAMING_KEEPALIVE_S", "36000")
    os.environ.setdefault("BLLM_KVTRANS_FSNAMING_TOLERATE_S", "360000")
    os.environ.setdefault("BLLM_KVTRANS_RDMA_SP", "2")      # connections per target of the TCP / SHM transports
    os.environ.setdefault("BLLM_KVTRANS_SDH_KIND", "2")


def support_async_sched() -> bool:
    """The connector assumes the engine schedules synchronously (blade_kvt/__init__.py:10-11)."""
    return False


def is_nv_gpu() -> bool:
    import torch

    return torch.cuda.is_available() and "nvidia" in torch.cuda.get_device_name().lower()


def is_erdma() -> bool:
    """Whether the host's RDMA devices are Alibaba eRDMA (blade_kvt/__init__.py:21-39 asks the verbs tools
    and the module list); False on hosts without an RDMA stack, which is every host this build targets."""
    import subprocess

    for cmd in ("ibv_devinfo -l", "ibv_devices", "lsmod"):
        try:
            out = subprocess.check_output(cmd, shell=True, stderr=subprocess.STDOUT, timeout=5)
        except Exception:
            continue
        if b"erdma" in out.lower():
            return True
    return False
