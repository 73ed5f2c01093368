"""Which GPU should a prefill rank send to, and how: NVLink / NVSwitch affinity.

The reference answers the RDMA version of this question: ``nic_affinity.generate`` runs an
external probe and writes, per GPU, the name of the closest NIC into a file that the C++
transport reads (blade_kvt/nic_affinity.py:24-52, kvtransfer/src/barex_protocol.cpp:262-302).
On a B200 box the data path is GPU-to-GPU stores through NVSwitch, so the table holds, per GPU
pair, whether peer stores are possible, the CUDA P2P performance rank, native atomics and, per
GPU, NVLS (multicast) capability and the number of NVLink links that are up.  ``generate``
writes the same kind of file for tools; ``best_peers`` is what schedulers use to pair prefill
and decode GPUs.  Everything is read-only: no GPU setting is touched.
"""
from __future__ import annotations

import json
import os
from typing import Optional

AFFINITY_FILE = "/tmp/llumnix_kv_b200_nvlink_affinity.json"


def discover() -> dict:
    """Topology of the GPUs visible to this process: {"gpus": [...], "links": [...]}."""
    from . import load_ops

    return json.loads(load_ops().discover_topology())


def generate(path: Optional[str] = None) -> str:
    """Write the topology to ``path`` (atomically) and return the path."""
    path = path or os.environ.get("LLUMNIX_KV_NVLINK_AFFINITY_FILE", AFFINITY_FILE)
    topo = discover()
    tmp = f"{path}.{os.getpid()}.tmp"
    with open(tmp, "w") as f:
        json.dump(topo, f, indent=1)
    os.replace(tmp, path)
    return path


def load(path: Optional[str] = None) -> dict:
    path = path or os.environ.get("LLUMNIX_KV_NVLINK_AFFINITY_FILE", AFFINITY_FILE)
    with open(path) as f:
        return json.load(f)


def best_peers(topo: dict, src: int) -> list:
    """Destination GPUs ``src`` can store into, best first (P2P performance rank, then index).
    Behind an NVSwitch every peer has the same rank, so the order is by index."""
    peers = [l for l in topo.get("links", []) if l["src"] == src and l["access"]]
    peers.sort(key=lambda l: (l["perf_rank"] if l["perf_rank"] >= 0 else 1 << 30, l["dst"]))
    return [l["dst"] for l in peers]


def pair_prefill_decode(topo: dict, n_prefill: int) -> list:
    """A one-to-one pairing of the first ``n_prefill`` GPUs with the remaining ones such that every
    pair has peer access; falls back to (i, i + n_prefill) where no better choice exists."""
    n = len(topo.get("gpus", []))
    free = set(range(n_prefill, n))
    pairs = []
    for p in range(n_prefill):
        choice = next((d for d in best_peers(topo, p) if d in free), None)
        if choice is None:
            choice = p + n_prefill if p + n_prefill in free else (min(free) if free else None)
        if choice is None:
            break
        free.discard(choice)
        pairs.append((p, choice))
    return pairs


def nvls_capable(topo: dict) -> bool:
    gpus = topo.get("gpus", [])
    return bool(gpus) and all(g.get("multicast_supported", -1) == 1 for g in gpus)
