"""Host-side collectives for the benchmark ranks.

The ranks of a benchmark serve one another: a decode rank's transfer server maps memory, opens
event handles and launches the pull kernels while its main thread waits for the prefill ranks to
finish their steps.  If that wait were a NCCL barrier, a NCCL kernel would sit on the decode GPU
spinning for a rank that in turn waits for work on that same GPU; device memory allocation and
handle-opening calls can queue behind such a kernel and never return.  So every barrier and every
exchange of small values between ranks goes over a gloo group on the host; NCCL carries only what
a measured arm sends through it."""
from __future__ import annotations

from typing import Any, List

import torch

_group = None


def _dist():
    import torch.distributed as dist

    return dist


def init() -> None:
    """Collective: every rank calls it once, right after the default process group exists."""
    global _group
    dist = _dist()
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1 and _group is None:
        _group = dist.new_group(backend="gloo")


def active() -> bool:
    return _group is not None


def barrier() -> None:
    if _group is not None:
        _dist().barrier(group=_group)


def all_reduce(t: torch.Tensor, op=None) -> torch.Tensor:
    """In-place reduction of a small tensor (any device) through host memory."""
    if _group is None:
        return t
    dist = _dist()
    c = t.detach().to("cpu", copy=True)
    dist.all_reduce(c, op=op if op is not None else dist.ReduceOp.SUM, group=_group)
    t.copy_(c)
    return t


def all_gather_object(out: List[Any], obj: Any) -> None:
    if _group is None:
        out[0] = obj
        return
    _dist().all_gather_object(out, obj, group=_group)
