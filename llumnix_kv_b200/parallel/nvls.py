"""NVLS fan-out of replicated KV blocks inside a tensor-parallel decode group.

Data that every TP rank of a decode instance holds identically (MLA latent and indexer caches,
replicated KV heads) is sent by the reference once per destination rank: a prefill rank fans out
to d/p decode ranks (blade_kvt/hybrid_connector/kvtbackend.py:637-664), so its link carries d/p
copies.  With the caches of the group allocated as one *symmetric* buffer bound to an NVLink
multicast object, the prefill rank pushes ONE copy to one member (the ordinary peer-store kernel)
and that member replicates the blocks with ``multimem.st``: its NVLink egress carries the bytes
once and NVSwitch writes them into every member's memory.

    group = tp_group_of_the_decode_instance
    cache = MulticastKVCache(num_layers, layer_bytes, group, device)     # every rank, same sizes
    ... prefill pushes the request's blocks into rank r0's cache.layers ...
    if group.rank() == r0:
        cache.fanout(block_ids, block_stride, num_blocks, flag_value=stepid)  # one kernel
    cache.wait(flag_value=stepid, slots=[r0], timeout_s=1.0)                   # bounded device wait

Better balanced: the prefill rank scatters the request's blocks over landing buffers of ALL members
(still one copy on its link), every member relays its share from its landing buffer
(``src_layers=...``) and signals in its own completion word, and everybody waits for all words: no
member receives more than 1 + 1/k copies, where the single-relay form makes r0 receive two.

Teardown is collective: every rank calls ``close()`` (barrier, then release) while all ranks are
alive.  Only stores are multicast; nothing loads through the multicast address.
"""
from __future__ import annotations

import collections
from typing import Optional, Sequence

import torch

from llumnix_kv_b200 import load_ops

_FLAG_BYTES = 256     # completion word + padding, at the end of the symmetric buffer

_live_caches: "list[MulticastKVCache]" = []     # caches of this process, for multicast_address_of()


def multicast_address_of(tensor: torch.Tensor):
    """``(multicast address, group size)`` of a tensor that lives inside a MulticastKVCache of this
    process, else None.  The transfer server uses it to tell senders that this worker can relay a
    request to its whole group."""
    ptr, end = tensor.data_ptr(), tensor.data_ptr() + tensor.numel() * tensor.element_size()
    for c in _live_caches:
        if c.buffer is not None and c.local_ptr <= ptr and end <= c.local_ptr + c.num_layers * c.layer_bytes:
            return c.mc_ptr + (ptr - c.local_ptr), c.world
    return None


class MulticastKVCache:
    """``num_layers`` cache tensors of ``layer_bytes`` each, in one symmetric allocation of the group."""

    def __init__(self, num_layers: int, layer_bytes: int, group, device: torch.device):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        assert layer_bytes % 16 == 0, "layers must be made of whole 16-byte words"
        self._dist = dist
        self.group = group
        self.device = torch.device(device)
        self.num_layers = num_layers
        self.layer_bytes = layer_bytes
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        total = num_layers * layer_bytes + _FLAG_BYTES
        self.buffer = symm.empty(total, dtype=torch.uint8, device=self.device)
        self.buffer.zero_()
        torch.cuda.synchronize(self.device)
        self._handle = symm.rendezvous(self.buffer, group)
        self.mc_ptr = int(self._handle.multicast_ptr)
        if self.mc_ptr == 0:
            raise RuntimeError("this GPU group has no NVLink multicast (NVLS) support")
        self.local_ptr = self.buffer.data_ptr()
        self.layers = [self.buffer[i * layer_bytes:(i + 1) * layer_bytes] for i in range(num_layers)]
        self._flag_off = num_layers * layer_bytes
        assert self.world * 8 <= _FLAG_BYTES
        self.flags = self.buffer[self._flag_off:self._flag_off + _FLAG_BYTES].view(torch.int64)   # one word per rank
        dev = self.device
        self._src_layers = torch.tensor([self.local_ptr + i * layer_bytes for i in range(num_layers)], dtype=torch.int64,
                                        device=dev)
        self._mc_layers = torch.tensor([self.mc_ptr + i * layer_bytes for i in range(num_layers)], dtype=torch.int64,
                                       device=dev)
        self._status = torch.zeros(4, dtype=torch.int32, device=dev)
        self._wait_status = torch.zeros(4, dtype=torch.int32, device=dev)
        self._counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self._ops = load_ops()
        self._closed = False
        self._keep = collections.deque(maxlen=256)
        _live_caches.append(self)

    # ---- the member that received the blocks -----------------------------------------------------------
    def _ids(self, block_ids) -> torch.Tensor:
        if isinstance(block_ids, torch.Tensor):
            return block_ids.to(device=self.device, dtype=torch.int32)
        return torch.tensor(list(block_ids), dtype=torch.int32, device=self.device)

    def fanout(self, block_ids, block_stride: int, num_blocks: int, block_off: int = 0, block_len: Optional[int] = None,
               layers: Optional[Sequence[int]] = None, flag_value: int = 0, flag_slot: Optional[int] = None, grid: int = 0,
               stream: Optional[torch.cuda.Stream] = None, src_layers: Optional[torch.Tensor] = None,
               src_block_ids=None, src_block_stride: Optional[int] = None, src_num_blocks: Optional[int] = None) -> None:
        """Replicate blocks of layers ``[layers[0], layers[1])`` into ``block_ids`` of every member.

        In place by default: the source is this member's own cache (the sender pushed into it).  With
        ``src_layers`` (an int64 device tensor of per-layer base addresses of any local memory, for
        instance a landing buffer that the sender reaches over CUDA-IPC) the blocks are read from there,
        at ``src_block_ids`` with ``src_block_stride``.  ``block_ids`` may be lists or int32 device tensors.
        With ``flag_value`` != 0 completion word ``flag_slot`` (default: this rank's) of every member
        receives it after the data: when several members relay shares of one request, each signals in
        its own word and ``wait`` looks at all of them."""
        ids = self._ids(block_ids)
        sids = ids if src_block_ids is None else self._ids(src_block_ids)
        assert sids.numel() == ids.numel()
        lo, hi = (0, self.num_layers) if layers is None else layers
        assert 0 <= lo <= hi <= self.num_layers
        assert num_blocks * block_stride <= self.layer_bytes
        sstride = block_stride if src_block_stride is None else src_block_stride
        snum = num_blocks if src_num_blocks is None else src_num_blocks
        blen = min(block_stride, sstride) - block_off if block_len is None else block_len
        src = self._src_layers if src_layers is None else src_layers
        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        self._keep.append((ids, sids, src))   # the launches are asynchronous: keep their arguments alive for a while
        self._ops.kvt_launch_mc_fanout(
            src.data_ptr(), self._mc_layers.data_ptr(), lo, hi, sstride, block_stride, snum, num_blocks, sids.data_ptr(),
            ids.data_ptr(), ids.numel(), block_off, blen, self._status.data_ptr(), self._counter.data_ptr(),
            (self.mc_ptr + self._flag_off + 8 * (self.rank if flag_slot is None else flag_slot)) if flag_value else 0,
            flag_value, grid, st.cuda_stream)

    def check_status(self) -> None:
        code, detail = (int(x) for x in self._status[:2].tolist())
        if code != 0:
            self._status.zero_()
            raise RuntimeError(f"fan-out kernel reported status {code} (detail {detail})")

    # ---- the other members -----------------------------------------------------------------------------
    def wait(self, flag_value: int, timeout_s: float = 1.0, stream: Optional[torch.cuda.Stream] = None,
             slots: Optional[Sequence[int]] = None, sync: bool = True) -> bool:
        """Device-side wait, bounded by ``timeout_s`` per word, until this member's completion words
        ``slots`` (default: one per rank of the group) reach ``flag_value``; returns False when a wait ran
        out (the context stays usable).  With ``sync=False`` the waits are only enqueued; read
        ``wait_failed()`` after synchronising the stream."""
        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        self._wait_status.zero_()
        for slot in (range(self.world) if slots is None else slots):
            self._ops.kvt_launch_wait_flag(self.flags[slot:].data_ptr(), flag_value, int(timeout_s * 1e9),
                                           self._wait_status.data_ptr(), st.cuda_stream)
        if not sync:
            return True
        st.synchronize()
        return not self.wait_failed()

    def wait_failed(self) -> bool:
        return int(self._wait_status[0].item()) != 0

    # ---- collective teardown ---------------------------------------------------------------------------
    def close(self) -> None:
        """Every rank calls this while all ranks of the group are alive: no rank may go away while
        its memory is still bound to the multicast object."""
        if self._closed:
            return
        self._closed = True
        if self in _live_caches:
            _live_caches.remove(self)
        torch.cuda.synchronize(self.device)
        self._dist.barrier(self.group)
        self.layers = []
        self.flags = None
        self._handle = None
        self.buffer = None
        torch.cuda.synchronize(self.device)
        self._dist.barrier(self.group)
