"""Block pool and per-request block bookkeeping of the minimal engine.

Blocks carry a reference count: the scheduler holds one reference per request that uses a
block, and the connector takes an extra one while a save is in flight so that the blocks
outlive the request until the transfer has finished (the contract behind
sched_acquire_blocks / sched_free_blocks in blade_kvt/hybrid_connector/engine_proxy.py:231-253).
Block 0 is the null block: never handed out, always zero.
"""
from __future__ import annotations

from collections import deque
from typing import Iterable, Optional

from .types import KVCacheBlock, KVCacheBlocks, Request


class BlockPool:
    def __init__(self, num_blocks: int):
        assert num_blocks >= 2
        self.blocks = [KVCacheBlock(i) for i in range(num_blocks)]
        self.blocks[0].is_null = True
        self.null_block = self.blocks[0]
        self._free: deque = deque(self.blocks[1:])

    def num_free_blocks(self) -> int:
        return len(self._free)

    def get_new_blocks(self, n: int) -> list:
        if n > len(self._free):
            raise RuntimeError("out of KV blocks")
        out = []
        for _ in range(n):
            b = self._free.popleft()
            assert b.ref_cnt == 0
            b.ref_cnt = 1
            out.append(b)
        return out

    def free_blocks(self, blocks: Iterable[KVCacheBlock]) -> None:
        for b in blocks:
            if b.is_null:
                continue
            assert b.ref_cnt > 0, f"double free of block {b.block_id}"
            b.ref_cnt -= 1
            if b.ref_cnt == 0:
                self._free.append(b)


class KVCacheManager:
    """Allocates blocks per KV-cache group.  ``group_types`` lists the groups in physical order:
    "attn" / "indexer" groups grow with the token count, "gdn" / "ple" groups hold one state
    block per request."""

    def __init__(self, num_blocks: int, block_size: int, group_types: Optional[list] = None):
        self.block_size = block_size
        self.block_pool = BlockPool(num_blocks)
        self.group_types = list(group_types or ["attn"])
        self._req_blocks: dict[str, list] = {}      # reqid -> per-group block lists
        self._pending_zero: set = set()
        self.enable_caching = False

    def _needed(self, gtype: str, num_tokens: int) -> int:
        if gtype in ("gdn", "ple"):
            return 1
        return (num_tokens + self.block_size - 1) // self.block_size

    def get_blocks(self, reqid: str) -> tuple:
        groups = self._req_blocks.get(reqid)
        if groups is None:
            return tuple([] for _ in self.group_types)
        return tuple(list(g) for g in groups)

    def get_block_ids(self, reqid: str) -> list:
        return [[b.block_id for b in g] for g in self.get_blocks(reqid)]

    def allocate_slots(self, req: Request, num_tokens_total: int, skip_new_block_zeroing: bool = False
                       ) -> Optional[KVCacheBlocks]:
        """Make sure the request owns enough blocks for ``num_tokens_total`` tokens; returns the
        newly added blocks, or None when the pool cannot satisfy it."""
        groups = self._req_blocks.setdefault(req.request_id, [[] for _ in self.group_types])
        need = [max(0, self._needed(t, num_tokens_total) - len(g)) for t, g in zip(self.group_types, groups)]
        if sum(need) > self.block_pool.num_free_blocks():
            if not any(groups):
                self._req_blocks.pop(req.request_id, None)
            return None
        new = []
        for g, n in zip(groups, need):
            blks = self.block_pool.get_new_blocks(n)
            g.extend(blks)
            new.append(blks)
            if not skip_new_block_zeroing:
                self._pending_zero.update(b.block_id for b in blks)
        return KVCacheBlocks(tuple(new))

    def discard_new_block_ids(self, block_ids: Iterable[int]) -> None:
        """Blocks about to be filled by a connector load must not be zeroed afterwards."""
        self._pending_zero.difference_update(block_ids)

    def take_pending_zero(self) -> list:
        ids = sorted(self._pending_zero)
        self._pending_zero.clear()
        return ids

    def free(self, req: Request) -> None:
        groups = self._req_blocks.pop(req.request_id, None)
        if groups is None:
            return
        for g in groups:
            self.block_pool.free_blocks(reversed(g))

    def usage(self) -> float:
        total = len(self.block_pool.blocks) - 1
        return 1.0 - self.block_pool.num_free_blocks() / total if total > 0 else 0.0
