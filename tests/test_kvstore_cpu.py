"""Shared host-DRAM block store: index semantics (reserve / seal / discard / pin / TTL / LRU /
dead-writer reaping / cross-process sharing) and the CPU data path."""
import multiprocessing as mp
import os

import pytest
import torch

from llumnix_kv_b200 import load_ops
from llumnix_kv_b200.kvstore import PinnedKVStore, block_keys
from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape


def k(i: int) -> bytes:
    return i.to_bytes(8, "little") + (i * 7919 + 1).to_bytes(8, "little")


@pytest.fixture
def store():
    K = load_ops()
    name = f"kvx_test_{os.getpid()}"
    s = K.KvStore.open(name, 4096, 8, True, "t")
    yield K, s, name
    K.KvStore.unlink(name)


def test_reserve_seal_lookup_discard(store):
    K, s, _ = store
    assert s.lookup_prefix(k(1) + k(2)) == 0
    code, slot = s.reserve(k(1))
    assert code == K.STORE_RESERVE_NEW and slot == 0
    assert s.reserve(k(1))[0] == K.STORE_RESERVE_BUSY          # still being written
    assert s.lookup_prefix(k(1)) == 0                            # not visible before seal
    assert s.seal(k(1)) and not s.seal(k(1))
    assert s.reserve(k(1))[0] == K.STORE_RESERVE_EXISTS
    assert s.reserve(k(2)) == (K.STORE_RESERVE_NEW, 1)
    s.seal(k(2))
    assert s.lookup_prefix(k(1) + k(2) + k(3)) == 2
    assert s.lookup_prefix(k(3) + k(1)) == 0                     # a prefix stops at the first miss
    assert s.discard(k(1)) and s.lookup_prefix(k(1)) == 0
    st = s.stats()
    assert st["used"] == 1 and st["sealed"] == 1 and st["discards"] == 1


def test_lru_eviction_skips_pinned_and_writing(store):
    K, s, _ = store
    for i in range(8):
        assert s.reserve(k(i))[0] == K.STORE_RESERVE_NEW
        if i != 7:
            s.seal(k(i))                                         # entry 7 stays WRITING
    assert s.pin_prefix(k(0)) == [0]                             # pin the oldest
    s.lookup_prefix(k(1))                                        # touch 1: now 2 is the LRU victim
    code, slot = s.reserve(k(100))
    assert code == K.STORE_RESERVE_NEW and slot == 2
    assert s.lookup_prefix(k(2)) == 0 and s.lookup_prefix(k(0)) == 1 and s.lookup_prefix(k(1)) == 1
    assert s.stats()["evictions"] == 1
    s.unpin(k(0))
    assert s.stats()["pinned"] == 0


def test_full_when_nothing_evictable(store):
    K, s, _ = store
    for i in range(8):
        s.reserve(k(i))                                          # all WRITING
    assert s.reserve(k(50))[0] == K.STORE_RESERVE_FULL
    assert s.stats()["reserve_fail"] == 1
    assert s.discard(k(3))
    assert s.reserve(k(50)) == (K.STORE_RESERVE_NEW, 3)


def test_ttl_expiry(store):
    K, s, _ = store
    s.reserve(k(1), 1000)
    s.seal(k(1))
    s.reserve(k(2), 0)
    s.seal(k(2))
    assert s.lookup_prefix(k(1)) == 1
    s.advance_clock_for_test(1500)
    assert s.lookup_prefix(k(1)) == 0 and s.lookup_prefix(k(2)) == 1   # no TTL = never expires
    assert s.stats()["expired"] == 1 and s.stats()["used"] == 1


def test_many_keys_survive_deletions(store):
    """Backward-shift deletion keeps every remaining key reachable."""
    K, s, name = store
    big = K.KvStore.open(name + "_big", 64, 512, True, "t")
    try:
        for i in range(512):
            assert big.reserve(k(i))[0] == K.STORE_RESERVE_NEW
            big.seal(k(i))
        for i in range(0, 512, 3):
            assert big.discard(k(i))
        for i in range(512):
            assert big.lookup_prefix(k(i)) == (0 if i % 3 == 0 else 1), i
        for i in range(0, 512, 3):
            assert big.reserve(k(1000 + i))[0] == K.STORE_RESERVE_NEW
        assert big.stats()["used"] == 512
    finally:
        K.KvStore.unlink(name + "_big")


def _child_writer(name, q):
    K = load_ops()
    s = K.KvStore.open(name, 4096, 8, False, "t")
    s.reserve(k(9))
    s.seal(k(9))
    s.reserve(k(10))          # left WRITING when the process exits
    q.put("ok")


def test_shared_between_processes_and_dead_writer_reaped(store):
    K, s, name = store
    with pytest.raises(RuntimeError):
        K.KvStore.open(name, 4096, 8, False, "other-format")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_child_writer, args=(name, q))
    p.start()
    assert q.get(timeout=60) == "ok"
    p.join(30)
    assert s.lookup_prefix(k(9)) == 1                            # sealed by the other process
    assert s.reserve(k(10))[0] == K.STORE_RESERVE_BUSY
    assert s.reap_dead_writers() == 1
    assert s.reserve(k(10))[0] == K.STORE_RESERVE_NEW


def test_block_keys_are_prefix_chained():
    a = block_keys(list(range(64)), 16, 4)
    b = block_keys(list(range(48)) + [999] * 16, 16, 4)
    assert a[:3] == b[:3] and a[3] != b[3]
    c = block_keys([7] + list(range(1, 64)), 16, 4)
    assert all(x != y for x, y in zip(a, c))                     # a change in block 0 changes every key
    assert block_keys(list(range(64)), 16, 4, b"rank1") != a


@pytest.mark.parametrize("shape", [CacheShape.FLASH, CacheShape.FLASHINFER])
def test_cpu_round_trip_across_layouts(shape):
    """Saved from one layout, loaded into another: pages are layout-independent."""
    name = f"kvx_rt_{os.getpid()}"
    src_l = AttnLayout(shape, 12, 16, 4, 32, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER if shape == CacheShape.FLASH else CacheShape.FLASH, 12, 16, 4, 32, 2)
    src = [src_l.alloc("cpu", fill="normal", seed=i) for i in range(3)]
    dst = [dst_l.alloc("cpu") for _ in range(3)]
    a = PinnedKVStore(name, src_l, src, 0, 1, 16, create=True)
    b = PinnedKVStore(name, dst_l, dst, 0, 1, 16, create=False)
    try:
        toks = list(range(100, 100 + 80))
        keys = a.keys(toks, 5)
        new, full = a.reserve(keys)
        assert not full and [i for i, _ in new] == [0, 1, 2, 3, 4]
        blocks = [7, 3, 9, 1, 5]
        a.save_layers(0, 3, blocks, [s for _, s in new])
        assert b.lookup(keys) == 0
        a.seal(keys)
        assert b.lookup(keys) == 5 and b.lookup(b.keys(toks[:48] + [1] * 32, 5)) == 3
        slots = b.pin(keys)
        assert len(slots) == 5
        into = [2, 4, 6, 8, 10]
        b.load_layers(0, 3, into, slots)
        b.unpin(keys)
        for layer in range(3):
            sv = src_l.view(src[layer], torch.int16)[blocks]
            dv = dst_l.view(dst[layer], torch.int16)[into]
            assert torch.equal(sv, dv)
        assert a.reserve(keys) == ([], False)                    # everything already stored
    finally:
        a.close()
        b.close()
        load_ops().KvStore.unlink(name)


def _child_reader(name, q):
    K = load_ops()
    s = K.KvStore.open(name, 4096, 8, False, "t")
    q.put(s.pin_prefix(k(0) + k(1)))          # exits holding both pins


def test_pins_of_a_dead_reader_are_released_and_clear_keeps_pinned_slots(store):
    K, s, name = store
    for i in range(4):
        s.reserve(k(i))
        s.seal(k(i))
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_child_reader, args=(name, q))
    p.start()
    assert q.get(timeout=60) == [0, 1]
    p.join(30)
    assert s.pin_prefix(k(1)) == [1]                             # our own pin on top of the dead reader's
    assert not s.discard(k(0)) and s.stats()["pinned"] == 2
    assert s.reap_dead_readers() == 2                            # the child's two pins, not ours
    assert s.discard(k(0)) and not s.discard(k(1))
    assert s.clear() == 1                                        # entry 1 is being read: it stays
    assert s.lookup_prefix(k(1)) == 1 and s.lookup_prefix(k(2)) == 0 and s.stats()["used"] == 1
    assert s.reserve(k(2))[0] == K.STORE_RESERVE_NEW             # freed slots are usable again
    s.unpin(k(1))
    assert s.reap_dead_readers() == 0 and s.clear() == 0 and s.stats()["used"] == 0


def test_recency_list_matches_a_model_under_random_traffic(store):
    """Evictions come from the recency list, never from a scan of the table.  Random reserve / seal / lookup /
    discard / pin traffic against a model that keeps the same order: every eviction must take the model's
    least recently used unpinned sealed key, through thousands of deletions that move entries between buckets."""
    import random

    K, s, _ = store          # 8 slots
    rng = random.Random(7)
    order: list = []         # sealed keys, least recent first
    writing: set = set()
    pinned: dict = {}
    for step in range(6000):
        i = rng.randrange(40)
        op = rng.random()
        if op < 0.45:
            code, _slot = s.reserve(k(i))
            if i in order:
                assert code == K.STORE_RESERVE_EXISTS
                order.remove(i)
                order.append(i)
            elif i in writing:
                assert code == K.STORE_RESERVE_BUSY
            else:
                used = len(order) + len(writing)
                if used == 8:
                    victims = [x for x in order if pinned.get(x, 0) == 0]
                    if not victims:
                        assert code == K.STORE_RESERVE_FULL
                        continue
                    order.remove(victims[0])
                    assert s.lookup_prefix(k(victims[0])) == 0, (step, victims[0])      # exactly that key went
                assert code == K.STORE_RESERVE_NEW, (step, code)
                writing.add(i)
        elif op < 0.70:
            if i in writing:
                assert s.seal(k(i))
                writing.discard(i)
                order.append(i)
        elif op < 0.85:
            hit = s.lookup_prefix(k(i))
            assert hit == (1 if i in order else 0)
            if i in order:
                order.remove(i)
                order.append(i)
        elif op < 0.92:
            ok = s.discard(k(i))
            assert ok == ((i in order and pinned.get(i, 0) == 0) or i in writing)
            if ok:
                writing.discard(i)
                if i in order:
                    order.remove(i)
        elif op < 0.97:
            got = s.pin_prefix(k(i))
            assert len(got) == (1 if i in order else 0)
            if i in order:
                pinned[i] = pinned.get(i, 0) + 1
                order.remove(i)
                order.append(i)
        else:
            if pinned.get(i, 0) > 0:
                s.unpin(k(i))
                pinned[i] -= 1
        st = s.stats()
        assert st["used"] == len(order) + len(writing) and st["sealed"] == len(order), step


def _hammer(name, seed, n_ops, q):
    """One of several processes on one store: random reserve + write + seal / pin + verify + unpin / discard."""
    import ctypes
    import random

    K = load_ops()
    s = K.KvStore.open(name, 4096, 16, False, "t")
    rng = random.Random(seed)
    base, sb = s.data_ptr, s.slot_bytes
    held = []                                   # (key index, slot) pinned by this process
    torn = written = verified = 0
    for _ in range(n_ops):
        i = rng.randrange(48)
        op = rng.random()
        if op < 0.40:
            code, slot = s.reserve(k(i))
            if code == K.STORE_RESERVE_NEW:
                # the slot is this process's until it seals: fill it with the key's pattern, first and last word last
                pat = (i * 0x01010101 + 0x5A5A5A5A) & 0xFFFFFFFF
                buf = (ctypes.c_uint32 * (sb // 4)).from_address(base + slot * sb)
                for w in range(1, sb // 4 - 1, 61):
                    buf[w] = pat
                buf[0] = buf[sb // 4 - 1] = pat
                if rng.random() < 0.9:
                    s.seal(k(i))
                else:
                    s.discard(k(i))
                written += 1
        elif op < 0.75:
            got = s.pin_prefix(k(i))
            if got:
                slot = got[0]
                pat = (i * 0x01010101 + 0x5A5A5A5A) & 0xFFFFFFFF
                buf = (ctypes.c_uint32 * (sb // 4)).from_address(base + slot * sb)
                # a pinned, sealed slot must hold its key's bytes for as long as the pin lasts
                if buf[0] != pat or buf[sb // 4 - 1] != pat or buf[1] != pat:
                    torn += 1
                held.append((i, slot))
                verified += 1
        elif op < 0.90:
            if held:
                i2, slot = held.pop(rng.randrange(len(held)))
                pat = (i2 * 0x01010101 + 0x5A5A5A5A) & 0xFFFFFFFF
                buf = (ctypes.c_uint32 * (sb // 4)).from_address(base + slot * sb)
                if buf[0] != pat or buf[sb // 4 - 1] != pat:
                    torn += 1                   # evicted or rewritten under the pin
                s.unpin(k(i2))
        elif op < 0.95:
            s.discard(k(i))
        else:
            s.lookup_prefix(k(i) + k((i + 1) % 48))
    for i2, _slot in held:
        s.unpin(k(i2))
    q.put((torn, written, verified))


def test_four_processes_hammering_one_store_never_see_a_torn_or_stolen_slot(store):
    """Writers fill a reserved slot with a pattern of its key and seal it; readers pin a key and check the slot
    holds that key's pattern when pinned and still when unpinned later, while the other processes keep reserving
    (evicting), discarding and looking up.  Nothing is ever seen half-written or replaced under a pin, the index
    ends consistent and no pin is left."""
    K, _s8, _ = store
    name = f"kvx_hammer_{os.getpid()}"
    s = K.KvStore.open(name, 4096, 16, True, "t")
    try:
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        procs = [ctx.Process(target=_hammer, args=(name, 100 + i, 4000, q)) for i in range(4)]
        for p in procs:
            p.start()
        results = [q.get(timeout=180) for _ in procs]
        for p in procs:
            p.join(30)
            assert p.exitcode == 0
        assert sum(r[0] for r in results) == 0, results
        assert sum(r[1] for r in results) > 500 and sum(r[2] for r in results) > 500, results
        st = s.stats()
        assert st["pinned"] == 0 and st["writing"] == 0 and st["used"] == st["sealed"] <= 16, st
        assert s.reap_dead_readers() == 0 and s.reap_dead_writers() == 0
    finally:
        K.KvStore.unlink(name)
