"""The store flavours (Vineyard / Mooncake / v6d_object, and the v6d_object+kvt composite) over the shared
host-DRAM store: each one's block names at rest, when a step's pages leave, who seals them, and that a second
request still loads what the first one saved."""
import hashlib
import os
import struct
import time

import pytest
import torch
import xxhash

from pd_helpers import make_cfg, make_req
from llumnix_kv_b200 import load_ops
from llumnix_kv_b200.engine.core import MiniEngineCore
from llumnix_kv_b200.engine.types import Request
from llumnix_kv_b200.hybrid_connector.backend import get_backend_cls
from llumnix_kv_b200.hybrid_connector.kvs_flavours import (MooncakeKVSBackend, V6dObjectBackend, mooncake_block_name,
                                                         name_to_store_key)
from llumnix_kv_b200.hybrid_connector.kvsbackend import KVSBackend
from test_kvs_cpu import run, spy, wait_free


@pytest.fixture
def store_name():
    name = f"kvx_flv_{os.getpid()}_{time.monotonic_ns() & 0xffff}"
    yield name
    load_ops().KvStore.unlink(name)


def engine(name, store, backend, **extra):
    e = {"kvs_name": store, "kvs_slots": 64}
    e.update(extra)
    return MiniEngineCore(make_cfg("kv_both", name, backend=backend, extra=e))


def test_selection_table_names_a_class_per_flavour():
    for backend, extra, cls in (("kvs", {}, KVSBackend), ("kvs", {"kvs_backend": "mooncake"}, MooncakeKVSBackend),
                                ("mooncake", {}, MooncakeKVSBackend), ("v6d_object", {}, V6dObjectBackend)):
        assert get_backend_cls(make_cfg("kv_both", "x", backend=backend, extra=extra)) is cls
    from llumnix_kv_b200.hybrid_connector.kvsp import KVSP, V6dObjectKVTBackend

    assert get_backend_cls(make_cfg("kv_producer", "x", backend="v6d_object+kvt")) is V6dObjectKVTBackend
    assert get_backend_cls(make_cfg("kv_producer", "x", backend="kvt+kvs")) is KVSP
    with pytest.raises(ValueError):
        get_backend_cls(make_cfg("kv_consumer", "x", backend="v6d_object+kvt"))


def test_block_names_at_rest():
    """Golden names: a Mooncake block is "<hex of the engine's block hash>_<tp rank>" and is found in the shared
    store under BLAKE2b-128 of that name; a v6d / Vineyard (request-hash mode) block is xxh64 of the block hash."""
    r = Request("r", list(range(1, 50)))
    hashes = r.compute_block_hashes(16)
    assert len(hashes) == 3 and all(len(h) == 32 for h in hashes)
    # the chain: hash_i = sha256(hash_{i-1} || tokens of block i as little-endian int64)
    h0 = hashlib.sha256(struct.pack("<16q", *range(1, 17))).digest()
    h1 = hashlib.sha256(h0 + struct.pack("<16q", *range(17, 33))).digest()
    assert hashes[0] == h0 and hashes[1] == h1
    assert mooncake_block_name(h0, 3) == h0.hex() + "_3"
    assert mooncake_block_name(bytes(range(32)), 0) == \
        "000102030405060708090a0b0c0d0e0f101112131415161718191a1b1c1d1e1f_0"
    assert name_to_store_key("abc_1") == hashlib.blake2b(b"abc_1", digest_size=16).digest()
    cfg = make_cfg("kv_both", "x", backend="mooncake", extra={"kvs_name": "unused"})
    from llumnix_kv_b200.hybrid_connector.engine_proxy import KVConnectorRole

    mc = MooncakeKVSBackend(cfg, KVConnectorRole.WORKER)
    assert mc.block_names([], hashes, 2, 1) == [h0.hex() + "_1", h1.hex() + "_1"]
    assert mc.store_keys([], hashes, 2, 1) == [hashlib.blake2b(n.encode(), digest_size=16).digest()
                                               for n in (h0.hex() + "_1", h1.hex() + "_1")]
    v6 = V6dObjectBackend(make_cfg("kv_both", "x", backend="v6d_object", extra={"kvs_name": "unused"}), KVConnectorRole.WORKER)
    assert v6.block_names([], hashes, 2, 0) == [xxhash.xxh64(h0).intdigest(), xxhash.xxh64(h1).intdigest()]
    assert v6.store_keys([], hashes, 1, 0) == [struct.pack("<QII", xxhash.xxh64(h0).intdigest(), 0, 1)]


@pytest.mark.parametrize("backend", ["mooncake", "v6d_object"])
def test_flavour_round_trip(store_name, backend):
    e = engine("A", store_name, backend)
    try:
        cap = spy(e)
        r1 = run(e, "a", 100)
        assert cap["a"][0] == 0
        assert wait_free(e, 63) == 63
        be = e.workers[0].connector._worker._backend
        assert type(be).FLAVOUR == backend
        # sealed blocks: by the worker after the step's last layer (mooncake), by the scheduler's cleanup (v6d_object)
        deadline = time.time() + 5
        while time.time() < deadline and be._store.stats()["sealed"] != 6:
            time.sleep(0.01)
        st = be._store.stats()
        assert st["sealed"] == 6 and st["writing"] == 0
        # the blocks are found under the flavour's own names
        hashes = Request("x", r1.prompt_token_ids).compute_block_hashes(16)
        keys = be.store_keys(r1.prompt_token_ids, hashes, 6, 0)
        assert be._store.lookup(keys) == 6
        for t in e.workers[0].kv_caches.values():
            t.zero_()
        r2 = run(e, "b", 100)
        computed, blocks = cap["b"]
        assert computed == 96
        w = e.workers[0]
        for layer in range(2):
            assert torch.equal(w.read_kv(layer, blocks[0], 0, 96), w.expected_kv(layer, r2.prompt_token_ids, 0, 96))
    finally:
        e.shutdown()


def test_vineyard_request_hash_mode(store_name, monkeypatch):
    monkeypatch.setenv("VLLM_KVS_USE_REQUEST_HASH", "1")
    e = engine("A", store_name, "kvs")
    try:
        cap = spy(e)
        r1 = run(e, "a", 70)
        assert wait_free(e, 63) == 63
        be = e.workers[0].connector._worker._backend
        hashes = Request("x", r1.prompt_token_ids).compute_block_hashes(16)
        keys = [struct.pack("<QII", xxhash.xxh64(h).intdigest(), 0, 1) for h in hashes[:4]]
        assert be._store.lookup(keys) == 4
        for t in e.workers[0].kv_caches.values():
            t.zero_()
        run(e, "b", 70)
        assert cap["b"][0] == 64
    finally:
        e.shutdown()


def test_v6d_object_failed_store_is_discarded_by_the_scheduler(store_name):
    """The worker reports a failed store with n == 0 in its save-done; the scheduler's cleanup then discards the
    request's pending blocks instead of sealing them, and a later request finds nothing."""
    e = engine("A", store_name, "v6d_object")
    try:
        be = e.workers[0].connector._worker._backend
        orig = be._store.check_status

        def boom():
            raise RuntimeError("injected store failure")

        be._store.check_status = boom
        cap = spy(e)
        run(e, "a", 100)
        assert wait_free(e, 63) == 63
        deadline = time.time() + 5
        while time.time() < deadline and be._store.stats()["writing"] != 0:
            time.sleep(0.01)
        st = be._store.stats()
        assert st["sealed"] == 0 and st["writing"] == 0
        be._store.check_status = orig
        run(e, "b", 100)
        assert cap["b"][0] == 0
    finally:
        e.shutdown()
