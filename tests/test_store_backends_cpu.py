"""The file backend and the store+KVT composites end to end on CPU."""
import os
import time

import pytest
import torch

from pd_helpers import make_cfg, make_req
from llumnix_kv_b200 import load_ops
from llumnix_kv_b200.engine.core import MiniEngineCore
from test_kvs_cpu import run, spy, wait_free


def test_file_backend_round_trip_and_format(tmp_path):
    e = MiniEngineCore(make_cfg("kv_both", "F", backend="local_file", extra={"cachedir": str(tmp_path)}))
    try:
        cap = spy(e)
        r1 = run(e, "a", 50)
        assert cap["a"][0] == 0 and wait_free(e, 63) == 63
        # at-rest format: <tokens joined by _>/<rank>.<layer name>.data + ready
        d = tmp_path / "_".join(str(t) for t in r1.prompt_token_ids[:16])
        assert (d / "ready").is_file()
        blk = torch.load(d / "0.model.layers.1.self_attn.attn.data")
        assert tuple(blk.shape) == (2, 16, 8, 32)
        w = e.workers[0]
        assert torch.equal(blk, w.expected_kv(1, r1.prompt_token_ids, 0, 16).transpose(0, 1))
        assert len(list(tmp_path.iterdir())) == 3
        for t in w.kv_caches.values():
            t.zero_()
        r2 = run(e, "b", 50)
        computed, blocks = cap["b"]
        assert computed == 48
        for layer in range(2):
            assert torch.equal(w.read_kv(layer, blocks[0], 0, 48), w.expected_kv(layer, r2.prompt_token_ids, 0, 48))
        assert wait_free(e, 63) == 63
    finally:
        e.shutdown()


def _pd_with_store(p_cfg):
    p = MiniEngineCore(p_cfg)
    d = MiniEngineCore(make_cfg("kv_consumer", "D"))
    return p, d


def _check_pd(p, d, rid, n):
    cap = spy(d)
    req = make_req(rid, n, max_tokens=2, params={"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()})
    d.add_request(req)
    out = d.wait_finished(rid, 30)
    assert out is not None and out.finish_reason.name == "LENGTH"
    computed, blocks = cap[rid]
    assert computed == n - 1
    w = d.workers[0]
    for layer in range(2):
        assert torch.equal(w.read_kv(layer, blocks[0], 0, n - 1), w.expected_kv(layer, req.prompt_token_ids, 0, n - 1))
    return req


def test_file_plus_kvt_prefill_engine(tmp_path):
    """kv_both + kvt: the prefill engine sends to the decode engine AND keeps the blocks on disk;
    the second identical prompt is served from disk on P and still transferred to D."""
    p, d = _pd_with_store(make_cfg("kv_both", "P", backend="kvt", extra={"cachedir": str(tmp_path)}))
    try:
        pcap = spy(p)
        _check_pd(p, d, "r1", 70)
        assert wait_free(p, 63) == 63
        assert len([x for x in tmp_path.iterdir() if (x / "ready").is_file()]) == 4
        for t in p.workers[0].kv_caches.values():
            t.zero_()
        _check_pd(p, d, "r2", 70)
        assert pcap["r2"][0] == 64          # P loaded 4 blocks from disk instead of recomputing them
        assert wait_free(p, 63) == 63 and wait_free(d, 63) == 63
    finally:
        d.shutdown()
        p.shutdown()


def test_kvs_plus_kvt_prefill_engine():
    name = f"kvx_kvsp_{os.getpid()}"
    p, d = _pd_with_store(make_cfg("kv_producer", "P", backend="kvt+kvs", extra={"kvs_name": name, "kvs_slots": 32}))
    try:
        pcap = spy(p)
        _check_pd(p, d, "r1", 90)
        assert wait_free(p, 63) == 63
        for t in p.workers[0].kv_caches.values():
            t.zero_()
        _check_pd(p, d, "r2", 90)
        assert pcap["r2"][0] == 80
        assert wait_free(p, 63) == 63 and wait_free(d, 63) == 63
        stats = p.connector.get_hybrid_connector_stats(64)
        assert stats.save_done_count_by_source.get("kvs") == 2 and stats.save_done_count_by_source.get("kvt") == 2
    finally:
        d.shutdown()
        p.shutdown()
        load_ops().KvStore.unlink(name)


def _find_store(backend, depth=0):
    """The store object behind a (possibly composite) worker backend."""
    st = getattr(backend, "_store", None)
    if st is not None and hasattr(st, "stats"):
        return st
    if depth < 3:
        for v in vars(backend).values():
            if hasattr(v, "__dict__") and type(v).__module__.startswith("llumnix_kv_b200.hybrid_connector"):
                found = _find_store(v, depth + 1)
                if found is not None:
                    return found
    return None


@pytest.mark.parametrize("backend,seed", [("kvt+kvs", 1), ("v6d_object+kvt", 2), ("file+kvt", 3)])
def test_random_requests_and_aborts_through_a_prefill_engine_that_also_stores(backend, seed, tmp_path):
    """A prefill engine that sends every prompt to the decode engine AND keeps it (shared store, object store
    flavour, or files): each request has two save sources on it, repeated prompts are served from what was kept,
    some requests are aborted on the decode side at random moments, a few transfers hit an injected fault.
    Every request ends, an untouched one decodes what its prompt always decodes, both engines get every block
    back and nothing stays reserved in the store."""
    import random

    from llumnix_kv_b200 import load_ops as _ops

    ops = _ops()
    rng = random.Random(seed)
    name = f"kvx_cmp_{os.getpid()}_{seed}"
    if backend == "file+kvt":
        p_cfg = make_cfg("kv_both", "P", backend="kvt", max_batched=64, extra={"cachedir": str(tmp_path)})
    else:
        p_cfg = make_cfg("kv_producer", "P", backend=backend, max_batched=64, extra={"kvs_name": name, "kvs_slots": 24})
    p, d = _pd_with_store(p_cfg)
    params = {"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()}
    try:
        lens = [30, 70, 120, 180]
        want = {}
        issued, touched = [], set()
        for i in range(24):
            k = rng.randrange(len(lens))
            rid = f"m{seed}.{i}"
            if rng.random() < 0.12:
                ops.fault_inject_arm(rng.randint(1, 3))
                touched.add("fault")
            d.add_request(make_req(rid, lens[k], max_tokens=2, seed=k, params=params))
            issued.append((rid, k))
            if rng.random() < 0.25:
                time.sleep(rng.choice([0.0, 0.004, 0.03, 0.1]))
                d.abort_requests([rid])
                touched.add(rid)
            if rng.random() < 0.4:
                time.sleep(rng.choice([0.01, 0.06]))
        ops.fault_inject_arm(0)
        for rid, k in issued:
            out = d.wait_finished(rid, 60)
            assert out is not None, rid
            how = out.finish_reason.name
            assert how in ("LENGTH", "ABORT"), (rid, how)
            if how == "LENGTH":
                want.setdefault(k, d.output_tokens(rid))
                assert d.output_tokens(rid) == want[k], rid
            else:
                assert rid in touched or "fault" in touched, rid
        deadline = time.time() + 20
        pools = [e.scheduler.kv_cache_manager.block_pool for e in (p, d)]
        while time.time() < deadline and (any(pl.num_free_blocks() != 63 for pl in pools) or p.connector._sched._saving
                                          or d.connector._sched._loading):
            time.sleep(0.01)
        left = {"free": [pl.num_free_blocks() for pl in pools], "p_saving": list(p.connector._sched._saving),
                "p_loading": list(p.connector._sched._loading), "d_loading": list(d.connector._sched._loading)}
        assert left["free"] == [63, 63] and not left["p_saving"] and not left["d_loading"], left
        if backend != "file+kvt":
            store = _find_store(p.workers[0].connector._worker._backend)
            assert store is not None
            end = time.time() + 10
            while time.time() < end and (store.stats()["writing"] or store.stats()["pinned"]):
                time.sleep(0.02)
            st = store.stats()
            assert st["writing"] == 0 and st["pinned"] == 0, st
    finally:
        ops.fault_inject_arm(0)
        d.shutdown()
        p.shutdown()
        if backend != "file+kvt":
            ops.KvStore.unlink(name)


def test_a_stored_block_that_cannot_be_read_is_a_miss_not_a_failed_request(tmp_path):
    """The second request finds its prefix in the file store, but one block's data has been damaged since it was
    written.  The load reports nothing loaded, the engine computes the prompt itself, and the request decodes
    what it always decodes: a cache that cannot deliver costs time, never the request (and never the worker:
    a failure object in a completion report used to end its process)."""
    e = MiniEngineCore(make_cfg("kv_both", "F", backend="local_file", extra={"cachedir": str(tmp_path)}))
    try:
        cap = spy(e)
        r1 = run(e, "a", 50)
        want = e.output_tokens("a")
        assert wait_free(e, 63) == 63
        d = tmp_path / "_".join(str(t) for t in r1.prompt_token_ids[:16])           # the first block of the prefix
        assert (d / "ready").is_file()
        (d / "0.model.layers.1.self_attn.attn.data").write_bytes(b"not a tensor")
        for t in e.workers[0].kv_caches.values():
            t.zero_()
        run(e, "b", 50)
        assert cap["b"][0] == 0                       # nothing counted as loaded: everything was computed here
        assert e.output_tokens("b") == want
        assert wait_free(e, 63) == 63 and not e.connector._sched._loading
    finally:
        e.shutdown()
