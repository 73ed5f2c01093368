"""The "kvs" backend end to end on CPU: prefixes saved to the shared host-DRAM store by one
request are loaded by the next, by another engine of the node, and across cache layouts."""
import os
import time

import pytest
import torch

from pd_helpers import make_cfg, make_req
from llumnix_kv_b200 import load_ops
from llumnix_kv_b200.engine.core import MiniEngineCore


def make_kvs(name, store, **kw):
    extra = {"kvs_name": store, "kvs_slots": 64}
    extra.update(kw.pop("extra", {}))
    return MiniEngineCore(make_cfg("kv_both", name, backend="kvs", extra=extra, **kw))


def spy(e):
    captured = {}
    orig = e.scheduler.add_request

    def f(r):
        captured[r.request_id] = (r.num_computed_tokens, e.scheduler.kv_cache_manager.get_block_ids(r.request_id))
        orig(r)

    e.scheduler.add_request = f
    return captured


def wait_free(e, n, t=5.0):
    pool = e.scheduler.kv_cache_manager.block_pool
    end = time.time() + t
    while time.time() < end and pool.num_free_blocks() != n:
        time.sleep(0.01)
    return pool.num_free_blocks()


@pytest.fixture
def store_name():
    name = f"kvx_kvs_{os.getpid()}_{time.monotonic_ns() & 0xffff}"
    yield name
    load_ops().KvStore.unlink(name)


def run(e, rid, n, max_tokens=2, seed=0, params=None):
    req = make_req(rid, n, max_tokens=max_tokens, seed=seed, params=params)
    e.add_request(req)
    out = e.wait_finished(rid, 30)
    assert out is not None and out.finish_reason.name == "LENGTH", rid
    return req


def test_second_request_loads_what_the_first_saved(store_name):
    e = make_kvs("A", store_name)
    try:
        cap = spy(e)
        r1 = run(e, "a", 100)
        assert cap["a"][0] == 0                         # nothing in the store yet
        assert wait_free(e, 63) == 63                   # save finished, extra references dropped
        st = e.workers[0].connector._worker._backend._store.stats()
        assert st["sealed"] == 6 and st["writing"] == 0  # 100 tokens = 6 full blocks of 16
        # wipe the engine's own cache so that only the store can supply the prefix
        for t in e.workers[0].kv_caches.values():
            t.zero_()
        r2 = run(e, "b", 100)
        computed, blocks = cap["b"]
        assert computed == 96
        w = e.workers[0]
        for layer in range(2):
            assert torch.equal(w.read_kv(layer, blocks[0], 0, 96), w.expected_kv(layer, r2.prompt_token_ids, 0, 96))
        assert e.output_tokens("a") == e.output_tokens("b")
        # a prompt that shares only the first 40 tokens reuses 2 blocks
        toks = list(r1.prompt_token_ids[:40]) + [5] * 60
        from llumnix_kv_b200.engine.types import EngineCoreRequest, SamplingParams
        e.add_request(EngineCoreRequest("c", toks, SamplingParams(max_tokens=1, extra_args={"kv_transfer_params": {}}), None))
        assert e.wait_finished("c", 30) is not None
        assert cap["c"][0] == 32
        assert wait_free(e, 63) == 63
        stats = e.connector.get_hybrid_connector_stats(64)
        assert stats.save_done_count == 3 and stats.load_done_count >= 2 and stats.save_failed_count == 0
    finally:
        e.shutdown()


@pytest.mark.parametrize("gran", ["layer", "step"])
def test_chunked_prefill_saves_block_by_block(store_name, gran):
    e = make_kvs("A", store_name, max_batched=40, extra={"kvs_save_granularity": gran})
    try:
        run(e, "a", 130)
        assert wait_free(e, 63) == 63
        st = e.workers[0].connector._worker._backend._store.stats()
        assert st["sealed"] == 8 and st["writing"] == 0
        assert e.steps >= 4
        # what was stored is what was computed: load it back into a wiped cache
        cap = spy(e)
        for t in e.workers[0].kv_caches.values():
            t.zero_()
        r = run(e, "b", 130)
        computed, blocks = cap["b"]
        assert computed == 128
        w = e.workers[0]
        for layer in range(2):
            assert torch.equal(w.read_kv(layer, blocks[0], 0, 128), w.expected_kv(layer, r.prompt_token_ids, 0, 128))
    finally:
        e.shutdown()


def test_another_engine_with_another_layout_loads_it(store_name):
    a = make_kvs("A", store_name, cache_shape=2)
    b = make_kvs("B", store_name, cache_shape=5)
    try:
        r = run(a, "x", 70)
        assert wait_free(a, 63) == 63
        cap = spy(b)
        run(b, "y", 70)
        computed, blocks = cap["y"]
        assert computed == 64
        w = b.workers[0]
        for layer in range(2):
            assert torch.equal(w.read_kv(layer, blocks[0], 0, 64), w.expected_kv(layer, r.prompt_token_ids, 0, 64))
    finally:
        a.shutdown()
        b.shutdown()


def test_tp2_needs_every_rank(store_name):
    e = make_kvs("A", store_name, tp=2)
    try:
        cap = spy(e)
        r = run(e, "a", 50)
        assert wait_free(e, 63) == 63
        # drop rank 1's copy of the second block: only one block can be loaded now
        be = e.workers[1].connector._worker._backend
        keys = be._store.keys(r.prompt_token_ids, 3)
        assert be._store.kv.discard(keys[1])
        run(e, "b", 50)
        assert cap["b"][0] == 16
    finally:
        e.shutdown()


def test_abort_mid_prefill_discards_unsealed_blocks(store_name):
    e = make_kvs("A", store_name, max_batched=16, extra={"kvs_abort_grace_s": 0.05})
    try:
        e.add_request(make_req("a", 960, max_tokens=2))     # 60 engine steps of 16 tokens: still prefilling below
        time.sleep(0.02)
        e.abort_requests(["a"])
        out = e.wait_finished("a", 20)
        assert out is not None and out.finish_reason.name == "ABORT"
        assert wait_free(e, 63) == 63
        st = e.workers[0].connector._worker._backend._store.stats()
        assert st["writing"] == 0
        assert not e.connector._sched._saving
    finally:
        e.shutdown()


def test_nosave_and_min_length(store_name, monkeypatch):
    e = make_kvs("A", store_name)
    try:
        run(e, "a", 60, params={"kvs_nosave": True})
        assert e.workers[0].connector._worker._backend._store.stats()["used"] == 0
        monkeypatch.setenv("VLLM_KVS_ON_MIN_LENGTH", "100")
        run(e, "b", 60)
        assert e.workers[0].connector._worker._backend._store.stats()["used"] == 0
    finally:
        e.shutdown()


def test_many_concurrent_requests_with_shared_prefixes(store_name):
    """Two batches of 16 concurrent requests over 4 distinct prompts while the store is smaller than what they would
    need without sharing: every request finishes with the right tokens, nothing stays reserved or
    pinned, and later copies of a prompt are served from the store."""
    e = make_kvs("A", store_name, num_blocks=256, max_batched=256, extra={"kvs_slots": 40})
    try:
        cap = spy(e)
        lens = [70, 150, 230, 95]
        first = {}
        for half in (range(0, 4), range(4, 8)):
            for wave in half:
                for k, n in enumerate(lens):
                    e.add_request(make_req(f"w{wave}k{k}", n, max_tokens=2, seed=k))
            for wave in half:
                for k, n in enumerate(lens):
                    rid = f"w{wave}k{k}"
                    out = e.wait_finished(rid, 60)
                    assert out is not None and out.finish_reason.name == "LENGTH", rid
                    first.setdefault(k, e.output_tokens(rid))
                    assert e.output_tokens(rid) == first[k]
        assert wait_free(e, 255, 10) == 255
        st = e.workers[0].connector._worker._backend._store.stats()
        assert st["writing"] == 0 and st["pinned"] == 0 and st["sealed"] <= 40
        reused = sum(1 for rid, (computed, _) in cap.items() if computed > 0)
        assert reused >= 16, reused      # the second half looked up after the first half had sealed
    finally:
        e.shutdown()


def test_nan_in_hidden_states_keeps_the_step_out_of_the_store(store_name, monkeypatch):
    """With the NaN check on, a forward pass whose hidden states hold a NaN seals nothing: the
    request finishes, its blocks are released, and the next request with that prompt finds no prefix."""
    monkeypatch.setenv("VLLM_KVS_STORE_NAN_CHECK", "1")
    e = make_kvs("A", store_name)
    try:
        cap = spy(e)
        w = e.workers[0]
        poisoned = {"on": True}
        w.hidden_states_hook = lambda n: torch.tensor([1.0, float("nan") if poisoned["on"] else 2.0])
        run(e, "a", 100)
        assert wait_free(e, 63) == 63
        st = w.connector._worker._backend._store.stats()
        assert st["sealed"] == 0 and st["writing"] == 0 and st["used"] == 0
        poisoned["on"] = False
        run(e, "b", 100)
        assert cap["b"][0] == 0                         # nothing was kept from the poisoned pass
        assert wait_free(e, 63) == 63
        assert w.connector._worker._backend._store.stats()["sealed"] == 6
        run(e, "c", 100)
        assert cap["c"][0] == 96
    finally:
        e.shutdown()


def test_trace_context_reaches_the_store_operations(store_name):
    """A request that carries a W3C traceparent header has its save and its load tagged with child
    spans of that trace (same trace id, another span id per operation), start and end marked."""
    e = make_kvs("A", store_name)
    try:
        tp = "00-0af7651916cd43dd8448eb211c80319c-b7ad6b7169203331-01"
        for rid in ("a", "b"):
            req = make_req(rid, 100, max_tokens=2)
            req.trace_headers = {"traceparent": tp}
            e.add_request(req)
            assert e.wait_finished(rid, 30) is not None
            assert wait_free(e, 63) == 63
        ctx = list(e.workers[0].connector._worker._backend.request_contexts)
        saves = [c for c in ctx if c.startswith("a;")]
        assert len(saves) == 2 and saves[0].endswith(";op=start") and saves[1].endswith(";op=end")
        child = saves[0].split(";")[1]
        ver, trace_id, span, flags = child.split("-")
        assert (ver, trace_id, flags) == ("00", "0af7651916cd43dd8448eb211c80319c", "01")
        assert len(span) == 16 and span != "b7ad6b7169203331"
        loads = [c for c in ctx if c.startswith("b;") and "op=" not in c]
        assert len(loads) == 1 and loads[0].split(";")[1].split("-")[1] == trace_id
        assert loads[0].split(";")[1].split("-")[2] not in (span, "b7ad6b7169203331")     # kv_load is its own span
        # requests without the header are tagged with their id alone
        run(e, "c", 40)
        assert "c" in [c for c in e.workers[0].connector._worker._backend.request_contexts if c.startswith("c")]
    finally:
        e.shutdown()


@pytest.mark.parametrize("backend,seed,tp", [("kvs", 1, 1), ("kvs", 2, 1), ("mooncake", 3, 1), ("v6d_object", 4, 1), ("kvs", 5, 2)])
def test_random_requests_and_aborts_on_two_engines_sharing_a_store(store_name, seed, backend, tp):
    """Two engines of a node share one store (any flavour) that is too small for everything; requests over a handful of prompts
    (so prefixes are shared, saved by one engine and loaded by the other) arrive at random and some are aborted
    while they load, prefill or save.  Every request that was not aborted produces the tokens its prompt always
    produces, both engines get every block back, and the store keeps nothing reserved or pinned.  With ``tp`` 2
    every rank of an engine keeps its own pages of a block and a prefix counts only when all ranks have it."""
    import random

    rng = random.Random(seed)
    extra = {"kvs_name": store_name, "kvs_slots": 24, "kvs_abort_grace_s": 0.05}
    a, b = (MiniEngineCore(make_cfg("kv_both", n, backend=backend, num_blocks=128, max_batched=64, tp=tp, extra=dict(extra)))
            for n in "AB")
    try:
        lens = [40, 75, 130, 200, 260]
        want = {}
        for k, n in enumerate(lens):                              # what each prompt decodes to
            run(a, f"ref{k}", n, max_tokens=3, seed=k)
            want[k] = a.output_tokens(f"ref{k}")
        issued, aborted = [], set()
        for i in range(40):
            k = rng.randrange(len(lens))
            e = rng.choice((a, b))
            rid = f"s{seed}.{i}"
            e.add_request(make_req(rid, lens[k], max_tokens=3, seed=k))
            issued.append((rid, k, e))
            if rng.random() < 0.25:
                time.sleep(rng.choice([0.0, 0.003, 0.02, 0.08]))
                e.abort_requests([rid])
                aborted.add(rid)
            if rng.random() < 0.3:
                time.sleep(rng.choice([0.01, 0.05]))
        done = 0
        for rid, k, e in issued:
            out = e.wait_finished(rid, 60)
            assert out is not None, rid
            if out.finish_reason.name == "LENGTH":
                assert e.output_tokens(rid) == want[k], rid
                done += 1
            else:
                assert out.finish_reason.name == "ABORT" and rid in aborted, (rid, out.finish_reason.name)
        assert done >= len(issued) - len(aborted)
        for e in (a, b):
            assert wait_free(e, 127, 15) == 127
            assert not e.connector._sched._saving and not e.connector._sched._loading
        deadline = time.time() + 10
        store = a.workers[0].connector._worker._backend._store
        while time.time() < deadline and (store.stats()["writing"] or store.stats()["pinned"]):
            time.sleep(0.02)
        st = store.stats()
        assert st["writing"] == 0 and st["pinned"] == 0 and st["sealed"] <= 24, st
    finally:
        a.shutdown()
        b.shutdown()
