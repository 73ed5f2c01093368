"""Live migration between engines on CPU: a frontend hands requests to engines, moves them while
they decode, and gets one uninterrupted token stream whichever engines produced it."""
import time

import pytest
import torch

from pd_helpers import make_cfg, make_req
from llumnix_kv_b200.engine.core import MiniEngineCore
from llumnix_kv_b200.hybrid_connector.migration import int2ipport, ipport2int, is_migration
from llumnix_kv_b200.hybrid_connector.migration.frontend import MigrationCli

LOCAL = {"ali_llumnix_disagg": False}


def make_engine(name, **kw):
    return MiniEngineCore(make_cfg("kv_both", name, backend="kvt+migration", **kw))


def addr(e):
    return ("127.0.0.1", e.proxy.rpc_port())


def baseline_tokens(n_prompt, max_tokens, seed=0):
    """What one engine produces for this prompt without any migration."""
    e = MiniEngineCore(make_cfg("kv_both", "base", backend="kvt+migration"))
    try:
        e.add_request(make_req("b", n_prompt, max_tokens=max_tokens, seed=seed, params=LOCAL))
        assert e.wait_finished("b", 30) is not None
        return e.output_tokens("b")
    finally:
        e.shutdown()


def wait_free(e, n, t=5.0):
    pool = e.scheduler.kv_cache_manager.block_pool
    end = time.time() + t
    while time.time() < end and pool.num_free_blocks() != n:
        time.sleep(0.01)
    return pool.num_free_blocks()


def test_ipport_roundtrip():
    v = ipport2int("10.1.2.3", 40000)
    assert is_migration(v) and int2ipport(v) == ("10.1.2.3", 40000) and not is_migration(7)


@pytest.fixture
def two():
    a, b = make_engine("A"), make_engine("B")
    yield a, b
    a.shutdown()
    b.shutdown()


def test_outputs_reach_the_frontend_without_migration(two):
    a, b = two
    cli = MigrationCli([addr(a), addr(b)])
    try:
        cli.add_request(make_req("r", 30, max_tokens=5, params=LOCAL))
        st = cli.wait("r", 30)
        assert st is not None and st.finish_reason == 1 and st.tokens == baseline_tokens(30, 5)
        assert st.migrations == 0
    finally:
        cli.close()


def test_migrate_while_decoding_moves_kv_and_continues_the_stream(two):
    a, b = two
    cli = MigrationCli([addr(a), addr(b)], migrate_after_first_token=True)
    try:
        slow = a.step
        a.step = lambda: (time.sleep(0.01), slow())[1]       # keep the source decoding while it is asked to let go
        cli.add_request(make_req("m", 45, max_tokens=40, params=LOCAL), engine=addr(a))
        st = cli.wait("m", 60)
        assert st is not None and st.finish_reason == 1
        assert st.migrations == 1 and st.engines_seen == [addr(a), addr(b)]
        assert st.tokens == baseline_tokens(45, 40)
        assert b.steps > 3                                    # the destination really decoded
        assert wait_free(a, 63) == 63 and wait_free(b, 63) == 63
        assert not a.connector._sched._saving and not b.connector._sched._loading
        assert b.connector._sched._backend.migration_status() == {"migrate_in": {}, "migrate_out": []}
    finally:
        cli.close()


def test_migrate_before_first_token_restarts_on_destination(two):
    a, b = two
    cli = MigrationCli([addr(a), addr(b)])
    try:
        a._stop = True           # the source engine loop is frozen: the request stays waiting there
        a.input_queue.put_nowait((None, None))
        time.sleep(0.1)
        cli.add_request(make_req("w", 33, max_tokens=4, params=LOCAL), engine=addr(a))
        a._stop = False
        a.start()
        code = cli.migrate("w", addr(b))
        assert code == 0
        st = cli.wait("w", 60)
        assert st is not None and st.tokens == baseline_tokens(33, 4)
    finally:
        cli.close()


def test_admission_control_rejects_when_busy(two, monkeypatch):
    a, b = two
    cli = MigrationCli([addr(a), addr(b)])
    try:
        monkeypatch.setenv("LLUMNIX_MAX_REQ_MIG_IN", "0")
        cli.add_request(make_req("x", 20, max_tokens=30, params=LOCAL), engine=addr(a))
        assert cli.migrate("x", addr(b)) == 1001
        assert cli.rejected == 1
        st = cli.wait("x", 60)                                # it simply finishes where it was
        assert st is not None and st.migrations == 0 and len(st.tokens) == 30
    finally:
        cli.close()


def test_abort_through_the_frontend(two):
    a, b = two
    cli = MigrationCli([addr(a), addr(b)])
    try:
        cli.add_request(make_req("k", 20, max_tokens=100000, params=LOCAL), engine=addr(a))
        time.sleep(0.2)
        cli.abort("k")
        st = cli.wait("k", 30)
        assert st is not None and st.finish_reason == 2
        assert wait_free(a, 63) == 63
    finally:
        cli.close()


_VARIANTS = {
    "plain": {},
    "tp2": dict(tp=2),
    "gdn": dict(cache_shape=3, layers=8, gdn_groups=3),
    "mla": dict(cache_shape=4, mla=(64, 16, 36), block_size=64, num_blocks=64),
}


@pytest.mark.parametrize("variant,seed", [("plain", 1), ("plain", 2), ("tp2", 3), ("gdn", 4), ("mla", 5)])
def test_random_migrations_on_every_kind_of_engine(variant, seed):
    """The random migrations below on tensor-parallel engines, on a hybrid model (recurrent state pages travel with
    the attention pages) and on an MLA model."""
    kw = _VARIANTS[variant]
    a, b = make_engine("A", **kw), make_engine("B", **kw)
    try:
        test_random_migrations_keep_every_stream_intact((a, b), seed, kw)
    finally:
        a.shutdown()
        b.shutdown()


@pytest.mark.parametrize("seed", [6])
def test_random_migrations_keep_every_stream_intact(two, seed, kw=None):
    """Several requests decode on two engines while the frontend keeps asking, at random moments, to move a
    random one of them to the other engine (some asks come too early, some too late, some are refused).
    Whatever happened to a request on the way, its token stream is the one a single engine produces, every
    block returns to its pool and no engine remembers a migration."""
    import random

    rng = random.Random(seed)
    a, b = two
    for e in (a, b):
        step = e.step
        e.step = (lambda s: lambda: (time.sleep(0.004), s())[1])(step)       # slow decoding: migrations land mid-stream
    cli = MigrationCli([addr(a), addr(b)])
    shapes = [(rng.randint(10, 70), rng.randint(15, 40)) for _ in range(6)]
    try:
        # the reference streams, from one engine, before anything migrates
        ref = MiniEngineCore(make_cfg("kv_both", "base", backend="kvt+migration", **(kw or {})))
        try:
            for i, (n, m) in enumerate(shapes):
                ref.add_request(make_req(f"b{i}", n, max_tokens=m, seed=seed * 50 + i, params=LOCAL))
            want = []
            for i in range(len(shapes)):
                assert ref.wait_finished(f"b{i}", 60) is not None
                want.append(ref.output_tokens(f"b{i}"))
        finally:
            ref.shutdown()
        for i, (n, m) in enumerate(shapes):
            cli.add_request(make_req(f"q{i}", n, max_tokens=m, seed=seed * 50 + i, params=LOCAL))
        codes = []
        end = time.time() + 1.5
        while time.time() < end:
            i = rng.randrange(len(shapes))
            st = cli._reqs[f"q{i}"]
            other = addr(b) if st.engine == addr(a) else addr(a)
            codes.append(cli.migrate(f"q{i}", other))
            time.sleep(rng.choice([0.0, 0.01, 0.05]))
        moved = 0
        for i in range(len(shapes)):
            st = cli.wait(f"q{i}", 90)
            assert st is not None and st.finish_reason == 1, (i, codes)
            assert st.tokens == want[i], (i, st.migrations, codes)
            moved += st.migrations
        assert moved >= 1, codes                                  # the test did migrate something
        free_all = a.cfg.cache_config.num_gpu_blocks - 1
        assert wait_free(a, free_all, 15) == free_all and wait_free(b, free_all, 15) == free_all
        for e in (a, b):
            assert not e.connector._sched._saving and not e.connector._sched._loading
            assert e.connector._sched._backend.migration_status() == {"migrate_in": {}, "migrate_out": []}
    finally:
        cli.close()
