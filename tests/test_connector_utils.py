"""Unit tests of the connector's small parts: completion counting, the native engine's send-done wire
formats, peer records, operation-plan merging, cleanup reference counts."""
import asyncio
import struct

import pytest

from llumnix_kv_b200.engine.types import Request
from llumnix_kv_b200.hybrid_connector.backend import (dec_cleanup_rc, inc_cleanup_rc, merge_operation_plans,
                                                       set_operation_sources)
from llumnix_kv_b200.hybrid_connector.engine_proxy import get_param
from llumnix_kv_b200.hybrid_connector.utils import (CodeError, IoRet, IoState, PeerInfo, PeerManager, ConnManager,
                                                     handle_done_req, try_advance)


def test_io_state_counts_ranks_and_signals():
    st = {"r": IoState(signals_per_worker=2)}
    assert try_advance(st, IoRet(reqid="r", n=10), 0, 2) is None
    assert try_advance(st, IoRet(reqid="r", n=12), 0, 2) is None          # rank 0 complete, rank 1 missing
    assert try_advance(st, IoRet(reqid="r", n=9), 0, 2) is None           # a third signal from rank 0 is a duplicate
    assert try_advance(st, IoRet(reqid="r", n=11), 1, 2) is None
    done = try_advance(st, IoRet(reqid="r", n=13), 1, 2)
    assert done is st["r"] and done.merge().n == 10                       # the minimum over all signals
    assert try_advance(st, IoRet(reqid="unknown"), 0, 2) is None


def test_io_state_with_named_sources():
    s = IoState(signals_per_worker=2)
    s.expected_sources = ("kvs", "kvt")
    st = {"r": s}
    assert try_advance(st, IoRet(reqid="r", source="kvs"), 0, 1) is None
    assert try_advance(st, IoRet(reqid="r", source="kvs"), 0, 1) is None   # same source twice: ignored
    assert try_advance(st, IoRet(reqid="r", source="other"), 0, 1) is None
    assert try_advance(st, IoRet(reqid="r", source="kvt"), 0, 1) is s


def test_merge_keeps_the_first_failure():
    s = IoState()
    st = {"r": s}
    try_advance(st, IoRet(reqid="r", n=5), 0, 2)
    try_advance(st, IoRet(reqid="r", n=0, ex=CodeError(500, "boom")), 1, 2)
    m = s.merge()
    assert isinstance(m.ex, CodeError) and m.ex.code == 500


class _Writer:
    def __init__(self):
        self.buf = b""

    def write(self, b):
        self.buf += b

    async def drain(self):
        pass


def _parse(body: bytes):
    got = []

    async def main():
        reader = asyncio.StreamReader()
        reader.feed_data(body)
        reader.feed_eof()
        w = _Writer()
        await handle_done_req(reader, w, lambda rank, r: got.append((rank, r.reqid, r.n, getattr(r.ex, "code", None))), 77)
        return w.buf

    resp = asyncio.run(main())
    assert resp == struct.pack("=I", 77)
    return got


def test_send_done_version2_body():
    body = struct.pack("=II", 3 | 0x40000000, 2)
    body += struct.pack("=III", 100, 0, 2) + b"r1" + struct.pack("=III", 0, 500, 3) + b"bad"
    assert _parse(body) == [(3, "r1", 100, None), (3, "bad", 0, 500)]


def test_send_done_version1_bodies():
    plain = struct.pack("=II", 1, 2) + struct.pack("=I", 1) + b"a" + struct.pack("=I", 2) + b"bb"
    assert _parse(plain) == [(1, "a", None, None), (1, "bb", None, None)]
    with_plen = struct.pack("=II", 1 | 0x80000000, 2) + struct.pack("=I", 1) + b"a" + struct.pack("=I", 2) + b"bb" + \
        struct.pack("=II", 40, 41)
    assert _parse(with_plen) == [(1, "a", 40, None), (1, "bb", 41, None)]


def test_peer_info_round_trip_and_bad_input():
    p = PeerInfo(role="prefill", tpsize=4, ctime_us=123456, addr="10.0.0.7", port=33001, dprank=2)
    assert p.serialize() == "prefill:4:123456:10.0.0.7:33001:2"
    assert PeerInfo.deserialize(p.serialize()) == p
    with pytest.raises(ValueError):
        PeerInfo.deserialize("prefill:4:1")


class _FakeNaming:
    def __init__(self):
        self.data = {}

    def list(self):
        return list(self.data)

    def search(self, inst, prefix):
        return [v for k, v in self.data[inst].items() if k.startswith(prefix)]


def test_peer_manager_notices_new_restarted_and_departed_peers():
    nm = _FakeNaming()
    nm.data["p1"] = {"endpoint0": PeerInfo("prefill", 1, 10, "127.0.0.1", 4001, 0).serialize()}
    nm.data["d1"] = {"endpoint0": PeerInfo("decode", 1, 11, "127.0.0.1", 4002, 0).serialize()}
    pm = PeerManager(nm, "prefill", ConnManager(8))
    asyncio.run(pm.refresh())
    assert pm.get_peer() == ("127.0.0.1", 4001)                           # the decode instance is not of interest
    assert pm.get_peer(exclude=("127.0.0.1", 4001)) is None
    nm.data["p1"] = {"endpoint0": PeerInfo("prefill", 1, 99, "127.0.0.1", 4011, 0).serialize()}   # restarted elsewhere
    asyncio.run(pm.refresh())
    assert pm.get_peer() == ("127.0.0.1", 4011)
    del nm.data["p1"]
    asyncio.run(pm.refresh())
    assert pm.get_peer() is None


def test_operation_plans_and_cleanup_refcount():
    assert merge_operation_plans((1, 0, ("kvs",), ()), (0, 1, (), ("kvt",)), (0, 1, (), ("kvs",))) == \
        (1, 2, ("kvs",), ("kvt", "kvs"))
    req = Request("r", [1, 2, 3])
    set_operation_sources(req, load_sources=("kvs",), save_sources=("kvt", "kvs"))
    assert get_param(req, "_HybridBackend_SAVE_SOURCES") == ("kvt", "kvs")
    assert inc_cleanup_rc(req) == 1 and inc_cleanup_rc(req) == 2
    assert dec_cleanup_rc(req) == 1 and dec_cleanup_rc(req) == 0
    with pytest.raises(AssertionError):
        dec_cleanup_rc(req)


def test_backend_selection_table():
    from pd_helpers import make_cfg
    from llumnix_kv_b200.hybrid_connector.backend import get_backend_cls

    def pick(backend, role):
        return get_backend_cls(make_cfg(role, "x", backend=backend)).__name__

    assert pick("kvt", "kv_producer") == "PBackend" and pick("kvt", "kv_consumer") == "DBackend"
    assert pick("kvt", "kv_both") == "FilePBackend"
    assert pick("migration", "kv_both") == "MigrationBackend"
    assert pick("kvt+migration", "kv_both") == pick("migration+kvt", "kv_both") == "KVTMigration"
    assert pick("kvt+kvs", "kv_producer") == pick("kvs+kvt", "kv_producer") == "KVSP"
    assert pick("local_file", "kv_both") == "FileBackend"
    for b, cls in (("kvs", "KVSBackend"), ("mooncake", "MooncakeKVSBackend"), ("v6d_object", "V6dObjectBackend")):
        assert pick(b, "kv_both") == cls
        with pytest.raises(AssertionError):
            pick(b, "kv_producer")
    assert pick("v6d_object+kvt", "kv_producer") == pick("kvt+v6d_object", "kv_both") == "V6dObjectKVTBackend"
    with pytest.raises(ValueError):
        pick("v6d_object+kvt", "kv_consumer")
    with pytest.raises(ValueError):
        pick("nope", "kv_both")


def test_wrapped_cache_objects_resolve_to_their_raw_buffer():
    """A TurboQuant-style cache object (key / value index views of one allocation) is registered as the
    flat int8 view of that allocation; plain tensors pass through; row size helper."""
    import types

    import torch

    from llumnix_kv_b200.hybrid_connector.kvtbackend import resolve_raw_cache_tensors, turboquant_last_dim_bytes

    raw = torch.arange(4 * 2 * 8 * 6, dtype=torch.int8).view(4, 2, 8, 6)
    wrapped = types.SimpleNamespace(key_cache=types.SimpleNamespace(indices=raw[:, 0]),
                                    value_cache=types.SimpleNamespace(indices=raw[:, 1]))
    plain = torch.zeros(16, dtype=torch.bfloat16)
    out = resolve_raw_cache_tensors({"model.layers.0.attn": wrapped, "model.layers.1.attn": plain})
    got = out["model.layers.0.attn"]
    assert got.dtype == torch.int8 and got.numel() == raw.numel() and got.data_ptr() == raw.data_ptr()
    assert torch.equal(got, raw.reshape(-1))
    assert out["model.layers.1.attn"] is plain
    other = torch.zeros(4, 8, 6, dtype=torch.int8)
    bad = types.SimpleNamespace(key_cache=types.SimpleNamespace(indices=raw[:, 0]), value_cache=types.SimpleNamespace(indices=other))
    import pytest
    with pytest.raises(AssertionError):
        resolve_raw_cache_tensors({"l.0": bad})
    assert turboquant_last_dim_bytes(64, 128, fast=True) == 66 and turboquant_last_dim_bytes(64, 256, fast=True) == 68
    assert turboquant_last_dim_bytes(64, 128, fast=False) == 80


def test_role_and_model_probes():
    from pd_helpers import make_cfg

    import llumnix_kv_b200 as pkg
    from llumnix_kv_b200.hybrid_connector import engine_proxy as ep

    assert pkg.support_async_sched() is False and pkg.is_erdma() is False
    d = make_cfg("kv_consumer", "D")
    p = make_cfg("kv_producer", "P")
    assert ep.is_kvt_consumer_backend(d) and not ep.is_kvt_consumer_backend(p)
    assert not ep.is_kvt_consumer_backend(make_cfg("kv_both", "S", backend="kvs", extra={"kvs_name": "x"}))
    hybrid = make_cfg("kv_consumer", "H", gdn_groups=3)
    assert ep.is_statemodel(hybrid) and not ep.is_statemodel(d)
    assert not ep.use_kvt_decode_prefix_cache(d)


def test_set_envs_fills_defaults_without_overriding(monkeypatch):
    import os

    import llumnix_kv_b200 as pkg

    monkeypatch.delenv("BLLM_KVTRANS_RDMA_SP", raising=False)
    monkeypatch.setenv("BLLM_KVTRANS_FSNAMING_KEEPALIVE_S", "7")
    pkg.set_envs()
    assert os.environ["BLLM_KVTRANS_RDMA_SP"] == "2"                 # two connections per target, as the reference's Python layer
    assert os.environ["BLLM_KVTRANS_FSNAMING_KEEPALIVE_S"] == "7"    # what the operator set stays
    monkeypatch.delenv("BLLM_KVTRANS_RDMA_SP", raising=False)


def test_relay_choice_for_replicated_caches(monkeypatch):
    """One decode worker takes a request for its whole group only when every target holds the same bytes
    (a single KV head or the MLA latent per prefill rank), every target advertises a multicast group that
    covers them, and the knob is on; the choice depends on the request id alone."""
    from llumnix_kv_b200.hybrid_connector.kvtbackend import choose_relay, multicast_kwargs

    def winfo(mcn):
        tail = f";mcn={mcn}" if mcn else ""
        return f"D|0|4,0,4,0,4096,256,8,2,4,16,0,1,0,10.0.0.1,x:dev=0;heads=1{tail};pid=1;port=2;shape=4"

    four = [("D", i, winfo(4)) for i in range(4)]
    r = choose_relay("req-1", four, total_kv_heads=1, src_tpsize=1)
    assert r is not None and 0 <= r < 4 and r == choose_relay("req-1", four, 1, 1)      # stable per request
    assert {choose_relay(f"req-{i}", four, 1, 1) for i in range(64)} == {0, 1, 2, 3}     # spread over the group
    assert choose_relay("req-1", four, total_kv_heads=8, src_tpsize=2) is None           # distinct head slices
    assert choose_relay("req-1", four, total_kv_heads=2, src_tpsize=2) is not None       # one head per prefill rank
    assert choose_relay("req-1", four[:1], 1, 1) is None                                 # a single target
    assert choose_relay("req-1", [("D", i, winfo(2)) for i in range(4)], 1, 1) is None   # group smaller than the targets
    assert choose_relay("req-1", [("D", 0, winfo(4)), ("D", 1, winfo(0))], 1, 1) is None
    assert choose_relay("req-1", [("D", 0, winfo(4)), ("D", 1, None)], 1, 1) is None     # worker info unknown here
    monkeypatch.setenv("VLLM_KVT_NVLS_FANOUT", "0")
    assert choose_relay("req-1", four, 1, 1) is None
    import torch
    assert multicast_kwargs([torch.zeros(16)]) == {}                                     # plain memory: nothing advertised


# ---- the ledger against a recomputation from the full signal history -------------------------------
def _replay(history, names, quota, tpsize):
    """What a ledger that rescans every signal on each arrival would answer: which signals count, how many
    ranks are complete, and the merged outcome."""
    accepted, per_rank = [], {}
    for rank, sig in history:
        got = per_rank.setdefault(rank, [])
        if names:
            if sig.source not in names or any(s.source == sig.source for s in got):
                continue
        elif len(got) >= quota:
            continue
        got.append(sig)
        accepted.append((rank, sig))
    need = len(names) if names else quota
    full = sum(1 for got in per_rank.values() if len(got) == need)
    merged = None
    if accepted:
        sigs = [s for _, s in accepted]
        failure = next((s.ex for s in sigs if s.ex is not None), None)
        n = None if any(s.n is None for s in sigs) else min(s.n for s in sigs)
        merged = (failure, n)
    return [id(s) for _, s in accepted], full, merged, full >= tpsize


def test_ledger_agrees_with_a_recomputation_over_random_signal_histories():
    from hypothesis import given, settings, strategies as st

    signal = st.tuples(st.integers(0, 3),                                   # rank
                       st.sampled_from([None, "kvt", "kvs", "other"]),      # source
                       st.one_of(st.none(), st.integers(0, 50)),            # token count
                       st.booleans())                                       # failed

    @settings(max_examples=300, deadline=None)
    @given(st.lists(signal, max_size=24), st.sampled_from([(), ("kvt",), ("kvt", "kvs")]), st.integers(1, 3), st.integers(1, 4))
    def run(raw, names, quota, tpsize):
        led = IoState(signals_per_worker=quota)
        led.expected_sources = names
        table = {"r": led}
        history, counted = [], []
        for rank, source, n, failed in raw:
            sig = IoRet(reqid="r", n=n, ex=CodeError(500, f"rank {rank}") if failed else None, source=source)
            history.append((rank, sig))
            done = try_advance(table, sig, rank, tpsize, on_signal_advanced=lambda _s, s: counted.append(id(s)))
            want_ids, want_full, want_merged, want_done = _replay(history, names, quota, tpsize)
            assert counted == want_ids
            assert led.full_ranks() == want_full
            # the ledger is handed out by the signal that completes the request and by every accepted one after it
            assert (done is led) == (want_done and bool(counted) and counted[-1] == id(sig))
            if want_merged is not None:
                m = led.merge()
                assert (m.ex, m.n) == want_merged
            for src in ("kvt", "kvs"):
                seen = [s for _, s in history if id(s) in want_ids and s.source == src]
                assert led.ranks_reporting(src) == len(seen)
                assert led.source_moved_nothing(src) == any(s.n == 0 for s in seen)

    run()


def test_a_workers_failure_travels_in_its_completion_report():
    """A worker backend that reports a failed load or save puts the exception into the IoRet; on its way to the
    scheduler the exception becomes text and comes out as an exception again (msgspec cannot encode exception
    objects, and a worker that tried used to end its process)."""
    import msgspec

    from llumnix_kv_b200.hybrid_connector.backend import IoDoneReqs
    from llumnix_kv_b200.hybrid_connector.worker import _failure_as_text

    enc = msgspec.msgpack.Encoder(enc_hook=_failure_as_text)
    dec = msgspec.msgpack.Decoder(IoDoneReqs)
    report = IoDoneReqs(worker_tprank=1, reqids=[IoRet(reqid="a", n=0, ex=FileNotFoundError("block 7 is gone"), source="local_file"),
                                                 IoRet(reqid="b", n=32, source="kvs")])
    back = dec.decode(enc.encode(report))
    assert back.worker_tprank == 1 and back.reqids[1] == IoRet(reqid="b", n=32, source="kvs")
    assert back.reqids[0].ex == "FileNotFoundError: block 7 is gone" and back.reqids[0].n == 0
    with pytest.raises(NotImplementedError):
        enc.encode(IoDoneReqs(worker_tprank=0, reqids=[IoRet(reqid="c", ex=object())]))


def test_what_the_native_stub_encodes_is_what_the_scheduler_parses():
    """Random finished-request lists through the C++ send-done encoder and the scheduler's parser: ranks, request
    ids (any UTF-8), token counts and outcomes arrive as sent, under both head kinds."""
    from hypothesis import given, settings, strategies as st

    import llumnix_kv_b200

    ops = llumnix_kv_b200.load_ops()
    reqs = st.lists(st.tuples(st.text(min_size=1, max_size=24).filter(lambda s: "\\x00" not in s), st.integers(0, (1 << 31) - 1),
                              st.booleans()), min_size=1, max_size=12)

    @settings(max_examples=150, deadline=None)
    @given(st.integers(0, 0xFFFE), reqs, st.sampled_from([1, 2]))
    def run(rank, rs, head_kind):
        buf, _resp = ops.encode_send_done(rank, rs, head_kind)
        body = bytes(buf)
        if head_kind == 2:
            half = len(body) // 2
            assert body[4:half] == body[half + 4:]          # the same body again under the save-done head
            body = body[:half]
        assert struct.unpack_from("=I", body, 0)[0] == 0x20181219
        got = _parse(body[4:])
        assert got == [(rank, rid, plen, None if ok else 500) for rid, plen, ok in rs]

    run()
