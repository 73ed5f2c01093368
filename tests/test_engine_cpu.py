"""Engine tests that need no GPU: codecs, naming, the client/step/stub pipeline over the TCP and
shared-memory transports with host-resident caches, failure handling and send-done reporting.

The scenarios mirror what the reference covers with fakes in kvtransfer/tests/client_test.cpp,
send_stub_test.cpp (FaultTolerantTest, CreateChannelFaultTolerantTest), naming_test.cpp and
common_test.cpp - here the real transports run, between threads of one process and between
two processes.
"""
import multiprocessing as mp
import os
import random
import socket
import struct
import threading
import time

import pytest
import torch

os.environ.setdefault("BLLM_KVTRANS_QUIET_ENV", "1")

from llumnix_kv_b200.kv_transfer_impl import (KVTransferClient, KVTransferProtocolType as PT, KVTransferServer,
                                              ReqMeta, encode_send_done)

L, H, D, T, NB = 2, 8, 128, 16, 64
TOK = 2 * H * D * 2
BLK = TOK * T


def make_cache(seed=None, device="cpu"):
    if seed is None:
        return [torch.zeros(2, NB, T, H, D, dtype=torch.float16, device=device) for _ in range(L)]
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(2, NB, T, H, D, dtype=torch.float16, generator=g).to(device) for _ in range(L)]


def check_tokens(src, dst, sb, db, lo, hi):
    for layer in range(L):
        for t in range(lo, hi):
            assert torch.equal(src[layer][:, sb[t // T], t % T], dst[layer][:, db[t // T], t % T]), (layer, t)


class SendDoneSink:
    """Stands in for the scheduler's RPC port: records every send-done message."""

    def __init__(self):
        self.sock = socket.socket()
        self.sock.bind(("127.0.0.1", 0))
        self.sock.listen(16)
        self.port = self.sock.getsockname()[1]
        self.msgs = []
        self.stop = False
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _recvn(self, c, n):
        buf = b""
        while len(buf) < n:
            chunk = c.recv(n - len(buf))
            if not chunk:
                raise EOFError
            buf += chunk
        return buf

    def _serve(self, c):
        try:
            while True:
                head, rank, n = struct.unpack("=III", self._recvn(c, 12))
                reqs = []
                for _ in range(n):
                    plen, code, rlen = struct.unpack("=III", self._recvn(c, 12))
                    reqs.append((self._recvn(c, rlen).decode(), plen, code))
                self.msgs.append((head, rank & 0xFFFF, bool(rank & 0x40000000), reqs))
                c.sendall(struct.pack("=I", 0x91218102))
        except (EOFError, OSError):
            pass

    def _run(self):
        while not self.stop:
            try:
                c, _ = self.sock.accept()
            except OSError:
                return
            threading.Thread(target=self._serve, args=(c,), daemon=True).start()

    def wait_for(self, n, timeout=10):
        t0 = time.time()
        while len(self.msgs) < n and time.time() - t0 < timeout:
            time.sleep(0.01)
        return list(self.msgs)

    def close(self):
        self.stop = True
        self.sock.close()


@pytest.fixture
def sink(ops):
    s = SendDoneSink()
    os.environ["BLLM_KVTRANS_SEND_DONE_ADDR"] = f"127.0.0.1:{s.port}"
    ops.envcfg_reset_for_test()
    yield s
    s.close()
    os.environ.pop("BLLM_KVTRANS_SEND_DONE_ADDR", None)
    ops.envcfg_reset_for_test()


# ---- codecs ------------------------------------------------------------------------------------
def test_worker_info_round_trip_and_back_compat(ops):
    W = ops.WorkerInfo
    s = "inst|0|2,3,2,1,65536|4096,4096|256,100,32,6,16,0,1,0,10.0.0.7"
    w = W.from_string(s)
    assert (w.inst_id, w.worker_id, w.engine_tp_size, w.worker_tp_rank) == ("inst|0|2", 3, 2, 1)
    assert w.block_sizes == [65536, 4096] and w.token_sizes == [4096, 256]
    assert (w.layer_num_blocks, w.num_layers, w.transfer_protocols) == (100, 32, 6)
    assert (w.attn_kernel_blk_ntpb, w.indexer_blk_ntpb, w.attn_pack_size, w.kda_page_stride, w.addr) == (16, 0, 1, 0, "10.0.0.7")
    assert w.to_string() == s
    # 11 fields: legacy without attn_pack_size / addr
    w = W.from_string("a,0,1,0,16384,1024,8,4,2,16,0")
    assert (w.attn_pack_size, w.kda_page_stride, w.addr) == (1, 0, "")
    # 12 fields: numeric -> attn_pack_size, otherwise address
    assert W.from_string("a,0,1,0,16384,1024,8,4,2,16,0,2").attn_pack_size == 2
    assert W.from_string("a,0,1,0,16384,1024,8,4,2,16,0,10.1.2.3").addr == "10.1.2.3"
    # 13 fields: {pack, addr} or {pack, stride}
    w = W.from_string("a,0,1,0,16384,1024,8,4,2,16,0,2,fe80::1")
    assert (w.attn_pack_size, w.addr) == (2, "fe80::1")
    w = W.from_string("a,0,1,0,16384,1024,8,4,2,16,0,2,40960")
    assert (w.attn_pack_size, w.kda_page_stride) == (2, 40960)
    # extension field survives a round trip and is ignored by the positional rules
    w = W.from_string("a,0,1,0,16384,1024,8,4,2,16,0,1,0,10.0.0.1,x:dev=3;port=4000;shape=5")
    assert w.ext == {"dev": "3", "port": "4000", "shape": "5"} and w.addr == "10.0.0.1"
    assert W.from_string(w.to_string()).ext == w.ext
    for bad in ("a,b", "a,0,1,0,1,1,1,1,1,1,1,1,1,1,1,1"):
        with pytest.raises(Exception):
            W.from_string(bad)


def test_send_done_wire_format(ops):
    buf, resp = ops.encode_send_done(3, [("req-a", 100, True), ("req-bb", 7, False)], 2)
    assert resp == 8
    expect = encode_send_done(3, [("req-a", 100, 0), ("req-bb", 7, 500)], 2)
    assert buf == expect
    head, rank, n = struct.unpack_from("=III", buf, 0)
    assert head == 0x20181219 and rank == (3 | 0x40000000) and n == 2
    half = len(buf) // 2
    assert struct.unpack_from("=I", buf, half)[0] == 0x20181223 and buf[4:half] == buf[half + 4:]
    buf1, resp1 = ops.encode_send_done(0, [("r", 1, True)], 1)
    assert resp1 == 4 and len(buf1) == 12 + 12 + 1


# ---- naming ------------------------------------------------------------------------------------
def test_file_naming(ops, tmp_path):
    os.environ["BLLM_KVTRANS_FSNAMING_KEEPALIVE_S"] = "1"
    os.environ["BLLM_KVTRANS_FSNAMING_TOLERATE_S"] = "3"
    ops.envcfg_reset_for_test()
    a = ops.connect_naming("instA", f"file:{tmp_path}")
    b = ops.connect_naming("instB", f"file:{tmp_path}")
    a.store("worker_0", "hello")
    a.store("worker_1", "world")
    a.store("other", "x")
    assert b.get("instA", "worker_0") == "hello"
    assert sorted(b.search("instA", "worker_")) == ["hello", "world"]
    assert b.get("instA", "missing") is None and b.get("nobody", "worker_0") is None
    assert sorted(b.list()) == ["instA", "instB"]
    a.remove("other")
    assert b.get("instA", "other") is None
    with pytest.raises(Exception):
        a.store("bad/key", "v")
    # a stale instance (old timestamp, nobody refreshing it) drops out of the listing
    stale = tmp_path / "ghost"
    stale.mkdir()
    (stale / "_timestamp_").write_text(str(int(time.time()) - 100) + "\n")
    time.sleep(2.1)
    assert "ghost" not in b.list() and "instA" in b.list()
    ts1 = int(b.get("instA", "_timestamp_"))
    time.sleep(1.3)
    assert int(b.get("instA", "_timestamp_")) >= ts1


def test_tcpstore_and_mem_naming(ops):
    srv = ops.KvStoreServer()
    port = srv.start(0)
    try:
        a = ops.connect_naming("i1", f"tcpstore:127.0.0.1:{port}")
        b = ops.connect_naming("i2", f"tcpstore://127.0.0.1:{port}")
        a.store("worker_3", "w3")
        a.store("endpoint0", "e0")
        assert b.get("i1", "worker_3") == "w3" and b.get("i1", "nope") is None
        assert b.search("i1", "worker_") == ["w3"]
        assert sorted(b.list()) == ["i1", "i2"]
        a.remove("worker_3")
        assert b.get("i1", "worker_3") is None
    finally:
        srv.stop()
    m1 = ops.connect_naming("x", "mem:space1")
    m2 = ops.connect_naming("y", "mem:space1")
    m1.store("k", "v")
    assert m2.get("x", "k") == "v" and m2.list() == ["x"]


def test_eas_document_parser(ops):
    ok, ver, doc = ops.parse_eas_document(
        '{"version": 7, "instances": {"p0": {"worker_0": "a,b", "endpoint0": "1.2.3.4:5"}, "d0": {}}}')
    assert ok and ver == 7 and doc == {"p0": {"worker_0": "a,b", "endpoint0": "1.2.3.4:5"}, "d0": {}}
    assert not ops.parse_eas_document('{"version": ')[0]


def test_eas_naming_over_http(ops):
    import http.server

    state = {"version": 1, "instances": {"d0": {"worker_0": "first"}}}

    class Handler(http.server.BaseHTTPRequestHandler):
        def do_GET(self):
            import json
            body = json.dumps(state).encode()
            self.send_response(200)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def log_message(self, *a):
            pass

    httpd = http.server.HTTPServer(("127.0.0.1", 0), Handler)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    try:
        c = ops.connect_naming("me", f"eas:127.0.0.1:{httpd.server_port}/discovery")
        assert c.get("d0", "worker_0") == "first" and c.list() == ["d0"]
        state["version"] = 2
        state["instances"]["d1"] = {"worker_0": "second"}
        time.sleep(1.1)  # the document is re-fetched at most once a second
        assert c.get("d1", "worker_0") == "second" and sorted(c.list()) == ["d0", "d1"]
        c.store("mine", "local")  # the service is read-only: own keys live in an overlay
        assert c.get("me", "mine") == "local"
    finally:
        httpd.shutdown()


# ---- transfers ---------------------------------------------------------------------------------
@pytest.mark.parametrize("proto", [PT.TCP, PT.SHM])
def test_config1_ten_requests_bit_exact(proto, sink):
    """BASELINE config 1 inside one process: 2 layers, 8 KV heads, head_dim 128, block 16, 64 blocks,
    fp16 N(0,1), NHD; 10 requests with random block tables, verified bit-exactly."""
    src, dst = make_cache(1), make_cache()
    srv = KVTransferServer("D|0|1", 1, 0, 0, BLK, TOK, "fake://", dst, [proto], num_kv_heads=H, cache_shape=2)
    cli = KVTransferClient("P|0|1", 1, 0, 0, BLK, TOK, "fake://", src, [proto], num_kv_heads=H, cache_shape=2)
    try:
        rng = random.Random(7)
        done = []
        stepid = 1024
        for batch in range(5):
            free_s, free_d = list(range(NB)), list(range(NB))
            rng.shuffle(free_s)
            rng.shuffle(free_d)
            reqs = []
            for r in range(2):
                nb = rng.randint(4, 32)
                sb, db = [free_s.pop() for _ in range(nb)], [free_d.pop() for _ in range(nb)]
                ntok = nb * T - rng.randint(0, T - 1)
                rid = f"req-{batch}-{r}"
                reqs.append((rid, sb, db, ntok))
                cli.submit_req_send2("D|0|1", 0, rid, 0, ntok, True, sb, db, srv.worker_info(), stepid=stepid)
            cli.start_send_step(stepid, 1)
            for layer in range(L):
                cli.record_event(layer)
            cli.flush_send_step()
            cli.drain()
            for rid, sb, db, ntok in reqs:
                check_tokens(src, dst, sb, db, 0, ntok)
                done.append(rid)
            stepid += 1
        msgs = sink.wait_for(10)
        got = {r[0]: r[2] for m in msgs if m[0] == 0x20181219 for r in m[3]}
        assert got == {rid: 0 for rid in done}
    finally:
        srv.stop()


def test_chunked_prefill_deltas_and_unknown_delta(sink):
    src, dst = make_cache(2), make_cache()
    srv = KVTransferServer("D|0|1", 1, 0, 0, BLK, TOK, "fake://", dst, [PT.TCP], num_kv_heads=H, cache_shape=2)
    cli = KVTransferClient("P|0|1", 1, 0, 0, BLK, TOK, "fake://", src, [PT.TCP], num_kv_heads=H, cache_shape=2)
    try:
        sb, db = [5, 9, 11, 2], [40, 41, 3, 8]
        total = 3 * T + 5
        chunks = [(0, 20, False), (20, 21, False), (41, total - 41, True)]
        for i, (seen, new, last) in enumerate(chunks):
            if i == 0:
                cli.submit_req_send2("D|0|1", 0, "chunky", seen, new, last, sb, db, srv.worker_info(), stepid=2000 + i)
            else:
                cli.submit_delta_send("chunky", seen, new, last, stepid=2000 + i)
            cli.submit_delta_send("never-submitted", 0, 4, True, stepid=2000 + i)  # warns and is ignored
            cli.start_send_step(2000 + i, 1)
            for layer in range(L):
                cli.record_event(layer)
            cli.flush_send_step()
            cli.drain()
            check_tokens(src, dst, sb, db, 0, seen + new)
            # nothing beyond the chunk has been written yet
            if not last:
                nxt = seen + new
                assert float(dst[0][:, db[nxt // T], nxt % T].abs().sum()) == 0.0
        msgs = sink.wait_for(1)
        sd = [m for m in msgs if m[0] == 0x20181219]
        assert len(sd) == 1 and sd[0][3] == [("chunky", total, 0)]
        # an empty step returns without opening anything
        cli.start_send_step(3000, 0)
        cli.flush_send_step()
    finally:
        srv.stop()


def test_freeze_send_and_substeps(sink):
    src, dst = make_cache(3), make_cache()
    srv = KVTransferServer("D|0|1", 1, 0, 0, BLK, TOK, "fake://", dst, [PT.SHM], num_kv_heads=H, cache_shape=2)
    cli = KVTransferClient("P|0|1", 1, 0, 0, BLK, TOK, "fake://", src, [PT.SHM], num_kv_heads=H, cache_shape=2)
    try:
        def meta(rid, sb, db, n):
            m = ReqMeta()
            m.dst_inst, m.dst_worker, m.reqid, m.seen_tokens, m.new_tokens = "D|0|1", 0, rid, 0, n
            m.src_block_ids, m.dst_block_ids, m.dst_worker_info = [sb], [db], srv.worker_info()
            return m
        # freeze: data complete, no layer events involved
        cli.start_req_send([meta("frozen", [1, 2], [3, 4], 30)], 100, 0)
        cli.drain()
        check_tokens(src, dst, [1, 2], [3, 4], 0, 30)
        # substep for a step that has not started yet: parked, sent when the step opens
        cli.start_send_substep(200, 1, [meta("parked", [5], [6], 10)])
        cli.drain()
        assert float(dst[0][:, 6].abs().sum()) == 0.0
        cli.start_send_step(200, 1)
        # substep attached to the running step
        cli.start_send_substep(200, 2, [meta("attached", [7], [8], 16)])
        for layer in range(L):
            cli.record_event(layer)
        cli.flush_send_step()
        cli.drain()
        check_tokens(src, dst, [5], [6], 0, 10)
        check_tokens(src, dst, [7], [8], 0, 16)
        # substep for a step that is already over: becomes its own frozen step
        cli.start_send_substep(200, 3, [meta("late", [9], [10], 16)])
        cli.drain()
        check_tokens(src, dst, [9], [10], 0, 16)
        names = sorted(r[0] for m in sink.wait_for(4) if m[0] == 0x20181219 for r in m[3])
        assert names == ["attached", "frozen", "late", "parked"]
    finally:
        srv.stop()


def test_step_protocol_violations(ops):
    src = make_cache(4)
    cli = KVTransferClient("P|0|1", 1, 0, 0, BLK, TOK, "fake://", src, [PT.TCP], num_kv_heads=H, cache_shape=2)
    cli.record_event(0)  # before any step: ignored (warm-up)
    cli.start_send_step(10, 1)
    with pytest.raises(RuntimeError):
        cli.start_send_step(11, 1)
    cli.flush_send_step()
    cli.flush_send_step()  # idempotent once closed
    with pytest.raises(Exception):
        cli.submit_req_send2("D", 0, "r", 0, 0, True, [1], [1], None)  # new_tokens must be positive
    cli.submit_req_send2("D", 0, "r", 0, 4, False, [1], [1], None, stepid=20)
    with pytest.raises(Exception):
        cli.submit_req_send2("D", 0, "r2", 0, 4, False, [1], [1], None, stepid=21)  # one step id per step


def test_failure_marks_batch_failed_and_next_batch_recovers(ops, sink):
    src, dst = make_cache(5), make_cache()
    srv = KVTransferServer("D|0|1", 1, 0, 0, BLK, TOK, "fake://", dst, [PT.TCP], num_kv_heads=H, cache_shape=2)
    cli = KVTransferClient("P|0|1", 1, 0, 0, BLK, TOK, "fake://", src, [PT.TCP], num_kv_heads=H, cache_shape=2)
    try:
        def step(stepid, reqs):
            for rid, sb, db, n, last in reqs:
                cli.submit_req_send2("D|0|1", 0, rid, 0, n, last, sb, db, srv.worker_info(), stepid=stepid)
            cli.start_send_step(stepid, 1)
            for layer in range(L):
                cli.record_event(layer)
            cli.flush_send_step()
            cli.drain()
        # first batch connects fine
        step(1, [("warm", [1], [1], 8, True)])
        # the 1st fault point hit from now on throws: the send of this batch fails after connect
        ops.fault_inject_arm(1)
        step(2, [("a", [2], [2], 16, True), ("b", [3], [3], 10, False)])
        ops.fault_inject_arm(0)
        # a later chunk of the failed request stays failed; a new request on a fresh channel works
        cli.submit_delta_send("b", 10, 6, True, stepid=3)
        step(3, [("c", [4], [4], 16, True)])
        check_tokens(src, dst, [4], [4], 0, 16)
        codes = {r[0]: r[2] for m in sink.wait_for(3) if m[0] == 0x20181219 for r in m[3]}
        assert codes == {"warm": 0, "a": 500, "b": 500, "c": 0}
    finally:
        ops.fault_inject_arm(0)
        srv.stop()


def test_unreachable_destination_fails_requests_not_the_engine(ops, sink):
    src = make_cache(6)
    cli = KVTransferClient("P|0|1", 1, 0, 0, BLK, TOK, "fake://", src, [PT.TCP], num_kv_heads=H, cache_shape=2)
    os.environ["BLLM_KVTRANS_RPC_TIMEOUT_S"] = "1"
    ops.envcfg_reset_for_test()
    ghost = ops.WorkerInfo.from_string(f"D|0|1,0,1,0,{BLK},{TOK},{NB},{L},2,16,0,1,0,127.0.0.1,x:port=1;shape=2")
    cli.submit_req_send2("D|0|1", 0, "lost", 0, 8, True, [1], [1], ghost.to_string(), stepid=1)
    cli.start_send_step(1, 1)
    for layer in range(L):
        cli.record_event(layer)
    cli.flush_send_step()
    cli.drain()
    codes = {r[0]: r[2] for m in sink.wait_for(1) if m[0] == 0x20181219 for r in m[3]}
    assert codes == {"lost": 500}
    os.environ.pop("BLLM_KVTRANS_RPC_TIMEOUT_S")
    ops.envcfg_reset_for_test()


def test_target_lru_shrink(ops):
    src = make_cache(7)
    dsts = [make_cache() for _ in range(3)]
    srvs = [KVTransferServer(f"D{i}|0|1", 1, 0, 0, BLK, TOK, "fake://", dsts[i], [PT.TCP], num_kv_heads=H,
                             cache_shape=2) for i in range(3)]
    cli = KVTransferClient("P|0|1", 1, 0, 0, BLK, TOK, "fake://", src, [PT.TCP], num_kv_heads=H, cache_shape=2)
    try:
        for i, s in enumerate(srvs):
            cli.submit_req_send2(f"D{i}|0|1", 0, f"r{i}", 0, 8, True, [i + 1], [i + 1], s.worker_info(), stepid=1)
        cli.start_send_step(1, 1)
        for layer in range(L):
            cli.record_event(layer)
        cli.flush_send_step()
        cli.drain()
        assert cli._c.target_size() == 3
        cli._c.target_try_shrink(1)
        assert cli._c.target_size() == 1
        # evicted targets are recreated on demand
        cli.submit_req_send2("D0|0|1", 0, "again", 0, 8, True, [9], [9], srvs[0].worker_info(), stepid=2)
        cli.start_send_step(2, 1)
        for layer in range(L):
            cli.record_event(layer)
        cli.flush_send_step()
        cli.drain()
        check_tokens(src, dsts[0], [9], [9], 0, 8)
    finally:
        for s in srvs:
            s.stop()


def test_receiver_rejects_out_of_range_destination(ops, sink):
    """A sender whose idea of the destination is too big is refused by the receiver's own check."""
    src, dst = make_cache(8), make_cache()
    srv = KVTransferServer("D|0|1", 1, 0, 0, BLK, TOK, "fake://", dst, [PT.TCP], num_kv_heads=H, cache_shape=2)
    cli = KVTransferClient("P|0|1", 1, 0, 0, BLK, TOK, "fake://", src, [PT.TCP], num_kv_heads=H, cache_shape=2)
    try:
        lie = ops.WorkerInfo.from_string(srv.worker_info())
        lie.layer_num_blocks = NB * 4
        cli.submit_req_send2("D|0|1", 0, "oob", 0, 8, True, [1], [NB * 2], lie.to_string(), stepid=1)
        cli.start_send_step(1, 1)
        for layer in range(L):
            cli.record_event(layer)
        cli.flush_send_step()
        cli.drain()
        codes = {r[0]: r[2] for m in sink.wait_for(1) if m[0] == 0x20181219 for r in m[3]}
        assert codes == {"oob": 500}
        assert all(float(d.abs().sum()) == 0.0 for d in dst)
    finally:
        srv.stop()


# ---- two processes ---------------------------------------------------------------------------------
def _decode_proc(naming_dir, proto_name, ready, go, result):
    os.environ["BLLM_KVTRANS_QUIET_ENV"] = "1"
    from llumnix_kv_b200.kv_transfer_impl import KVTransferProtocolType as P2, KVTransferServer as Srv
    dst = make_cache()
    srv = Srv("D|0|1", 1, 0, 0, BLK, TOK, f"file:{naming_dir}", dst, [P2[proto_name]], num_kv_heads=H, cache_shape=2)
    ready.set()
    go.wait(60)
    result.put([d.numpy().copy() for d in dst])  # by value: the process exits right after
    srv.stop()


@pytest.mark.parametrize("proto", ["TCP", "SHM"])
def test_config1_two_processes_with_file_naming(proto, tmp_path, ops):
    ctx = mp.get_context("spawn")
    ready, go, result = ctx.Event(), ctx.Event(), ctx.Queue()
    p = ctx.Process(target=_decode_proc, args=(str(tmp_path), proto, ready, go, result))
    p.start()
    try:
        assert ready.wait(120)
        src = make_cache(11)
        # no destination info in the request: resolved through the naming directory
        cli = KVTransferClient("P|0|1", 1, 0, 0, BLK, TOK, f"file:{tmp_path}", src, [PT[proto]], num_kv_heads=H,
                               cache_shape=2)
        rng = random.Random(3)
        free_s, free_d = list(range(NB)), list(range(NB))
        rng.shuffle(free_s)
        rng.shuffle(free_d)
        reqs = []
        for r in range(10):
            nb = rng.randint(4, 6)
            sb, db = [free_s.pop() for _ in range(nb)], [free_d.pop() for _ in range(nb)]
            ntok = nb * T - rng.randint(0, T - 1)
            reqs.append((sb, db, ntok))
            cli.submit_req_send2("D|0|1", 0, f"r{r}", 0, ntok, True, sb, db, None, stepid=1)
        cli.start_send_step(1, 1)
        for layer in range(L):
            cli.record_event(layer)
        cli.flush_send_step()
        cli.drain()
        go.set()
        dst = [torch.from_numpy(a) for a in result.get(timeout=60)]
        for sb, db, ntok in reqs:
            check_tokens(src, dst, sb, db, 0, ntok)
    finally:
        go.set()
        p.join(30)
        if p.is_alive():
            p.kill()


def test_bf16_to_e4m3_host_conversion_matches_torch(ops):
    """Every finite bf16 value whose magnitude e4m3 can hold converts like torch's round-to-nearest-even
    cast; larger ones saturate to 448, NaN stays NaN, signed zero keeps its sign."""
    bits = torch.arange(0, 1 << 16, dtype=torch.int32)
    vals = bits.to(torch.int16).view(torch.bfloat16)
    mask = vals.float().abs() <= 448
    want = vals[mask].to(torch.float8_e4m3fn).view(torch.uint8).tolist()
    got = [ops.kvt_bf16_to_e4m3(int(b)) for b in bits[mask].tolist()]
    assert got == want
    assert ops.kvt_bf16_to_e4m3(0x7F80) == 0x7E and ops.kvt_bf16_to_e4m3(0xFF80) == 0xFE      # +-inf saturate
    assert ops.kvt_bf16_to_e4m3(0x4480) == 0x7E                                              # 1024 saturates
    assert ops.kvt_bf16_to_e4m3(0x7FC0) & 0x7F == 0x7F                                       # NaN
    assert ops.kvt_bf16_to_e4m3(0x8000) == 0x80 and ops.kvt_bf16_to_e4m3(0x0000) == 0x00


@pytest.mark.parametrize("proto", [PT.TCP, PT.SHM])
def test_staged_transfer_casts_bf16_to_fp8_for_a_smaller_decode_tp(proto, ops, sink, monkeypatch):
    """BLLM_KVTRANS_BF162FP8_CONV=1 (the reference's staged cast, tcp_channel.cpp:411-447): two prefill
    TP ranks with bf16 caches fill their head slices of one decode rank's fp8 cache; every byte on the
    decode side is the unscaled e4m3 cast of the prefill value."""
    monkeypatch.setenv("BLLM_KVTRANS_BF162FP8_CONV", "1")
    ops.envcfg_reset_for_test()
    hp = H // 2
    g = torch.Generator().manual_seed(3)
    srcs = [[torch.randn(2, NB, T, hp, D, generator=g).to(torch.bfloat16) for _ in range(L)] for _ in range(2)]
    dst = [torch.zeros(2, NB, T, H, D, dtype=torch.uint8) for _ in range(L)]
    p_tok, d_tok = 2 * hp * D * 2, 2 * H * D
    srv = KVTransferServer("D|0|1", 1, 0, 0, d_tok * T, d_tok, "fake://", dst, [proto], num_kv_heads=H, cache_shape=2)
    clis = [KVTransferClient("P|0|2", 2, r, r, p_tok * T, p_tok, "fake://", srcs[r], [proto], num_kv_heads=H, cache_shape=2)
            for r in range(2)]
    try:
        sb, db, ntok = [5, 9, 2], [7, 1, 30], 41
        for r, cli in enumerate(clis):
            cli.submit_req_send2("D|0|1", 0, "q", 0, ntok, True, sb, db, srv.worker_info(), stepid=7)
            cli.start_send_step(7, 1)
            for layer in range(L):
                cli.record_event(layer)
            cli.flush_send_step()
            cli.drain()
        for layer in range(L):
            for t in range(ntok):
                for r in range(2):
                    want = srcs[r][layer][:, sb[t // T], t % T].to(torch.float8_e4m3fn).view(torch.uint8)
                    got = dst[layer][:, db[t // T], t % T, r * hp:(r + 1) * hp]
                    assert torch.equal(got, want), (layer, t, r)
        # slots past the request stay untouched
        assert int(dst[0][:, db[2], ntok % T:].sum()) == 0
    finally:
        srv.stop()
        monkeypatch.delenv("BLLM_KVTRANS_BF162FP8_CONV")
        ops.envcfg_reset_for_test()


def test_server_refuses_oversized_frames_and_oversized_shm_attach(ops):
    """A peer that announces a frame no sender of ours produces is dropped before anything is read or
    pinned for it; a shared-memory attach larger than the segment is refused; the server stays up."""
    import socket
    from multiprocessing import shared_memory

    dst = make_cache()
    srv = KVTransferServer("D|0|1", 1, 0, 0, BLK, TOK, "fake://", dst, [PT.TCP], num_kv_heads=H, cache_shape=2)
    port = int(ops.WorkerInfo.from_string(srv.worker_info()).ext["port"])

    def rpc(sock, magic, body=b""):
        msg = struct.pack("=IQ", magic, 7) + body
        sock.sendall(struct.pack("=I", len(msg)) + msg)
        n = struct.unpack("=I", sock.recv(4, socket.MSG_WAITALL))[0]
        return sock.recv(n, socket.MSG_WAITALL)

    seg = shared_memory.SharedMemory(create=True, size=8192)
    try:
        with socket.create_connection(("127.0.0.1", port), timeout=10) as c:
            c.sendall(struct.pack("=I", 0xFFFFFF00))
            assert c.recv(4) == b""                               # closed, nothing allocated for 4 GiB
        with socket.create_connection(("127.0.0.1", port), timeout=10) as c:
            assert struct.unpack("=I", rpc(c, 0x4B565069)[12:16])[0] == 0          # ping still answered
            name = ("/" + seg.name.lstrip("/")).encode()
            attach = struct.pack("=I", len(name)) + name
            assert struct.unpack("=I", rpc(c, 0x4B565341, attach + struct.pack("=Q", 1 << 30))[12:16])[0] == 400
            assert struct.unpack("=I", rpc(c, 0x4B565341, attach + struct.pack("=Q", 8192))[12:16])[0] == 0
    finally:
        seg.close()
        seg.unlink()
        srv.stop()


def test_relayed_transfer_is_refused_by_host_transports(ops, sink):
    """fanout=k hands the request to one worker of a multicast group for all k: only the NVLINK transport
    with a pull session on a worker that advertises such a group can do that.  Anything else fails the
    request (once, not k times) instead of reporting k deliveries after one."""
    src, dst = make_cache(8), make_cache()
    srv = KVTransferServer("D|0|1", 1, 0, 0, BLK, TOK, "fake://", dst, [PT.TCP], num_kv_heads=H, cache_shape=2)
    cli = KVTransferClient("P|0|1", 1, 0, 0, BLK, TOK, "fake://", src, [PT.TCP], num_kv_heads=H, cache_shape=2)
    try:
        cli.submit_req_send2("D|0|1", 0, "fan", 0, 8, True, [1], [2], srv.worker_info(), stepid=1, fanout=3)
        cli.start_send_step(1, 1)
        for layer in range(L):
            cli.record_event(layer)
        cli.flush_send_step()
        cli.drain()
        reports = [r for m in sink.wait_for(1) if m[0] == 0x20181219 for r in m[3]]
        assert [(r[0], r[2]) for r in reports] == [("fan", 500)] * 3       # one report per worker it stood for
        assert cli.failed_batches() == 1
        assert all(float(d.abs().sum()) == 0.0 for d in dst)
    finally:
        srv.stop()


# ---- end-to-end transfer check ------------------------------------------------------------------
def _term(k, w):
    key = (k * 0x85EBCA77) & 0xFFFFFFFF
    x = ((w * 0x9E3779B1) & 0xFFFFFFFF) ^ (((key << 13) | (key >> 19)) & 0xFFFFFFFF)
    x ^= x >> 15
    x = (x * 0xC2B2AE3D) & 0xFFFFFFFF
    x ^= x >> 13
    return x


def _piece_sum(data: bytes, index0=0):
    """A piece as little-endian 32-bit words, the last padded with zero bytes; word k adds term(index0 + k, word)."""
    padded = data + b"\0" * (-len(data) % 4)
    words = struct.unpack(f"<{len(padded) // 4}I", padded)
    return sum(_term((index0 + k) & 0xFFFFFFFF, w) for k, w in enumerate(words)) & 0xFFFFFFFFFFFFFFFF


def _rotl64(v, r):
    r &= 63
    return v if r == 0 else ((v << r) | (v >> (64 - r))) & 0xFFFFFFFFFFFFFFFF


def test_checksum_function_matches_its_definition(ops):
    rng = random.Random(3)
    data = bytes(rng.randrange(256) for _ in range(1000))
    assert ops.kvt_checksum_host(data) == _piece_sum(data)
    assert ops.kvt_checksum_host(data[100:], 25) == _piece_sum(data[100:], 25)
    assert ops.kvt_checksum_host(data[:997]) == _piece_sum(data[:997])            # a ragged tail is one padded word
    # a piece cut at word boundaries into chunks that carry their starting word index sums to the whole piece
    cuts = [0, 16, 256, 640, 1000]
    assert sum(ops.kvt_checksum_host(data[a:b], a // 4) for a, b in zip(cuts, cuts[1:])) & 0xFFFFFFFFFFFFFFFF == _piece_sum(data)
    # the value depends on where a byte sits in its piece, not only on the multiset of bytes
    swapped = bytearray(data)
    swapped[3], swapped[4] = swapped[4], swapped[3]
    assert data[3] != data[4] and ops.kvt_checksum_host(bytes(swapped)) != _piece_sum(data)


def test_server_answers_a_check_request_with_the_checksum_of_its_cache(ops):
    """CHECK_REQ names byte ranges per tensor for a span of layers; the answer is the sum over layers of the
    rotated per-layer sums.  Ranges outside the tensor are refused, not read."""
    dst = make_cache(21)
    srv = KVTransferServer("D|0|1", 1, 0, 0, BLK, TOK, "fake://", dst, [PT.TCP], num_kv_heads=H, cache_shape=2)
    port = int(ops.WorkerInfo.from_string(srv.worker_info()).ext["port"])
    ranges = [(5 * BLK // 2 + 64, 300), (40 * BLK // 2, 4096), (7, 1)]
    cap = dst[0].numel() * 2

    def ask(c, lb, le, rs):
        body = struct.pack("=IIII", lb, le, 1, 0) + struct.pack("=Q", len(rs)) + b"".join(struct.pack("=QQ", o, n) for o, n in rs)
        msg = struct.pack("=IQ", 0x4B56436B, 9) + body
        c.sendall(struct.pack("=I", len(msg)) + msg)
        n = struct.unpack("=I", c.recv(4, socket.MSG_WAITALL))[0]
        resp = c.recv(n, socket.MSG_WAITALL)
        magic, reqid, status, total = struct.unpack("=IQIQ", resp[:24])
        assert (magic, reqid) == (0x4B56436B, 9)
        return status, total

    def expect(lb, le):
        total = 0
        for layer in range(lb, le):
            raw = dst[layer].numpy().tobytes()
            total += _rotl64(sum(_piece_sum(raw[o:o + n]) for o, n in ranges) & 0xFFFFFFFFFFFFFFFF, layer * 7)
        return total & 0xFFFFFFFFFFFFFFFF

    try:
        with socket.create_connection(("127.0.0.1", port), timeout=10) as c:
            assert ask(c, 0, L, ranges) == (0, expect(0, L))
            assert ask(c, 1, 2, ranges) == (0, expect(1, 2))
            before = expect(0, L)
            dst[1].view(torch.int16).view(-1)[(40 * BLK // 2) // 2 + 9] ^= 0x0100       # one bit of one byte in a checked range
            after = ask(c, 0, L, ranges)
            assert after == (0, expect(0, L)) and after[1] != before
            assert ask(c, 0, L, [(cap - 8, 16)])[0] == 400
            assert ask(c, 0, L + 1, ranges)[0] == 400
    finally:
        srv.stop()


@pytest.mark.parametrize("proto", [PT.TCP, PT.SHM])
def test_transfer_check_passes_intact_batches_and_fails_a_mismatch(proto, ops, sink):
    """BLLM_KVTRANS_CRC=1: after a batch has landed the sender compares a checksum of its source ranges with
    the destination's checksum of the ranges it wrote.  Intact batches finish as before; a batch whose two
    sums differ (the sender's sum perturbed through the host-side hook) reports its requests failed, and
    the stub carries on with the next batch."""
    os.environ["BLLM_KVTRANS_CRC"] = "1"
    ops.envcfg_reset_for_test()
    src, dst = make_cache(31), make_cache()
    srv = KVTransferServer("D|0|1", 1, 0, 0, BLK, TOK, "fake://", dst, [proto], num_kv_heads=H, cache_shape=2)
    cli = KVTransferClient("P|0|1", 1, 0, 0, BLK, TOK, "fake://", src, [proto], num_kv_heads=H, cache_shape=2)
    try:
        def step(stepid, reqs):
            for rid, sb, db, n in reqs:
                cli.submit_req_send2("D|0|1", 0, rid, 0, n, True, sb, db, srv.worker_info(), stepid=stepid)
            cli.start_send_step(stepid, 1)
            for layer in range(L):
                cli.record_event(layer)
            cli.flush_send_step()
            cli.drain()

        step(1, [("a", [3, 9, 4], [7, 1, 8], 41), ("b", [20], [21], 16)])
        check_tokens(src, dst, [3, 9, 4], [7, 1, 8], 0, 41)
        ops.fault_inject_arm_corrupt_check(1)
        step(2, [("c", [5], [6], 12)])
        step(3, [("d", [11, 12], [13, 14], 32)])
        check_tokens(src, dst, [11, 12], [13, 14], 0, 32)
        codes = {r[0]: r[2] for m in sink.wait_for(3) if m[0] == 0x20181219 for r in m[3]}
        assert codes == {"a": 0, "b": 0, "c": 500, "d": 0}
        assert cli.failed_batches() == 1
    finally:
        ops.fault_inject_arm_corrupt_check(0)
        srv.stop()
        os.environ.pop("BLLM_KVTRANS_CRC", None)
        ops.envcfg_reset_for_test()


# ---- randomized ------------------------------------------------------------------------------------
@pytest.mark.parametrize("proto,seed", [(PT.TCP, 1), (PT.SHM, 2), (PT.TCP, 3)])
def test_random_chunked_requests_to_several_destinations_with_faults(proto, seed, ops, sink):
    random_chunked_requests(proto, seed, ops, sink, "cpu")


def random_chunked_requests(proto, seed, ops, sink, device, drop_completions=False):
    """One client, four destinations, forty steps: every step starts some requests (random block tables,
    random destination) and continues some that are in flight with another chunk; now and then a fault is
    armed so that a batch fails somewhere on its way.  Steps are not drained one by one, so batches of
    several steps and destinations overlap.  At the end every request has been reported exactly once; one
    reported good has every token of every chunk at its destination; one reported failed stayed failed
    whatever was sent for it afterwards; the client has nothing in flight.  ``drop_completions`` (device
    transports) also leaves out a batch's completion record now and then, so that its deadline has to fail it."""
    rng = random.Random(seed)
    src = make_cache(40 + seed, device)
    n_dst = 4
    dsts = [make_cache(None, device) for _ in range(n_dst)]
    srvs = [KVTransferServer(f"D{i}|0|1", 1, 0, 0, BLK, TOK, "fake://", dsts[i], [proto], num_kv_heads=H, cache_shape=2)
            for i in range(n_dst)]
    cli = KVTransferClient("P|0|1", 1, 0, 0, BLK, TOK, "fake://", src, [proto], num_kv_heads=H, cache_shape=2)
    free_d = [list(range(1, NB)) for _ in range(n_dst)]
    for f in free_d:
        rng.shuffle(f)
    live, finished = {}, {}          # rid -> dict(dst, sb, db, total, sent)
    try:
        stepid = 5000
        n_req = 0
        for step in range(40):
            if rng.random() < 0.15:
                ops.fault_inject_arm(rng.randint(1, 4))
            if drop_completions and rng.random() < 0.08:
                ops.fault_inject_arm_drop_completion(1)
            submitted = 0
            for rid, r in list(live.items()):           # continue some of the requests in flight
                if rng.random() < 0.6:
                    new = min(r["total"] - r["sent"], rng.randint(1, 40))
                    last = r["sent"] + new == r["total"]
                    cli.submit_delta_send(rid, r["sent"], new, last, stepid=stepid)
                    r["sent"] += new
                    submitted += 1
                    if last:
                        finished[rid] = live.pop(rid)
            for _ in range(rng.randint(0, 3)):            # start new ones
                i = rng.randrange(n_dst)
                nb = rng.randint(1, 5)
                if len(free_d[i]) < nb:
                    continue
                total = nb * T - rng.randint(0, T - 1)
                sb = [rng.randrange(1, NB) for _ in range(nb)]
                db = [free_d[i].pop() for _ in range(nb)]
                rid = f"z{seed}.{n_req}"
                n_req += 1
                new = rng.randint(1, total)
                last = new == total
                cli.submit_req_send2(f"D{i}|0|1", 0, rid, 0, new, last, sb, db, srvs[i].worker_info(), stepid=stepid)
                rec = dict(dst=i, sb=sb, db=db, total=total, sent=new)
                (finished if last else live)[rid] = rec
                submitted += 1
            cli.start_send_step(stepid, 1 if submitted else 0)
            if submitted:
                for layer in range(L):
                    cli.record_event(layer)
            cli.flush_send_step()
            stepid += 1
            if rng.random() < 0.2:
                assert cli.wait_inflight(0, 30.0)
        ops.fault_inject_arm(0)
        for rid, r in list(live.items()):                # close what is still open
            cli.submit_delta_send(rid, r["sent"], r["total"] - r["sent"], True, stepid=stepid)
            r["sent"] = r["total"]
            finished[rid] = live.pop(rid)
        cli.start_send_step(stepid, 1)
        for layer in range(L):
            cli.record_event(layer)
        cli.flush_send_step()
        assert cli.wait_inflight(0, 30.0) and cli.inflight() == 0
        deadline = time.time() + 10
        def reports():
            return [r for m in list(sink.msgs) if m[0] == 0x20181219 for r in m[3]]
        while time.time() < deadline and len(reports()) < len(finished):
            time.sleep(0.01)
        got = {}
        for rid, plen, code in reports():
            assert rid not in got, f"{rid} reported twice"
            got[rid] = (plen, code)
        assert set(got) == set(finished)
        good = 0
        for rid, r in finished.items():
            plen, code = got[rid]
            assert code in (0, 500), (rid, code)
            if code == 0:
                assert plen == r["total"]
                check_tokens(src, dsts[r["dst"]], r["sb"], r["db"], 0, r["total"])
                good += 1
        assert good >= max(1, len(finished) // 5), (good, len(finished))
    finally:
        ops.fault_inject_arm(0)
        ops.fault_inject_arm_drop_completion(0)
        for s in srvs:
            s.stop()


def test_server_survives_malformed_and_mutated_frames(ops):
    """Hundreds of frames that no sender of ours produces - valid messages of every kind with bytes flipped,
    fields blown up, tails cut off or junk appended, and pure noise - against one server.  It answers or hangs
    up, never crashes, never writes outside the ranges a well-formed message names, and still serves a
    well-formed transfer afterwards."""
    rng = random.Random(99)
    dst = make_cache()
    srv = KVTransferServer("D|0|1", 1, 0, 0, BLK, TOK, "fake://", dst, [PT.TCP], num_kv_heads=H, cache_shape=2)
    port = int(ops.WorkerInfo.from_string(srv.worker_info()).ext["port"])
    payload = bytes(rng.randrange(256) for _ in range(512))

    def data_msg():
        blocks = [(0, 3 * BLK // 2 + 64, 256), (256, 9 * BLK // 2, 256)]            # src (in blob), dst, len
        body = struct.pack("=QQ", 1, 1) + struct.pack("=Q", len(blocks)) + b"".join(struct.pack("=QQQ", *b) for b in blocks)
        return struct.pack("=IQ", 0x4B564361, 5) + body + struct.pack("=Q", len(payload)) + payload

    def check_msg():
        rs = [(64, 128), (BLK, 4096)]
        return (struct.pack("=IQ", 0x4B56436B, 6) + struct.pack("=IIII", 0, L, 1, 0) + struct.pack("=Q", len(rs))
                + b"".join(struct.pack("=QQ", *r) for r in rs))

    def check_rows_msg():
        layout = struct.pack("=8q6I", BLK // 2, NB * BLK // 2, H * D * 2, D * 2, 0, 0, 0, 0, T, H, D * 2, NB, 2, 0)
        reqs = struct.pack("=6I", 0, 2, 0, 20, 0, 0)
        return (struct.pack("=IQ", 0x4B56436C, 7) + struct.pack("=IIII", 0, L, 0, H) + layout + struct.pack("=II", 1, 2) + reqs
                + struct.pack("=II", 3, 4))

    def attach_msg():
        name = b"/kvx_no_such_segment"
        return struct.pack("=IQ", 0x4B565341, 8) + struct.pack("=I", len(name)) + name + struct.pack("=Q", 4096)

    seeds = [data_msg(), check_msg(), check_rows_msg(), attach_msg(), struct.pack("=IQ", 0x20181218, 9),
             struct.pack("=IQ", 0x4B56504F, 10) + b"\\0" * 64, struct.pack("=IQ", 0x4B565050, 11) + b"\\0" * 40,
             struct.pack("=IQ", 0x4B565069, 12)]

    def mutate(m: bytes) -> bytes:
        b = bytearray(m)
        kind = rng.randrange(6)
        if kind == 0 and len(b) > 12:
            for _ in range(rng.randint(1, 6)):
                b[rng.randrange(4, len(b))] = rng.randrange(256)
        elif kind == 1 and len(b) > 20:
            at = rng.randrange(12, len(b) - 7)
            b[at:at + 8] = struct.pack("=Q", rng.choice([0, 1 << 31, 1 << 40, (1 << 64) - 1, 1 << 62]))
        elif kind == 2 and len(b) > 13:
            del b[rng.randrange(12, len(b)):]
        elif kind == 3:
            b += bytes(rng.randrange(256) for _ in range(rng.randint(1, 64)))
        elif kind == 4:
            b = bytearray(rng.randrange(256) for _ in range(rng.randint(0, 80)))
        return bytes(b)

    def talk(c, msg):
        c.sendall(struct.pack("=I", len(msg)) + msg)
        head = c.recv(4, socket.MSG_WAITALL)
        if len(head) < 4:
            return None
        return c.recv(struct.unpack("=I", head)[0], socket.MSG_WAITALL)

    try:
        c = socket.create_connection(("127.0.0.1", port), timeout=5)
        answered = hung_up = 0
        for i in range(400):
            msg = mutate(rng.choice(seeds)) if i % 5 else rng.choice(seeds[:3] + seeds[7:])
            try:
                r = talk(c, msg)
            except (OSError, socket.timeout):
                r = None
            if r is None:
                hung_up += 1
                c.close()
                c = socket.create_connection(("127.0.0.1", port), timeout=5)
            else:
                answered += 1
        assert answered > 50 and hung_up > 20, (answered, hung_up)
        # still in service: a ping, and an intact transfer lands where it says
        assert struct.unpack("=I", talk(c, struct.pack("=IQ", 0x4B565069, 1))[12:16])[0] == 0
        for d in dst:
            d.zero_()
        assert struct.unpack("=I", talk(c, data_msg())[12:16])[0] == 0
        flat = dst[1].view(torch.uint8).flatten()
        assert bytes(flat[3 * BLK // 2 + 64:3 * BLK // 2 + 64 + 256].tolist()) == payload[:256]
        assert bytes(flat[9 * BLK // 2:9 * BLK // 2 + 256].tolist()) == payload[256:]
        assert int(flat.count_nonzero()) <= 512 and int(dst[0].count_nonzero()) == 0
        c.close()
    finally:
        srv.stop()


def test_shm_transport_leaves_no_name_behind(sink):
    """The segment that carries the SHM transport's data is unlinked as soon as both sides have mapped it: while
    transfers run there is no name of this process under /dev/shm, so a process that dies, or never closes its
    channels, leaves nothing behind."""
    import glob

    src, dst = make_cache(77), make_cache()
    srv = KVTransferServer("D|0|1", 1, 0, 0, BLK, TOK, "fake://", dst, [PT.SHM], num_kv_heads=H, cache_shape=2)
    cli = KVTransferClient("P|0|1", 1, 0, 0, BLK, TOK, "fake://", src, [PT.SHM], num_kv_heads=H, cache_shape=2)
    try:
        for step, nb in enumerate((2, 30)):              # the second batch outgrows the first segment
            sb, db = list(range(1, 1 + nb)), list(range(30, 30 + nb))
            cli.submit_req_send2("D|0|1", 0, f"s{step}", 0, nb * T, True, sb, db, srv.worker_info(), stepid=step + 1)
            cli.start_send_step(step + 1, 1)
            for layer in range(L):
                cli.record_event(layer)
            cli.flush_send_step()
            cli.drain()
            check_tokens(src, dst, sb, db, 0, nb * T)
            assert glob.glob(f"/dev/shm/kvx_{os.getpid()}_*") == []
    finally:
        srv.stop()


def test_worker_info_survives_a_round_trip_whatever_it_holds(ops):
    """Random worker descriptions (several block groups, every optional field, addresses with and without colons,
    extension entries) through to_string / from_string, and malformed strings that must be refused, not crash."""
    from hypothesis import given, settings, strategies as st

    W = ops.WorkerInfo
    name = st.text(alphabet="abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789-_.", min_size=1, max_size=12)
    addr = st.sampled_from(["", "10.0.0.7", "fe80::1", "host-3.cluster.local", "127.0.0.1"])
    ext = st.dictionaries(st.sampled_from(["dev", "port", "shape", "host", "pid", "mx", "mcn", "heads"]),
                          st.integers(0, 1 << 40).map(str), max_size=5)

    @settings(max_examples=200, deadline=None)
    @given(name, st.integers(0, 7), st.integers(0, 64), st.sampled_from([1, 2, 4, 8, 16]),
           st.lists(st.tuples(st.integers(1, 1 << 24), st.integers(1, 1 << 16)), min_size=1, max_size=5),
           st.integers(1, 1 << 20), st.integers(1, 128), st.integers(0, 255), st.integers(1, 256), st.integers(0, 256),
           st.integers(1, 8), st.integers(0, 1 << 20), addr, ext)
    def run(inst, dp, wid, tp, groups, nblocks, layers, protos, ntpb, idx_ntpb, pack, stride, address, extension):
        w = W()
        w.inst_id = f"{inst}|{dp}|{tp}"
        w.worker_id, w.engine_tp_size, w.worker_tp_rank = wid, tp, wid % tp
        w.block_sizes, w.token_sizes = [g[0] for g in groups], [g[1] for g in groups]
        w.layer_num_blocks, w.num_layers, w.transfer_protocols = nblocks, layers, protos
        w.attn_kernel_blk_ntpb, w.indexer_blk_ntpb, w.attn_pack_size, w.kda_page_stride = ntpb, idx_ntpb, pack, stride
        w.addr = address
        w.ext = extension
        back = W.from_string(w.to_string())
        for f in ("inst_id", "worker_id", "engine_tp_size", "worker_tp_rank", "block_sizes", "token_sizes", "layer_num_blocks",
                  "num_layers", "transfer_protocols", "attn_kernel_blk_ntpb", "indexer_blk_ntpb", "attn_pack_size",
                  "kda_page_stride", "addr", "ext"):
            assert getattr(back, f) == getattr(w, f), (f, w.to_string())
        assert back.to_string() == w.to_string()

    run()

    @settings(max_examples=200, deadline=None)
    @given(st.text(alphabet="a0,|:;=x.-", max_size=60))
    def noise(s):
        try:
            W.from_string(s)
        except Exception:
            pass

    noise()
