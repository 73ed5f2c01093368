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
