"""Prefill/decode separation end to end on CPU: two minimal engines, each with its
HybridConnector, the native KVT engine over TCP / shared memory in between."""
import time

import pytest
import torch

from pd_helpers import make_pd, make_req


def check_decode_cache(d, rid, toks, blocks, hi):
    for w in d.workers:
        for layer in range(d.cfg.model_config.num_layers):
            got = w.read_kv(layer, blocks, 0, hi)
            exp = w.expected_kv(layer, toks, 0, hi)
            assert torch.equal(got, exp), (rid, layer)


@pytest.fixture
def pd():
    p, d = make_pd()
    yield p, d
    d.shutdown()
    p.shutdown()


def test_push_mode_prefill_on_p_decode_on_d(pd):
    p, d = pd
    req = make_req("r1", 37, max_tokens=3, params={"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()})
    captured = {}
    orig = d.scheduler.add_request

    def spy(r):
        captured[r.request_id] = (r.num_computed_tokens, d.scheduler.kv_cache_manager.get_block_ids(r.request_id))
        orig(r)

    d.scheduler.add_request = spy
    d.add_request(req)
    out = d.wait_finished("r1", 30)
    assert out is not None and out.finish_reason is not None and out.finish_reason.name == "LENGTH"
    assert len(d.output_tokens("r1")) == 3
    computed, blocks = captured["r1"]
    assert computed == 36   # everything but the last prompt token came over the wire
    check_decode_cache(d, "r1", req.prompt_token_ids, blocks[0], 36)
    # the prefill engine released the request's blocks once its save was acknowledged
    deadline = time.time() + 5
    while time.time() < deadline and p.scheduler.kv_cache_manager.block_pool.num_free_blocks() != 63:
        time.sleep(0.01)
    assert p.scheduler.kv_cache_manager.block_pool.num_free_blocks() == 63
    assert not p.connector._sched._saving and not d.connector._sched._loading
