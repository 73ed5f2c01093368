"""Prefill/decode separation through the connector with the caches on a B200: the prefill
engine's NHD cache is pushed layer by layer into the decode engine's HND cache by the fused
transfer kernel (same GPU here; across NVLink in the multi-GPU file)."""
import time

import pytest
import torch

from pd_helpers import make_pd, make_req

pytestmark = pytest.mark.gpu

LLAMA = dict(layers=4, heads=8, head_dim=128, num_blocks=96)


def spy_add(d):
    captured = {}
    orig = d.scheduler.add_request

    def spy(r):
        captured[r.request_id] = (r.num_computed_tokens, d.scheduler.kv_cache_manager.get_block_ids(r.request_id))
        orig(r)

    d.scheduler.add_request = spy
    return captured


def check_cache(d, toks, blocks, hi):
    from llumnix_kv_b200.ops.p2d_attn import mx_dequantize_reference, mx_quantize_reference

    for w in d.workers:
        for layer in range(d.cfg.model_config.num_layers):
            if d.cfg.cache_config.mx_scaled:
                codes, exps = w.read_kv_mx(layer, blocks, 0, hi)
                exp = w.expected_kv(layer, toks, 0, hi, dtype=torch.bfloat16)
                qc, qe = mx_quantize_reference(exp.float())
                assert torch.equal(exps, qe) and torch.equal(codes, qc), layer
                assert (mx_dequantize_reference(codes, exps).float() - exp.float()).abs().max() <= 0.25
            else:
                assert torch.equal(w.read_kv(layer, blocks, 0, hi), w.expected_kv(layer, toks, 0, hi)), layer


def run_pd(p_kw, d_kw, n_prompt=200, dual=False):
    p, d = make_pd(p_kw=p_kw, d_kw=d_kw)
    try:
        cap = spy_add(d)
        params = {"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()}
        if dual:
            params["do_remote_prefill"] = True
            p.add_request(make_req("g", n_prompt, max_tokens=1, params={"do_remote_decode": True}))
        req = make_req("g", n_prompt, max_tokens=2, params=params)
        d.add_request(req)
        out = d.wait_finished("g", 60)
        assert out is not None and out.finish_reason.name == "LENGTH"
        computed, blocks = cap["g"]
        assert computed == n_prompt - 1
        check_cache(d, req.prompt_token_ids, blocks[0], n_prompt - 1)
        deadline = time.time() + 5
        pool = p.scheduler.kv_cache_manager.block_pool
        while time.time() < deadline and pool.num_free_blocks() != p_kw["num_blocks"] - 1:
            time.sleep(0.01)
        assert pool.num_free_blocks() == p_kw["num_blocks"] - 1
    finally:
        d.shutdown()
        p.shutdown()


def test_pd_nhd_to_hnd_same_gpu():
    run_pd(dict(device="cuda:0", cache_shape=2, **LLAMA), dict(device="cuda:0", cache_shape=5, **LLAMA))


def test_pd_dual_request_chunked_same_gpu():
    run_pd(dict(device="cuda:0", cache_shape=2, max_batched=64, **LLAMA),
           dict(device="cuda:0", cache_shape=5, **LLAMA), n_prompt=333, dual=True)


def test_pd_tp2_to_tp1_block_scaled_fp8():
    run_pd(dict(device="cuda:0", cache_shape=2, tp=2, **LLAMA),
           dict(device="cuda:0", cache_shape=5, tp=1, mx_scaled=True, **LLAMA), n_prompt=150)


@pytest.mark.multigpu
def test_pd_across_nvlink():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_pd(dict(device="cuda:0", cache_shape=2, **LLAMA), dict(device="cuda:1", cache_shape=5, **LLAMA), n_prompt=500)


@pytest.mark.multigpu
def test_pd_tp_mismatch_across_four_gpus():
    if torch.cuda.device_count() < 3:
        pytest.skip("needs three GPUs")
    p, d = None, None
    from pd_helpers import make_cfg
    from llumnix_kv_b200.engine.core import MiniEngineCore

    p = MiniEngineCore(make_cfg("kv_producer", "P", tp=2, cache_shape=2, **LLAMA), devices=["cuda:0", "cuda:1"])
    d = MiniEngineCore(make_cfg("kv_consumer", "D", tp=1, cache_shape=5, **LLAMA), devices=["cuda:2"])
    try:
        cap = spy_add(d)
        req = make_req("x", 130, max_tokens=2, params={"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()})
        d.add_request(req)
        out = d.wait_finished("x", 60)
        assert out is not None and out.finish_reason.name == "LENGTH"
        check_cache(d, req.prompt_token_ids, cap["x"][1][0], 129)
    finally:
        d.shutdown()
        p.shutdown()


def test_pd_hybrid_gdn_model_on_gpu():
    """Hybrid pages (3 GDN groups + attention sharing physical tensors), prefill TP=2 -> decode TP=1:
    no fused kernel for this shape, the planner's ranges drive the descriptor copy kernel over the
    NVLink transport; recurrent state is re-sliced across the TP change."""
    from test_pd_cpu import _check_hybrid, _snapshot_states

    kw = dict(cache_shape=3, layers=8, gdn_groups=3, heads=8, head_dim=64, num_blocks=48)
    p, d = make_pd(p_kw=dict(device="cuda:0", tp=2, max_batched=64, **kw), d_kw=dict(device="cuda:0", tp=1, **kw))
    try:
        cap = spy_add(d)
        states = {}
        orig = d.scheduler.add_request

        def snap(r):
            torch.cuda.synchronize()
            states[r.request_id] = _snapshot_states(d, d.scheduler.kv_cache_manager.get_block_ids(r.request_id))
            orig(r)

        d.scheduler.add_request = snap
        req = make_req("h", 150, max_tokens=2, params={"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()})
        d.add_request(req)
        out = d.wait_finished("h", 60)
        assert out is not None and out.finish_reason.name == "LENGTH"
        computed, blocks = cap["h"]
        assert computed == 149
        _check_hybrid(d, req, blocks, 149, states["h"])
    finally:
        d.shutdown()
        p.shutdown()


def test_pd_mla_latent_and_indexer_on_gpu():
    kw = dict(cache_shape=4, mla=(512, 64, 132), block_size=64, num_blocks=24, layers=3)
    p, d = make_pd(p_kw=dict(device="cuda:0", tp=2, max_batched=128, **kw), d_kw=dict(device="cuda:0", tp=1, **kw))
    try:
        cap = spy_add(d)
        req = make_req("m", 300, max_tokens=2, params={"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()})
        d.add_request(req)
        out = d.wait_finished("m", 60)
        assert out is not None and out.finish_reason.name == "LENGTH"
        computed, blocks = cap["m"]
        assert computed == 299
        for w in d.workers:
            for layer in range(3):
                for t in range(2):
                    assert torch.equal(w.read_rows(layer, t, blocks[0], 0, 299),
                                       w.expected_rows(layer, t, req.prompt_token_ids, 0, 299)), (layer, t)
    finally:
        d.shutdown()
        p.shutdown()
