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


def _spy_add(d):
    captured = {}
    orig = d.scheduler.add_request

    def spy(r):
        captured[r.request_id] = (r.num_computed_tokens, d.scheduler.kv_cache_manager.get_block_ids(r.request_id))
        orig(r)

    d.scheduler.add_request = spy
    return captured


def _dual_params(p):
    return {"do_remote_prefill": True, "remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()}


@pytest.mark.parametrize("p_first", [True, False])
def test_dual_request_mode_either_arrival_order(pd, p_first):
    """The frontend sends one half of the request to P (do_remote_decode) and one to D
    (do_remote_prefill); whichever arrives first waits for the other."""
    p, d = pd
    cap = _spy_add(d)
    rid = f"dual{int(p_first)}"
    preq = make_req(rid, 50, max_tokens=1, params={"do_remote_decode": True})
    dreq = make_req(rid, 50, max_tokens=2, params=_dual_params(p))
    if p_first:
        p.add_request(preq)
        time.sleep(0.2)
        d.add_request(dreq)
    else:
        d.add_request(dreq)
        time.sleep(0.3)      # D polls P and gets 404 a few times
        p.add_request(preq)
    out = d.wait_finished(rid, 30)
    assert out is not None and out.finish_reason.name == "LENGTH"
    computed, blocks = cap[rid]
    assert computed == 49
    check_decode_cache(d, rid, dreq.prompt_token_ids, blocks[0], 49)
    deadline = time.time() + 5
    while time.time() < deadline and p.scheduler.kv_cache_manager.block_pool.num_free_blocks() != 63:
        time.sleep(0.01)
    assert p.scheduler.kv_cache_manager.block_pool.num_free_blocks() == 63


def test_dual_request_gone_on_p_fails_the_load(pd):
    """A request P has aborted answers 410: D gives up at once instead of retrying."""
    p, d = pd
    preq = make_req("gone", 40, max_tokens=1, params={"do_remote_decode": True})
    p.add_request(preq)
    time.sleep(0.3)
    p.abort_requests(["gone"])
    time.sleep(0.3)
    d.add_request(make_req("gone", 40, max_tokens=2, params=_dual_params(p)))
    out = d.wait_finished("gone", 20)
    assert out is not None and out.finish_reason.name == "ABORT"
    deadline = time.time() + 5
    while time.time() < deadline and d.scheduler.kv_cache_manager.block_pool.num_free_blocks() != 63:
        time.sleep(0.01)
    assert d.scheduler.kv_cache_manager.block_pool.num_free_blocks() == 63
    assert p.scheduler.kv_cache_manager.block_pool.num_free_blocks() == 63


def test_chunked_prefill_sends_deltas():
    """A prompt longer than the prefill engine's token budget goes out chunk by chunk."""
    p, d = make_pd(p_kw={"max_batched": 32})
    try:
        cap = _spy_add(d)
        req = make_req("chunky", 150, max_tokens=2,
                       params={"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()})
        d.add_request(req)
        out = d.wait_finished("chunky", 30)
        assert out is not None and out.finish_reason.name == "LENGTH"
        computed, blocks = cap["chunky"]
        assert computed == 149
        check_decode_cache(d, "chunky", req.prompt_token_ids, blocks[0], 149)
        assert p.steps >= 5
    finally:
        d.shutdown()
        p.shutdown()


@pytest.mark.parametrize("ptp,dtp", [(2, 1), (1, 2), (4, 2), (2, 2)])
def test_tp_mismatch(ptp, dtp):
    p, d = make_pd(p_kw={"tp": ptp}, d_kw={"tp": dtp})
    try:
        cap = _spy_add(d)
        req = make_req("tp", 45, max_tokens=2, params={"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()})
        d.add_request(req)
        out = d.wait_finished("tp", 30)
        assert out is not None and out.finish_reason.name == "LENGTH"
        computed, blocks = cap["tp"]
        assert computed == 44
        check_decode_cache(d, "tp", req.prompt_token_ids, blocks[0], 44)
    finally:
        d.shutdown()
        p.shutdown()


def test_many_concurrent_requests(pd):
    p, d = pd
    cap = _spy_add(d)
    reqs = [make_req(f"c{i}", 20 + 7 * i, max_tokens=2, seed=i,
                     params={"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()}) for i in range(6)]
    for r in reqs:
        d.add_request(r)
    for r in reqs:
        out = d.wait_finished(r.request_id, 30)
        assert out is not None and out.finish_reason.name == "LENGTH", r.request_id
        computed, blocks = cap[r.request_id]
        n = len(r.prompt_token_ids) - 1
        assert computed == n
    # decode blocks are released after finish; the caches were checked at admission time above
    deadline = time.time() + 5
    while time.time() < deadline and p.scheduler.kv_cache_manager.block_pool.num_free_blocks() != 63:
        time.sleep(0.01)
    assert p.scheduler.kv_cache_manager.block_pool.num_free_blocks() == 63
    assert d.scheduler.kv_cache_manager.block_pool.num_free_blocks() == 63


def test_abort_on_decode_side_releases_everything(pd):
    """Abort while the load is outstanding: D drops the request, tells P, both free their blocks."""
    p, d = pd
    # P never gets its half, so D keeps polling
    d.add_request(make_req("ab", 40, max_tokens=2, params=_dual_params(p)))
    time.sleep(0.3)
    d.abort_requests(["ab"])
    out = d.wait_finished("ab", 20)
    assert out is not None and out.finish_reason.name == "ABORT"
    deadline = time.time() + 5
    while time.time() < deadline and d.scheduler.kv_cache_manager.block_pool.num_free_blocks() != 63:
        time.sleep(0.01)
    assert d.scheduler.kv_cache_manager.block_pool.num_free_blocks() == 63
    assert not d.connector._sched._loading


def _snapshot_states(d, blocks_by_group):
    """The recurrent-state pages as they are when the load has finished (the decode engine advances
    them as soon as it computes its own first token)."""
    mc = d.cfg.model_config
    return [{layer: w.read_state(layer, blocks_by_group[mc.layer_group(layer)][0])
             for layer in range(mc.num_layers) if mc.is_gdn_layer(layer)} for w in d.workers]


def _check_hybrid(d, req, blocks_by_group, n_ctx, states):
    mc = d.cfg.model_config
    for w, snap in zip(d.workers, states):
        for layer in range(mc.num_layers):
            if mc.is_gdn_layer(layer):
                conv, ssm = snap[layer]
                ec, es = w.expected_state(layer, req.prompt_token_ids, n_ctx)
                assert torch.equal(conv, ec) and torch.equal(ssm, es), ("state", layer)
            else:
                got = w.read_kv(layer, blocks_by_group[-1], 0, n_ctx)
                assert torch.equal(got, w.expected_kv(layer, req.prompt_token_ids, 0, n_ctx)), ("kv", layer)


@pytest.mark.parametrize("ptp,dtp", [(1, 1), (2, 1), (1, 2)])
def test_hybrid_gdn_model_state_and_attention_pages(ptp, dtp):
    """Qwen3-Next-like model: 3 GDN groups + 1 attention group, 8 logical layers in 2 physical tensors.
    The prefill engine drops the last prompt token, ships attention KV as it is computed and the
    recurrent state of every GDN layer with the last chunk; TP-mismatched ranks re-slice both."""
    kw = dict(cache_shape=3, layers=8, gdn_groups=3)
    p, d = make_pd(p_kw=dict(tp=ptp, max_batched=48, **kw), d_kw=dict(tp=dtp, **kw))
    try:
        cap = _spy_add(d)
        states = {}
        orig_add = d.scheduler.add_request

        def snap(r):
            states[r.request_id] = _snapshot_states(d, d.scheduler.kv_cache_manager.get_block_ids(r.request_id))
            orig_add(r)

        d.scheduler.add_request = snap
        req = make_req("h", 101, max_tokens=2, params={"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()})
        d.add_request(req)
        out = d.wait_finished("h", 30)
        assert out is not None and out.finish_reason.name == "LENGTH"
        computed, blocks = cap["h"]
        assert computed == 100 and len(blocks) == 4 and [len(g) for g in blocks[:3]] == [1, 1, 1]
        _check_hybrid(d, req, blocks, 100, states["h"])
        deadline = time.time() + 5
        free_all = p.cfg.cache_config.num_gpu_blocks - 1
        while time.time() < deadline and p.scheduler.kv_cache_manager.block_pool.num_free_blocks() != free_all:
            time.sleep(0.01)
        assert p.scheduler.kv_cache_manager.block_pool.num_free_blocks() == free_all
    finally:
        d.shutdown()
        p.shutdown()


@pytest.mark.parametrize("ptp,dtp,shape,mla", [(1, 1, 4, (64, 16, 36)), (2, 1, 4, (64, 16, 36)), (1, 2, 4, (64, 16, 36)),
                                              (2, 1, 1, (64, 16, 0))])
def test_mla_latent_and_indexer_caches(ptp, dtp, shape, mla):
    """DeepSeek-style caches: one head-less latent+rope row per token (and, for sparse attention, an
    indexer-key row in a second tensor of the layer), identical on every TP rank: with more prefill
    ranks than decode ranks only one of them sends, with fewer each one feeds several."""
    kw = dict(cache_shape=shape, mla=mla, block_size=64 if shape == 4 else 16, num_blocks=24)
    p, d = make_pd(p_kw=dict(tp=ptp, max_batched=100, **kw), d_kw=dict(tp=dtp, **kw))
    try:
        cap = _spy_add(d)
        req = make_req("m", 230, max_tokens=2, params={"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()})
        d.add_request(req)
        out = d.wait_finished("m", 30)
        assert out is not None and out.finish_reason.name == "LENGTH"
        computed, blocks = cap["m"]
        assert computed == 229
        for w in d.workers:
            for layer in range(2):
                for t in range(len(w.row_widths)):
                    assert torch.equal(w.read_rows(layer, t, blocks[0], 0, 229),
                                       w.expected_rows(layer, t, req.prompt_token_ids, 0, 229)), (layer, t)
    finally:
        d.shutdown()
        p.shutdown()


def test_cross_layout_over_a_byte_range_transport_fails_the_request_cleanly():
    """NHD -> HND needs the fused kernel (GPU caches, NVLINK transport).  Between host-memory caches
    the transfer is refused: the prefill side marks the request failed, the decode side aborts it
    and nobody keeps blocks; no misplaced bytes are delivered."""
    p, d = make_pd(p_kw=dict(cache_shape=2), d_kw=dict(cache_shape=5))
    try:
        d.add_request(make_req("x", 40, max_tokens=2, params={"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()}))
        out = d.wait_finished("x", 30)
        assert out is not None and out.finish_reason.name == "ABORT"
        for e in (p, d):
            deadline = time.time() + 5
            while time.time() < deadline and e.scheduler.kv_cache_manager.block_pool.num_free_blocks() != 63:
                time.sleep(0.01)
            assert e.scheduler.kv_cache_manager.block_pool.num_free_blocks() == 63
        assert not any(t.any() for t in d.workers[0].kv_caches.values())
    finally:
        d.shutdown()
        p.shutdown()


def test_peer_discovery_and_worker_info_through_file_naming(tmp_path):
    """With a naming service nothing travels inside the request: the decode engine finds a prefill
    engine through the registry (role "prefill"), and the prefill engine's native stubs look the
    decode workers' WorkerInfo up there as well."""
    url = f"file:{tmp_path}"
    p, d = make_pd(p_kw=dict(extra={"naming_url": url}), d_kw=dict(extra={"naming_url": url}, tp=2))
    try:
        cap = _spy_add(d)
        deadline = time.time() + 10
        while time.time() < deadline and d.connector._sched._backend.get_peer() is None:
            time.sleep(0.05)
        assert d.connector._sched._backend.get_peer() == ("127.0.0.1", p.proxy.rpc_port())
        req = make_req("n", 55, max_tokens=2)            # no remote_host / remote_port
        d.add_request(req)
        out = d.wait_finished("n", 30)
        assert out is not None and out.finish_reason.name == "LENGTH"
        computed, blocks = cap["n"]
        assert computed == 54
        check_decode_cache(d, "n", req.prompt_token_ids, blocks[0], 54)
        names = {x.name for x in tmp_path.iterdir()}
        assert {"P", "D"} <= names
    finally:
        d.shutdown()
        p.shutdown()


def test_bypass_substep_delivers_a_late_transfer_without_a_forward_pass(monkeypatch):
    """Dual-request mode with the prefill half finished long before the decode half arrives: the
    transfer is handed to the workers as a substep of the last engine step over the bypass channel
    (ZMQ publish / subscribe), not by running another model step."""
    monkeypatch.setenv("VLLM_ENABLE_BYPASS_TASK", "1")
    p, d = make_pd()
    try:
        cap = _spy_add(d)
        p.add_request(make_req("late", 50, max_tokens=1, params={"do_remote_decode": True}))
        time.sleep(0.5)
        steps_before = p.workers[0].forward_passes
        dreq = make_req("late", 50, max_tokens=2, params=_dual_params(p))
        d.add_request(dreq)
        out = d.wait_finished("late", 30)
        assert out is not None and out.finish_reason.name == "LENGTH"
        computed, blocks = cap["late"]
        assert computed == 49
        check_decode_cache(d, "late", dreq.prompt_token_ids, blocks[0], 49)
        assert p.bypass_substeps >= 1
        assert p.workers[0].forward_passes == steps_before      # no extra forward pass on the prefill engine
    finally:
        d.shutdown()
        p.shutdown()


def test_injected_transport_failures_fail_requests_cleanly_and_later_ones_recover(pd):
    """Transport faults injected on the host while requests stream through a P/D pair: a request whose
    batch failed ends with ABORT on D (the 500 of the send stub travels P scheduler -> KVTResp -> load
    failure), every other request decodes the right tokens, and nothing stays referenced on either side."""
    from llumnix_kv_b200 import load_ops

    ops = load_ops()
    p, d = pd
    params = {"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()}
    outcomes = {}
    try:
        for i in range(10):
            if i in (2, 5, 6):
                ops.fault_inject_arm(1)          # the next fault point any sender passes throws
            rid = f"x{i}"
            d.add_request(make_req(rid, 24 + 5 * i, max_tokens=2, seed=i, params=params))
            out = d.wait_finished(rid, 30)
            ops.fault_inject_arm(0)
            assert out is not None, rid
            outcomes[rid] = out.finish_reason.name
        assert set(outcomes.values()) <= {"LENGTH", "ABORT"}
        assert [outcomes[f"x{i}"] for i in (0, 1, 3, 4, 7, 8, 9)] == ["LENGTH"] * 7, outcomes
        assert any(outcomes[f"x{i}"] == "ABORT" for i in (2, 5, 6)), outcomes
        # a request that went through decodes exactly what a colocated engine would
        assert d.output_tokens("x9") and len(d.output_tokens("x9")) == 2
        deadline = time.time() + 10
        pools = [e.scheduler.kv_cache_manager.block_pool for e in (p, d)]
        while time.time() < deadline and any(pl.num_free_blocks() != 63 for pl in pools):
            time.sleep(0.01)
        assert [pl.num_free_blocks() for pl in pools] == [63, 63]
        assert not p.connector._sched._saving and not d.connector._sched._loading
    finally:
        ops.fault_inject_arm(0)


def test_prefill_worker_hands_replicated_requests_to_one_decode_worker():
    """A prefill worker (TP 1) of an MLA model whose decode instance has four workers submits every chunk
    to each of them - unless they advertise a multicast group: then one of them gets the request with
    fanout=4, the same one for every chunk of that request."""
    from pd_helpers import make_cfg

    from llumnix_kv_b200.engine.core import MiniEngineCore
    from llumnix_kv_b200.hybrid_connector.kvtbackend import KVTPMeta, PReqMeta

    p = MiniEngineCore(make_cfg("kv_producer", "PX", cache_shape=4, mla=(512, 64, 132), block_size=64, num_blocks=16))
    try:
        backend = p.workers[0].connector._worker._backend
        calls = []

        class Recorder:
            def submit_req_send2(self, inst, wid, reqid, seen, new, last, sb, db, winfo, stepid=0, fanout=0):
                calls.append((inst, wid, reqid, seen, new, fanout))

            def submit_delta_send(self, *a, **k):
                calls.append(("delta",) + a)

            def start_send_step(self, **k):
                pass

        backend._kvt_cli = Recorder()

        def winfo(rank, mcn):
            tail = f";mcn={mcn}" if mcn else ""
            return f"DX|0|4,{rank},4,{rank},4096,256,8,2,4,16,0,1,0,10.0.0.1,x:dev={rank};heads=1{tail};pid=1;port=2;shape=4"

        def step(stepid, reqid, seen, new, infos):
            meta = KVTPMeta(stepid=stepid, sched_tokens=new)
            meta.nonfreeze_metas = [PReqMeta(reqid=reqid, d_inst_id="DX|0|4", p_block_ids=[[1, 2]], d_block_ids=[[3, 4]],
                                             new_tokens=new, has_last_token=False, seen_tokens=seen, d_workers_info=infos)]
            backend.bind_backend_metadata(meta)

        step(1, "plain", 0, 64, [winfo(r, 0) for r in range(4)])
        assert [(c[1], c[5]) for c in calls] == [(0, 0), (1, 0), (2, 0), (3, 0)]        # one send per decode worker
        calls.clear()
        step(2, "grouped", 0, 64, [winfo(r, 4) for r in range(4)])
        step(3, "grouped", 64, 32, [winfo(r, 4) for r in range(4)])
        assert len(calls) == 2 and calls[0][5] == calls[1][5] == 4 and calls[0][1] == calls[1][1]    # one relay, kept
        relays = set()
        for i in range(32):
            calls.clear()
            step(10 + i, f"r{i}", 0, 64, [winfo(r, 4) for r in range(4)])
            relays.add(calls[0][1])
        assert relays == {0, 1, 2, 3}                                                   # the group shares the work
    finally:
        p.shutdown()


_MODELS = {
    "llama": (dict(), 63),
    "gdn": (dict(cache_shape=3, layers=8, gdn_groups=3), 63),
    "mla": (dict(cache_shape=4, mla=(64, 16, 36), block_size=64, num_blocks=24), 23),
}


@pytest.mark.parametrize("model,ptp,dtp,seed", [("llama", 1, 1, 1), ("llama", 1, 1, 2), ("llama", 2, 1, 3), ("gdn", 1, 1, 4),
                                                ("gdn", 2, 1, 5), ("mla", 1, 2, 6)])
def test_random_arrivals_aborts_and_transport_faults_leak_nothing(model, ptp, dtp, seed):
    """Requests arrive in bursts with random prompt lengths; some are aborted on the decode side at a random
    moment (before the prefill engine has them, while their KV is moving, or while they decode), and a few
    transfers hit an injected transport fault.  Whatever the interleaving: every request ends (LENGTH or
    ABORT), one that was neither aborted nor hit by a fault decodes its tokens, both engines get every block
    back and neither connector keeps a request."""
    import random

    from llumnix_kv_b200 import load_ops

    ops = load_ops()
    rng = random.Random(seed)
    kw, free_all = _MODELS[model]
    p, d = make_pd(p_kw=dict(tp=ptp, max_batched=64, **kw), d_kw=dict(tp=dtp, **kw))
    params = {"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()}
    reqs, aborted = [], set()
    faults = 0
    try:
        for burst in range(4):
            batch = [make_req(f"s{seed}.{burst}.{i}", rng.randint(5, 90), max_tokens=rng.randint(1, 4), seed=seed * 100 + burst * 10 + i,
                              params=params) for i in range(rng.randint(2, 5))]
            if rng.random() < 0.5:
                ops.fault_inject_arm(rng.randint(1, 3))      # one of the next few fault points throws
                faults += 1
            for r in batch:
                d.add_request(r)
                reqs.append(r)
                if rng.random() < 0.3:
                    time.sleep(rng.choice([0.0, 0.002, 0.02, 0.1]))
                    d.abort_requests([r.request_id])
                    aborted.add(r.request_id)
            time.sleep(rng.choice([0.0, 0.05, 0.2]))
        ops.fault_inject_arm(0)
        ended = {}
        for r in reqs:
            out = d.wait_finished(r.request_id, 60)
            assert out is not None, r.request_id
            ended[r.request_id] = out.finish_reason.name
        assert set(ended.values()) <= {"LENGTH", "ABORT"}, ended
        clean = [rid for rid, how in ended.items() if how == "LENGTH"]
        # one fault fails the whole batch it hits: up to a burst of five requests
        assert len(clean) >= len(reqs) - len(aborted) - 6 * faults, (ended, aborted, faults)
        for r in reqs:
            if ended[r.request_id] == "LENGTH":
                assert len(d.output_tokens(r.request_id)) == r.sampling_params.max_tokens, r.request_id
        deadline = time.time() + 15
        pools = [e.scheduler.kv_cache_manager.block_pool for e in (p, d)]
        while time.time() < deadline and (any(pl.num_free_blocks() != free_all for pl in pools) or p.connector._sched._saving
                                          or d.connector._sched._loading):
            time.sleep(0.01)
        left = {"free": [pl.num_free_blocks() for pl in pools], "p_saving": list(p.connector._sched._saving),
                "d_loading": list(d.connector._sched._loading)}
        assert left["free"] == [free_all, free_all] and not left["p_saving"] and not left["d_loading"], left
    finally:
        ops.fault_inject_arm(0)
        d.shutdown()
        p.shutdown()


@pytest.mark.parametrize("ptp,dtp,seed,bypass", [(1, 1, 1, False), (2, 1, 2, False), (1, 2, 3, False), (1, 1, 4, True), (2, 2, 5, True)])
def test_random_dual_requests_with_aborts_on_either_side(ptp, dtp, seed, bypass, monkeypatch):
    """Dual-request mode under a careless frontend: the two halves of a request reach the prefill and the
    decode engine in either order and at random distances, prompts are longer than the prefill engine's token
    budget (chunked prefill, deltas), the engines may be tensor-parallel with different sizes, and some
    requests are aborted on the prefill side, on the decode side or on both, at random moments.  Every
    decode-side request ends; one that nobody aborted decodes; both engines get every block back and neither
    connector keeps a request.  With ``bypass`` the engines run with bypass tasks and substeps on."""
    import random

    rng = random.Random(seed)
    # a prefill half whose decode half never comes (aborted before it got in touch) is given up after this long
    monkeypatch.setenv("VLLM_PD_TRY_CONNECT_TIMEOUT_SECONDS", "1.5")
    if bypass:          # late transfers go to the workers as substeps, without a forward pass
        monkeypatch.setenv("VLLM_ENABLE_BYPASS_TASK", "1")
        monkeypatch.setenv("VLLM_ENABLE_BYPASS_SUBSTEP", "1")
    p, d = make_pd(p_kw={"tp": ptp, "max_batched": 48}, d_kw={"tp": dtp})
    try:
        reqs, touched = [], set()
        for i in range(14):
            rid = f"u{seed}.{i}"
            n = rng.randint(8, 140)
            preq = make_req(rid, n, max_tokens=1, seed=i, params={"do_remote_decode": True})
            dreq = make_req(rid, n, max_tokens=rng.randint(1, 3), seed=i, params=_dual_params(p))
            first, second = ((p, preq), (d, dreq)) if rng.random() < 0.5 else ((d, dreq), (p, preq))
            first[0].add_request(first[1])
            time.sleep(rng.choice([0.0, 0.0, 0.01, 0.06]))
            second[0].add_request(second[1])
            reqs.append(dreq)
            roll = rng.random()
            if roll < 0.35:
                time.sleep(rng.choice([0.0, 0.005, 0.03, 0.1]))
                if roll < 0.15:
                    p.abort_requests([rid])
                elif roll < 0.3:
                    d.abort_requests([rid])
                else:
                    d.abort_requests([rid])
                    p.abort_requests([rid])
                touched.add(rid)
        for r in reqs:
            out = d.wait_finished(r.request_id, 60)
            assert out is not None, r.request_id
            how = out.finish_reason.name
            assert how in ("LENGTH", "ABORT"), (r.request_id, how)
            if r.request_id not in touched:
                assert how == "LENGTH", r.request_id
                assert len(d.output_tokens(r.request_id)) == r.sampling_params.max_tokens
        deadline = time.time() + 20
        pools = [e.scheduler.kv_cache_manager.block_pool for e in (p, d)]
        while time.time() < deadline and (any(pl.num_free_blocks() != 63 for pl in pools) or p.connector._sched._saving
                                          or d.connector._sched._loading):
            time.sleep(0.01)
        left = {"free": [pl.num_free_blocks() for pl in pools], "p_saving": list(p.connector._sched._saving),
                "d_loading": list(d.connector._sched._loading), "p_running": [r.request_id for r in p.scheduler.running],
                "p_waiting": [r.request_id for r in p.scheduler.waiting], "d_running": [r.request_id for r in d.scheduler.running],
                "touched": sorted(touched)}
        assert left["free"] == [63, 63], left
        assert not p.connector._sched._saving and not d.connector._sched._loading
    finally:
        d.shutdown()
        p.shutdown()


def test_prefill_engine_goes_away_mid_stream_and_a_new_one_serves_the_next_requests():
    """The prefill engine stops while the decode engine has requests with it (some being computed, some
    queued, some moving).  Every one of them ends on the decode side in bounded time - none waits for an answer
    that cannot come - the decode engine gets its blocks back, and requests sent to a fresh prefill engine
    afterwards decode as usual."""
    p, d = make_pd(p_kw={"max_batched": 32})
    p2 = None
    try:
        params = {"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()}
        slow = p.step
        p.step = lambda: (time.sleep(0.01), slow())[1]                  # keep requests in the prefill engine for a while
        reqs = [make_req(f"g{i}", 60 + 20 * i, max_tokens=2, seed=i, params=params) for i in range(6)]
        for r in reqs:
            d.add_request(r)
        time.sleep(0.08)
        p.shutdown()                                                    # RPC server, workers and transfer client go away
        ended = {}
        for r in reqs:
            out = d.wait_finished(r.request_id, 60)
            assert out is not None, r.request_id
            ended[r.request_id] = out.finish_reason.name
        assert set(ended.values()) <= {"LENGTH", "ABORT"} and "ABORT" in ended.values(), ended
        deadline = time.time() + 15
        pool = d.scheduler.kv_cache_manager.block_pool
        while time.time() < deadline and (pool.num_free_blocks() != 63 or d.connector._sched._loading):
            time.sleep(0.01)
        assert pool.num_free_blocks() == 63 and not d.connector._sched._loading
        from pd_helpers import make_cfg
        from llumnix_kv_b200.engine.core import MiniEngineCore

        p2 = MiniEngineCore(make_cfg("kv_producer", "P2"))
        params2 = {"remote_host": "127.0.0.1", "remote_port": p2.proxy.rpc_port()}
        for i in range(3):
            d.add_request(make_req(f"n{i}", 50 + i, max_tokens=2, seed=20 + i, params=params2))
        for i in range(3):
            out = d.wait_finished(f"n{i}", 30)
            assert out is not None and out.finish_reason.name == "LENGTH", i
    finally:
        d.shutdown()
        if p2 is not None:
            p2.shutdown()


def test_decode_engine_goes_away_mid_stream_and_the_prefill_engine_lets_go_of_everything():
    """The mirror image: the decode engine stops while the prefill engine computes and ships its requests.  The
    transfers fail on the host (nobody listens any more), the prefill engine finishes or fails every request, gets
    every block back, keeps no request in its connector, and serves a fresh decode engine afterwards."""
    p, d = make_pd(p_kw={"max_batched": 32})
    d2 = None
    try:
        params = {"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()}
        slow = p.step
        p.step = lambda: (time.sleep(0.01), slow())[1]
        for i in range(6):
            d.add_request(make_req(f"v{i}", 60 + 20 * i, max_tokens=2, seed=i, params=params))
        time.sleep(0.08)
        d.shutdown()
        deadline = time.time() + 30
        pool = p.scheduler.kv_cache_manager.block_pool
        sched = p.connector._sched
        while time.time() < deadline and (pool.num_free_blocks() != 63 or sched._saving or p.scheduler.running or p.scheduler.waiting):
            time.sleep(0.01)
        left = {"free": pool.num_free_blocks(), "saving": list(sched._saving), "running": [r.request_id for r in p.scheduler.running],
                "waiting": [r.request_id for r in p.scheduler.waiting]}
        assert left == {"free": 63, "saving": [], "running": [], "waiting": []}, left
        from pd_helpers import make_cfg
        from llumnix_kv_b200.engine.core import MiniEngineCore

        d2 = MiniEngineCore(make_cfg("kv_consumer", "D2"))
        for i in range(3):
            d2.add_request(make_req(f"w{i}", 50 + i, max_tokens=2, seed=30 + i, params=params))
        for i in range(3):
            out = d2.wait_finished(f"w{i}", 30)
            assert out is not None and out.finish_reason.name == "LENGTH", i
    finally:
        p.shutdown()
        if d2 is not None:
            d2.shutdown()


def test_engines_come_and_go_behind_a_naming_service(tmp_path, monkeypatch):
    """With a registry, the engines find each other by name and role.  The decode engine is replaced by a new
    one under the same name (new process in real life: new ports, new worker infos), then the prefill engine is
    replaced as well: each side notices through the registry, drops what it knew about the old peer, and the
    requests that follow a replacement are served as the first ones were."""
    from pd_helpers import make_cfg
    from llumnix_kv_b200.engine.core import MiniEngineCore

    from llumnix_kv_b200.hybrid_connector.utils import PeerManager

    monkeypatch.setattr(PeerManager, "POLL_S", 0.2)          # the registry is polled every 7 s in production
    url = f"file:{tmp_path}"
    ex = {"naming_url": url}
    p = MiniEngineCore(make_cfg("kv_producer", "P", extra=dict(ex)))
    d = MiniEngineCore(make_cfg("kv_consumer", "D", extra=dict(ex)))
    engines = [p, d]

    def serve(dec, pre, tag, n=3):
        deadline = time.time() + 20
        want = ("127.0.0.1", pre.proxy.rpc_port())
        while time.time() < deadline and dec.connector._sched._backend.get_peer() != want:
            time.sleep(0.05)
        assert dec.connector._sched._backend.get_peer() == want, tag
        cap = _spy_add(dec)
        reqs = [make_req(f"{tag}{i}", 40 + 9 * i, max_tokens=2, seed=i) for i in range(n)]
        for r in reqs:
            dec.add_request(r)
        for r in reqs:
            out = dec.wait_finished(r.request_id, 30)
            assert out is not None and out.finish_reason.name == "LENGTH", r.request_id
            computed, blocks = cap[r.request_id]
            check_decode_cache(dec, r.request_id, r.prompt_token_ids, blocks[0], computed)

    try:
        serve(d, p, "a")
        d.shutdown()
        d = MiniEngineCore(make_cfg("kv_consumer", "D", extra=dict(ex)))      # same name, everything else new
        engines[1] = d
        serve(d, p, "b")
        p.shutdown()
        p = MiniEngineCore(make_cfg("kv_producer", "P", extra=dict(ex)))
        engines[0] = p
        serve(d, p, "c")
    finally:
        for e in engines:
            e.shutdown()


def test_control_plane_survives_malformed_messages(pd, monkeypatch):
    """Every RPC the two schedulers answer, with bodies no peer of ours sends (noise, truncated msgpack, wrong
    types, absurd lengths) and with unknown heads: the sender loses its connection at most; both engines stay
    up, with the default setting that aborts the process on a failed background task, and serve the next
    request."""
    import random
    import socket
    import struct

    import llumnix_kv_b200.hybrid_connector.utils as U

    monkeypatch.setattr(U, "ABORT_ON_TASK_EXCEPTION", True)          # production default; the tests run with it off
    rng = random.Random(5)
    p, d = pd
    heads = [0x20181218, 0x20210912, 0x20181219, 20250820, 0x20181221, 0x20181222, 0x20181223, 0x20181224, 0x20181226,
             20080818, 20080901, 20080903, 20080828, 0x20240912, 0xDEADBEEF, 0]
    bodies = [b"", b"\\xff" * 7, struct.pack("=I", 5) + b"\\x93\\x01\\x02", struct.pack("=I", 1 << 30) + b"x" * 16,
              struct.pack("=I", 12) + b"\\x91\\xa3abc" + b"\\0" * 8, struct.pack("=II", 0x40000001, 3) + b"\\0" * 11]
    for eng in (p, d):
        port = eng.proxy.rpc_port()
        for head in heads:
            for _ in range(4):
                body = rng.choice(bodies) if rng.random() < 0.7 else bytes(rng.randrange(256) for _ in range(rng.randint(1, 60)))
                try:
                    with socket.create_connection(("127.0.0.1", port), timeout=2) as c:
                        c.sendall(struct.pack("=I", head) + body)
                        c.settimeout(0.05)
                        try:
                            c.recv(64)
                        except (socket.timeout, OSError):
                            pass
                except OSError:
                    pass
    req = make_req("after", 44, max_tokens=2, params={"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()})
    d.add_request(req)
    out = d.wait_finished("after", 30)
    assert out is not None and out.finish_reason.name == "LENGTH"
