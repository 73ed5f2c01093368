"""Auxiliary subsystems on CPU: process monitor line protocol, gdrcopy shim, CRC, NVLink affinity
table helpers, KV specs of the model families."""
import os
import socket
import zlib

from llumnix_kv_b200 import load_ops, nvlink_affinity
from llumnix_kv_b200.models.kv_spec import DEEPSEEK_V32, LLAMA3_8B, LLAMA3_70B, QWEN3_NEXT_80B, SPECS
from llumnix_kv_b200.ops.layouts import CacheShape


def test_monitor_line_protocol(tmp_path):
    K = load_ops()
    port = K.monitor_start()
    assert port > 0 and K.monitor_port() == port and K.monitor_start() == port    # idempotent
    try:
        s = socket.create_connection(("127.0.0.1", port), timeout=5)
        f = s.makefile("rw")

        def cmd(line):
            f.write(line + "\n")
            f.flush()
            return f.readline().strip()

        assert cmd("prof active").startswith("prev=")        # -33 without jemalloc, 0/1 with it
        assert cmd("prof deactive").startswith("prev=")
        dump = tmp_path / "heap.out"
        assert cmd(f"prof dump {dump}") == "ok" and dump.stat().st_size > 0
        assert cmd("prof dump ") == "empty filepath"
        stats = cmd("stats")
        assert "rss_bytes=" in stats and "malloc_in_use=" in stats
        assert cmd("bogus") == "unknown command"
        f.write("quit\n")
        f.flush()
        assert f.readline() == ""                               # server closed the connection
        s.close()
    finally:
        K.monitor_stop()
    assert K.monitor_port() == 0


def test_env_dump_lists_resolved_settings():
    K = load_ops()
    K.env_port_base()
    assert "BLLM_KVTRANS_PORT_BASE=" in K.envcfg_dump()


def test_gdr_shim_reports_unavailable_and_crc_matches_zlib():
    K = load_ops()
    ok, why = K.gdr_available()
    assert ok or "libgdrapi" in why
    data = bytes(range(256)) * 37
    assert K.crc32_bytes(data) == zlib.crc32(data)
    assert K.crc32_bytes(data[100:], K.crc32_bytes(data[:100])) == zlib.crc32(data)


def test_affinity_helpers_on_a_synthetic_switch_topology():
    n = 8
    topo = {"gpus": [{"index": i, "multicast_supported": 1, "nvlink_links_up": 18} for i in range(n)],
            "links": [{"src": a, "dst": b, "access": 1, "perf_rank": 0, "native_atomics": 1}
                      for a in range(n) for b in range(n) if a != b]}
    assert nvlink_affinity.best_peers(topo, 2) == [0, 1, 3, 4, 5, 6, 7]
    assert nvlink_affinity.pair_prefill_decode(topo, 4) == [(0, 4), (1, 5), (2, 6), (3, 7)]
    assert nvlink_affinity.nvls_capable(topo)
    topo["links"] = [l for l in topo["links"] if not (l["src"] == 0 and l["dst"] == 4)]
    assert nvlink_affinity.pair_prefill_decode(topo, 4)[0] == (0, 5)
    topo["gpus"][3]["multicast_supported"] = 0
    assert not nvlink_affinity.nvls_capable(topo)


def test_affinity_file_roundtrip(tmp_path):
    path = nvlink_affinity.generate(str(tmp_path / "aff.json"))   # no GPU here: an empty but valid table
    topo = nvlink_affinity.load(path)
    assert "gpus" in topo and "links" in topo


def test_kv_specs():
    assert LLAMA3_8B.token_bytes() == 4096 and LLAMA3_8B.token_bytes(tp=4) == 1024
    assert LLAMA3_70B.heads_on_rank(16) == 1                    # GQA heads replicate beyond 8-way TP
    lay = LLAMA3_8B.attn_layout(CacheShape.FLASHINFER, 10, tp=2)
    assert lay.num_heads == 4 and lay.block_bytes == 2 * 16 * 4 * 128 * 2
    mla = DEEPSEEK_V32.attn_layout(CacheShape.DPSK_V32_SPARSE_MLA, 4)
    assert mla.kv_count == 1 and mla.block_bytes == 64 * 576 * 2
    assert QWEN3_NEXT_80B.linear_state_bytes(tp=2) == 3 * 4096 * 2 + 16 * 128 * 128 * 4
    assert set(SPECS) >= {"llama-3-8b", "deepseek-v3.2", "kimi-k3"}


def test_prefill_worker_fills_the_paged_cache_and_calls_the_layer_hook():
    import torch

    from benchmarks.llama_prefill import TINY_GEOMETRY, PrefillWorker

    w = PrefillWorker(TINY_GEOMETRY, "cpu", 12)
    toks = torch.randint(0, TINY_GEOMETRY.vocab, (70,))
    blocks = torch.tensor([3, 5, 7, 9, 1])
    calls = []
    t1 = w.prefill(toks, blocks, after_layer=calls.append)
    assert calls == [0, 1]
    view = w.layout.view(w.kv_caches[1], torch.bfloat16)
    used = view[blocks]
    assert used[:4].abs().sum() > 0 and used[4, :, :6].abs().sum() > 0      # 70 tokens = 4 blocks + 6 slots
    assert view[[0, 2, 4, 6, 8, 10, 11]].abs().sum() == 0 and used[4, :, 6:].abs().sum() == 0
    # same prompt, same first token; the KV of a prefix does not depend on what follows it (causal)
    before = view[blocks[:2]].clone()
    t2 = w.prefill(toks, blocks)
    assert torch.equal(t1, t2)
    w.prefill(torch.cat([toks[:32], torch.randint(0, TINY_GEOMETRY.vocab, (38,))]), blocks)
    assert torch.equal(view[blocks[:2]], before)


def test_cache_shape_selection_and_prefix_alignment(monkeypatch):
    import pytest

    from pd_helpers import make_cfg
    from llumnix_kv_b200.hybrid_connector import engine_proxy as ep

    cfg = make_cfg("kv_producer", "x")
    monkeypatch.delenv("VLLM_ATTENTION_BACKEND", raising=False)
    assert ep.kvt_cache_shape(cfg) == 2
    monkeypatch.setenv("VLLM_ATTENTION_BACKEND", "FLASHINFER")
    assert ep.kvt_cache_shape(cfg, sm_major=10) == 5
    with pytest.raises(ValueError):
        ep.kvt_cache_shape(cfg, sm_major=12)
    with pytest.raises(ValueError):
        ep.kvt_cache_shape(cfg, sm_major=9)
    cfg.model_config.is_hybrid = True
    assert ep.kvt_cache_shape(cfg, sm_major=10) == 7 and ep.kvt_cache_shape(cfg, sm_major=12) == 3
    monkeypatch.setenv("VLLM_ATTENTION_BACKEND", "FLASHMLA_SPARSE")
    assert ep.use_sparse_mla() and ep.kvt_cache_shape(cfg) == 4
    monkeypatch.setenv("VLLM_ATTENTION_BACKEND", "FLASH_ATTN")
    cfg.cache_config.cache_dtype = "tq4"
    assert ep.kvt_cache_shape(cfg) == 6
    # attention blocks of 16 striped over 2 DCP ranks, indexer blocks of 64 replicated: lcm(32, 64) = 64
    assert ep.align_seen_tokens_for_kvt([200, 130], [16, 64], dcp_world_size=2, replicated=[False, True]) == 128
    assert ep.align_seen_tokens_for_kvt([50], [16]) == 48 and ep.align_seen_tokens_for_kvt([], []) == 0


def test_copy_policy_static_rule_and_buckets(ops):
    """Without a measurement the copy engines take a descriptor list only when it is short and every
    run is long (the reference's rule, kvtransfer/src/copy_kernels.cpp:495-510); bucket edges."""
    K, M = 0, 1
    assert ops.copy_policy_choose("static", 0, 16, 16 * (256 << 10), 256 << 10) == M
    assert ops.copy_policy_choose("static", 0, 17, 17 * (256 << 10), 256 << 10) == K
    assert ops.copy_policy_choose("static", 1, 4, 4 << 20, (256 << 10) - 1) == K
    assert ops.copy_policy_choose("kernel", 1, 1, 8 << 20, 8 << 20) == K
    assert ops.copy_policy_choose("memcpy", 0, 5000, 5000 * 64, 64) == M
    assert ops.copy_policy_choose("memcpy", 0, 0, 0, 0) == K          # nothing to move
    assert ops.copy_policy_bucket(4, 16 << 10) == (0, 0)
    assert ops.copy_policy_bucket(5, (16 << 10) + 1) == (1, 1)
    assert ops.copy_policy_bucket(512, 2 << 20) == (2, 2)
    assert ops.copy_policy_bucket(513, (2 << 20) + 1) == (3, 3)


def test_log_line_format_and_level_filter():
    """The native logger writes glog-style lines to stderr ("date time.us:pid:tid L file:line] text") and
    drops INFO lines unless LLMOPS_CPP_MIN_LOG_LEVEL=0 (kvtransfer/third_party/logging.cpp:106-147)."""
    import os
    import re
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    probe = ("import llumnix_kv_b200 as p\nK = p.load_ops()\n"
             "try:\n    K.plan_ipc_blocks(K.WorkerInfo(), K.WorkerInfo(), 2, [('x', 0, 4, True, [[1]], [[1]])])\n"
             "except Exception:\n    pass\nprint(K.new_id(), K.new_id())\n")
    for level, want_info in (("0", True), ("1", False)):
        env = dict(os.environ, LLMOPS_CPP_MIN_LOG_LEVEL=level, BLLM_KVTRANS_QUIET_ENV="1")
        r = subprocess.run([sys.executable, "-c", probe], cwd=root, env=env, capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, r.stderr[-500:]
        a, b = (int(x) for x in r.stdout.split())
        assert a >= 20181218 and b == a + 1                     # ids count up from the reference's seed
        lines = [ln for ln in r.stderr.splitlines() if "]" in ln and re.match(r"\d{4}-\d\d-\d\d ", ln)]
        assert lines, r.stderr[-500:]                            # the failed plan logs an ERROR line at either level
        for ln in lines:
            assert re.match(r"\d{4}-\d\d-\d\d \d\d:\d\d:\d\d\.\d{6}:\d+:\d+ [IWEF] [\w.]+:\d+\] ", ln), ln
        assert any(" E " in ln for ln in lines)
        if not want_info:
            assert not any(re.search(r":\d+ I ", ln) for ln in lines)


def test_bulk_copy_round_count_covers_the_longest_descriptor(ops):
    """rounds x units-per-descriptor x 8 KiB must reach the end of the longest descriptor; the
    kernel splits a descriptor over at most 65536 units, so beyond 512 MiB the rounds grow."""
    seg, max_segs = 8192, 65536

    def segs(n):
        return 1 if n <= seg else min(-(-n // seg), max_segs)

    for first, longest in ((100, 100), (41984, 41984), (100, 3 * seg + 40), (1 << 30, 1 << 30),
                           ((1 << 29) + 16, 3 << 30), (seg, (4 << 30) - 16), (5 << 20, 700 << 20)):
        r = ops.kvt_bulk_rounds(first, longest)
        assert r * segs(first) * seg >= longest, (first, longest, r)
        assert r == 1 or (r - 1) * segs(first) * seg < longest, (first, longest, r)   # and no more than needed
    assert ops.kvt_bulk_rounds(1 << 30, 1 << 30) == 2          # 131072 segments over 65536 units


def test_crash_trace_prints_native_frames_then_chains(ops):
    """A child process with BLLM_KVTRANS_CRASH_TRACE=1 that dereferences a null pointer on the host
    writes its native frames to stderr before it dies of the signal."""
    import subprocess
    import sys

    code = ("import ctypes, llumnix_kv_b200\n"
            "llumnix_kv_b200.load_ops()\n"
            "ctypes.string_at(0)\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=120,
                       env=dict(os.environ, BLLM_KVTRANS_CRASH_TRACE="1"))
    assert r.returncode == -11, (r.returncode, r.stderr[-500:])
    assert "kvtransfer crash trace: signal 11" in r.stderr and "end of trace" in r.stderr
    assert "(+0x" in r.stderr or "[0x" in r.stderr
