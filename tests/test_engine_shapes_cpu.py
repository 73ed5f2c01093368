"""Every cache shape through the whole engine on CPU memory (client -> step -> send stub -> planner ->
TCP / SHM channel -> server -> destination tensors), checked against the planner's IpcBlocks applied
by hand.  The planner itself is checked against the reference's ParseBlock in test_planner.py; this
file checks the plumbing around it: multi-tensor layers, block groups, TP relations, the bf16 -> fp8
cast of the host-staged path."""
import os
import random

import pytest
import torch

os.environ.setdefault("BLLM_KVTRANS_QUIET_ENV", "1")

from llumnix_kv_b200.kv_transfer_impl import KVTransferClient, KVTransferProtocolType as PT, KVTransferServer

L = 2


@pytest.fixture(autouse=True)
def _end_to_end_check_on(ops):
    """Every transfer of this file also runs the end-to-end check (byte-range form): multi-tensor layers, block
    groups, zero fills and every TP relation must give the same sum on both sides."""
    os.environ["BLLM_KVTRANS_CRC"] = "1"
    ops.envcfg_reset_for_test()
    yield
    os.environ.pop("BLLM_KVTRANS_CRC", None)
    ops.envcfg_reset_for_test()


def _tensors(sizes, nblocks, fill):
    g = torch.Generator().manual_seed(11)
    out = []
    for _ in range(L):
        layer = []
        for bs in sizes:
            t = torch.randint(1, 255, (bs * nblocks,), dtype=torch.uint8, generator=g) if fill else \
                torch.zeros(bs * nblocks, dtype=torch.uint8)
            if fill:
                t[:bs] = 0      # block 0 is the engine's all-zero block
            layer.append(t)
        out.append(layer)
    return out


def _run(ops, shape, p, d, tasks, kw_p=None, kw_d=None, proto=PT.TCP):
    """p / d: (tp, rank, block_sizes, token_sizes, nblocks).  tasks: [(rid, total, src_groups, dst_groups)]."""
    kw_p, kw_d = dict(kw_p or {}), dict(kw_d or {})
    src = _tensors(p[2], p[4], True)
    dst = _tensors(d[2], d[4], False)
    d_inst, p_inst = f"D|0|{d[0]}", f"P|0|{p[0]}"
    srv = KVTransferServer(d_inst, d[0], d[1], d[1], list(d[2]), list(d[3]), "fake://", dst, [proto], cache_shape=shape, **kw_d)
    cli = KVTransferClient(p_inst, p[0], p[1], p[1], list(p[2]), list(p[3]), "fake://", src, [proto], cache_shape=shape, **kw_p)
    try:
        for rid, total, sb, db in tasks:
            cli.submit_req_send2(d_inst, d[1], rid, 0, total, True, sb, db, srv.worker_info(), stepid=1)
        cli.start_send_step(1, 1)
        for layer in range(L):
            cli.record_event(layer)
        cli.flush_send_step()
        cli.drain()
        assert cli.failed_batches() == 0
        W = ops.WorkerInfo
        pw, dw = W.from_string(cli.worker_info()), W.from_string(srv.worker_info())
        for w, kw in ((pw, kw_p), (dw, kw_d)):
            for k, v in kw.items():
                setattr(w, k, v)
        per_tensor = ops.plan_ipc_blocks(pw, dw, shape, [(rid, 0, total, True, sb, db) for rid, total, sb, db in tasks])[0]
        assert len(per_tensor) == len(p[2])
        moved = 0
        for layer in range(L):
            for t, blocks in enumerate(per_tensor):
                expect = torch.zeros_like(dst[layer][t])
                for s_off, d_off, n in blocks:
                    expect[d_off:d_off + n] = src[layer][t][s_off:s_off + n]
                    moved += n
                assert torch.equal(dst[layer][t], expect), (layer, t)
        assert moved > 0
        return per_tensor
    finally:
        srv.stop()


def _blocks(rng, n, hi):
    ids = list(range(1, hi))
    rng.shuffle(ids)
    return [ids.pop() for _ in range(n)]


@pytest.mark.parametrize("proto", [PT.TCP, PT.SHM])
def test_shape1_ragged_and_shape5_hnd_p_gt_d(ops, proto):
    rng = random.Random(1)
    tok = 2 * 4 * 64 * 2
    _run(ops, 1, (1, 0, [tok * 16], [tok], 24), (1, 0, [tok * 16], [tok], 30),
         [("a", 37, [_blocks(rng, 3, 24)], [_blocks(rng, 3, 30)])], dict(num_kv_heads=4), dict(num_kv_heads=4), proto)
    # HND, prefill TP2 rank 1 (2 heads) -> decode TP1 (4 heads): lands in the second half of each K / V plane
    p_tok, d_tok = 2 * 2 * 64 * 2, 2 * 4 * 64 * 2
    _run(ops, 5, (2, 1, [p_tok * 16], [p_tok], 24), (1, 0, [d_tok * 16], [d_tok], 30),
         [("b", 50, [_blocks(rng, 4, 24)], [_blocks(rng, 4, 30)])], dict(num_kv_heads=4), dict(num_kv_heads=4), proto)


def test_shape4_two_tensors_per_layer(ops):
    """Sparse-MLA style: indexer keys (132 B/token) and latent+rope (656 B/token) as two tensors of a layer."""
    rng = random.Random(2)
    toks, ntpb = [132, 656], 64
    sizes = [t * ntpb for t in toks]
    per_tensor = _run(ops, 4, (2, 1, sizes, toks, 20), (2, 1, sizes, toks, 26),
                      [("m", 150, [_blocks(rng, 3, 20)], [_blocks(rng, 3, 26)])], dict(num_kv_heads=1), dict(num_kv_heads=1))
    assert len(per_tensor) == 2 and per_tensor[0] and per_tensor[1]


@pytest.mark.parametrize("shape", [3, 7])
def test_hybrid_pages_with_gdn_groups_p_gt_d(ops, shape):
    rng = random.Random(3)
    rows, dims_p, hd = 3, [32, 32, 64], 64
    p_tok, d_tok = 2 * 2 * hd * 2, 2 * 4 * hd * 2
    kw_p = dict(num_kv_heads=4, num_gdn_layers=2, conv_state_shape=[1, rows, sum(dims_p)], ssm_state_shape=[1, 4, 8, 8],
                gdn_conv_channel_dims=dims_p, gdn_conv_elem_size=2, gdn_ssm_elem_size=4)
    kw_d = dict(kw_p, conv_state_shape=[1, rows, 2 * sum(dims_p)], gdn_conv_channel_dims=[2 * x for x in dims_p],
                ssm_state_shape=[1, 8, 8, 8])
    sb = [[5], [9], _blocks(rng, 3, 24)]
    db = [[2], [3], _blocks(rng, 3, 30)]
    _run(ops, shape, (2, 1, [p_tok * 16], [p_tok], 24), (1, 0, [d_tok * 16], [d_tok], 30), [("h", 41, sb, db)], kw_p, kw_d)


@pytest.mark.parametrize("dim_first", [False, True])
def test_shape8_kda_pages_with_mla_prefix(ops, dim_first):
    rng = random.Random(4)
    kb, mla_tok, n_kda, tp = 16, 576, 2, 2
    dims = [d * 4 // tp for d in (32, 32, 64)]
    conv = [1, sum(dims), 3] if dim_first else [1, 3, sum(dims)]
    ssm = [1, 8 // tp, 16, 16]
    page = max(sum(dims) * 3 * 2 + ssm[1] * 16 * 16 * 4, 64 * mla_tok)
    page = (page + 255) // 256 * 256
    kw = dict(num_kv_heads=1, num_gdn_layers=n_kda, conv_state_shape=conv, ssm_state_shape=ssm,
              gdn_conv_channel_dims=dims, gdn_conv_elem_size=2, gdn_ssm_elem_size=4, kda_conv_dim_first=dim_first,
              hybrid_attn_token_size=mla_tok, kda_page_stride=page)
    sizes, toks = [64 * (page // 64)], [page // 64]
    ids_s, ids_d = _blocks(rng, 5, 20), _blocks(rng, 5, 20)
    sb = [[ids_s[0]], [ids_s[1]], ids_s[2:]]
    db = [[ids_d[0]], [ids_d[1]], ids_d[2:]]
    _run(ops, 8, (tp, 1, sizes, toks, 20), (tp, 1, sizes, toks, 20), [("k", 130, sb, db)], kw, kw)
