"""The block-table walk kernel (csrc/kernels/kvt_walk.cu) against the CPU planner, byte for byte.

Every cache shape that has no TMA-tiled kernel of its own (hybrid GDN pages in both attention layouts,
multi-tensor MLA, KDA pages) and, for completeness, the plain attention shapes, in every TP relation:
the planner records walk ops, the kernel expands them on the GPU, and the destination must equal what
the planner's byte ranges produce when they are applied on the host.  The configurations are the
randomised ones of tests/test_planner.py.
"""
import os
import random

import numpy as np
import pytest
import torch

import test_planner as tp

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
N_LAYERS = 2


@pytest.fixture(scope="module")
def K(ops):
    os.environ["BLLM_KVTRANS_QUIET_ENV"] = "1"
    return ops


def launch_plan(K, plan, blob, sp, dp, nt, src_caps, dst_caps, status, grid=0, layers=(0, N_LAYERS)):
    """The copies, then (same stream) the zero fills: the order the NVLINK channel launches them in."""
    stream = torch.cuda.current_stream().cuda_stream
    pool = blob.data_ptr() + plan.pool_offset
    if plan.n_bulk + plan.n_simt:
        K.kvt_launch_walk(sp.data_ptr(), dp.data_ptr(), nt, layers[0], layers[1], src_caps, dst_caps, blob.data_ptr(), plan.n_bulk,
                          plan.n_simt, plan.bulk_units, plan.simt_units, pool, plan.pool_len, status.data_ptr(), grid, stream)
    if plan.n_zero:
        zero_ops = blob.data_ptr() + (plan.n_bulk + plan.n_simt) * K.KVT_WALK_OP_BYTES
        K.kvt_launch_walk(sp.data_ptr(), dp.data_ptr(), nt, layers[0], layers[1], src_caps, dst_caps, zero_ops, 0, plan.n_zero, 0,
                          plan.zero_units, pool, plan.pool_len, status.data_ptr(), grid, stream)


def run_walk(K, shape, src, dst, tasks, pad=True, grid=0):
    src_caps = [bs * src.layer_num_blocks for bs in src.block_sizes]
    dst_caps = [bs * dst.layer_num_blocks for bs in dst.block_sizes]
    nt = len(src_caps)
    rng = np.random.default_rng(shape * 131 + len(tasks))
    for task in tasks:
        s_host = [[rng.integers(1, 256, cap, dtype=np.uint8) for cap in src_caps] for _ in range(N_LAYERS)]
        for layer in range(N_LAYERS):
            for t, bs in enumerate(src.block_sizes):
                for g in task[4]:
                    if g:
                        s_host[layer][t][g[0] * bs:(g[0] + 1) * bs] = 0
        d_host = [[rng.integers(1, 256, cap, dtype=np.uint8) for cap in dst_caps] for _ in range(N_LAYERS)]
        blocks = K.plan_ipc_blocks(src, dst, shape, [task], False, pad, False)[0]
        want = [[d.copy() for d in layer] for layer in d_host]
        for layer in range(N_LAYERS):
            for t, lst in enumerate(blocks):
                for so, do, n in lst:
                    want[layer][t][do:do + n] = s_host[layer][t][so:so + n]
        plan = K.plan_walk(src, dst, shape, [task], pad)
        s_dev = [[torch.from_numpy(a).to(DEV) for a in layer] for layer in s_host]
        d_dev = [[torch.from_numpy(a).to(DEV) for a in layer] for layer in d_host]
        if plan.n_ops:
            blob = torch.frombuffer(bytearray(plan.blob()), dtype=torch.uint8).to(DEV)
            sp = torch.tensor([t.data_ptr() for layer in s_dev for t in layer], dtype=torch.int64, device=DEV)
            dp = torch.tensor([t.data_ptr() for layer in d_dev for t in layer], dtype=torch.int64, device=DEV)
            status = torch.zeros(4, dtype=torch.int32, device=DEV)
            launch_plan(K, plan, blob, sp, dp, nt, src_caps, dst_caps, status, grid)
            torch.cuda.synchronize()
            assert status[:2].tolist() == [0, 0]
        for layer in range(N_LAYERS):
            for t in range(nt):
                got = d_dev[layer][t].cpu().numpy()
                if not np.array_equal(got, want[layer][t]):
                    bad = int(np.flatnonzero(got != want[layer][t])[0])
                    raise AssertionError(f"shape {shape} layer {layer} tensor {t}: first difference at byte {bad} "
                                         f"(task seen={task[1]} new={task[2]} last={task[3]}, {plan.n_ops} ops, "
                                         f"{plan.n_bulk} bulk)")


@pytest.fixture()
def via_kernel(K, monkeypatch):
    """Routes the configuration generators of test_planner.py through the kernel."""
    monkeypatch.setattr(tp, "check", lambda K_, oracle, shape, fn, src, dst, tasks, pad=True: run_walk(K_, shape, src, dst, tasks, pad))
    return K


@pytest.mark.parametrize("seed", range(2))
def test_walk_plain_attention_shapes(via_kernel, seed):
    tp.test_diff_plain_shapes(via_kernel, None, seed)


@pytest.mark.parametrize("seed", range(2))
def test_walk_multi_tensor_mla(via_kernel, seed):
    tp.test_diff_multi_tensor(via_kernel, None, seed)


@pytest.mark.parametrize("hnd", [False, True])
@pytest.mark.parametrize("seed", range(2))
def test_walk_hybrid_gdn_pages(via_kernel, hnd, seed):
    tp.test_diff_hybrid(via_kernel, None, hnd, seed)


@pytest.mark.parametrize("dim_first", [False, True])
def test_walk_kda_pages(via_kernel, dim_first):
    tp.test_diff_kimi_k3(via_kernel, None, dim_first, 0)


def test_walk_long_request_few_ops_and_small_grid(K):
    """A 32k-token MLA request is a handful of ops (not 2 x 512 descriptors), and any grid moves it whole."""
    ntpb, toks = 64, [132, 656]
    src = tp.mk_worker(K, "p", 0, 1, 0, [t * ntpb for t in toks], toks, 600, num_kv_heads=1)
    dst = tp.mk_worker(K, "d", 0, 1, 0, [t * ntpb for t in toks], toks, 600, num_kv_heads=1)
    rng = random.Random(3)
    n = 32768
    sb, db = rng.sample(range(1, 600), n // ntpb), rng.sample(range(1, 600), n // ntpb)
    task = ("long", 0, n, True, [sb], [db])
    plan = K.plan_walk(src, dst, 4, [task], True)
    assert plan.n_ops == 2 and plan.bytes == n * sum(toks)
    for grid in (0, 3):
        run_walk(K, 4, src, dst, [task], grid=grid)


def test_walk_reports_a_table_that_is_too_short(K):
    """A request whose block table does not cover its tokens sets the status word; nothing faults."""
    ntpb, tok = 16, 512
    src = tp.mk_worker(K, "p", 0, 1, 0, [tok * ntpb], [tok], 16, num_kv_heads=1)
    dst = tp.mk_worker(K, "d", 0, 1, 0, [tok * ntpb], [tok], 16, num_kv_heads=1)
    plan = K.plan_walk(src, dst, 1, [("short", 0, 40, True, [[1, 2]], [[3, 4]])], True)     # 40 tokens need 3 blocks
    s = torch.zeros(16 * tok * ntpb, dtype=torch.uint8, device=DEV)
    d = torch.zeros_like(s)
    blob = torch.frombuffer(bytearray(plan.blob()), dtype=torch.uint8).to(DEV)
    sp = torch.tensor([s.data_ptr()], dtype=torch.int64, device=DEV)
    dp = torch.tensor([d.data_ptr()], dtype=torch.int64, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    launch_plan(K, plan, blob, sp, dp, 1, [s.numel()], [d.numel()], status, layers=(0, 1))
    torch.cuda.synchronize()
    assert int(status[0]) == 1      # KVT_ERR_BLOCK_RANGE
