"""Planner (CPU IpcBlock generation) tests.

* truth table of ``compute_valid_ranks_pd`` and interval merging (values from the reference's
  tests: kvtransfer/tests/send_stub_test.cpp:1212-1277, 1552-1559, 2739-2802);
* golden literals for the simple shapes, derived by hand from the layout definitions;
* a differential test against the reference's own ParseBlock functions, compiled at test time
  from a reference checkout when one is available (skipped otherwise), over randomised
  configurations of every cache shape and TP relation.
"""
import os
import random
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference's sources: LLUMNIX_KV_REFERENCE, else a "reference" folder next to this repository's checkout
REF = os.environ.get("LLUMNIX_KV_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


@pytest.fixture(scope="module")
def K(ops):
    os.environ["BLLM_KVTRANS_QUIET_ENV"] = "1"
    return ops


def mk_worker(K, inst, wid, tp, rank, block_sizes, token_sizes, nblocks, **kw):
    w = K.WorkerInfo()
    w.inst_id, w.worker_id, w.engine_tp_size, w.worker_tp_rank = inst, wid, tp, rank
    w.block_sizes, w.token_sizes, w.layer_num_blocks = list(block_sizes), list(token_sizes), nblocks
    ntpb = block_sizes[0] // token_sizes[0]
    w.attn_pack_size = kw.pop("attn_pack_size", 1)
    w.attn_kernel_blk_ntpb = kw.pop("attn_kernel_blk_ntpb", ntpb // w.attn_pack_size)
    for k, v in kw.items():
        setattr(w, k, v)
    return w


# ---------------------------------------------------------------------------------------------
def test_valid_ranks_truth_table(K):
    f = K.compute_valid_ranks_pd

    def bits(s):
        return [i for i, c in enumerate(reversed(s)) if c == "1"]

    assert bits(f(4, 2, 8)) == [0, 1, 2, 3]          # a head or more per prefill rank: all valid
    assert bits(f(8, 2, 2)) == [0, 4]                # replicated heads, d_tp <= heads: one rank per head
    assert bits(f(8, 4, 2)) == [0, 2, 4, 6]          # d_tp > heads: first rank of each decode subgroup
    assert bits(f(8, 8, 2)) == list(range(0, 8, 1)) or bits(f(8, 8, 2)) == [0, 1, 2, 3, 4, 5, 6, 7]
    assert bits(f(2, 8, 4)) == [0, 1]                # fan-out: every prefill rank sends
    assert bits(f(4, 1, -1)) == [0, 1, 2, 3]         # unknown head count
    assert bits(f(16, 4, 4)) == [0, 4, 8, 12]
    assert bits(f(4, 4, 1)) == [0, 1, 2, 3]


def test_merge_interval(K):
    merged, mn, mx, total, cnt = K.merge_interval([(100, 1100, 50), (0, 1000, 100), (150, 1150, 10), (400, 9000, 8)])
    assert merged == [(0, 1000, 160), (400, 9000, 8)]
    assert (mn, mx, total, cnt) == (8, 160, 168, 2)
    # adjacent in the source but not in the destination: not merged
    merged, *_ = K.merge_interval([(0, 0, 16), (16, 64, 16)])
    assert merged == [(0, 0, 16), (16, 64, 16)]
    assert K.merge_interval([])[0] == []


def test_flash_nhd_eq_golden(K):
    # [2, blocks, 16 slots, heads*dim]: token K bytes = 256, block K bytes = 4096, 10 blocks
    src = mk_worker(K, "p", 0, 1, 0, [8192], [512], 10, num_kv_heads=2)
    dst = mk_worker(K, "d", 0, 1, 0, [8192], [512], 20, num_kv_heads=2)
    tasks = [("r", 5, 30, True, [[3, 7, 2]], [[9, 1, 4]])]
    per_tensor, kind, *_ = K.plan_ipc_blocks(src, dst, 2, tasks)
    assert kind == "PEQD"
    k = [(3 * 4096 + 5 * 256, 9 * 4096 + 5 * 256, 11 * 256), (7 * 4096, 1 * 4096, 4096), (2 * 4096, 4 * 4096, 3 * 256)]
    v = [(s + 4096 * 10, d + 4096 * 20, n) for s, d, n in k]
    assert per_tensor == [k + v]


def test_hnd_p_gt_d_golden(K):
    # prefill TP4 (1 head/rank), decode TP2 (2 heads/rank); rank 3 -> decode rank 1, slot 1
    hd = 64
    src = mk_worker(K, "p", 3, 4, 3, [2 * 1 * 16 * hd], [2 * 1 * hd], 8, num_kv_heads=4)
    dst = mk_worker(K, "d", 1, 2, 1, [2 * 2 * 16 * hd], [2 * 2 * hd], 8, num_kv_heads=4)
    per_tensor, kind, valid, kvt_size, kvt_rank = K.plan_ipc_blocks(src, dst, 5, [("r", 14, 4, False, [[5, 6]], [[2, 3]])])
    assert (kind, kvt_size, kvt_rank) == ("PGTD", 4, 3)
    pb, db = 2 * 16 * hd, 4 * 16 * hd
    exp = []
    for blk_i, (t0, n) in enumerate([(14, 2), (0, 2)]):
        sk = [5, 6][blk_i] * pb + t0 * hd
        dk = [2, 3][blk_i] * db + 1 * (16 * hd) + t0 * hd
        exp += [(sk, dk, n * hd), (sk + pb // 2, dk + db // 2, n * hd)]
    assert per_tensor == [exp]


def test_bounds_violation_is_rejected(K):
    src = mk_worker(K, "p", 0, 1, 0, [8192], [512], 4, num_kv_heads=2)
    dst = mk_worker(K, "d", 0, 1, 0, [8192], [512], 4, num_kv_heads=2)
    with pytest.raises(Exception):
        K.plan_ipc_blocks(src, dst, 2, [("r", 0, 16, True, [[9]], [[0]])])
    with pytest.raises(Exception):
        K.plan_ipc_blocks(src, dst, 2, [("r", 0, 40, True, [[1]], [[2]])])  # block table too short


# ---------------------------------------------------------------------------------------------
# differential oracle
# ---------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def oracle(tmp_path_factory):
    """Path of the reference's ParseBlock functions built as a command-line oracle, or None without a
    reference checkout: the randomised configurations below then still check the walk ops against the
    byte ranges (check_walk), only the comparison with the reference's output is left out."""
    root = os.path.join(REF, "kvtransfer")
    if not os.path.isdir(root) or shutil.which("g++") is None:
        return None
    out = tmp_path_factory.mktemp("oracle")
    srcs = ["parse_block_common", "parse_block_flash", "parse_block_flashinfer", "parse_block_ragged",
            "parse_block_dpsk", "parse_block_qwen3_next", "parse_block_qwen3_next_flashinfer", "parse_block_kda",
            "parse_block_kimi_k3", "parse_block_turboquant", "common", "envcfg", "third_party/logging"]
    cmd = ["g++", "-std=c++17", "-O1", "-DNDEBUG", f"-I{root}/include", f"-I{root}/src", "-o", str(out / "ref_oracle"),
           os.path.join(HERE, "oracle", "ref_oracle_main.cpp")] + [f"{root}/src/{s}.cpp" for s in srcs] + ["-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        return None
    return str(out / "ref_oracle")


def _vec(v):
    return f"{len(v)} " + " ".join(str(x) for x in v)


def _ser_worker(w):
    return " ".join(str(x) for x in [
        w.inst_id, w.worker_id, w.engine_tp_size, w.worker_tp_rank, _vec(w.block_sizes), _vec(w.token_sizes),
        w.layer_num_blocks, w.attn_kernel_blk_ntpb, w.indexer_blk_ntpb, w.attn_pack_size, w.kda_page_stride,
        w.num_kv_heads, w.num_gdn_layers, w.hybrid_indexer_token_size, w.gdn_conv_elem_size, w.gdn_ssm_elem_size,
        _vec(w.conv_state_shape), _vec(w.ssm_state_shape), _vec(w.gdn_conv_channel_dims), w.num_ple_layers,
        w.ple_block_group, w.ple_conv_elem_size, _vec(w.ple_conv_state_shape), int(w.kda_conv_dim_first),
        w.hybrid_attn_token_size])


def _ser_blocks(groups):
    return f"{len(groups)} " + " ".join(_vec(g) for g in groups)


def run_oracle(oracle, fn, valid, kvt_size, kvt_rank, src, dst, tasks, env=None):
    text = f"{fn} {valid} {kvt_size} {kvt_rank}\n{_ser_worker(src)}\n{_ser_worker(dst)}\n{len(tasks)}\n"
    for rid, seen, new, last, sb, db in tasks:
        text += f"{rid} {seen} {new} {int(last)} {_ser_blocks(sb)} {_ser_blocks(db)}\n"
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run([oracle], input=text, capture_output=True, text=True, env=e, timeout=60)
    assert r.returncode == 0, r.stderr
    out, cur = [], None
    for line in r.stdout.splitlines():
        if line.startswith("kvtenv"):
            continue
        if line.startswith("EXC"):
            return "EXC"
        if line.startswith("T "):
            cur = []
            out.append(cur)
            continue
        s, d, n = line.split()
        cur.append((int(s), int(d), int(n)))
    return out


def check_walk(K, shape, src, dst, tasks, pad=True):
    """The walk ops of a request (what the device kernel expands, csrc/kernels/kvt_walk.h) move exactly the
    bytes the planner's byte ranges move.  Both are applied to random caches, request by request; the first
    block of every block group holds zeros, as the engine keeps it, because the byte ranges pad a tail by
    copying from there while the ops write zeros."""
    import numpy as np

    src_caps = [bs * src.layer_num_blocks for bs in src.block_sizes]
    dst_caps = [bs * dst.layer_num_blocks for bs in dst.block_sizes]
    rng = np.random.default_rng(len(tasks) * 7919 + shape)
    for task in tasks:
        sb = task[4]
        s_mem = [rng.integers(1, 256, cap, dtype=np.uint8) for cap in src_caps]
        for t, bs in enumerate(src.block_sizes):
            for g in sb:
                if g:
                    s_mem[t][g[0] * bs:(g[0] + 1) * bs] = 0
        d0 = [rng.integers(1, 256, cap, dtype=np.uint8) for cap in dst_caps]
        want = [d.copy() for d in d0]
        blocks = K.plan_ipc_blocks(src, dst, shape, [task], False, pad, False)[0]
        for t, lst in enumerate(blocks):
            for so, do, n in lst:
                want[t][do:do + n] = s_mem[t][so:so + n]
        got = [d.copy() for d in d0]
        plan = K.plan_walk(src, dst, shape, [task], pad)
        moved = 0
        for t, zero, so, do, n in plan.expand(src_caps, dst_caps):
            got[t][do:do + n] = 0 if zero else s_mem[t][so:so + n]
            moved += n
        assert moved == plan.bytes
        for t in range(len(want)):
            if not np.array_equal(got[t], want[t]):
                bad = int(np.flatnonzero(got[t] != want[t])[0])
                raise AssertionError(f"shape {shape}: walk ops differ from the byte ranges in tensor {t} at byte {bad} "
                                     f"(task {task[0]} seen={task[1]} new={task[2]} last={task[3]})")
        # a long request costs a handful of ops, not one descriptor per piece
        assert plan.n_ops <= 64


def check(K, oracle, shape, fn, src, dst, tasks, pad=True):
    check_walk(K, shape, src, dst, tasks, pad)
    if oracle is None:
        return
    mine, kind, valid, kvt_size, kvt_rank = K.plan_ipc_blocks(src, dst, shape, tasks, False, pad, False)
    ref = run_oracle(oracle, fn, valid, kvt_size, kvt_rank, src, dst, tasks,
                     {"BLLM_KVTRANS_PAD_LAST_ATTN_BLOCK": "1" if pad else "0"})
    assert ref != "EXC"
    ref = [t for t in ref]
    mine = [t for t in mine]
    # the reference leaves send_blocks empty when a rank has nothing to send
    while len(ref) < len(mine):
        ref.append([])
    while len(mine) < len(ref):
        mine.append([])
    assert mine == ref, f"{fn}: first diff at " + str(next(
        (i, a, b) for t in range(len(ref)) for i, (a, b) in enumerate(zip(mine[t] + [None], ref[t] + [None])) if a != b))


def rand_task(rng, rid, nblocks_s, nblocks_d, ntpb_s, ntpb_d, groups_extra=0, chunked=True, max_tokens=120):
    total = rng.randint(1, max_tokens)
    nb_s = (total + ntpb_s - 1) // ntpb_s + rng.randint(0, 1)
    nb_d = (total + ntpb_d - 1) // ntpb_d + rng.randint(0, 1)
    sb = rng.sample(range(1, nblocks_s), nb_s)
    db = rng.sample(range(1, nblocks_d), nb_d)
    if chunked:
        seen = rng.randint(0, total - 1)
        new = rng.randint(1, total - seen)
    else:
        seen, new = 0, total
    last = seen + new == total
    return (rid, seen, new, last, [sb], [db])


@pytest.mark.parametrize("seed", range(6))
def test_diff_plain_shapes(K, oracle, seed):
    rng = random.Random(seed)
    hd = rng.choice([32, 64, 256])
    ntpb = rng.choice([8, 16, 32])
    heads_total = 8
    # ---- equal TP -------------------------------------------------------------------------
    H = rng.choice([1, 2, 4])
    tok, bs = 2 * H * hd, 2 * H * hd * ntpb
    for shape, fn in ((1, "ragged_eq"), (2, "flash_eq"), (5, "hnd_eq")):
        src = mk_worker(K, "p", 0, 2, 1, [bs], [tok], 40, num_kv_heads=2 * H)
        dst = mk_worker(K, "d", 0, 2, 1, [bs], [tok], 50, num_kv_heads=2 * H)
        tasks = [rand_task(rng, f"r{i}", 40, 50, ntpb, ntpb) for i in range(3)]
        check(K, oracle, shape, fn, src, dst, tasks)
    # ---- P > D ----------------------------------------------------------------------------
    for p_tp, d_tp in ((4, 2), (8, 2), (4, 1)):
        hp, hdd = heads_total // p_tp, heads_total // d_tp
        p_tok, d_tok = 2 * hp * hd, 2 * hdd * hd
        for shape, fn in ((1, "ragged_gt"), (2, "flash_gt"), (5, "hnd_gt")):
            rank = rng.randrange(p_tp)
            g_n = p_tp // d_tp
            src = mk_worker(K, "p", rank, p_tp, rank, [p_tok * ntpb], [p_tok], 40, num_kv_heads=heads_total)
            dst = mk_worker(K, "d", rank // g_n, d_tp, rank // g_n, [d_tok * ntpb], [d_tok], 50, num_kv_heads=heads_total)
            tasks = [rand_task(rng, f"r{i}", 40, 50, ntpb, ntpb) for i in range(3)]
            check(K, oracle, shape, fn, src, dst, tasks)
    # ---- P < D (ragged only in the reference) ------------------------------------------------
    p_tp, d_tp = 2, 4
    hp, hdd = heads_total // p_tp, heads_total // d_tp
    d_rank = rng.randrange(d_tp)
    src = mk_worker(K, "p", 0, p_tp, d_rank // 2, [2 * hp * hd * ntpb], [2 * hp * hd], 40, num_kv_heads=heads_total)
    dst = mk_worker(K, "d", d_rank, d_tp, d_rank, [2 * hdd * hd * ntpb], [2 * hdd * hd], 50, num_kv_heads=heads_total)
    check(K, oracle, 1, "ragged_lt", src, dst, [rand_task(rng, "r", 40, 50, ntpb, ntpb)])
    # ---- replicated (MLA-like) ragged cache, P > D -------------------------------------------------
    for rank in (0, 1):
        src = mk_worker(K, "p", rank, 2, rank, [576 * ntpb], [576], 40, num_kv_heads=-1)
        dst = mk_worker(K, "d", 0, 1, 0, [576 * ntpb], [576], 50, num_kv_heads=-1)
        check(K, oracle, 1, "ragged_gt_dpsk", src, dst, [rand_task(rng, "r", 40, 50, ntpb, ntpb)])


@pytest.mark.parametrize("seed", range(4))
def test_diff_multi_tensor(K, oracle, seed):
    rng = random.Random(100 + seed)
    ntpb = 64
    toks = [132, 656]
    src = mk_worker(K, "p", 0, 2, 1, [t * ntpb for t in toks], toks, 30, num_kv_heads=1)
    dst = mk_worker(K, "d", 0, 2, 1, [t * ntpb for t in toks], toks, 36, num_kv_heads=1)
    tasks = [rand_task(rng, f"r{i}", 30, 36, ntpb, ntpb, max_tokens=300) for i in range(3)]
    check(K, oracle, 4, "multi_eq", src, dst, tasks)
    # replicated latent, P TP 4 -> D TP 1: rank 0 only
    for rank in (0, 2):
        src = mk_worker(K, "p", rank, 4, rank, [t * ntpb for t in toks], toks, 30, num_kv_heads=-1)
        dst = mk_worker(K, "d", 0, 1, 0, [t * ntpb for t in toks], toks, 36, num_kv_heads=-1)
        check(K, oracle, 4, "multi_gt", src, dst, tasks)
    # sliced multi-tensor caches
    p_toks, d_toks = [64, 256], [128, 512]
    src = mk_worker(K, "p", 1, 2, 1, [t * ntpb for t in p_toks], p_toks, 30, num_kv_heads=8)
    dst = mk_worker(K, "d", 0, 1, 0, [t * ntpb for t in d_toks], d_toks, 36, num_kv_heads=8)
    check(K, oracle, 4, "multi_gt", src, dst, tasks)
    src = mk_worker(K, "p", 0, 1, 0, [t * ntpb for t in d_toks], d_toks, 30, num_kv_heads=8)
    dst = mk_worker(K, "d", 1, 2, 1, [t * ntpb for t in p_toks], p_toks, 36, num_kv_heads=8)
    check(K, oracle, 4, "multi_lt", src, dst, tasks)


def hybrid_workers(K, rng, hnd, p_tp, d_tp, p_rank, d_rank, indexer, ple, pack, heads_total=8):
    """Qwen3-Next-like page: GDN groups | indexer? | attention | PLE?; one tensor per layer."""
    hd = 64
    n_gdn = rng.choice([1, 3])
    hp = max(1, heads_total // p_tp)
    hdd = max(1, heads_total // d_tp)
    p_tok, d_tok = 2 * hp * hd, 2 * hdd * hd
    kb = 16
    ntpb = kb * rng.choice([1, 2]) * pack
    p_bs, d_bs = p_tok * ntpb, d_tok * ntpb
    # GDN state sized to fit the smaller page; channel dims sharded by engine TP
    base_dims = [64, 64, 128]
    rows = 3

    def dims(tp):
        return [d * 4 // tp for d in base_dims]

    def state(tp):
        cd = dims(tp)
        return dict(conv_state_shape=[1, rows, sum(cd)], ssm_state_shape=[1, 16 // tp if tp <= 16 else 1, 8, 8],
                    gdn_conv_channel_dims=cd, gdn_conv_elem_size=2, gdn_ssm_elem_size=4)

    extra = dict(num_gdn_layers=n_gdn, num_kv_heads=heads_total, attn_pack_size=pack, attn_kernel_blk_ntpb=kb)
    if indexer:
        extra.update(indexer_blk_ntpb=ntpb // pack, hybrid_indexer_token_size=32)
    n_groups = n_gdn + (1 if indexer else 0) + 1
    if ple:
        extra.update(num_ple_layers=1, ple_block_group=n_groups, ple_conv_elem_size=2)
        n_groups += 1
    pe, de = dict(extra), dict(extra)
    pe.update(state(p_tp))
    de.update(state(d_tp))
    if ple:
        pe.update(ple_conv_state_shape=[1, 2, 48])
        de.update(ple_conv_state_shape=[1, 2, 48])
    src = mk_worker(K, "p", p_rank, p_tp, p_rank, [p_bs], [p_tok], 64, **pe)
    dst = mk_worker(K, "d", d_rank, d_tp, d_rank, [d_bs], [d_tok], 64, **de)
    return src, dst, n_gdn, indexer, ple, ntpb // pack if not hnd else ntpb


def hybrid_task(rng, rid, n_gdn, indexer, ple, layer_ntpb_s, layer_ntpb_d, last=None):
    total = rng.randint(1, 150)
    seen = rng.randint(0, total - 1)
    new = rng.randint(1, total - seen)
    is_last = (seen + new == total) if last is None else last
    if last:
        new = total - seen
    nb_s = (total + layer_ntpb_s - 1) // layer_ntpb_s + rng.randint(0, 1)
    nb_d = (total + layer_ntpb_d - 1) // layer_ntpb_d
    if layer_ntpb_s == layer_ntpb_d:
        nb_d = nb_s
    pool_s = list(range(1, 64))
    pool_d = list(range(1, 64))
    rng.shuffle(pool_s)
    rng.shuffle(pool_d)
    sb, db = [], []
    for _ in range(n_gdn):
        sb.append([pool_s.pop()])
        db.append([pool_d.pop()])
    if indexer:
        sb.append([pool_s.pop() for _ in range(nb_s)])
        db.append([pool_d.pop() for _ in range(nb_d)])
    sb.append([pool_s.pop() for _ in range(nb_s)])
    db.append([pool_d.pop() for _ in range(nb_d)])
    if ple:
        sb.append([pool_s.pop()])
        db.append([pool_d.pop()])
    return (rid, seen, new, is_last, sb, db)


@pytest.mark.parametrize("hnd", [False, True])
@pytest.mark.parametrize("seed", range(5))
def test_diff_hybrid(K, oracle, hnd, seed):
    rng = random.Random(1000 * hnd + seed)
    shape = 7 if hnd else 3
    pre = "hyb_hnd" if hnd else "hyb_nhd"
    for indexer in (False, True):
        for ple in (False, True):
            pack = 1 if hnd else rng.choice([1, 2])
            # P == D
            src, dst, n_gdn, ix, pl, lntpb = hybrid_workers(K, rng, hnd, 2, 2, 1, 1, indexer, ple, pack)
            tasks = [hybrid_task(rng, f"r{i}", n_gdn, ix, pl, lntpb, lntpb) for i in range(3)]
            check(K, oracle, shape, pre + "_eq", src, dst, tasks)
            # P > D, with and without tail padding
            for p_tp, d_tp in ((4, 2), (4, 1)):
                p_rank = rng.randrange(p_tp)
                src, dst, n_gdn, ix, pl, lntpb = hybrid_workers(K, rng, hnd, p_tp, d_tp, p_rank, p_rank // (p_tp // d_tp),
                                                                indexer, ple, pack)
                tasks = [hybrid_task(rng, f"r{i}", n_gdn, ix, pl, lntpb, lntpb) for i in range(3)]
                check(K, oracle, shape, pre + "_gt", src, dst, tasks, pad=True)
            # P < D
            d_rank = rng.randrange(4)
            src, dst, n_gdn, ix, pl, lntpb = hybrid_workers(K, rng, hnd, 2, 4, d_rank // 2, d_rank, indexer, ple, pack)
            tasks = [hybrid_task(rng, f"r{i}", n_gdn, ix, pl, lntpb, lntpb) for i in range(3)]
            check(K, oracle, shape, pre + "_lt", src, dst, tasks, pad=True)


@pytest.mark.parametrize("dim_first", [False, True])
@pytest.mark.parametrize("seed", range(3))
def test_diff_kimi_k3(K, oracle, dim_first, seed):
    rng = random.Random(7000 + seed)
    kb, mla_tok = 16, 576
    n_kda = 2

    def worker(name, tp, rank):
        dims = [d * 4 // tp for d in (32, 32, 64)]
        state_len = 3
        conv = [1, sum(dims), state_len] if dim_first else [1, state_len, sum(dims)]
        ssm = [1, 8 // tp if tp <= 8 else 1, 16, 16]
        page = sum(dims) * state_len * 2 + ssm[1] * 16 * 16 * 4
        page = max(page, 64 * mla_tok)
        page = (page + 255) // 256 * 256
        # the manager sees logical MLA blocks of 64 tokens inside KDA-sized physical pages
        return mk_worker(K, name, rank, tp, rank, [64 * (page // 64)], [page // 64], 48, num_kv_heads=1,
                         num_gdn_layers=n_kda, conv_state_shape=conv, ssm_state_shape=ssm, gdn_conv_channel_dims=dims,
                         gdn_conv_elem_size=2, gdn_ssm_elem_size=4, kda_conv_dim_first=dim_first,
                         hybrid_attn_token_size=mla_tok, kda_page_stride=page, attn_kernel_blk_ntpb=kb)

    def task(rid):
        total = rng.randint(1, 200)
        seen = rng.randint(0, total - 1)
        new = rng.randint(1, total - seen)
        nb = (total + 63) // 64 + rng.randint(0, 1)
        ps, pd = list(range(1, 48)), list(range(1, 48))
        rng.shuffle(ps)
        rng.shuffle(pd)
        sb = [[ps.pop()] for _ in range(n_kda)] + [[ps.pop() for _ in range(nb)]]
        db = [[pd.pop()] for _ in range(n_kda)] + [[pd.pop() for _ in range(nb)]]
        return (rid, seen, new, seen + new == total, sb, db)

    for p_tp, d_tp, fn in ((2, 2, "k3_eq"), (4, 2, "k3_gt"), (2, 4, "k3_lt")):
        if p_tp >= d_tp:
            p_rank = rng.randrange(p_tp)
            d_rank = p_rank // (p_tp // d_tp)
        else:
            d_rank = rng.randrange(d_tp)
            p_rank = d_rank // (d_tp // p_tp)
        src, dst = worker("p", p_tp, p_rank), worker("d", d_tp, d_rank)
        check(K, oracle, 8, fn, src, dst, [task(f"r{i}") for i in range(3)])


def test_merge_interval_moves_the_same_bytes_as_the_unmerged_list(K):
    """Random lists of ranges (runs adjacent on both sides, on one side only, gaps, shuffled order; the reference's
    test also feeds it overlapping prompt-cache ranges, kvtransfer/tests/send_stub_test.cpp:1212-1277, which carry
    the same bytes twice): applying the merged list to a memory image gives what the original list gives, the
    merged list is sorted by source offset with no two neighbours adjacent on both sides, and the statistics
    describe it."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=200, deadline=None)
    @given(st.lists(st.tuples(st.integers(1, 6), st.integers(0, 3), st.integers(0, 3), st.booleans()), min_size=0, max_size=40),
           st.randoms(use_true_random=False))
    def run(spec, rnd):
        blocks, s, d = [], 0, 4096
        for length, sgap, dgap, dup in spec:
            s += sgap * 8
            d += dgap * 8
            blocks.append((s, d, length * 8))
            if dup:
                blocks.append((s, d, length * 8))          # the same range twice
            s += length * 8
            d += length * 8
        rnd.shuffle(blocks)
        src = bytes((i * 7 + 3) & 0xFF for i in range(s + 64))
        want = bytearray(d + 64)
        for so, do, n in blocks:
            want[do:do + n] = src[so:so + n]
        merged, mn, mx, total, cnt = K.merge_interval(blocks)
        got = bytearray(d + 64)
        for so, do, n in merged:
            got[do:do + n] = src[so:so + n]
        assert got == want
        assert [m[0] for m in merged] == sorted(m[0] for m in merged)
        for (s0, d0, n0), (s1, d1, _n1) in zip(merged, merged[1:]):
            assert not (s0 + n0 == s1 and d0 + n0 == d1)
        if merged:
            assert (mn, mx, total, cnt) == (min(m[2] for m in merged), max(m[2] for m in merged), sum(m[2] for m in merged), len(merged))

    run()
