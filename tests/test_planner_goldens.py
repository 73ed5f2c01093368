"""Literal offset goldens of the planner, usable without a reference checkout.

The numbers are the expectations of the reference's own tests, read as data:
  * ragged cache, prefill TP 16 -> decode TP 4, 16 KV heads x 256 dims, 64-token blocks, first 8 tokens of a
    request with source blocks {0, 1, 2} and destination blocks {4, 5, 6}, prefill ranks 0-3 feeding decode
    rank 0 (kvtransfer/tests/send_stub_test.cpp:286-497);
  * KDA state pages, rows-first ("SD") and channels-first ("DS") conv layouts, P == D, P > D, P < D, and the
    Kimi-K3 page with its replicated MLA prefix (kvtransfer/tests/parse_block_kda_test.cpp:78-260).
"""
import pytest
import torch

from test_planner import mk_worker


@pytest.fixture(scope="module")
def K(ops):
    return ops


# ---- ragged P > D --------------------------------------------------------------------------------------
RAGGED_DST0 = {0: 1048576, 1: 1049088, 2: 1049600, 3: 1050112}   # first destination offset written by each prefill rank


@pytest.mark.parametrize("p_rank", [0, 1, 2, 3])
def test_ragged_p16_to_d4_literals(K, p_rank):
    heads, hd, ntpb = 16, 256, 64
    p_tok, d_tok = 2 * (heads // 16) * hd * 2, 2 * (heads // 4) * hd * 2
    assert (p_tok, d_tok) == (1024, 4096)
    src = mk_worker(K, "0", 0, 16, p_rank, [p_tok * ntpb], [p_tok], 8, num_kv_heads=heads)
    dst = mk_worker(K, "1", 0, 4, 0, [d_tok * ntpb], [d_tok], 8, num_kv_heads=heads)
    got = K.plan_ipc_blocks(src, dst, 1, [("req", 0, 8, False, [[0, 1, 2]], [[4, 5, 6]])])[0][0]
    # per token: the K slice then the V slice; source steps of 512, destination: 4096 per token, V 2048 after K
    want = []
    for i in range(8):
        want.append((1024 * i, RAGGED_DST0[p_rank] + 4096 * i, 512))
        want.append((1024 * i + 512, RAGGED_DST0[p_rank] + 4096 * i + 2048, 512))
    # spot literals copied from the reference's table
    table = {0: [(0, 1048576, 512), (512, 1050624, 512), (7680, 1079296, 512)],
             1: [(0, 1049088, 512), (512, 1051136, 512), (7680, 1079808, 512)],
             2: [(0, 1049600, 512), (512, 1051648, 512), (7680, 1080320, 512)],
             3: [(0, 1050112, 512), (512, 1052160, 512), (7680, 1080832, 512)]}[p_rank]
    # the planner emits all K slices of a chunk, then all V slices; the channel sorts by source offset before it
    # sends, which is the order of the reference's table
    by_src = sorted(got)
    assert [by_src[0], by_src[1], by_src[-1]] == table
    assert by_src == want


# ---- KDA pages -----------------------------------------------------------------------------------------
def kda_workers(K, p_tp, p_rank, d_tp, d_rank, p_bs, d_bs, conv=None, rec=None, dims=None, dim_first=False, mla=None):
    kw = dict(num_gdn_layers=1, num_kv_heads=1)
    if conv is not None:
        kw.update(conv_state_shape=conv, ssm_state_shape=rec, gdn_conv_channel_dims=dims, gdn_conv_elem_size=1,
                  gdn_ssm_elem_size=4, kda_conv_dim_first=dim_first)
    src = mk_worker(K, "src", 0, p_tp, p_rank, [p_bs], [1], 8, **kw)
    dst = mk_worker(K, "dst", 0, d_tp, d_rank, [d_bs], [1], 8, num_gdn_layers=1, num_kv_heads=1)
    for w, bs in ((src, p_bs), (dst, d_bs)):
        kernel, manager = mla or (4, 4)
        w.attn_kernel_blk_ntpb = kernel
        w.hybrid_attn_token_size = 2
        w.token_sizes = [bs // manager]
        w.kda_page_stride = bs
    return src, dst


def kda_pieces(K, src, dst, sb, db, last=True, p_page=None):
    """Pieces of the KDA page (source block 1): the MLA group's pieces are looked at separately."""
    got = K.plan_ipc_blocks(src, dst, 8, [("kda", 0, 1, last, sb, db)])[0]
    blocks = got[0] if got else []
    lo, hi = p_page
    return [b for b in blocks if lo <= b[0] < hi], [b for b in blocks if not lo <= b[0] < hi]


def test_kda_p_eq_d_copies_the_full_padded_page(K):
    src, dst = kda_workers(K, 2, 1, 2, 1, 64, 64)
    kda, _ = kda_pieces(K, src, dst, [[1], [3]], [[2], [4]], p_page=(64, 128))
    assert kda == [(64, 128, 64)]
    # mutable state does not leave before the request's last chunk
    kda, _ = kda_pieces(K, src, dst, [[1], [3]], [[2], [4]], last=False, p_page=(64, 128))
    assert kda == []


def test_kda_p_gt_d_merges_rows_first_components(K):
    src, dst = kda_workers(K, 4, 1, 2, 0, 32, 64, conv=[8, 2, 6], rec=[8, 1, 2, 2], dims=[2, 2, 2])
    kda, _ = kda_pieces(K, src, dst, [[1], [3]], [[2], [4]], p_page=(32, 64))
    assert kda == [(32, 130, 2), (34, 134, 2), (36, 138, 2),     # row 0: Q, K, V
                   (38, 142, 2), (40, 146, 2), (42, 150, 2),     # row 1
                   (44, 168, 16)]                                # recurrent state


def test_kda_p_gt_d_merges_channels_first_components(K):
    src, dst = kda_workers(K, 4, 1, 2, 0, 32, 64, conv=[8, 6, 2], rec=[8, 1, 2, 2], dims=[2, 2, 2], dim_first=True)
    kda, _ = kda_pieces(K, src, dst, [[1], [3]], [[2], [4]], p_page=(32, 64))
    assert kda == [(32, 132, 4), (36, 140, 4), (40, 148, 4), (44, 168, 16)]


def test_kda_p_lt_d_splits_rows_first_components(K):
    src, dst = kda_workers(K, 2, 0, 4, 1, 64, 32, conv=[8, 2, 12], rec=[8, 2, 2, 2], dims=[4, 4, 4])
    kda, _ = kda_pieces(K, src, dst, [[1], [3]], [[2], [4]], p_page=(64, 128))
    assert kda == [(66, 64, 2), (70, 66, 2), (74, 68, 2), (78, 70, 2), (82, 72, 2), (86, 74, 2), (104, 76, 16)]


def test_kda_p_lt_d_splits_channels_first_components(K):
    src, dst = kda_workers(K, 2, 0, 4, 1, 64, 32, conv=[8, 12, 2], rec=[8, 2, 2, 2], dims=[4, 4, 4], dim_first=True)
    kda, _ = kda_pieces(K, src, dst, [[1], [3]], [[2], [4]], p_page=(64, 128))
    assert kda == [(68, 64, 4), (76, 68, 4), (84, 72, 4), (104, 76, 16)]


def test_kimi_k3_p_eq_d_copies_mla_prefix_and_kda_page(K):
    src, dst = kda_workers(K, 2, 1, 2, 1, 64, 64)
    got = K.plan_ipc_blocks(src, dst, 8, [("k3", 0, 1, True, [[1], [3]], [[2], [4]])])[0][0]
    assert got == [(3 * 64, 4 * 64, 8),     # replicated MLA: one manager block of 4 tokens x 2 bytes
                   (1 * 64, 2 * 64, 64)]    # full KDA page


def test_bulk_pieces_are_cut_into_even_segments(K):
    """A 41984-byte MLA page travels as six segments of about 7 KiB (multiples of 16 bytes, none above the
    8 KiB stage), not five of 8 KiB and a 1 KiB tail.  The indexer page (64 rows of 132 bytes: rows that are
    not whole 16-byte words) belongs to the SIMT class and stays one piece."""
    from llumnix_kv_b200.kv_transfer_impl import KVTransferClient, KVTransferProtocolType as PT, KVTransferServer

    toks, ntpb, nb = [132, 656], 64, 8
    sizes = [t * ntpb for t in toks]

    def alloc():
        return [[torch.zeros(bs * nb, dtype=torch.uint8) for bs in sizes] for _ in range(2)]

    cli = KVTransferClient("P|0|1", 1, 0, 0, list(sizes), list(toks), "fake://", alloc(), [PT.TCP], cache_shape=4, num_kv_heads=1)
    srv = KVTransferServer("D|0|1", 1, 0, 0, list(sizes), list(toks), "fake://", alloc(), [PT.TCP], cache_shape=4, num_kv_heads=1)
    try:
        pw, dw = K.WorkerInfo.from_string(cli.worker_info()), K.WorkerInfo.from_string(srv.worker_info())
        for w in (pw, dw):
            w.num_kv_heads = 1
        plan = K.plan_walk(pw, dw, 4, [("x", 0, 192, True, [[3, 5, 6]], [[2, 4, 7]])])
        caps = [bs * nb for bs in sizes]
        pieces = plan.expand(caps, caps)
        by_tensor = {0: [], 1: []}
        for t, zero, so, do, n in pieces:
            assert not zero and n % 4 == 0 and (t == 0 or (n % 16 == 0 and 0 < n <= 8192))
            by_tensor[t].append((so, do, n))
        assert sorted(n for _, _, n in by_tensor[1]) == sorted([7008] * 5 * 3 + [6944] * 3)      # three latent pages
        assert sorted(n for _, _, n in by_tensor[0]) == [8448] * 3                                 # three indexer pages
        for t, src_b, dst_b in ((1, 3, 2), (1, 5, 4), (1, 6, 7), (0, 3, 2)):                       # the segments tile the page
            segs = sorted(p for p in by_tensor[t] if src_b * sizes[t] <= p[0] < (src_b + 1) * sizes[t])
            pos = src_b * sizes[t]
            for so, do, n in segs:
                assert so == pos and do - dst_b * sizes[t] == so - src_b * sizes[t]
                pos += n
            assert pos == (src_b + 1) * sizes[t]
    finally:
        srv.stop()
