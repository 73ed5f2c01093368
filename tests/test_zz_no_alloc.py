"""The allocation-free block-copy entry point, called through its exported C symbol and compared
with a numpy copy of the same descriptors and with the ordinary entry point, twice in a row."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_DESCS = 4096
ERR_TOO_MANY = -1


def _lib():
    from llumnix_kv_b200 import load_ops

    ops = load_ops()
    lib = ctypes.CDLL(ops.__file__)
    fn = lib.kvt_copy_blocks_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64,
                   ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
    return ops, fn


def _descs(rng, n, src_bytes, dst_bytes):
    """Non-overlapping destination ranges of mixed sizes and alignments."""
    out, dof = [], 0
    for i in range(n):
        ln = int(rng.choice([16, 48, 256, 1000, 4096, 5, 8192]))
        if i % 3 == 0:
            ln = ln // 16 * 16 or 16
        so = int(rng.integers(0, src_bytes - ln))
        if i % 3 == 0:
            so = so // 16 * 16
            dof = (dof + 15) // 16 * 16
        if dof + ln > dst_bytes:
            break
        out.append((so, dof, ln))
        dof += ln + int(rng.integers(0, 7))
    return out


def _run_pair(ops, fn, seed, n):
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    rng = np.random.default_rng(seed)
    src = torch.randint(0, 256, (8 << 20,), dtype=torch.uint8, device=dev)
    want = torch.zeros(16 << 20, dtype=torch.uint8, device=dev)
    got = torch.zeros_like(want)
    trip = _descs(rng, n, src.numel(), want.numel())
    host = np.asarray(trip, dtype=np.uint64).reshape(-1)
    # ordinary entry point: descriptors and status in caller-allocated device memory
    t_dev = torch.from_numpy(host.astype(np.int64)).to(dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    ops.kvt_launch_copy_blocks(src.data_ptr(), want.data_ptr(), t_dev.data_ptr(), len(trip), src.numel(),
                               want.numel(), status.data_ptr(), 0, stream)
    # allocation-free entry point: descriptors in host memory, status back to host memory
    hstat = np.full(2, 0xFFFFFFFF, dtype=np.uint32)
    rc = fn(src.data_ptr(), got.data_ptr(), host.ctypes.data, len(trip), src.numel(), got.numel(),
            hstat.ctypes.data, stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert status[0].item() == 0 and hstat[0] == 0
    # the oracle: the same byte ranges copied on the host, independent of either kernel
    src_h = src.cpu().numpy()
    oracle = np.zeros(want.numel(), dtype=np.uint8)
    for so, dof, ln in trip:
        oracle[dof:dof + ln] = src_h[so:so + ln]
    assert np.array_equal(got.cpu().numpy(), oracle)
    assert torch.equal(got, want)
    assert got.any()
    return len(trip)


def test_noalloc_matches_ordinary_entry_point_twice():
    ops, fn = _lib()
    n1 = _run_pair(ops, fn, seed=1, n=700)
    n2 = _run_pair(ops, fn, seed=2, n=MAX_DESCS)      # second call reuses the scratch; status was cleared
    assert n1 > 100 and n2 > 1000


def test_noalloc_reports_out_of_range_then_recovers():
    ops, fn = _lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    src = torch.arange(4096, dtype=torch.uint8, device=dev)
    dst = torch.zeros(4096, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    bad = np.asarray([0, 0, 64, 4000, 0, 200], dtype=np.uint64)      # second descriptor runs past src
    hstat = np.zeros(2, dtype=np.uint32)
    assert fn(src.data_ptr(), dst.data_ptr(), bad.ctypes.data, 2, 4096, 4096, hstat.ctypes.data, stream) == 0
    torch.cuda.synchronize()
    assert hstat[0] == 1 and hstat[1] == 1                          # KVT_ERR_BLOCK_RANGE at descriptor 1
    assert torch.equal(dst[:64], src[:64]) and not dst[64:].any()   # the bad one was skipped, not executed
    good = np.asarray([128, 256, 512], dtype=np.uint64)
    assert fn(src.data_ptr(), dst.data_ptr(), good.ctypes.data, 1, 4096, 4096, hstat.ctypes.data, stream) == 0
    torch.cuda.synchronize()
    assert hstat[0] == 0                                            # cleared before the launch
    assert torch.equal(dst[256:768], src[128:640])


def test_noalloc_rejects_more_than_the_maximum():
    _, fn = _lib()
    torch.cuda.set_device(0)
    host = np.zeros(3 * (MAX_DESCS + 1), dtype=np.uint64)
    rc = fn(1 << 20, 1 << 20, host.ctypes.data, MAX_DESCS + 1, 0, 0, None, None)
    assert rc == ERR_TOO_MANY
    assert fn(0, 0, None, 0, 0, 0, None, None) == 0                 # empty call is a no-op
