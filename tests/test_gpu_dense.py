"""The unquantized fp32 aggregation arm (gradientBits = 32) against its CPU restatement: the sum over the ranks in ascending
rank order, one fp32 rounding per addition (oracle.exchange.dense_sum).  K ranks live in one process on one device and
exchange through their windows, exactly as the multi-GPU path does over NVLink."""
import numpy as np
import pytest

from oracle import exchange as ox

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

SHAPES = [(2048, 40), (9304, 3), (256, 1), (89, 23), (1, 135), (64, 147), (5, 1), (1000, 8)]


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cntk_b200 import lib as L
    return L


@pytest.mark.parametrize("K", [1, 2, 3, 8])
def test_dense_sum_bit_exact(lib, K):
    dev = "cuda:0"
    comms = lib.Comm.local_group(K, 0)
    aggs = [lib.DenseAggregator(c, SHAPES) for c in comms]
    if K > 1:
        hs = [a.peer_handle() for a in aggs]
        for a in aggs:
            a.enable_peer(hs)
    rng = np.random.default_rng(17 + K)
    try:
        for step in range(3):
            # wide dynamic range, so that the order of the additions shows in the low bits
            host = [[(rng.standard_normal((N, M)) * 10.0 ** rng.integers(-4, 3, size=(N, M))).astype(np.float32) for (M, N) in SHAPES] for _ in range(K)]
            dg = [[torch.from_numpy(a).to(dev) for a in host[r]] for r in range(K)]
            lib.dense_step_group(aggs, [[t.data_ptr() for t in dg[r]] for r in range(K)])
            torch.cuda.synchronize()
            want = ox.dense_sum(host)
            for r in range(K):
                for i in range(len(SHAPES)):
                    got = dg[r][i].cpu().numpy()
                    assert np.array_equal(got.view(np.uint32), want[i].view(np.uint32)), f"step {step} rank {r} tensor {i}"
        for a in aggs:
            a.check()
        if K > 1:
            flat4 = sum((m * n + 3) // 4 for m, n in SHAPES)
            assert aggs[0].wire_bytes == 2 * (K - 1) * ((flat4 + K - 1) // K) * 16
    finally:
        for a in aggs:
            a.destroy()
        for c in comms:
            c.destroy()


def test_dense_unaligned_tensors_and_empty_ones(lib):
    """Tensor starts that are not 16-byte aligned (views into a larger buffer) and empty tensors."""
    dev = "cuda:0"
    K = 2
    shapes = [(7, 3), (0, 5), (33, 1), (4, 0), (129, 2)]
    comms = lib.Comm.local_group(K, 0)
    aggs = [lib.DenseAggregator(c, shapes) for c in comms]
    hs = [a.peer_handle() for a in aggs]
    for a in aggs:
        a.enable_peer(hs)
    rng = np.random.default_rng(3)
    try:
        host, ptrs, bufs = [], [], []
        for r in range(K):
            buf = torch.zeros(1024, dtype=torch.float32, device=dev)
            off, row_h, row_p = 1, [], []  # start one float past an aligned address
            for (M, N) in shapes:
                a = (rng.standard_normal((N, M)) * 1e-2).astype(np.float32)
                buf[off:off + M * N].copy_(torch.from_numpy(a.reshape(-1)))
                row_h.append(a)
                row_p.append(buf.data_ptr() + 4 * off)
                off += M * N + 1
            host.append(row_h)
            ptrs.append(row_p)
            bufs.append((buf, off))
        lib.dense_step_group(aggs, ptrs)
        torch.cuda.synchronize()
        want = ox.dense_sum(host)
        for r in range(K):
            buf, _ = bufs[r]
            off = 1
            for i, (M, N) in enumerate(shapes):
                got = buf[off:off + M * N].cpu().numpy().reshape(N, M)
                assert np.array_equal(got.view(np.uint32), want[i].view(np.uint32)), f"rank {r} tensor {i}"
                assert float(buf[off + M * N]) == 0.0, "wrote past the end of a tensor"
                off += M * N + 1
    finally:
        for a in aggs:
            a.destroy()
        for c in comms:
            c.destroy()


@pytest.mark.parametrize("K", [2, 3, 8])
def test_dense_fp16_transport_bit_exact(lib, K):
    """useFP16AllReduce: values cast to half, summed as halves in ascending rank order, cast back (oracle.exchange.dense_sum_fp16);
    switching it off again gives the fp32 sum; the wire bytes halve."""
    dev = "cuda:0"
    comms = lib.Comm.local_group(K, 0)
    aggs = [lib.DenseAggregator(c, SHAPES) for c in comms]
    hs = [a.peer_handle() for a in aggs]
    for a in aggs:
        a.enable_peer(hs)
    rng = np.random.default_rng(29 + K)
    try:
        full = aggs[0].wire_bytes
        for step in range(4):
            half = step != 2
            for a in aggs:
                a.set_fp16(half)
            # values across the half range, including some that overflow it and some below its smallest subnormal
            host = [[(rng.standard_normal((N, M)) * 10.0 ** rng.integers(-9, 6, size=(N, M))).astype(np.float32) for (M, N) in SHAPES] for _ in range(K)]
            dg = [[torch.from_numpy(a).to(dev) for a in host[r]] for r in range(K)]
            lib.dense_step_group(aggs, [[t.data_ptr() for t in dg[r]] for r in range(K)])
            torch.cuda.synchronize()
            with np.errstate(over="ignore", invalid="ignore"):
                want = ox.dense_sum_fp16(host) if half else ox.dense_sum(host)
            for r in range(K):
                for i in range(len(SHAPES)):
                    got = dg[r][i].cpu().numpy()
                    same = (got.view(np.uint32) == want[i].view(np.uint32)) | (np.isnan(got) & np.isnan(want[i]))
                    assert same.all(), f"step {step} rank {r} tensor {i} (fp16 {half})"
            assert aggs[0].wire_bytes == (full // 2 if half else full)
        for a in aggs:
            a.check()
    finally:
        for a in aggs:
            a.destroy()
        for c in comms:
            c.destroy()
