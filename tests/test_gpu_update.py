"""GPU parity of the fused learner step (consumer fusion): the momentum-SGD update taken straight from the packed aggregate
must leave the parameters and smoothed gradients byte-identical to "unquantize, then update" on the CPU checker
(oracle_sgd_update restates Matrix::MomentumSGDUpdate, Source/Math/Matrix.cpp:1681-1698, 5415-5429)."""
import numpy as np
import pytest

from oracle import exchange as ox

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

RULES = [(0.1, 0.9, 0.1), (0.05, 0.0, 1.0), (0.02, 1.0, 1.0), (1e-3, 0.5, 0.5)]  # (learn rate, momentum, unit-gain factor)


@pytest.fixture(scope="module")
def G():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util
    return gpu_util


@pytest.mark.parametrize("n,offset", [(1, 0), (3, 0), (1000, 0), (4099, 1), ((1 << 20) + 3, 0), (70000, 3)])
@pytest.mark.parametrize("rule", RULES)
def test_plain_update_kernel(G, oracle_port, n, offset, rule):
    """qagg_sgd_update over a gradient in memory, aligned and unaligned bases, all three forms of ScaleAndAdd."""
    from cntk_b200 import lib
    lr, mom, ug = rule
    rng = np.random.default_rng(n + offset)
    w = rng.standard_normal(n).astype(np.float32)
    g = (rng.standard_normal(n) * 1e-2).astype(np.float32)
    s = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    bufs = [torch.zeros(n + 8, dtype=torch.float32, device=G.DEV) for _ in range(3)]
    views = [b[offset:offset + n] for b in bufs]
    for v, a in zip(views, (w, g, s)):
        v.copy_(torch.from_numpy(a))
    for _ in range(2):
        lib.sgd_update(views[0].data_ptr(), views[1].data_ptr(), views[2].data_ptr(), n, lr, mom, ug)
        oracle_port.sgd_update(w, g, s, lr, mom, ug)
    G.assert_same_bits(G.host(views[0]), w, "parameters")
    G.assert_same_bits(G.host(views[2]), s, "smoothed gradients")
    G.assert_same_bits(G.host(views[1]), g, "gradients untouched")
    for b in bufs:  # nothing written outside the n values
        assert float(b[:offset].abs().sum()) == 0.0 and float(b[offset + n:].abs().sum()) == 0.0


@pytest.mark.parametrize("M,N", [(2048, 64), (9304, 8), (70, 5), (1000, 3), (64, 1), (1, 9), (4096, 33), (50000, 2)])
@pytest.mark.parametrize("bits", [1, 2, 4])
def test_unquantize_update_single_matrix(G, oracle_port, M, N, bits):
    """qagg_unquantize_sgd: every mapping of the unquantize kernel (vector, scalar, row-major) in update mode."""
    from cntk_b200 import lib
    lr, mom, ug = RULES[(M + bits) % len(RULES)]
    rng = np.random.default_rng(M * 31 + N + bits)
    grad = (rng.standard_normal((N, M)) * 1e-3).astype(np.float32)
    res = np.zeros((N, M), dtype=np.float32)
    packed = np.zeros(N * oracle_port.packed_col_bytes(M, bits), dtype=np.uint8)
    oracle_port.quantize(grad, res, res, packed, bits, True)
    agg = np.zeros((N, M), dtype=np.float32)
    oracle_port.unquantize(packed, agg, bits, False)
    w = rng.standard_normal((N, M)).astype(np.float32)
    s = (rng.standard_normal((N, M)) * 1e-4).astype(np.float32)
    dw, ds, dp = G.dev(w), G.dev(s), G.dev(packed)
    for _ in range(2):
        lib.unquantize_sgd(dp.data_ptr(), dw.data_ptr(), ds.data_ptr(), M, N, bits, lr, mom, ug)
        oracle_port.sgd_update(w.reshape(-1), agg.reshape(-1), s.reshape(-1), lr, mom, ug)
    G.assert_same_bits(G.host(dw), w, "parameters")
    G.assert_same_bits(G.host(ds), s, "smoothed gradients")


def test_unquantize_update_rejects_bad_arguments(G):
    from cntk_b200 import lib
    t = torch.zeros(64, dtype=torch.float32, device=G.DEV)
    with pytest.raises(lib.QaggError):
        lib.unquantize_sgd(t.data_ptr(), t.data_ptr(), t.data_ptr(), 8, 2, 1, 0.1, 1.5, 1.0)
    with pytest.raises(lib.QaggError):
        lib.sgd_update(t.data_ptr(), 0, t.data_ptr(), 8, 0.1, 0.5, 1.0)


@pytest.mark.parametrize("K,bits,peer", [(1, 1, False), (2, 1, False), (4, 1, True), (3, 4, False), (8, 1, True)])
def test_aggregator_fused_update(G, oracle_port, K, bits, peer):
    """While qagg_agg_set_update is on, a step ends in the update of the bound parameter and smoothed-gradient matrices and
    leaves the gradient buffers alone; switched off again, it writes aggregated gradients as before, with the residual
    state carried through both kinds of step."""
    from cntk_b200 import lib
    shapes = [(256, 40), (100, 7), (2048, 16), (9304, 3), (256, 1)]
    comms = lib.Comm.local_group(K, 0)
    aggs = [lib.Aggregator(c, shapes, bits) for c in comms]
    if peer:
        handles = [a.peer_handle() for a in aggs]
        for a in aggs:
            a.enable_peer(handles)
    st = ox.ExchangeState(shapes, K)
    rng = np.random.default_rng(100 * K + bits)
    w = [[rng.standard_normal((N, M)).astype(np.float32) for (M, N) in shapes] for _ in range(K)]
    s = [[np.zeros((N, M), dtype=np.float32) for (M, N) in shapes] for _ in range(K)]
    dw = [[G.dev(a) for a in w[r]] for r in range(K)]
    ds = [[G.dev(a) for a in s[r]] for r in range(K)]
    try:
        for r in range(K):
            with pytest.raises(lib.QaggError):
                aggs[r].set_update(True, 0.1, 0.9, 0.1)  # nothing bound yet
            aggs[r].bind_update([t.data_ptr() for t in dw[r]], [t.data_ptr() for t in ds[r]])
        for step in range(5):
            lr, mom, ug = RULES[step % len(RULES)]
            fused = step != 3
            grads = [[(rng.standard_normal((N, M)) * 1e-3).astype(np.float32) for (M, N) in shapes] for _ in range(K)]
            local = [[a.copy() for a in grads[r]] for r in range(K)]
            dg = [[G.dev(a) for a in grads[r]] for r in range(K)]
            ox.aggregate_step(oracle_port, st, grads, bits)  # grads now hold the aggregate
            for r in range(K):
                aggs[r].set_update(fused, lr, mom, ug)
            lib.step_group(aggs, [[t.data_ptr() for t in dg[r]] for r in range(K)])
            torch.cuda.synchronize()
            for r in range(K):
                for i in range(len(shapes)):
                    if fused:
                        oracle_port.sgd_update(w[r][i].reshape(-1), grads[r][i].reshape(-1), s[r][i].reshape(-1), lr, mom, ug)
                        G.assert_same_bits(G.host(dg[r][i]), local[r][i], f"step {step} rank {r} tensor {i}: gradient buffer left alone")
                    else:
                        G.assert_same_bits(G.host(dg[r][i]), grads[r][i], f"step {step} rank {r} tensor {i}: aggregate")
                    G.assert_same_bits(G.host(dw[r][i]), w[r][i], f"step {step} rank {r} tensor {i}: parameters")
                    G.assert_same_bits(G.host(ds[r][i]), s[r][i], f"step {step} rank {r} tensor {i}: smoothed gradients")
        for a in aggs:
            a.check()
            a.bind_update(None, None)
            with pytest.raises(lib.QaggError):
                a.set_update(True, 0.1, 0.9, 0.1)
    finally:
        for a in aggs:
            a.destroy()
        for c in comms:
            c.destroy()


def test_identity_aggregator_refuses_update(G):
    from cntk_b200 import lib
    comms = lib.Comm.local_group(1, 0)
    a = lib.Aggregator(comms[0], [(64, 4)], 1, lib.ZERO_THRESHOLD | lib.SELF_QUANTIZED | lib.V2_IDENTITY_K1)
    t = torch.zeros(256, dtype=torch.float32, device=G.DEV)
    try:
        with pytest.raises(lib.QaggError):
            a.bind_update([t.data_ptr()], [t.data_ptr()])
    finally:
        a.destroy()
        comms[0].destroy()


def test_fused_update_behind_the_form_walk_quantize_path(G, oracle_port, monkeypatch):
    """The fused learner step is the last kernel of a step whatever quantized the gradients: here the form + walk pair takes
    every matrix with 2048 rows or more, the streaming kernel the others."""
    monkeypatch.setenv("QAGG_TALL_ROWS", "2048")
    test_aggregator_fused_update(G, oracle_port, 4, 1, True)
