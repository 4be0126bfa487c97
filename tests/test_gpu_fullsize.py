"""Full-size runs of the benchmark configurations, checked through properties that do not need the oracle to process
the whole set, plus bit-exact spot checks: columns are quantized independently of each other, so the CPU oracle can
reproduce any sampled column of a full-size tensor exactly.

  * conservation (Tests/UnitTests/MathTests/MatrixQuantizerTests.cpp:327-338): in + old residual == new residual + output
  * every rank of a group ends with byte-identical aggregates
  * multi-rank runs: sampled columns of every tensor replayed through the whole exchange on the CPU checker, bit-exact
  * a 1-bit column's output takes at most two values, and padding bits of the packed words are zero
  * sampled columns: packed words, reconstruction values and residuals identical to the oracle's
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def env():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cntk_b200 import lib, workloads
    from oracle import backend
    backend.build()
    return lib, workloads, backend.OracleBackend()


def device_normal(shape, sigma, seed, dev="cuda:0"):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    return torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * sigma


def spot_check_quantize(lib, oracle, g, r_old, r_new, packed, M, N, bits, zero_thr, rng, ncols=24):
    C = lib.packed_col_bytes(M, bits)
    cols = sorted(set(int(c) for c in rng.integers(0, N, size=min(ncols, N))) | {0, N - 1})
    idx = torch.tensor(cols, device=g.device)
    gs, ro, rn = g[idx].cpu().numpy(), r_old[idx].cpu().numpy(), r_new[idx].cpu().numpy()
    pk = packed.view(N, C)[idx].cpu().numpy()
    exp_r = ro.copy()
    exp_p = np.zeros(len(cols) * C, np.uint8)
    oracle.quantize(np.ascontiguousarray(gs), exp_r, exp_r, exp_p, bits, zero_thr)
    assert np.array_equal(pk.reshape(-1), exp_p), "sampled columns: packed words / reconstruction values differ from the oracle"
    assert np.array_equal(rn.view(np.uint32), exp_r.view(np.uint32)), "sampled columns: residual differs from the oracle"


def test_speech_dnn_full_size_single_rank(env):
    """Config 2 at full size (45,122,648 values), one rank, three error-feedback steps."""
    lib, workloads, oracle = env
    shapes = workloads.speech_dnn()
    dev = "cuda:0"
    rng = np.random.default_rng(1)
    comm = lib.Comm.create(None, 0, 1, 0)
    agg = lib.Aggregator(comm, shapes, 1)
    try:
        r_old = [torch.zeros((N, M), dtype=torch.float32, device=dev) for (M, N) in shapes]
        for step in range(3):
            grads = [device_normal((N, M), 1e-3, 1000 * 0 + step * 97 + i) for i, (M, N) in enumerate(shapes)]
            work = [g.clone() for g in grads]
            agg.step([w.data_ptr() for w in work])
            torch.cuda.synchronize()
            for i, (M, N) in enumerate(shapes):
                r_new = torch.empty((N, M), dtype=torch.float32, device=dev)
                agg.copy_residual(i, 0, r_new.data_ptr())
                pk = torch.zeros(lib.packed_bytes(M, N, 1), dtype=torch.uint8, device=dev)
                agg.copy_packed(i, pk.data_ptr())
                torch.cuda.synchronize()
                lhs = grads[i] + r_old[i]
                err = (lhs - (r_new + work[i])).abs().max().item()
                assert err <= 8e-3 * 1e-4, f"conservation violated on tensor {i}: {err}"
                # two levels per column
                srt, _ = work[i].sort(dim=1)
                distinct = (srt[:, 1:] != srt[:, :-1]).sum(dim=1) + 1
                assert int(distinct.max()) <= 2, f"tensor {i}: a 1-bit column reconstructs to more than two values"
                # padding bits (rows >= M) of the packed words are zero
                Q = (M + 31) // 32
                words = pk.view(N, 8 + 4 * Q)[:, 8:].contiguous().view(torch.int32).view(N, Q)
                for w in range(Q):
                    nk = (M - w + Q - 1) // Q
                    if nk < 32:
                        assert int((words[:, w] >> nk).abs().max()) == 0 or int(((words[:, w].to(torch.int64) & 0xFFFFFFFF) >> nk).max()) == 0
                spot_check_quantize(lib, oracle, grads[i], r_old[i], r_new, pk, M, N, 1, True, rng)
                r_old[i] = r_new
    finally:
        agg.destroy()
        comm.destroy()


def run_group_fullsize(lib, oracle, shapes, K, bits, make_grad, steps, check_at, verify_ranks=None, peer=True):
    """K ranks on one device, full-size tensors, `steps` error-feedback steps.  At the steps in `check_at` a seeded sample
    of columns of every tensor (stripe edges included) is replayed on the CPU checker from the ranks' captured inputs and
    compared bit for bit: aggregates, residuals, stripe residuals, gathered packed columns (tests/parity_util.py).  Every
    step: all ranks end with byte-identical aggregates."""
    import parity_util as pu
    comms = lib.Comm.local_group(K, 0)
    aggs = [lib.Aggregator(c, shapes, bits) for c in comms]
    if peer and K > 1:
        hs = [a.peer_handle() for a in aggs]
        for a in aggs:
            a.enable_peer(hs)
    verify_ranks = sorted(set(verify_ranks if verify_ranks is not None else [0, K // 2, K - 1]))
    columns = 0
    try:
        for step in range(1, steps + 1):
            work = [[make_grad(r, step, i, M, N) for i, (M, N) in enumerate(shapes)] for r in range(K)]
            caps = None
            if step in check_at:
                cols = pu.pick_columns(shapes, K, seed=1000 + step)
                caps = [pu.RankCapture(lib, aggs[r], r, K, shapes, bits, cols) for r in range(K)]
                for r in range(K):
                    caps[r].before(work[r])
            lib.step_group(aggs, [[t.data_ptr() for t in work[r]] for r in range(K)])
            torch.cuda.synchronize()
            for i in range(len(shapes)):
                for r in range(1, K):
                    assert torch.equal(work[0][i].view(torch.int32), work[r][i].view(torch.int32)), f"step {step}: ranks 0 and {r} disagree on tensor {i}"
            if caps:
                inputs = [c.inp for c in caps]
                for r in verify_ranks:
                    caps[r].after(work[r])
                    columns += pu.verify(oracle, caps[r], inputs)
        for a in aggs:
            a.check()
    finally:
        for a in aggs:
            a.destroy()
        for c in comms:
            c.destroy()
    assert columns > 0
    return columns


def test_speech_dnn_full_size_8_ranks_100_steps(env):
    """Config 2 at full size (16 tensors, 45,122,648 values per rank, 1 bit, threshold 0), 8 ranks, 100 error-feedback
    steps; sampled columns against the CPU checker at steps 1, 25, 50, 75 and 100.  This is where the owner kernels meet
    full-height 9304-row and 2048-row stripes."""
    lib, workloads, oracle = env
    shapes = workloads.speech_dnn()

    def make(r, step, i, M, N):
        return device_normal((N, M), 1e-3, 1000 * r + step + 7919 * i)

    run_group_fullsize(lib, oracle, shapes, 8, 1, make, 100, {1, 25, 50, 75, 100})


@pytest.mark.parametrize("K", [2, 4])
def test_speech_dnn_full_size_2_and_4_ranks(env, K):
    """Config 2 at full size on 2 and 4 ranks, 10 steps, sampled columns at steps 1, 5 and 10."""
    lib, workloads, oracle = env

    def make(r, step, i, M, N):
        return device_normal((N, M), 1e-3, 77000 + 1000 * r + step + 7919 * i)

    run_group_fullsize(lib, oracle, workloads.speech_dnn(), K, 1, make, 10, {1, 5, 10}, verify_ranks=[0, K - 1])


def test_resnet50_full_size_4bit_8_ranks(env):
    """Config 3: 161 tensors, 25,557,032 values, 4 bits, Laplace(0, 1e-4), 8 ranks on one device, 20 steps; sampled columns
    against the CPU checker at steps 1, 10 and 20."""
    lib, workloads, oracle = env
    shapes = workloads.resnet50()
    assert len(shapes) == 161 and workloads.total_values(shapes) == 25557032

    def make(r, step, i, M, N):
        g = torch.Generator(device="cuda:0")
        g.manual_seed(500000 + 1000 * r + step + 104729 * i)
        u = (torch.rand((N, M), generator=g, device="cuda:0", dtype=torch.float32) - 0.5).clamp(-0.4999999, 0.4999999)
        return -1e-4 * torch.sign(u) * torch.log1p(-2 * u.abs())  # inverse-CDF Laplace(0, 1e-4)

    run_group_fullsize(lib, oracle, shapes, 8, 4, make, 20, {1, 10, 20})


def test_lstm_lm_full_size_ragged(env):
    """Config 4: 50000-row embedding with 90 % all-zero columns (columns taller than shared memory: streamed path),
    512 x 50000 softmax, bias vectors; 2 ranks (6 steps) and 8 ranks (3 steps) with sampled columns against the CPU checker;
    plus spot checks of the embedding through the single-matrix entry point."""
    lib, workloads, oracle = env
    shapes = workloads.lstm_lm()

    def make(r, step, i, M, N):
        a = device_normal((N, M), 5e-4, 900000 + 1000 * r + step + 15485863 * i)
        if i == 0:
            g = torch.Generator(device="cuda:0")
            g.manual_seed(77 + r + step)
            zero = torch.rand(N, generator=g, device="cuda:0") < 0.9
            a[zero] = 0.0
        return a

    run_group_fullsize(lib, oracle, shapes, 2, 1, make, 6, {1, 3, 6}, verify_ranks=[0, 1])
    run_group_fullsize(lib, oracle, shapes, 8, 1, make, 3, {1, 3}, verify_ranks=[0, 5])
    M, N = shapes[0]
    rng = np.random.default_rng(4)
    g = make(0, 0, 0, M, N)
    r_old = device_normal((N, M), 1e-4, 5)
    r_new = r_old.clone()
    pk = torch.zeros(lib.packed_bytes(M, N, 1), dtype=torch.uint8, device="cuda:0")
    lib.quantize(g.data_ptr(), r_new.data_ptr(), r_new.data_ptr(), pk.data_ptr(), M, N, 1, True)
    torch.cuda.synchronize()
    spot_check_quantize(lib, oracle, g, r_old, r_new, pk, M, N, 1, True, rng, ncols=12)
    # all-zero gradient columns with zero residual: range collapses, bits all one, residual zero
    z = torch.zeros((4, M), dtype=torch.float32, device="cuda:0")
    zr = torch.zeros_like(z)
    zp = torch.zeros(lib.packed_bytes(M, 4, 1), dtype=torch.uint8, device="cuda:0")
    lib.quantize(z.data_ptr(), zr.data_ptr(), zr.data_ptr(), zp.data_ptr(), M, 4, 1, True)
    torch.cuda.synchronize()
    assert not zr.any() and not zp.view(4, -1)[:, :8].any()


@pytest.mark.parametrize("bits", [1, 2])
def test_sweep_matrix_64m_values(env, bits):
    """Config 5 shape: 1024 rows x 65536 columns (64 Mi values), N(0,1) * 1e-3: quantize + unquantize, conservation and spot checks."""
    lib, _, oracle = env
    M, N = 1024, 65536
    rng = np.random.default_rng(bits)
    g = device_normal((N, M), 1e-3, 42 + bits)
    r_old = device_normal((N, M), 1e-4, 43 + bits)
    r_new = r_old.clone()
    pk = torch.zeros(lib.packed_bytes(M, N, bits), dtype=torch.uint8, device="cuda:0")
    out = torch.zeros((N, M), dtype=torch.float32, device="cuda:0")
    lib.quantize(g.data_ptr(), r_new.data_ptr(), r_new.data_ptr(), pk.data_ptr(), M, N, bits, True)
    lib.unquantize(pk.data_ptr(), out.data_ptr(), M, N, bits, False)
    torch.cuda.synchronize()
    assert float(((g + r_old) - (r_new + out)).abs().max()) <= 1e-2 * 1e-4
    spot_check_quantize(lib, oracle, g, r_old, r_new, pk, M, N, bits, True, rng)
