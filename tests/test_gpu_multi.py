"""Multi-GPU parity of the NCCL exchange (needs >= 2 GPUs; skipped otherwise)."""
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("K", [2, 4, 8])
def test_nccl_exchange_bit_exact(K):
    if not torch.cuda.is_available() or torch.cuda.device_count() < K:
        pytest.skip(f"needs {K} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "0"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={K}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "multi_gpu_check.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert f"multi-GPU parity ok on {K} ranks" in out.stdout


@pytest.mark.parametrize("K", [2, 4])
def test_cpp_mirror_classes_run_a_real_exchange(K, tmp_path, oracle_port):
    """tests/cpp/compat_check.cpp in mode "multi": K processes, one per GPU, tied together by a unique id passed through a
    file, drive the C++ mirror classes the way SGDLib and the V2 trainer drive the reference's: AllReduceDistGradAggregator,
    V2AllReduceDistGradAggregator (synchronous and buffered asynchronous) over QuantizedMPICommunicator with caller-owned
    residuals, QuantizedDataParallelDistributedLearner (checkpoint zeroes the residuals; over a momentum-SGD learner with and
    without the update fused into the exchange), SimpleDistGradAggregator and AllReduceDistGradAggregator<double>.
    Every rank's dumps are compared with the CPU checker bit for bit (the unquantized arm, whose all-reduce order is
    NCCL's, within 1e-5); the DistGradHeader sums are checked inside the program."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < K:
        pytest.skip(f"needs {K} GPUs")
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_golden as mg
    from oracle import exchange as ox
    from cntk_b200 import build
    build.build()
    exe = str(tmp_path / "compat_check")
    libdir = os.path.join(ROOT, "cntk_b200")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    res = subprocess.run(["g++", "-std=c++17", "-O1", f"-I{cuda}/include", os.path.join(ROOT, "tests", "cpp", "compat_check.cpp"), "-o", exe,
                          "-L", libdir, "-l:libqagg.so", f"-L{cuda}/lib64", "-lcudart", "-lpthread", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{cuda}/lib64"],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    M, N, bits, iters = 256, 37, 1, 3
    shapes = [(M, N), (M, 1)]
    inputs = [[[mg.normal_input(M, N, 1e-3, 100 * it + r), mg.normal_input(M, 1, 1e-3, 5000 + 100 * it + r)] for r in range(K)] for it in range(iters)]
    fin = str(tmp_path / "in.bin")
    np.concatenate([a.reshape(-1) for per_it in inputs for per_rank in per_it for a in per_rank]).astype(np.float32).tofile(fin)
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "0"))
    procs = [subprocess.Popen([exe, "multi", fin, str(tmp_path / f"out{r}.bin"), str(M), str(N), str(bits), "1", str(iters), str(r), str(K),
                               str(tmp_path / "id.bin")], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env) for r in range(K)]
    for r, p in enumerate(procs):
        out, err = p.communicate(timeout=300)
        assert p.returncode == 0 and "compat ok" in out, (r, p.returncode, out, err)

    def run_steps(state, its):
        outs = []
        for it in its:
            grads = [[a.copy() for a in inputs[it][r]] for r in range(K)]
            ox.aggregate_step(oracle_port, state, grads, bits)
            outs.append(grads)
        return outs

    st = ox.ExchangeState(shapes, K)
    seq = run_steps(st, range(iters))                       # A, B: consecutive steps from a fresh state
    first = run_steps(ox.ExchangeState(shapes, K), [0])[0]  # after a reset: like a first step
    stD = ox.ExchangeState(shapes, K)
    seqD = run_steps(stD, [0])
    stD.reset()                                             # the learner's checkpoint after its first step
    seqD += run_steps(stD, range(1, iters))
    dense = ox.dense_sum([[a for a in inputs[0][r]] for r in range(K)])
    from oracle import backend as ob
    st64, seq64, o64 = ox.ExchangeState(shapes, K, dtype=np.float64), [], ob.OracleBackendF64()
    for it in range(iters):
        g64 = [[a.astype(np.float64) for a in inputs[it][r]] for r in range(K)]
        ox.aggregate_step(o64, st64, g64, bits)
        seq64.append(g64)
    for r in range(K):
        dump = np.fromfile(str(tmp_path / f"out{r}.bin"), dtype=np.float32)
        off = 0

        def take(shape):
            nonlocal off
            n = int(np.prod(shape))
            a = dump[off:off + n].reshape(shape)
            off += n
            return a

        def same(a, b, what):
            assert np.array_equal(a.view(np.uint32), np.ascontiguousarray(b).view(np.uint32)), f"rank {r}: {what}"

        for it in range(iters):                             # A
            same(take((N, M)), seq[it][r][0], f"V1 aggregator step {it} tensor 0")
            same(take((1, M)), seq[it][r][1], f"V1 aggregator step {it} tensor 1")
        for it in range(iters):                             # B
            same(take((N, M)), seq[it][r][0], f"V2 aggregator step {it} tensor 0")
            same(take((1, M)), seq[it][r][1], f"V2 aggregator step {it} tensor 1")
        same(take((N, M)), st.res[r][0], "V2 aggregator: caller-owned residual after the steps")
        same(take((N, M)), first[r][0], "V2 aggregator after resetState tensor 0")
        same(take((1, M)), first[r][1], "V2 aggregator after resetState tensor 1")
        for it in range(iters + 1):                         # C: one call stale
            a, b = take((N, M)), take((1, M))
            if it == 0:
                assert not a.any() and not b.any(), f"rank {r}: buffered async: the first call must hand back zeros"
            else:
                same(a, seq[it - 1][r][0], f"buffered async call {it} tensor 0")
                same(b, seq[it - 1][r][1], f"buffered async call {it} tensor 1")
        for it in range(iters):                             # D
            same(take((N, M)), seqD[it][r][0], f"learner step {it} tensor 0")
            same(take((1, M)), seqD[it][r][1], f"learner step {it} tensor 1")
        assert np.allclose(take((N, M)), dense[0], rtol=1e-5, atol=1e-9), f"rank {r}: unquantized aggregator tensor 0"
        assert np.allclose(take((1, M)), dense[1], rtol=1e-5, atol=1e-9), f"rank {r}: unquantized aggregator tensor 1"
        # F: momentum-SGD learner (learning rate 0.05, momentum 0.9, unit gain), fused == unfused inside the program; here
        # against the CPU checker's update applied to the CPU checker's aggregates
        w = [(1.0 + 1000.0 * inputs[0][r][t]).astype(np.float32) for t in range(2)]
        sm = [np.zeros_like(a) for a in w]
        for it in range(iters):
            for t in range(2):
                oracle_port.sgd_update(w[t].reshape(-1), np.ascontiguousarray(seq[it][r][t]).reshape(-1), sm[t].reshape(-1), 0.05, 0.9, np.float32(1.0) - np.float32(0.9))
        for t, shape in enumerate([(N, M), (1, M)]):
            same(take(shape), w[t], f"fused learner: parameters of tensor {t}")
            same(take(shape), sm[t], f"fused learner: smoothed gradients of tensor {t}")
        for it in range(iters):                             # G: double gradients
            for t, shape in enumerate([(N, M), (1, M)]):
                got = take((shape[0], 2 * shape[1])).view(np.float64)
                assert np.array_equal(got.view(np.uint64), seq64[it][r][t].view(np.uint64)), f"rank {r}: double aggregator step {it} tensor {t}"
        assert off == dump.size
