"""The C++ mirror of the reference interfaces (cntk_b200/csrc/cntk_compat) driven as the reference's own callers drive
them: tests/cpp/compat_check.cpp is compiled with g++ against libqagg.so, run on the GPU, and its dumps are compared
bit for bit with the CPU oracle."""
import os
import subprocess
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as mg  # noqa: E402

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def exe(tmp_path_factory):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cntk_b200 import build
    build.build()
    out = str(tmp_path_factory.mktemp("compat") / "compat_check")
    libdir = os.path.join(ROOT, "cntk_b200")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++17", "-O1", f"-I{cuda}/include", os.path.join(ROOT, "tests", "cpp", "compat_check.cpp"), "-o", out,
           "-L", libdir, "-l:libqagg.so", f"-L{cuda}/lib64", "-lcudart", "-lpthread", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{cuda}/lib64"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return out


def run(exe, tmp_path, mode, inputs, M, N, bits, zero_thr):
    fin, fout = str(tmp_path / "in.bin"), str(tmp_path / "out.bin")
    np.concatenate([a.reshape(-1) for a in inputs]).astype(np.float32).tofile(fin)
    res = subprocess.run([exe, mode, fin, fout, str(M), str(N), str(bits), str(int(zero_thr)), str(len(inputs))], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "compat ok" in res.stdout, (res.returncode, res.stdout, res.stderr)
    return np.fromfile(fout, dtype=np.uint8)


@pytest.mark.parametrize("M,N,bits,zero_thr", [(489, 1, 1, True), (100, 50, 1, False), (89, 23, 4, True), (2048, 64, 1, True)])
def test_matrix_quantizer_impl_like_the_reference_unit_test(exe, tmp_path, oracle_port, M, N, bits, zero_thr):
    iters = 5
    inputs = [mg.uniform_input(M, N, -0.5, 0.5, 2515 + it) for it in range(iters)]
    dump = run(exe, tmp_path, "quantizer", inputs, M, N, bits, zero_thr)
    C = oracle_port.packed_col_bytes(M, bits)
    res = np.zeros((N, M), np.float32)
    out = np.zeros((N, M), np.float32)
    off = 0
    for it in range(iters):
        packed = np.zeros(N * C, np.uint8)
        oracle_port.quantize(inputs[it], res, res, packed, bits, zero_thr)
        oracle_port.unquantize(packed, out, bits, add=(it > 0))
        for name, ref in (("packed", packed), ("residual", res.view(np.uint8).reshape(-1)), ("output", out.view(np.uint8).reshape(-1))):
            got = dump[off:off + ref.size]
            off += ref.size
            assert np.array_equal(got, ref), f"iteration {it}: {name} differs"
    assert off == dump.size


def test_aggregator_and_v2_communicator_single_rank(exe, tmp_path, oracle_port):
    M, N, bits, iters = 256, 40, 1, 2
    inputs = [mg.normal_input(M, N, 1e-3, 77 + it) for it in range(iters)]
    dump = run(exe, tmp_path, "aggregator", inputs, M, N, bits, True)
    C = oracle_port.packed_col_bytes(M, bits)
    res0 = np.zeros((N, M), np.float32)
    res1 = np.zeros((1, M), np.float32)
    off = 0
    for it in range(iters):
        for g, res in ((inputs[it].copy(), res0), (inputs[it][:1].copy(), res1)):
            n = g.shape[0]
            packed = np.zeros(n * C, np.uint8)
            oracle_port.quantize(g, res, res, packed, bits, True)
            oracle_port.unquantize(packed, g, bits, add=False)
            ref = g.view(np.uint8).reshape(-1)
            assert np.array_equal(dump[off:off + ref.size], ref), f"step {it}: aggregate differs"
            off += ref.size
    assert off == dump.size


def test_aggregator_buffered_async_hands_back_the_previous_aggregate(exe, tmp_path, oracle_port):
    """useAsyncAggregation = true (Source/1BitSGD/AllReduceDistGradAggregator.h:156-229): call t returns the aggregate of the
    gradients given to call t - 1 (zeros after the reset); the residual chain is the same as without buffering."""
    M, N, bits, iters = 256, 40, 1, 3
    inputs = [mg.normal_input(M, N, 1e-3, 177 + it) for it in range(iters)]
    dump = run(exe, tmp_path, "aggregator_async", inputs, M, N, bits, True)
    C = oracle_port.packed_col_bytes(M, bits)
    res0 = np.zeros((N, M), np.float32)
    res1 = np.zeros((1, M), np.float32)
    per_call = (N * M + M) * 4
    assert dump.size == (iters + 1) * per_call
    assert not dump[:per_call].any(), "the first call must hand back zeros"
    off = per_call
    for it in range(iters):
        for g, res in ((inputs[it].copy(), res0), (inputs[it][:1].copy(), res1)):
            n = g.shape[0]
            packed = np.zeros(n * C, np.uint8)
            oracle_port.quantize(g, res, res, packed, bits, True)
            oracle_port.unquantize(packed, g, bits, add=False)
            ref = g.view(np.uint8).reshape(-1)
            assert np.array_equal(dump[off:off + ref.size], ref), f"call {it + 1}: aggregate of step {it} differs"
            off += ref.size
    assert off == dump.size


def test_per_epoch_bit_schedule_and_warm_start(exe, tmp_path, oracle_port):
    """DataParallelSGD (the bookkeeping of Source/SGDLib/SGD.cpp:427-432, 553-559, 2336-2359): gradientBits = 1:1:4:32 with
    parallelizationStartEpoch = 2 over five epochs of two minibatches.  Epoch 0 leaves the gradients alone; a change of bit
    width creates a new aggregator with zero residuals; every epoch's first minibatch resets the residuals; 32 bits is the
    unquantized sum (the identity on one rank)."""
    M, N = 256, 40
    inputs = [mg.normal_input(M, N, 1e-3, 900 + i) for i in range(10)]
    dump = run(exe, tmp_path, "schedule", inputs, M, N, 1, True)
    off = 0
    for epoch in range(5):
        bits = [None, 1, 4, 32, 32][epoch]
        for mb in range(2):
            if mb == 0:
                res = {}  # residuals per tensor shape: zero at every epoch's first minibatch
            x = inputs[2 * epoch + mb]
            for g in (x.copy(), x[:1].copy()):
                if bits not in (None, 32):
                    r = res.setdefault(g.shape, np.zeros(g.shape, np.float32))
                    packed = np.zeros(g.shape[0] * oracle_port.packed_col_bytes(M, bits), np.uint8)
                    oracle_port.quantize(g, r, r, packed, bits, True)
                    oracle_port.unquantize(packed, g, bits, add=False)
                ref = g.view(np.uint8).reshape(-1)
                assert np.array_equal(dump[off:off + ref.size], ref), f"epoch {epoch} minibatch {mb}: aggregate differs"
                off += ref.size
    assert off == dump.size
