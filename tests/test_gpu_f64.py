"""ElemType = double: the quantizer with 64-bit packed words (what the reference's 1-bit end-to-end tests run,
precision=double), through the C ABI and through MatrixQuantizerImpl<double>, bit for bit against the CPU checker's double
instantiation and the committed digests made from the reference's own headers (tests/golden/golden_digests_f64.json)."""
import json
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
def env():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cntk_b200 import lib
    from oracle import backend
    backend.build()
    return lib, backend.OracleBackendF64()


class GpuF64:
    """The oracle backend's interface on top of the C ABI, so that the fixture generator can drive the GPU."""

    def __init__(self, lib):
        self.lib = lib

    def packed_col_bytes(self, M, bits):
        return self.lib.packed_bytes_f64(M, 1, bits)

    def quantize(self, grad, res_in, res_out, packed, bits, zero_thr=True):
        N, M = grad.shape
        g, r = torch.from_numpy(grad).cuda(), torch.from_numpy(res_in).cuda()
        p = torch.zeros(packed.size, dtype=torch.uint8, device="cuda")
        self.lib.quantize_f64(g.data_ptr(), r.data_ptr(), r.data_ptr(), p.data_ptr(), M, N, bits, zero_thr)
        torch.cuda.synchronize()
        res_out[...] = r.cpu().numpy()
        packed[...] = p.cpu().numpy()

    def unquantize(self, packed, out, bits, add=False):
        N, M = out.shape
        p, o = torch.from_numpy(packed).cuda(), torch.from_numpy(out).cuda()
        self.lib.unquantize_f64(p.data_ptr(), o.data_ptr(), M, N, bits, add)
        torch.cuda.synchronize()
        out[...] = o.cpu().numpy()


def test_unit_grid_double_matches_reference_digests(env):
    lib, _ = env
    with open(os.path.join(ROOT, "tests", "golden", "golden_digests_f64.json")) as f:
        want = json.load(f)["unit"]
    got = mg.unit_digests_f64(GpuF64(lib))
    assert got.keys() == want.keys()
    for k in want:
        assert got[k] == want[k], k


@pytest.mark.parametrize("M,N", [(2048, 96), (9304, 5), (1, 7), (70, 3), (5000, 2)])
@pytest.mark.parametrize("bits,zero_thr", [(1, True), (1, False), (2, True), (8, True), (32, True), (64, True)])
def test_double_quantizer_bit_exact(env, M, N, bits, zero_thr):
    lib, oracle = env
    rng = np.random.default_rng(M * 31 + N + bits)
    gpu = GpuF64(lib)
    res_c = np.zeros((N, M))
    res_g = np.zeros((N, M))
    out_c = np.zeros((N, M))
    out_g = np.zeros((N, M))
    for it in range(3):
        g = rng.standard_normal((N, M)) * 1e-3
        if it == 1:
            g[0] = 0.0  # an all-zero column (zero residual in step 0 only where the column was zero before)
        pc = np.zeros(N * oracle.packed_col_bytes(M, bits), np.uint8)
        pg = np.zeros_like(pc)
        oracle.quantize(g, res_c, res_c, pc, bits, zero_thr)
        gpu.quantize(g, res_g, res_g, pg, bits, zero_thr)
        assert np.array_equal(pc, pg), f"iteration {it}: packed words differ"
        assert np.array_equal(res_c.view(np.uint64), res_g.view(np.uint64)), f"iteration {it}: residual differs"
        oracle.unquantize(pc, out_c, bits, add=(it > 0))
        gpu.unquantize(pg, out_g, bits, add=(it > 0))
        assert np.array_equal(out_c.view(np.uint64), out_g.view(np.uint64)), f"iteration {it}: output differs"


def test_double_argument_errors(env):
    lib, _ = env
    t = torch.zeros(64, dtype=torch.float64, device="cuda")
    p = torch.zeros(256, dtype=torch.uint8, device="cuda")
    with pytest.raises(lib.QaggError):
        lib.quantize_f64(t.data_ptr(), t.data_ptr(), t.data_ptr(), p.data_ptr(), 8, 8, 3)
    with pytest.raises(lib.QaggError):
        lib.quantize_f64(t.data_ptr() + 4, t.data_ptr(), t.data_ptr(), p.data_ptr(), 8, 4, 1)
    assert lib.packed_bytes_f64(2048, 3, 1) == 3 * (16 + 8 * 32)


def test_matrix_quantizer_impl_double_like_the_reference_unit_test(env, tmp_path):
    """MatrixQuantizerImpl<double> driven as TestRunQuantization drives it (compat_check.cpp, mode quantizer_f64)."""
    lib, oracle = env
    from cntk_b200 import build
    build.build()
    exe = str(tmp_path / "compat_check")
    libdir = os.path.join(ROOT, "cntk_b200")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    res = subprocess.run(["g++", "-std=c++17", "-O1", f"-I{cuda}/include", os.path.join(ROOT, "tests", "cpp", "compat_check.cpp"), "-o", exe,
                          "-L", libdir, "-l:libqagg.so", f"-L{cuda}/lib64", "-lcudart", "-lpthread", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{cuda}/lib64"],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    M, N, bits, iters = 489, 3, 1, 4
    inputs = [mg.uniform_input_f64(M, N, -0.5, 0.5, 2515 + it) for it in range(iters)]
    fin, fout = str(tmp_path / "in.bin"), str(tmp_path / "out.bin")
    np.concatenate([a.reshape(-1) for a in inputs]).tofile(fin)
    run = subprocess.run([exe, "quantizer_f64", fin, fout, str(M), str(N), str(bits), "1", str(iters)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and "compat ok" in run.stdout, (run.returncode, run.stdout, run.stderr)
    dump = np.fromfile(fout, dtype=np.uint8)
    C = oracle.packed_col_bytes(M, bits)
    res_c, out_c, off = np.zeros((N, M)), np.zeros((N, M)), 0
    for it in range(iters):
        packed = np.zeros(N * C, np.uint8)
        oracle.quantize(inputs[it], res_c, res_c, packed, bits, True)
        oracle.unquantize(packed, out_c, bits, add=(it > 0))
        for name, ref in (("packed", packed), ("residual", res_c.view(np.uint8).reshape(-1)), ("output", out_c.view(np.uint8).reshape(-1))):
            assert np.array_equal(dump[off:off + ref.size], ref), f"iteration {it}: {name} differs"
            off += ref.size
    assert off == dump.size


@pytest.mark.parametrize("K", [1, 2, 3, 8])
@pytest.mark.parametrize("bits,zero_thr,self_quant", [(1, True, True), (1, False, True), (1, True, False), (4, True, True), (64, True, True)])
def test_double_aggregator_bit_exact(env, K, bits, zero_thr, self_quant):
    """qagg_agg_f64_*: AllReduceDistGradAggregator<double> on an in-process group, four steps with the residuals carried:
    every rank's aggregate, residual and stripe residual byte-identical to the CPU restatement of the exchange run with
    the double checker (includes tensors with fewer columns than ranks, single columns, a column taller than one chunk)."""
    lib, oracle = env
    from oracle import exchange as ox
    shapes = [(70, 9), (256, 33), (1500, 2), (64, 1), (5, 16)]
    flags = (lib.ZERO_THRESHOLD if zero_thr else 0) | (lib.SELF_QUANTIZED if self_quant else 0)
    comms = lib.Comm.local_group(K, 0)
    aggs = [lib.AggregatorF64(c, shapes, bits, flags) for c in comms]
    st = ox.ExchangeState(shapes, K, dtype=np.float64)
    rng = np.random.default_rng(1000 * K + bits)
    dev = "cuda:0"
    try:
        for step in range(4):
            grads = [[(rng.standard_normal((N, M)) * 1e-3) for (M, N) in shapes] for _ in range(K)]
            dg = [[torch.from_numpy(a).to(dev) for a in grads[r]] for r in range(K)]
            ox.aggregate_step(oracle, st, grads, bits, zero_thr, self_quant)
            lib.step_group_f64(aggs, [[t.data_ptr() for t in dg[r]] for r in range(K)])
            torch.cuda.synchronize()
            for r in range(K):
                for i, (M, N) in enumerate(shapes):
                    what = f"K {K} bits {bits} step {step} rank {r} tensor {i}"
                    assert np.array_equal(dg[r][i].cpu().numpy().view(np.uint64), grads[r][i].view(np.uint64)), "aggregate: " + what
                    res = torch.zeros((N, M), dtype=torch.float64, device=dev)
                    aggs[r].copy_residual(i, 0, res.data_ptr())
                    torch.cuda.synchronize()
                    assert np.array_equal(res.cpu().numpy().view(np.uint64), st.res[r][i].view(np.uint64)), "residual: " + what
                    n = ox.stripe(N, r, K)[1]
                    if K > 1 and n:
                        sres = torch.zeros((n, M), dtype=torch.float64, device=dev)
                        aggs[r].copy_residual(i, 1, sres.data_ptr())
                        torch.cuda.synchronize()
                        assert np.array_equal(sres.cpu().numpy().view(np.uint64), st.sres[r][i].view(np.uint64)), "stripe residual: " + what
            if step == 1:
                for a in aggs:
                    a.reset_residuals()
                st.reset()
    finally:
        for a in aggs:
            a.destroy()
        for c in comms:
            c.destroy()

