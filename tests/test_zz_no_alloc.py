"""qagg_quantize_batch_noalloc -- the batched quantize entry point for callers that are not allowed to allocate
device memory when they call into the library (a plugin living inside a host framework's fixed memory pool, a step that
must not trigger the device-wide stall of cudaMalloc, a component with a start-up memory budget).

It runs the same kernel as the aggregator's quantize phase, but its scratch (descriptor tables, work items, work-queue
counters) sits in a fixed 64 KB array inside the library instead of cudaMalloc'ed buffers.  The check: through the C ABI,
two calls in a row (the second one continuing from the residuals the first one left, and reusing the scratch the first
one left behind) must give exactly the packed words and residuals that the existing per-matrix entry point
qagg_quantize gives -- bit for bit, the tolerance every other test here uses.  Batches beyond the fixed limits must be
refused with a clear message and launch nothing.

This file is collected last on purpose: a failure here cannot hide any other test from a run that stops at the first failure."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

SHAPES = [(2048, 40), (9304, 3), (256, 1), (89, 23), (1, 135), (512, 300), (64, 147), (1000, 8)]


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cntk_b200 import lib as L
    return L


@pytest.mark.parametrize("bits,zero_thr", [(1, True), (4, True)])
def test_two_calls_match_the_per_matrix_entry_point(lib, bits, zero_thr):
    dev = "cuda:0"
    rng = np.random.default_rng(123 + bits)
    res_new = [torch.zeros((N, M), dtype=torch.float32, device=dev) for (M, N) in SHAPES]
    res_old = [torch.zeros((N, M), dtype=torch.float32, device=dev) for (M, N) in SHAPES]
    for call in range(2):
        grads = [torch.from_numpy((rng.standard_normal((N, M)) * 1e-3).astype(np.float32)).to(dev) for (M, N) in SHAPES]
        packed_new = [torch.zeros(lib.packed_bytes(M, N, bits), dtype=torch.uint8, device=dev) for (M, N) in SHAPES]
        packed_old = [torch.zeros_like(p) for p in packed_new]
        lib.quantize_batch_noalloc([g.data_ptr() for g in grads], [r.data_ptr() for r in res_new], [r.data_ptr() for r in res_new],
                                   [p.data_ptr() for p in packed_new], SHAPES, bits, zero_thr)
        for g, r, p, (M, N) in zip(grads, res_old, packed_old, SHAPES):
            lib.quantize(g.data_ptr(), r.data_ptr(), r.data_ptr(), p.data_ptr(), M, N, bits, zero_thr)
        torch.cuda.synchronize()
        for i, (M, N) in enumerate(SHAPES):
            assert torch.equal(packed_new[i], packed_old[i]), f"call {call}, matrix {i} ({M}x{N}): packed words differ"
            assert torch.equal(res_new[i].view(torch.int32), res_old[i].view(torch.int32)), f"call {call}, matrix {i} ({M}x{N}): residual differs"


def test_batches_beyond_the_fixed_scratch_are_refused(lib):
    dev = "cuda:0"
    t = torch.zeros((1, 8), dtype=torch.float32, device=dev)
    p = torch.zeros(lib.packed_bytes(8, 1, 1), dtype=torch.uint8, device=dev)
    n = 33  # one more matrix than the array has descriptors for
    with pytest.raises(lib.QaggError) as e:
        lib.quantize_batch_noalloc([t.data_ptr()] * n, [t.data_ptr()] * n, [t.data_ptr()] * n, [p.data_ptr()] * n, [(8, 1)] * n, 1)
    assert "at most 32" in str(e.value)
    # one tall-and-wide matrix that needs more work items than the array holds (2 columns of 9304 rows per item)
    M, N = 9304, 2 * 4096 + 2
    with pytest.raises(lib.QaggError) as e:
        lib.quantize_batch_noalloc([t.data_ptr()], [t.data_ptr()], [t.data_ptr()], [p.data_ptr()], [(M, N)], 1)
    assert "work items" in str(e.value)
    torch.cuda.synchronize()
