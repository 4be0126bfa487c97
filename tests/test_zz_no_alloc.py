"""qagg_quantize_batch_noalloc -- the batched quantize entry point for callers that are not allowed to allocate
device memory when they call into the library (a plugin living inside a host framework's fixed memory pool, a step that
must not trigger the device-wide stall of cudaMalloc, a component with a start-up memory budget).

It runs the same kernel as the aggregator's quantize phase, but its scratch (descriptor tables, work items, work-queue
counters) sits in a fixed 64 KB array inside the library instead of cudaMalloc'ed buffers.  The check: through the C ABI,
two calls in a row (the second one continuing from the residuals the first one left, and reusing the scratch the first
one left behind) must give exactly the packed words and residuals that the existing per-matrix entry point
qagg_quantize gives -- bit for bit, the tolerance every other test here uses -- and exactly what the CPU checker
(oracle/qagg_oracle.c) computes from the same inputs.  Batches beyond the fixed limits must be refused with a clear
message and launch nothing.

This file is collected last on purpose: a failure here cannot hide any other test from a run that stops at the first failure."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

# the 20000-row matrix is taller than a CTA's shared memory: it takes the kernel's chunked path through this entry point
SHAPES = [(2048, 40), (9304, 3), (256, 1), (89, 23), (1, 135), (512, 300), (64, 147), (1000, 8), (20000, 3)]


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cntk_b200 import lib as L
    return L


@pytest.mark.parametrize("bits,zero_thr", [(1, True), (1, False), (4, True)])
def test_two_calls_match_the_per_matrix_entry_point(lib, oracle_port, bits, zero_thr):
    dev = "cuda:0"
    rng = np.random.default_rng(123 + bits)
    res_new = [torch.zeros((N, M), dtype=torch.float32, device=dev) for (M, N) in SHAPES]
    res_old = [torch.zeros((N, M), dtype=torch.float32, device=dev) for (M, N) in SHAPES]
    res_cpu = [np.zeros((N, M), np.float32) for (M, N) in SHAPES]
    for call in range(2):
        host = [(rng.standard_normal((N, M)) * 1e-3).astype(np.float32) for (M, N) in SHAPES]
        grads = [torch.from_numpy(h).to(dev) for h in host]
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
            packed_cpu = np.zeros(N * oracle_port.packed_col_bytes(M, bits), np.uint8)
            oracle_port.quantize(host[i], res_cpu[i], res_cpu[i], packed_cpu, bits, zero_thr)
            assert np.array_equal(packed_new[i].cpu().numpy(), packed_cpu), f"call {call}, matrix {i} ({M}x{N}): packed words differ from the CPU checker"
            assert np.array_equal(res_new[i].cpu().numpy().view(np.uint32), res_cpu[i].view(np.uint32)), \
                f"call {call}, matrix {i} ({M}x{N}): residual differs from the CPU checker"


def test_batches_beyond_the_fixed_scratch_are_refused(lib):
    dev = "cuda:0"
    t = torch.zeros((1, 8), dtype=torch.float32, device=dev)
    p = torch.zeros(lib.packed_bytes(8, 1, 1), dtype=torch.uint8, device=dev)
    n = 33  # one more matrix than the array has descriptors for; each is a valid 8 x 1 matrix
    with pytest.raises(lib.QaggError) as e:
        lib.quantize_batch_noalloc([t.data_ptr()] * n, [t.data_ptr()] * n, [t.data_ptr()] * n, [p.data_ptr()] * n, [(8, 1)] * n, 1)
    assert "at most 32" in str(e.value)
    # One short-and-wide matrix that needs more work items than the array holds however the kernel tiles it: an item never
    # has more than 128 columns, so 4096 * 128 + 1 columns need at least 4097 items.  All buffers have their true sizes
    # (about 17 MB each), so even a build that accepted the call would stay inside them.
    M, N = 8, 4096 * 128 + 1
    g = torch.zeros((N, M), dtype=torch.float32, device=dev)
    r = torch.zeros((N, M), dtype=torch.float32, device=dev)
    pk = torch.zeros(lib.packed_bytes(M, N, 1), dtype=torch.uint8, device=dev)
    with pytest.raises(lib.QaggError) as e:
        lib.quantize_batch_noalloc([g.data_ptr()], [r.data_ptr()], [r.data_ptr()], [pk.data_ptr()], [(M, N)], 1)
    assert "work items" in str(e.value)
    torch.cuda.synchronize()
    assert not bool(pk.any()), "a refused call must launch nothing"


def test_a_capturing_stream_is_refused(lib):
    """The tables are uploaded from the caller's stack, so the call cannot be recorded into a graph: it must say so."""
    dev = "cuda:0"
    M, N = 64, 5
    g = torch.zeros((N, M), dtype=torch.float32, device=dev)
    r = torch.zeros((N, M), dtype=torch.float32, device=dev)
    pk = torch.zeros(lib.packed_bytes(M, N, 1), dtype=torch.uint8, device=dev)
    args = ([g.data_ptr()], [r.data_ptr()], [r.data_ptr()], [pk.data_ptr()], [(M, N)], 1)
    lib.quantize_batch_noalloc(*args)  # set-up call, outside any capture
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        graph.capture_begin()
        try:
            with pytest.raises(lib.QaggError) as e:
                lib.quantize_batch_noalloc(*args, stream=side.cuda_stream)
            assert "captured" in str(e.value)
        finally:
            graph.capture_end()
    torch.cuda.synchronize()
