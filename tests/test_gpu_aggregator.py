"""GPU parity of the striped aggregator against the CPU restatement of the exchange (oracle/exchange.py).

K ranks live in one process on one device and exchange by device-to-device copies (qagg_comm_create_local_group),
which is how the reference's own multi-rank GPU tests ran (all ranks on GPU 0).  Every rank's aggregated gradients,
residuals, stripe residuals and the gathered packed words must be byte-identical to the oracle's, step after step."""
import json
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as mg  # noqa: E402

from oracle import exchange as ox  # noqa: E402

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def G():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util
    return gpu_util


def run_group(G, oracle, shapes, K, bits, zero_thr, self_quant, steps, make_inputs, check_every=1, v2_identity=False, peer=False):
    from cntk_b200 import lib
    flags = (lib.ZERO_THRESHOLD if zero_thr else 0) | (lib.SELF_QUANTIZED if self_quant else 0) | (lib.V2_IDENTITY_K1 if v2_identity else 0)
    comms = lib.Comm.local_group(K, 0)
    aggs = [lib.Aggregator(c, shapes, bits, flags) for c in comms]
    if peer:
        handles = [a.peer_handle() for a in aggs]
        for a in aggs:
            a.enable_peer(handles)
    st = ox.ExchangeState(shapes, K)
    dgrads = [[torch.zeros((N, M), dtype=torch.float32, device=G.DEV) for (M, N) in shapes] for _ in range(K)]
    try:
        for step in range(steps):
            grads = make_inputs(K, step)
            for r in range(K):
                for i in range(len(shapes)):
                    dgrads[r][i].copy_(torch.from_numpy(grads[r][i]))
            packed = ox.aggregate_step(oracle, st, grads, bits, zero_thr, self_quant, v2_identity_at_k1=v2_identity)
            lib.step_group(aggs, [[t.data_ptr() for t in dgrads[r]] for r in range(K)])
            if (step + 1) % check_every and step != steps - 1:
                continue
            for r in range(K):
                for i, (M, N) in enumerate(shapes):
                    G.assert_same_bits(G.host(dgrads[r][i]), grads[r][i], f"step {step} rank {r} tensor {i} aggregate")
                    if v2_identity and K == 1:
                        continue
                    res = torch.empty((N, M), dtype=torch.float32, device=G.DEV)
                    aggs[r].copy_residual(i, 0, res.data_ptr())
                    G.assert_same_bits(G.host(res), st.res[r][i], f"step {step} rank {r} tensor {i} residual")
                    n = ox.stripe(N, r, K)[1]
                    if n and K > 1:
                        sres = torch.empty((n, M), dtype=torch.float32, device=G.DEV)
                        aggs[r].copy_residual(i, 1, sres.data_ptr())
                        G.assert_same_bits(G.host(sres), st.sres[r][i], f"step {step} rank {r} tensor {i} stripe residual")
                    if packed is not None:
                        pk = torch.zeros(lib.packed_bytes(M, N, bits), dtype=torch.uint8, device=G.DEV)
                        aggs[r].copy_packed(i, pk.data_ptr())
                        G.assert_same_bits(G.host(pk), packed[r][i], f"step {step} rank {r} tensor {i} gathered packed words")
        for a in aggs:
            a.check()  # no bounded wait gave up
    finally:
        for a in aggs:
            a.destroy()
        for c in comms:
            c.destroy()


@pytest.mark.parametrize("K", [2, 3, 8])
@pytest.mark.parametrize("bits,zero_thr,self_quant", [(1, True, True), (1, True, False), (4, True, True)])
def test_peer_memory_exchange_bit_exact(G, oracle_port, K, bits, zero_thr, self_quant):
    """The exchange without collectives: the quantize kernel stores packed columns straight into their owner's receive
    slot and the owner's kernel stores its result into every rank's gather slot (here all windows are on one device, so
    the "peer" pointers are ordinary ones and the flag waits never spin: this checks routing, offsets and the protocol's
    bookkeeping; tests/test_gpu_multi.py runs it across GPUs)."""
    run_group(G, oracle_port, mg.EXCHANGE_SHAPES, K, bits, zero_thr, self_quant, 4, mg.exchange_inputs, peer=True)


def test_peer_memory_exchange_speech_shaped(G, oracle_port):
    run_group(G, oracle_port, SPEECH_SMALL, 4, 1, True, True, 12, speech_inputs, check_every=6, peer=True)


@pytest.mark.parametrize("chunks", [1, 3, 16])
def test_host_buffer_aggregator_pipelined(G, oracle_port, chunks):
    """qagg_hagg_*: gradients in pinned host memory, chunks of tensors pipelined over streams; one rank (V1 round trip).
    Results and the carried residuals (three steps) must equal the oracle's bit for bit, whatever the chunking."""
    from cntk_b200 import lib
    comm = lib.Comm.create(None, 0, 1, 0)
    h = lib.HostAggregator(comm, SPEECH_SMALL, 1, chunks=chunks)
    assert 1 <= h.chunks <= min(chunks, len(SPEECH_SMALL))
    st = ox.ExchangeState(SPEECH_SMALL, 1)
    host = [torch.empty((N, M), dtype=torch.float32).pin_memory() for (M, N) in SPEECH_SMALL]
    try:
        for step in range(3):
            grads = speech_inputs(1, step)
            for t, a in zip(host, grads[0]):
                t.copy_(torch.from_numpy(a))
            ox.aggregate_step(oracle_port, st, grads, 1)
            h.step([t.data_ptr() for t in host])
            for i in range(len(SPEECH_SMALL)):
                G.assert_same_bits(host[i].numpy(), grads[0][i], f"chunks {chunks} step {step} tensor {i}")
        h.check()
    finally:
        h.destroy()
        comm.destroy()


def test_bounded_wait_gives_up_and_reports(G):
    """Failure detection without a GPU fault: a wait on a flag that nothing sets runs out of polls, records it in the
    status word and returns; the context stays usable and a later wait on flags that ARE set passes."""
    from cntk_b200 import lib
    flags = torch.zeros(8, dtype=torch.int32, device=G.DEV)
    status = torch.zeros(1, dtype=torch.int32, device=G.DEV)
    lib.wait_flags(flags.data_ptr(), 4, 1, 1, 2000, status.data_ptr())
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    status.zero_()
    flags.fill_(7)
    lib.wait_flags(flags.data_ptr(), 4, 1, 7, 2000, status.data_ptr())
    lib.wait_flags(flags.data_ptr(), 4, 1, 5, 2000, status.data_ptr())
    torch.cuda.synchronize()
    assert int(status.item()) == 0


def test_streaming_kernel_wait_gives_up_and_reports(G):
    """The streaming quantize kernel waits on mbarriers for its copies into shared memory; every such wait is bounded.
    Here the kernel's own wait runs on a barrier that nothing completes: it gives up after the given number of polls, sets
    bit 1 of the status word and returns; a second wait in the same kernel returns at once; the context stays usable."""
    from cntk_b200 import lib
    status = torch.zeros(1, dtype=torch.int32, device=G.DEV)
    cycles = torch.zeros(2, dtype=torch.int64, device=G.DEV)
    lib.stream_wait_selftest(200, status.data_ptr(), cycles.data_ptr())
    torch.cuda.synchronize()
    assert int(status.item()) == 2
    first, second = [int(x) for x in cycles.tolist()]
    assert first > 200 * 100, "200 polls with a sleep in between take a while"
    assert second < first // 20, "once a wait has run out, later waits do not wait again"
    # the device is fine afterwards
    assert int((torch.ones(4, device=G.DEV) * 2).sum().item()) == 8


@pytest.mark.parametrize("K", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("bits,zero_thr", [(1, True), (1, False), (2, True), (4, True)])
@pytest.mark.parametrize("self_quant", [True, False])
def test_small_exchange_bit_exact(G, oracle_port, K, bits, zero_thr, self_quant):
    """The fixture gradient set (includes N < K and single-column tensors), three steps."""
    run_group(G, oracle_port, mg.EXCHANGE_SHAPES, K, bits, zero_thr, self_quant, mg.EXCHANGE_STEPS, mg.exchange_inputs)


def test_small_exchange_matches_committed_fixture(G, oracle_port):
    """Final aggregate of the K=2 and K=3 fixtures written by tests/golden/make_golden.py from the reference build."""
    small = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_small.npz"))
    from cntk_b200 import lib
    for K in (2, 3):
        comms = lib.Comm.local_group(K, 0)
        aggs = [lib.Aggregator(c, mg.EXCHANGE_SHAPES, 1) for c in comms]
        dgrads = None
        for step in range(mg.EXCHANGE_STEPS):
            grads = mg.exchange_inputs(K, step)
            dgrads = [[G.dev(g) for g in grads[r]] for r in range(K)]
            lib.step_group(aggs, [[t.data_ptr() for t in dgrads[r]] for r in range(K)])
        key = f"K{K}_b1_z1_s1"
        for i, (M, N) in enumerate(mg.EXCHANGE_SHAPES):
            G.assert_same_bits(G.host(dgrads[0][i]), small[f"exchange_{key}_final_agg_t{i}"], f"{key} tensor {i}")
            pk = torch.zeros(lib.packed_bytes(M, N, 1), dtype=torch.uint8, device=G.DEV)
            aggs[0].copy_packed(i, pk.data_ptr())
            G.assert_same_bits(G.host(pk), small[f"exchange_{key}_final_packed_t{i}"], f"{key} packed {i}")
        for a in aggs:
            a.destroy()
        for c in comms:
            c.destroy()


def test_v2_single_worker_is_identity(G, oracle_port):
    run_group(G, oracle_port, mg.EXCHANGE_SHAPES, 1, 1, True, True, 2, mg.exchange_inputs, v2_identity=True)


# speech-DNN-shaped gradient set scaled down 8x per dimension (same structure: weights + bias vectors)
SPEECH_SMALL = [(256, 54)] + [(256, 256)] * 6 + [(1163, 256)] + [(256, 1)] * 7 + [(1163, 1)]


def speech_inputs(K, step):
    return [[mg.normal_input(M, N, 1e-3, 1000 * r + step + 7919 * i) for i, (M, N) in enumerate(SPEECH_SMALL)] for r in range(K)]


@pytest.mark.parametrize("K", [1, 2, 4, 8])
def test_speech_shaped_set_100_steps_bit_exact(G, oracle_port, K):
    """1-bit SGD aggregation of a speech-DNN-shaped set, residual carried over 100 steps, seed = 1000*rank + step.
    Checked every 25 steps and at the end: aggregated gradients, both residual sets and packed words, all bit-exact."""
    run_group(G, oracle_port, SPEECH_SMALL, K, 1, True, True, 100, speech_inputs, check_every=25)


RESNET_SMALL = [(64, 147), (64, 64), (64, 576), (256, 64), (128, 1152), (512, 128), (64, 1), (256, 1), (512, 1), (100, 512), (100, 1)]


def resnet_inputs(K, step):
    out = []
    for r in range(K):
        row = []
        for i, (M, N) in enumerate(RESNET_SMALL):
            rng = np.random.default_rng(500000 + 1000 * r + step + 104729 * i)
            row.append(rng.laplace(0.0, 1e-4, size=(N, M)).astype(np.float32))
        out.append(row)
    return out


@pytest.mark.parametrize("K", [2, 8])
def test_resnet_shaped_set_4bit(G, oracle_port, K):
    """4-bit aggregation of conv-shaped tensors ([out_ch, in_ch*kh*kw]: few rows, many columns) plus BN vectors,
    Laplace(0, 1e-4) values, 20 steps."""
    run_group(G, oracle_port, RESNET_SMALL, K, 4, True, True, 20, resnet_inputs, check_every=10)


LSTM_SMALL = [(5000, 64), (512, 256), (512, 1), (512, 256), (512, 1), (64, 5000)]


def lstm_inputs(K, step):
    out = []
    for r in range(K):
        row = []
        for i, (M, N) in enumerate(LSTM_SMALL):
            rng = np.random.default_rng(900000 + 1000 * r + step + 15485863 * i)
            a = (rng.standard_normal((N, M)) * 5e-4).astype(np.float32)
            if i == 0:
                zero_cols = rng.random(N) < 0.9  # 90% of the embedding's columns exactly zero
                a[zero_cols] = 0.0
            row.append(a)
        out.append(row)
    return out


@pytest.mark.parametrize("K", [2, 4])
def test_lstm_shaped_set_ragged(G, oracle_port, K):
    """Tall embedding with 90% all-zero columns, wide softmax, bias vectors; 1 bit, 10 steps."""
    run_group(G, oracle_port, LSTM_SMALL, K, 1, True, True, 10, lstm_inputs, check_every=5)


@pytest.mark.parametrize("knob,value", [("QAGG_STREAM", "0"), ("QAGG_OWNER", "0"), ("QAGG_OWNER_SPLIT", "0"), ("QAGG_TALL_ROWS", "1000"),
                                        ("QAGG_TALL_ROWS", "200")])
def test_kernel_choice_knob_changes_no_result(G, oracle_port, knob, value, monkeypatch):
    """Tuning knobs read when an aggregator is created: QAGG_STREAM=0 = resident-column kernels only (plain residuals),
    QAGG_OWNER=0 = resident-column kernel for the owner's reduce-requantize only (plain stripe residuals),
    QAGG_OWNER_SPLIT=0 = one form and one walk launch instead of the tall matrices' walk on a stream of its own,
    QAGG_TALL_ROWS=n = matrices of n rows or more leave the streaming quantize kernel for the form + walk pair (default
    16384; here 1000 takes the tall matrix of the set, 200 all but the smallest, so the pair runs beside the streaming
    kernel and alone).  Either way
    aggregates, both residual sets and the gathered packed words stay bit-identical to the oracle (the default -- streaming
    quantize kernel, form + walk owner kernels, both residual sets deferred -- is what every other 1-bit zero-threshold
    test in this file runs)."""
    monkeypatch.setenv(knob, value)
    run_group(G, oracle_port, SPEECH_SMALL, 3, 1, True, True, 6, speech_inputs, check_every=3)
    run_group(G, oracle_port, mg.EXCHANGE_SHAPES, 2, 1, True, False, 4, mg.exchange_inputs, peer=True)
    if knob == "QAGG_TALL_ROWS":
        run_group(G, oracle_port, SPEECH_SMALL, 1, 1, True, True, 4, speech_inputs)
        run_group(G, oracle_port, LSTM_SMALL, 4, 1, True, True, 4, lstm_inputs, peer=True)


@pytest.mark.parametrize("K,peer", [(1, False), (2, False), (3, True), (8, True)])
def test_step_with_header_sums_it_in_rank_order(G, K, peer):
    """qagg_agg_step_group_header: the DistGradHeader values ride with the step and come back summed over the ranks in
    ascending rank order (exactly, as doubles); the gradients are aggregated as without a header."""
    from cntk_b200 import lib
    shapes = [(64, 9), (33, 2)]
    comms = lib.Comm.local_group(K, 0)
    aggs = [lib.Aggregator(c, shapes, 1) for c in comms]
    plain = [lib.Aggregator(c, shapes, 1) for c in comms]
    if peer:
        for group in (aggs, plain):
            hs = [a.peer_handle() for a in group]
            for a in group:
                a.enable_peer(hs)
    rng = np.random.default_rng(5)
    try:
        for step in range(3):
            n = 3 + 2 * step  # criterion, two sample counts, then evaluation pairs
            headers = [[float(rng.standard_normal() * 10.0 ** int(rng.integers(-3, 6))) for _ in range(n)] for _ in range(K)]
            g = [[torch.from_numpy((rng.standard_normal((N, M)) * 1e-3).astype(np.float32)).to(G.DEV) for (M, N) in shapes] for _ in range(K)]
            g2 = [[t.clone() for t in row] for row in g]
            lib.step_group(aggs, [[t.data_ptr() for t in row] for row in g], headers=headers)
            lib.step_group(plain, [[t.data_ptr() for t in row] for row in g2])
            expect = []
            for i in range(n):
                s = headers[0][i]
                for r in range(1, K):
                    s = s + headers[r][i]
                expect.append(s)
            for r in range(K):
                assert aggs[r].header_result(n) == expect, f"step {step} rank {r}"
                for a, b in zip(g[r], g2[r]):
                    assert torch.equal(a.view(torch.int32), b.view(torch.int32))
        with pytest.raises(lib.QaggError):
            lib.step_group(aggs, [[t.data_ptr() for t in row] for row in g], headers=[[0.0] * 65] * K)
    finally:
        for a in aggs + plain:
            a.destroy()
        for c in comms:
            c.destroy()


@pytest.mark.parametrize("keep_plain", [False, True])
def test_caller_owned_residual_buffers(G, oracle_port, keep_plain):
    """qagg_agg_bind_residuals: the error-feedback state lives in buffers the caller owns (the V2 interface's
    valueQuantizationResidues / stripeQuantizationResidues).  Their content at bind time is taken as plain residuals; with
    keep_plain they hold plain residuals after every step, otherwise after qagg_agg_materialize_residuals; zeroing them from
    outside and binding again starts over."""
    from cntk_b200 import lib
    K, bits = 3, 1
    shapes = [(256, 40), (100, 7), (256, 1)]
    comms = lib.Comm.local_group(K, 0)
    aggs = [lib.Aggregator(c, shapes, bits) for c in comms]
    rng = np.random.default_rng(8)
    st = ox.ExchangeState(shapes, K)
    # start from non-zero residuals, to show that bound content is used
    for r in range(K):
        for i, (M, N) in enumerate(shapes):
            st.res[r][i][...] = (rng.standard_normal((N, M)) * 1e-4).astype(np.float32)
            st.sres[r][i][...] = (rng.standard_normal(st.sres[r][i].shape) * 1e-4).astype(np.float32)
    vres = [[torch.from_numpy(st.res[r][i].copy()).to(G.DEV) for i in range(len(shapes))] for r in range(K)]
    sres = [[torch.from_numpy(st.sres[r][i].copy()).to(G.DEV) if st.sres[r][i].size else None for i in range(len(shapes))] for r in range(K)]

    def bind():
        for r in range(K):
            aggs[r].bind_residuals([t.data_ptr() for t in vres[r]], [t.data_ptr() if t is not None else 0 for t in sres[r]], keep_plain)

    def compare(what):
        for r in range(K):
            if not keep_plain:
                aggs[r].materialize_residuals()
            torch.cuda.synchronize()
            for i in range(len(shapes)):
                G.assert_same_bits(G.host(vres[r][i]), st.res[r][i], f"{what}: rank {r} tensor {i} residual buffer")
                if sres[r][i] is not None:
                    G.assert_same_bits(G.host(sres[r][i]), st.sres[r][i], f"{what}: rank {r} tensor {i} stripe residual buffer")

    try:
        bind()
        for step in range(4):
            grads = [[(rng.standard_normal((N, M)) * 1e-3).astype(np.float32) for (M, N) in shapes] for _ in range(K)]
            dg = [[torch.from_numpy(a).to(G.DEV) for a in grads[r]] for r in range(K)]
            ox.aggregate_step(oracle_port, st, grads, bits)
            lib.step_group(aggs, [[t.data_ptr() for t in dg[r]] for r in range(K)])
            torch.cuda.synchronize()
            for r in range(K):
                for i in range(len(shapes)):
                    G.assert_same_bits(G.host(dg[r][i]), grads[r][i], f"step {step} rank {r} tensor {i} aggregate")
            if step in (1, 3):
                compare(f"step {step}")
            if step == 1:
                # the caller zeroes its buffers (a checkpoint) and tells the aggregator by binding them again
                for r in range(K):
                    for t in vres[r] + [x for x in sres[r] if x is not None]:
                        t.zero_()
                st.reset()
                bind()
    finally:
        for a in aggs:
            a.destroy()
        for c in comms:
            c.destroy()


def _same_or_both_nan(a, b, what):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    assert a.shape == b.shape, what
    ok = (a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))
    assert ok.all(), f"{what}: {int((~ok).sum())} of {a.size} elements differ (NaN positions must agree, everything else bit for bit)"


@pytest.mark.parametrize("K,tall_rows,zero_thr", [(1, None, True), (3, None, True), (3, "200", True), (2, "0", True), (2, None, False)])
def test_nan_and_infinities_spread_like_the_reference(G, oracle_port, K, tall_rows, zero_thr, monkeypatch):
    """A NaN (or a pair of opposite infinities) in a gradient makes its column's range NaN in the reference
    (ColumnQuantizer.h:247-316: the value lands in the upper partition sum), its bit 0, and its residual NaN from then on;
    a lone infinity gives an infinite range.  Streaming kernel, form + walk pair (QAGG_TALL_ROWS) and owner kernels must
    spread them exactly the same way: NaN where the oracle has NaN, every other value and every packed bit identical.  Also
    with the mean as threshold (resident-column kernels), where a NaN makes the column's mean NaN.  (Multi-bit modes are left
    out: there the reference converts NaN to an integer, which C leaves undefined.)"""
    from cntk_b200 import lib
    if tall_rows is not None:
        monkeypatch.setenv("QAGG_TALL_ROWS", tall_rows)
    shapes = [(256, 24), (1163, 5), (64, 3)]
    comms = lib.Comm.local_group(K, 0)
    aggs = [lib.Aggregator(c, shapes, 1, (lib.ZERO_THRESHOLD if zero_thr else 0) | lib.SELF_QUANTIZED) for c in comms]
    st = ox.ExchangeState(shapes, K)
    rng = np.random.default_rng(77 + K)
    try:
        for step in range(3):
            grads = [[(rng.standard_normal((N, M)) * 1e-3).astype(np.float32) for (M, N) in shapes] for _ in range(K)]
            if step == 0:
                grads[0][0][2, 17] = np.nan                 # one NaN in column 2 of tensor 0
                grads[K - 1][1][1, 500] = np.inf            # a lone +inf
                grads[0][1][3, 7] = np.inf                  # +inf and -inf in one column
                grads[0][1][3, 900] = -np.inf
                grads[K - 1][2][0, :] = np.nan              # a whole column of NaN
            dg = [[G.dev(a) for a in grads[r]] for r in range(K)]
            with np.errstate(invalid="ignore", over="ignore"):
                packed = ox.aggregate_step(oracle_port, st, grads, 1, zero_thr)
            lib.step_group(aggs, [[t.data_ptr() for t in dg[r]] for r in range(K)])
            torch.cuda.synchronize()
            for r in range(K):
                for i, (M, N) in enumerate(shapes):
                    what = f"K {K} zero threshold {zero_thr} step {step} rank {r} tensor {i}"
                    _same_or_both_nan(G.host(dg[r][i]), grads[r][i], "aggregate: " + what)
                    res = torch.empty((N, M), dtype=torch.float32, device=G.DEV)
                    aggs[r].copy_residual(i, 0, res.data_ptr())
                    _same_or_both_nan(G.host(res), st.res[r][i], "residual: " + what)
                    pk = torch.zeros(lib.packed_bytes(M, N, 1), dtype=torch.uint8, device=G.DEV)
                    aggs[r].copy_packed(i, pk.data_ptr())
                    C = lib.packed_bytes(M, 1, 1)
                    got = G.host(pk).reshape(N, C)
                    want = packed[r][i].reshape(N, C)
                    assert np.array_equal(got[:, 8:], want[:, 8:]), "packed bits: " + what
                    _same_or_both_nan(got[:, :8].copy().view(np.float32), want[:, :8].copy().view(np.float32), "column ranges: " + what)
        for a in aggs:
            a.check()
    finally:
        for a in aggs:
            a.destroy()
        for c in comms:
            c.destroy()


def test_form_walk_quantize_path_with_caller_owned_residuals(G, oracle_port, monkeypatch):
    """The form + walk pair as the quantize kernel (QAGG_TALL_ROWS low enough to take every matrix of the set) keeps its
    state in caller-owned residual buffers like the streaming kernel does: bound content is used, the buffers hold plain
    residuals after qagg_agg_materialize_residuals, zeroing and binding again starts over."""
    monkeypatch.setenv("QAGG_TALL_ROWS", "100")
    test_caller_owned_residual_buffers(G, oracle_port, False)
