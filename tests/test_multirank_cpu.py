"""World-size-2 (and 3) `gloo` tests of the host side of the exchange, on CPU.

Each process is one rank.  The CPU oracle stands in for the device kernels (quantize / unquantize of stripes), but
every byte that crosses the process boundary is laid out by the product's own wire plan (qagg_plan_* in libqagg.so):
one message per peer holding that peer's stripes of all tensors, then an all-gather of equal-sized padded slots.  The
per-rank results must equal the single-process restatement of the exchange (oracle/exchange.py), which proves that the
plan's offsets and sizes describe the reference's stripes exactly, including N < K and single-column tensors."""
import os
import socket
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as mg  # noqa: E402

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, K, port, bits, steps, q):
    try:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=K)
        from cntk_b200 import lib
        from oracle import backend, exchange
        be = backend.OracleBackend()
        shapes = mg.EXCHANGE_SHAPES
        T = len(shapes)
        plan = lib.Plan(rank, K, shapes, bits)
        C = [lib.packed_col_bytes(M, bits) for (M, N) in shapes]
        # reference result: all K ranks simulated in this process
        ref_state = exchange.ExchangeState(shapes, K)
        # this rank's own state
        res = [np.zeros((N, M), np.float32) for (M, N) in shapes]
        sres = [np.zeros((lib.stripe(N, rank, K)[1], M), np.float32) for (M, N) in shapes]
        for step in range(steps):
            all_grads = mg.exchange_inputs(K, step)
            ref_grads = [[a.copy() for a in g] for g in all_grads]
            exchange.aggregate_step(be, ref_state, ref_grads, bits)
            grads = [a.copy() for a in all_grads[rank]]
            # K1: quantize everything, scatter columns into per-owner regions
            regions = [np.zeros(plan.region_bytes(p), np.uint8) for p in range(K)]
            for i, (M, N) in enumerate(shapes):
                packed = np.zeros(N * C[i], np.uint8)
                be.quantize(grads[i], res[i], res[i], packed, bits, True)
                for p in range(K):
                    s, n = lib.stripe(N, p, K)
                    o = plan.tensor_offset(p, i)
                    regions[p][o:o + n * C[i]] = packed[s * C[i]:(s + n) * C[i]]
            # X1: one message per peer
            recv = [np.zeros(plan.region_bytes(rank), np.uint8) for _ in range(K)]
            recv[rank][:] = regions[rank]
            reqs = []
            for p in range(K):
                if p == rank:
                    continue
                if regions[p].size:
                    reqs.append(dist.isend(torch.from_numpy(regions[p]), p))
                if recv[p].size:
                    reqs.append(dist.irecv(torch.from_numpy(recv[p]), p))
            for r_ in reqs:
                r_.wait()
            # K2: own stripe first, then sources by ascending rank; requantize into the gather slot
            slot = plan.gather_slot_bytes
            mine = np.zeros(slot, np.uint8)
            for i, (M, N) in enumerate(shapes):
                s, n = lib.stripe(N, rank, K)
                if n == 0:
                    continue
                o = plan.tensor_offset(rank, i)
                agg = np.zeros((n, M), np.float32)
                be.unquantize(recv[rank][o:o + n * C[i]], agg, bits, add=False)
                for src in range(K):
                    if src != rank:
                        be.unquantize(recv[src][o:o + n * C[i]], agg, bits, add=True)
                out = np.zeros(n * C[i], np.uint8)
                be.quantize(agg, sres[i], sres[i], out, bits, True)
                mine[o:o + n * C[i]] = out
            # X2: all-gather of equal-sized slots
            gathered = [torch.zeros(slot, dtype=torch.uint8) for _ in range(K)]
            dist.all_gather(gathered, torch.from_numpy(mine))
            # K3
            for i, (M, N) in enumerate(shapes):
                full = np.zeros(N * C[i], np.uint8)
                for p in range(K):
                    s, n = lib.stripe(N, p, K)
                    o = plan.tensor_offset(p, i)
                    full[s * C[i]:(s + n) * C[i]] = gathered[p].numpy()[o:o + n * C[i]]
                be.unquantize(full, grads[i], bits, add=False)
                assert np.array_equal(grads[i].view(np.uint32), ref_grads[rank][i].view(np.uint32)), (step, i)
                assert np.array_equal(res[i].view(np.uint32), ref_state.res[rank][i].view(np.uint32)), (step, i)
                assert np.array_equal(sres[i].view(np.uint32), ref_state.sres[rank][i].view(np.uint32)), (step, i)
        plan.destroy()
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # report instead of hanging the peers
        q.put((rank, f"{type(e).__name__}: {e}"))
        raise


@pytest.mark.parametrize("K,bits", [(2, 1), (3, 1), (2, 4)])
def test_wire_plan_across_processes(K, bits):
    from cntk_b200 import build
    build.build()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, K, port, bits, 2, q)) for r in range(K)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    results = {}
    while not q.empty():
        r, msg = q.get()
        results[r] = msg
    for p in procs:
        if p.is_alive():
            p.kill()
    assert results == {r: "ok" for r in range(K)}, results


def test_plan_properties():
    """Regions tile every packed matrix exactly once; offsets are 16-byte aligned; slots are equal and large enough."""
    from cntk_b200 import build, lib
    build.build()
    shapes = [(2048, 429), (9304, 2048), (2048, 1), (70, 3), (5, 16)]
    for K in (1, 2, 3, 8, 16):
        for bits in (1, 2, 4):
            plans = [lib.Plan(r, K, shapes, bits) for r in range(K)]
            for i, (M, N) in enumerate(shapes):
                C = lib.packed_col_bytes(M, bits)
                covered = 0
                for p in range(K):
                    s, n = lib.stripe(N, p, K)
                    assert s == covered
                    covered += n
                    off = plans[0].tensor_offset(p, i)
                    assert off % 16 == 0
                    nxt = plans[0].tensor_offset(p, i + 1) if i + 1 < len(shapes) else plans[0].region_bytes(p)
                    assert nxt - off >= n * C and nxt - off < n * C + 16
                assert covered == N
            for r in range(K):
                assert [plans[r].region_bytes(p) for p in range(K)] == [plans[0].region_bytes(p) for p in range(K)]
                assert plans[r].gather_slot_bytes >= max(plans[r].region_bytes(p) for p in range(K))
                assert plans[r].gather_slot_bytes % 256 == 0
            for p in plans:
                p.destroy()
