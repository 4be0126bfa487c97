"""One rank of the multi-GPU parity check; launched by tests/test_gpu_multi.py (and runnable by hand) as
    python -m torch.distributed.run --nnodes=1 --nproc-per-node K --master-addr 127.0.0.1 --master-port P tests/multi_gpu_check.py

Every rank builds all K ranks' seeded gradients, runs the CPU restatement of the exchange for all K ranks, runs ITS
aggregator step over NCCL on its own GPU, and compares its aggregated gradients, residuals, stripe residuals and gathered
packed words with the oracle's rank-r results, bit for bit, over several steps."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
import make_golden as mg  # noqa: E402

from cntk_b200 import lib  # noqa: E402
from oracle import backend, exchange  # noqa: E402

SHAPES = [(256, 54), (256, 256), (1163, 256), (256, 1), (1163, 1), (64, 147), (70, 3), (5, 16), (2048, 40)]


def inputs(K, step):
    return [[mg.normal_input(M, N, 1e-3, 1000 * r + step + 7919 * i) for i, (M, N) in enumerate(SHAPES)] for r in range(K)]


def run_checks(comm, rank, K, dev):
    """All checks of this module on an existing communicator (torch.distributed must be initialised: it carries the
    peer handles and the barriers).  Raises AssertionError on the first differing byte; returns the number of
    (configuration, step) pairs compared."""
    be = backend.OracleBackend()
    compared = 0
    # the communicator's own collectives: sum of rank-dependent doubles (exact) and the barrier
    vals = comm.allreduce_f64([float(rank + 1), 0.5 * rank, 2.0 ** rank, -1.0])
    assert vals == [K * (K + 1) / 2.0, 0.5 * K * (K - 1) / 2.0, float(2 ** K - 1), -float(K)], f"rank {rank}: allreduce_f64 gave {vals}"
    comm.barrier()
    # creation handshake: one rank asks for a different first tensor -> EVERY rank's creation fails, with a state error
    if K > 1:
        odd = [(SHAPES[0][0] + 1, SHAPES[0][1])] + list(SHAPES[1:]) if rank == K - 1 else SHAPES
        try:
            lib.Aggregator(comm, odd, 1)
            raised = False
        except lib.QaggError as e:
            raised = "do not describe the same exchange" in str(e)
        assert raised, f"rank {rank}: mismatched shapes were not refused at creation"
        try:
            lib.Aggregator(comm, SHAPES, 1 if rank else 2)
            raised = False
        except lib.QaggError:
            raised = True
        assert raised, f"rank {rank}: mismatched bit widths were not refused at creation"
        comm.barrier()
        # a rank that skips a step (between steps, nothing of its own in flight): the others' bounded flag waits give up
        # after the set number of polls, their kernels end normally, qagg_agg_check reports the time-out on the host and
        # keeps reporting it until it is cleared; the aggregator is then dropped (the ranks' step counts differ)
        agg = lib.Aggregator(comm, SHAPES, 1)
        mine = torch.frombuffer(bytearray(agg.peer_handle()), dtype=torch.uint8).to(dev)
        allh = [torch.zeros_like(mine) for _ in range(K)]
        dist.all_gather(allh, mine)
        agg.enable_peer([bytes(h.cpu().numpy().tobytes()) for h in allh])
        agg.set_wait_limit(20000)
        dg = [torch.zeros((N, M), dtype=torch.float32, device=dev) for (M, N) in SHAPES]
        if rank != K - 1:
            agg.step([t.data_ptr() for t in dg], torch.cuda.current_stream().cuda_stream)
            for attempt in range(2):
                try:
                    agg.check(torch.cuda.current_stream().cuda_stream)
                    reported = False
                except lib.QaggError as e:
                    reported = "wait" in str(e)
                assert reported, f"rank {rank}: a peer that skipped the step was not reported (attempt {attempt})"
            agg.clear_status(torch.cuda.current_stream().cuda_stream)
            agg.check(torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        comm.barrier()
        agg.destroy()
    for bits, zero_thr, self_q, peer in ((1, True, True, False), (1, False, True, False), (4, True, True, False), (1, True, False, False),
                                         (1, True, True, True), (4, True, True, True), (1, True, False, True)):
        flags = (lib.ZERO_THRESHOLD if zero_thr else 0) | (lib.SELF_QUANTIZED if self_q else 0)
        agg = lib.Aggregator(comm, SHAPES, bits, flags)
        if peer:
            # exchange the IPC handles of the ranks' windows, then switch the aggregator to the peer-memory path
            mine = torch.frombuffer(bytearray(agg.peer_handle()), dtype=torch.uint8).to(dev)
            allh = [torch.zeros_like(mine) for _ in range(K)]
            dist.all_gather(allh, mine)
            agg.enable_peer([bytes(h.cpu().numpy().tobytes()) for h in allh])
        st = exchange.ExchangeState(SHAPES, K)
        dg = [torch.zeros((N, M), dtype=torch.float32, device=dev) for (M, N) in SHAPES]
        for step in range(4):
            grads = inputs(K, step)
            for t, a in zip(dg, grads[rank]):
                t.copy_(torch.from_numpy(a))
            packed = exchange.aggregate_step(be, st, grads, bits, zero_thr, self_q)
            # the step carries a DistGradHeader: rank-dependent doubles, summed in rank order (exact in double)
            hdr = lambda r: [1.5 * (r + 1) + step, float(100 * r + 7), float(r), 0.125 * (r + 3), float(3 * r + step)]
            agg.step_header([t.data_ptr() for t in dg], hdr(rank), torch.cuda.current_stream().cuda_stream)
            got = agg.header_result(5, torch.cuda.current_stream().cuda_stream)
            want = [sum(hdr(r)[k] for r in range(K)) for k in range(5)]
            assert got == want, f"header sum: bits {bits} peer {peer} step {step} rank {rank}: {got} != {want}"
            torch.cuda.synchronize()
            for i, (M, N) in enumerate(SHAPES):
                what = f"bits {bits} zero {zero_thr} self {self_q} peer {peer} step {step} rank {rank} tensor {i}"
                assert np.array_equal(dg[i].cpu().numpy().view(np.uint32), grads[rank][i].view(np.uint32)), "aggregate: " + what
                r_ = torch.empty((N, M), dtype=torch.float32, device=dev)
                agg.copy_residual(i, 0, r_.data_ptr())
                torch.cuda.synchronize()
                assert np.array_equal(r_.cpu().numpy().view(np.uint32), st.res[rank][i].view(np.uint32)), "residual: " + what
                n = exchange.stripe(N, rank, K)[1]
                if n:
                    s_ = torch.empty((n, M), dtype=torch.float32, device=dev)
                    agg.copy_residual(i, 1, s_.data_ptr())
                    torch.cuda.synchronize()
                    assert np.array_equal(s_.cpu().numpy().view(np.uint32), st.sres[rank][i].view(np.uint32)), "stripe residual: " + what
                pk = torch.zeros(lib.packed_bytes(M, N, bits), dtype=torch.uint8, device=dev)
                agg.copy_packed(i, pk.data_ptr())
                torch.cuda.synchronize()
                assert np.array_equal(pk.cpu().numpy(), packed[rank][i]), "packed words: " + what
            compared += 1
        agg.check()
        dist.barrier()  # nobody unmaps a window that a peer may still be writing to
        agg.destroy()
    # the unquantized fp32 arm: peer-window kernels (rank-ordered sum: bit-exact) and the ncclAllReduce baseline (close)
    for peer in (True, False):
        dagg = lib.DenseAggregator(comm, SHAPES)
        if peer:
            mine = torch.frombuffer(bytearray(dagg.peer_handle()), dtype=torch.uint8).to(dev)
            allh = [torch.zeros_like(mine) for _ in range(K)]
            dist.all_gather(allh, mine)
            dagg.enable_peer([bytes(h.cpu().numpy().tobytes()) for h in allh])
        dg = [torch.zeros((N, M), dtype=torch.float32, device=dev) for (M, N) in SHAPES]
        for step in range(3):
            grads = inputs(K, step)
            for t, a in zip(dg, grads[rank]):
                t.copy_(torch.from_numpy(a))
            want = exchange.dense_sum(grads)
            dagg.step([t.data_ptr() for t in dg], torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            for i in range(len(SHAPES)):
                got = dg[i].cpu().numpy()
                if peer:
                    assert np.array_equal(got.view(np.uint32), want[i].view(np.uint32)), f"dense sum: step {step} rank {rank} tensor {i}"
                else:
                    assert np.allclose(got, want[i], rtol=1e-5, atol=1e-9), f"dense sum (nccl): step {step} rank {rank} tensor {i}"
            compared += 1
        dagg.check()
        dist.barrier()
        dagg.destroy()
    # host-buffer aggregator, chunks pipelined over streams, peer-memory exchange per chunk
    hagg = lib.HostAggregator(comm, SHAPES, 1, chunks=3)
    mine = torch.frombuffer(bytearray(hagg.peer_handles()), dtype=torch.uint8).to(dev)
    allh = [torch.zeros_like(mine) for _ in range(K)]
    dist.all_gather(allh, mine)
    hagg.enable_peer([bytes(h.cpu().numpy().tobytes()) for h in allh])
    st = exchange.ExchangeState(SHAPES, K)
    host = [torch.empty((N, M), dtype=torch.float32).pin_memory() for (M, N) in SHAPES]
    for step in range(3):
        grads = inputs(K, step)
        for t, a in zip(host, grads[rank]):
            t.copy_(torch.from_numpy(a))
        exchange.aggregate_step(be, st, grads, 1)
        hagg.step([t.data_ptr() for t in host])
        for i in range(len(SHAPES)):
            assert np.array_equal(host[i].numpy().view(np.uint32), grads[rank][i].view(np.uint32)), f"host aggregator: step {step} rank {rank} tensor {i}"
        compared += 1
    hagg.check()
    dist.barrier()
    hagg.destroy()
    dist.barrier()
    return compared


def main():
    rank, local, K = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    idt = torch.zeros(lib.UNIQUE_ID_BYTES, dtype=torch.uint8, device=dev)
    if rank == 0:
        idt.copy_(torch.frombuffer(bytearray(lib.unique_id()), dtype=torch.uint8))
    dist.broadcast(idt, 0)
    comm = lib.Comm.create(bytes(idt.cpu().numpy().tobytes()), rank, K, local)
    run_checks(comm, rank, K, dev)
    comm.destroy()
    dist.destroy_process_group()
    if rank == 0:
        print(f"multi-GPU parity ok on {K} ranks")


if __name__ == "__main__":
    main()
