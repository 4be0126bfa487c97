"""One rank of the multi-GPU parity check; launched by tests/test_gpu_multi.py as
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
    be = backend.OracleBackend()
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
            agg.step([t.data_ptr() for t in dg], torch.cuda.current_stream().cuda_stream)
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
        agg.check()
        dist.barrier()  # nobody unmaps a window that a peer may still be writing to
        agg.destroy()
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
    hagg.check()
    dist.barrier()
    hagg.destroy()
    dist.barrier()
    comm.destroy()
    dist.destroy_process_group()
    if rank == 0:
        print(f"multi-GPU parity ok on {K} ranks")


if __name__ == "__main__":
    main()
