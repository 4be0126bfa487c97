#!/usr/bin/env python
"""Benchmark of the quantized gradient aggregation step (CNTK 1-bit SGD path) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload speech_dnn|...]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

A "step" is one AggregateGradients call over the whole gradient set of one rank (default: the speech-DNN set,
16 tensors, 45,122,648 fp32 values, 1 bit, zero threshold, residual carried from step to step).  Rank 0 prints ONE
JSON line.  `value` is fp32-gradient GB/s summed over ranks (4 * values * ranks / step time, step time = max over
ranks of the CUDA-event time of the step); `per_gpu_value` is the per-GPU figure the metric is named after.

--impl reference times the reference's own CPU quantizer (its headers compiled in place, oracle/_ref) driving the
restated exchange with one thread per simulated rank on this box's host cores, and prints the same line shape.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "1-bit aggregated fp32-grad GB/s per GPU (max over ranks) at 1/2/4/8 B200"
UNIT = "GB/s of fp32 gradient, summed over GPUs (per_gpu_value = per GPU)"


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock/throttle samples of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of the quantize kernel, from the ncu capture
# summarised in profiles/k_stream1_speech_dnn_1bit.md (same build, same workload); None where no capture exists
NCU_TRAFFIC_BYTES = {"speech_dnn": 502.62e6}


def get_shapes(name):
    from cntk_b200 import workloads as w
    table = {"speech_dnn": (w.speech_dnn, 1), "resnet50": (w.resnet50, 4), "lstm_lm": (w.lstm_lm, 1), "round_trip_2048": (w.round_trip_2048, 1)}
    fn, bits = table[name]
    return fn(), bits


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# ------------------------------------------------------------------------------------------------ reference arm
def cpu_reference_run(shapes, bits, K, steps, warmup, col_div):
    """Times the CPU checker (reference headers when built, else the C port) on the restated exchange with K simulated
    ranks, one host thread each.  Columns are divided by col_div to bound the run."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor
    from oracle import backend, exchange
    be = backend.best_backend()
    sub = [(m, max(1, n // col_div)) for (m, n) in shapes]
    cores = min(K, os.cpu_count() or 1)
    st = exchange.ExchangeState(sub, K)
    rngs = [np.random.default_rng(1000 * r) for r in range(K)]
    pool = [[(rngs[r].standard_normal((n, m), dtype=np.float32) * np.float32(1e-3)) for (m, n) in sub] for r in range(K)]
    V = sum(m * n for m, n in sub)
    times = []
    with ThreadPoolExecutor(max_workers=cores) as ex:
        for s in range(warmup + steps):
            grads = [[a.copy() for a in pool[r]] for r in range(K)]
            t0 = time.perf_counter()
            exchange.aggregate_step(be, st, grads, bits, True, True, executor=ex if K > 1 else None)
            dt = time.perf_counter() - t0
            if s >= warmup:
                times.append(dt)
    t = sum(times) / len(times)
    return {"gbs_total": 4.0 * V * K / t / 1e9, "ms_per_step": t * 1e3, "cores": cores, "kind": be.kind, "values_per_rank": V,
            "sample": f"{'all' if col_div == 1 else '1/' + str(col_div)} of the columns of every tensor ({V} values per rank), "
                      f"{steps} steps after {warmup} warm-up, {K} simulated rank(s) on {cores} host thread(s)"}


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    shapes, bits = get_shapes(args.workload)
    K = args.gpus
    # bound the run to a few minutes: one rank-step of the full speech set costs ~0.8 s on one core
    col_div = 1 if K == 1 else (2 if K == 2 else 4)
    steps = min(args.steps, 10)
    warm = min(args.warmup, 1)
    r = cpu_reference_run(shapes, bits, K, steps, warm, col_div)
    line = {"impl": "reference", "metric": METRIC, "value": r["gbs_total"], "unit": UNIT, "per_gpu_value": r["gbs_total"] / K,
            "n_gpus": K, "steps": steps, "warmup": warm, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "bits": bits, "values_per_rank": r["values_per_rank"], "ranks": K,
                       "note": "reference CPU quantizer (MatrixQuantizerCPU arithmetic) + restated striped exchange on host cores"},
            "cpu_baseline": {"value": r["gbs_total"], "unit": UNIT, "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]},
            "e2e": {"value": r["gbs_total"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------ our arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    from cntk_b200 import lib, workloads

    rank, local_rank, world = dist_env()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    shapes, bits = get_shapes(args.workload)
    V = workloads.total_values(shapes)
    K = world

    if K > 1:
        dist.init_process_group("nccl", device_id=dev)
        idt = torch.zeros(lib.UNIQUE_ID_BYTES, dtype=torch.uint8, device=dev)
        if rank == 0:
            idt.copy_(torch.frombuffer(bytearray(lib.unique_id()), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        uid = bytes(idt.cpu().numpy().tobytes())
    else:
        uid = None
    comm = lib.Comm.create(uid, rank, K, local_rank)
    agg = lib.Aggregator(comm, shapes, bits)
    exchange = "none (1 rank)"
    if K > 1:
        exchange = "nccl send/recv + all-gather"
        if args.exchange == "p2p":
            # stores into the peers' windows over NVLink instead of collectives; all ranks must agree, so the outcome of
            # the set-up is reduced over ranks before anyone uses it
            ok = 1
            try:
                mine = torch.frombuffer(bytearray(agg.peer_handle()), dtype=torch.uint8).to(dev)
                allh = [torch.zeros_like(mine) for _ in range(K)]
                dist.all_gather(allh, mine)
            except Exception:
                ok = 0
            okt = torch.tensor([ok], device=dev)
            dist.all_reduce(okt, op=dist.ReduceOp.MIN)
            if int(okt.item()):
                try:
                    agg.enable_peer([bytes(h.cpu().numpy().tobytes()) for h in allh])
                except Exception as e:  # cannot map peer memory here: every rank must fall back together
                    ok = 0
                    print(f"[rank {rank}] peer mapping failed: {e}", file=sys.stderr)
                okt = torch.tensor([ok], device=dev)
                dist.all_reduce(okt, op=dist.ReduceOp.MIN)
                if int(okt.item()):
                    exchange = "peer-memory stores over NVLink + flag hand-shake (no collective)"
                else:
                    raise SystemExit("peer mapping succeeded on some ranks only; rerun with --exchange nccl")

    def barrier():
        if K > 1:
            dist.barrier()

    # gradients: persistent buffers (as a trainer's are) refreshed between steps from a pool of pre-generated sets
    POOL = 3
    gen = torch.Generator(device=dev)
    pool = []
    for s in range(POOL):
        gen.manual_seed(1000 * rank + s)
        pool.append([torch.randn((n, m), generator=gen, device=dev, dtype=torch.float32) * 1e-3 for (m, n) in shapes])
    grads = [torch.empty((n, m), device=dev, dtype=torch.float32) for (m, n) in shapes]
    ptrs = [g.data_ptr() for g in grads]
    stream = torch.cuda.current_stream().cuda_stream

    def refresh(s):
        for g, p in zip(grads, pool[s % POOL]):
            g.copy_(p)

    # clocks are sampled from the warm-up to the end of the host-buffer loop: the timed region alone lasts a few
    # milliseconds, shorter than one nvidia-smi polling period
    sampler = ClockSampler(local_rank)
    sampler.start()
    for s in range(args.warmup):
        refresh(s)
        agg.step(ptrs, stream)
    torch.cuda.synchronize()

    agg.set_profiling(True)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for s in range(args.steps):
        refresh(args.warmup + s)
        ev[s][0].record()
        agg.step(ptrs, stream)
        ev[s][1].record()
    torch.cuda.synchronize()
    barrier()
    wall = time.perf_counter() - t0
    step_ms = [a.elapsed_time(b) for a, b in ev]
    phases = agg.phase_ms()
    agg.set_profiling(False)
    t_step = sum(step_ms) / len(step_ms)
    tt = torch.tensor([t_step] + phases, device=dev, dtype=torch.float64)
    if K > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    t_step = float(tt[0])
    phases = [float(x) for x in tt[1:]]

    # end to end through the host-buffer entry point: pinned host gradients in, aggregated gradients back out, chunks of
    # tensors pipelined over streams inside the library (upload / kernels / download of different chunks overlap)
    hagg = lib.HostAggregator(comm, shapes, bits, chunks=args.e2e_chunks)
    if K > 1 and exchange.startswith("peer"):
        mine = torch.frombuffer(bytearray(hagg.peer_handles()), dtype=torch.uint8).to(dev)
        allh = [torch.zeros_like(mine) for _ in range(K)]
        dist.all_gather(allh, mine)
        hagg.enable_peer([bytes(h.cpu().numpy().tobytes()) for h in allh])
    hpool = [torch.empty((n, m), dtype=torch.float32).normal_(0, 1e-3).pin_memory() for (m, n) in shapes]
    hgrads = [torch.empty((n, m), dtype=torch.float32).pin_memory() for (m, n) in shapes]
    hptrs = [h.data_ptr() for h in hgrads]
    e2e_steps = max(3, min(args.steps, 10))
    e2e_t = []
    for s in range(2 + e2e_steps):
        for h, p in zip(hgrads, hpool):
            h.copy_(p)
        barrier()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        hagg.step(hptrs)  # returns after the results are back in host memory
        dt = time.perf_counter() - t1
        if s >= 2:
            e2e_t.append(dt)
    e2e_ms = sum(e2e_t) / len(e2e_t) * 1e3
    clocks = sampler.stop()
    te = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if K > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te[0])
    hagg.check()
    e2e_launches = e2e_steps * hagg.chunks * agg.launches_per_step
    barrier()
    hagg.destroy()

    if rank == 0:
        peak, peak_kind = load_peaks()
        alg = workloads.algorithmic_bytes(shapes, bits, K)
        k1_gbs = alg["quantize"] / (phases[0] * 1e-3) / 1e9 if phases[0] > 0 else 0.0
        kern_ms = phases[0] + phases[2] + phases[4]
        line = {
            "metric": METRIC, "value": 4.0 * V * K / (t_step * 1e-3) / 1e9, "unit": UNIT,
            "per_gpu_value": 4.0 * V / (t_step * 1e-3) / 1e9,
            "n_gpus": K, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "tensors": len(shapes), "values_per_rank": V, "bits": bits,
                       "zero_threshold": True, "self_stripe_quantized": True, "parallelism": f"dp{K} striped by columns", "exchange": exchange,
                       "l2": "inputs (361 MB gradient + residual per step) exceed the 126 MB L2; gradients are also re-copied "
                             "from a pre-generated pool between steps, outside the per-step events",
                       "timing": "CUDA events around each step on the launch stream, mean over steps, max over ranks"},
            "phases_ms": {"quantize": phases[0], "scatter": phases[1], "reduce_requantize": phases[2], "all_gather": phases[3],
                          "unquantize": phases[4]},
            "roofline": {"bound": "hbm", "kernel": "k_stream1 (quantize: level sums + pack + deferred residual)", "achieved": k1_gbs, "peak": peak,
                         "unit": "GB/s", "frac": k1_gbs / peak, "peak_kind": peak_kind, "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                         "algorithmic_bytes_per_launch": alg["quantize"],
                         "all_kernels": {"algorithmic_bytes": alg["total"], "ms": kern_ms,
                                         "frac": alg["total"] / (kern_ms * 1e-3) / 1e9 / peak if kern_ms > 0 else None}},
            "wire": {"bytes_per_step_per_gpu_each_way": agg.wire_bytes,
                     "nvlink_frac_of_770GBs": (agg.wire_bytes / ((phases[1] + phases[3]) * 1e-3) / 770e9) if K > 1 and (phases[1] + phases[3]) > 0 else None},
            "e2e": {"value": 4.0 * V * K / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": 4 * V, "d2h_bytes_per_step": 4 * V, "steps": e2e_steps,
                    "chunks": args.e2e_chunks, "api": "qagg_hagg_step (pinned host buffers, chunk-pipelined)"},
            "gpu_launches": agg.launches_per_step * args.steps, "gpu_launches_e2e": e2e_launches,
            "clocks": clocks, "wall_ms_per_step_including_refresh": wall / args.steps * 1e3,
        }
        if K == 1 and not args.no_cpu_baseline:
            r = cpu_reference_run(shapes, bits, 1, 3, 1, 1)
            line["cpu_baseline"] = {"value": r["gbs_total"], "unit": UNIT, "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]}
        print(json.dumps(line), flush=True)
    agg.check(stream)
    barrier()
    agg.destroy()
    comm.destroy()
    if K > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="speech_dnn", choices=["speech_dnn", "resnet50", "lstm_lm", "round_trip_2048"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-chunks", type=int, default=6, help="tensor chunks pipelined by the host-buffer entry point")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"], help="multi-GPU transport of the packed stripes")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
