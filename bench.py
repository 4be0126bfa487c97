#!/usr/bin/env python
"""Benchmark of the quantized gradient aggregation step (CNTK 1-bit SGD path) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload speech_dnn|resnet50|lstm_lm|sweep]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

A "step" is one AggregateGradients call over the whole gradient set of one rank, DistGradHeader included (default: the
speech-DNN set, 16 tensors, 45,122,648 fp32 values, 1 bit, zero threshold, residual carried from step to step).  Rank 0
prints ONE JSON line.  `value` is fp32-gradient GB/s summed over ranks (4 * values * ranks / step time, step time = max
over ranks of the mean CUDA-event time of a step); `per_gpu_value` is the per-GPU figure the metric is named after.

After the timed loops, and outside them, every rank checks results against the CPU checker (oracle/): a seeded sample of
columns of every tensor of one more full-size step is replayed through the whole exchange from all ranks' inputs, and with
more than one rank the small multi-rank parity set of tests/multi_gpu_check.py runs as well.  A differing byte ends the
process with a non-zero status; the line carries "parity": {"checked": true, ...}.

--impl reference times the reference's own CPU quantizer (its headers compiled in place, oracle/_ref; else the C port)
driving the restated exchange with one thread per simulated rank on this box's host cores, and prints the same line shape.
--local-ranks K (one GPU) steps K simulated ranks as an in-process group and prints each rank's kernel times per phase: the way
to look at the owner's reduce-requantize kernels, which a single rank never runs, on one device and under a profiler.  Its
line is a kernel-time table, not a bench value.  --fused-update adds the learner step (momentum SGD) fused into the last
kernel beside the unfused sequence.
--workload sweep runs BASELINE config 5 (1024 rows x 1 Mi .. 1 Gi values; 1, 2 and 32 bits) and reports a table in "sweep".
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
sys.path.insert(0, os.path.join(ROOT, "tests"))

METRIC = "1-bit aggregated fp32-grad GB/s per GPU (max over ranks) at 1/2/4/8 B200"
UNIT = "GB/s of fp32 gradient, summed over GPUs (per_gpu_value = per GPU)"
REFERENCE_STEP_CAP = 5  # a full-size CPU step takes about a second per rank-thread: the reference arm times at most this many


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


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of the quantize kernel at ONE rank, from the ncu
# capture summarised in profiles/k_stream1_speech_dnn_1bit.md (same workload).  Reported only for the configuration that
# was captured; null elsewhere.
NCU_TRAFFIC_BYTES = {("speech_dnn", 1): 504.58e6}


def get_shapes(name):
    from cntk_b200 import workloads as w
    table = {"speech_dnn": (w.speech_dnn, 1), "resnet50": (w.resnet50, 4), "lstm_lm": (w.lstm_lm, 1), "round_trip_2048": (w.round_trip_2048, 1)}
    fn, bits = table[name]
    return fn(), bits


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def bind_near_gpu(local_rank):
    """Runs this process on the CPUs next to its GPU, so that the pinned buffers it allocates afterwards land on that NUMA
    node (first touch).  Reads the topology from sysfs; changes no GPU setting.  Returns a short description."""
    try:
        import torch
        p = torch.cuda.get_device_properties(local_rank)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/local_cpulist") as f:
            spec = f.read().strip()
        cpus = set()
        for part in spec.split(","):
            if "-" in part:
                a, b = part.split("-")
                cpus.update(range(int(a), int(b) + 1))
            elif part:
                cpus.add(int(part))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            return f"host thread bound to {len(allowed)} CPUs local to GPU {bdf}"
        return "GPU-local CPUs not in this process's affinity mask: not bound"
    except Exception as e:  # no sysfs entry, container without the topology: run unbound
        return f"not bound ({type(e).__name__})"


# ------------------------------------------------------------------------------------------------ reference arm
def cpu_reference_run(shapes, bits, K, steps, warmup):
    """Times the CPU checker (reference headers when built, else the C port) on the restated exchange with K simulated
    ranks, one host thread each, on the FULL tensor set."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor
    from oracle import backend, exchange
    be = backend.best_backend()
    cores = min(K, len(os.sched_getaffinity(0)) or 1)
    st = exchange.ExchangeState(shapes, K)
    rngs = [np.random.default_rng(1000 * r) for r in range(K)]
    pool = [[(rngs[r].standard_normal((n, m), dtype=np.float32) * np.float32(1e-3)) for (m, n) in shapes] for r in range(K)]
    V = sum(m * n for m, n in shapes)
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
            "sample": f"all columns of every tensor ({V} values per rank), {steps} step(s) after {warmup} warm-up, "
                      f"{K} simulated rank(s) on {cores} host thread(s)"}


def workload_config(workload, shapes, V, bits, K):
    """The `config` object of a bench line: what is computed, identical for this build's arm and the reference arm (what
    differs between the arms -- transport, timing method, host binding -- goes under "arm")."""
    return {"workload": workload, "tensors": len(shapes), "values_per_rank": V, "bits": bits, "zero_threshold": True,
            "self_stripe_quantized": True, "parallelism": f"dp{K} striped by columns",
            "l2": f"inputs ({8 * V / 1e6:.0f} MB gradient + residual per rank and step) exceed the 126 MB L2"}


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    shapes, bits = get_shapes(args.workload if args.workload != "sweep" else "speech_dnn")
    K = args.gpus
    steps = max(1, min(args.steps, REFERENCE_STEP_CAP))
    warm = max(0, min(args.warmup, 1))
    r = cpu_reference_run(shapes, bits, K, steps, warm)
    line = {"impl": "reference", "metric": METRIC, "value": r["gbs_total"], "unit": UNIT, "per_gpu_value": r["gbs_total"] / K,
            "n_gpus": K, "steps": steps, "warmup": warm, "steps_requested": args.steps, "warmup_requested": args.warmup,
            "steps_cap": f"a full-size CPU step takes about a second: at most {REFERENCE_STEP_CAP} timed steps and 1 warm-up",
            "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.workload, shapes, r["values_per_rank"], bits, K),
            "arm": {"exchange": "reference CPU quantizer (MatrixQuantizerCPU arithmetic) + restated striped exchange in host memory, one thread per rank",
                    "timing": "host clock around each step, max over rank threads"},
            "cpu_baseline": {"value": r["gbs_total"], "unit": UNIT, "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]},
            "e2e": {"value": r["gbs_total"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------ our arm
class Ranks:
    """torch.distributed plumbing of one rank: NCCL for device data, a gloo group for waits that must not spin."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank, self.local, self.K = dist_env()
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.gloo = None
        if self.K > 1:
            dist.init_process_group("nccl", device_id=self.dev)
            self.gloo = dist.new_group(backend="gloo")

    def barrier(self):
        if self.K > 1:
            self.dist.barrier()

    def quiet_barrier(self):
        """Blocks in a socket, not in a GPU spin: used while rank 0 times host code."""
        if self.K > 1:
            self.dist.barrier(group=self.gloo)

    def max_over_ranks(self, values):
        t = self.torch.tensor(values, device=self.dev, dtype=self.torch.float64)
        if self.K > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t]

    def all_gather_bytes(self, blob):
        torch = self.torch
        mine = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(self.dev)
        out = [torch.zeros_like(mine) for _ in range(self.K)]
        self.dist.all_gather(out, mine)
        return [bytes(h.cpu().numpy().tobytes()) for h in out]

    def unique_id(self, lib):
        if self.K == 1:
            return None
        torch = self.torch
        idt = torch.zeros(lib.UNIQUE_ID_BYTES, dtype=torch.uint8, device=self.dev)
        if self.rank == 0:
            idt.copy_(torch.frombuffer(bytearray(lib.unique_id()), dtype=torch.uint8))
        self.dist.broadcast(idt, 0)
        return bytes(idt.cpu().numpy().tobytes())

    def close(self):
        if self.K > 1:
            self.dist.destroy_process_group()


def enable_peer(R, agg, handle_fn, enable_fn):
    """All ranks must agree on the transport: the outcome of every set-up stage is reduced over the ranks."""
    torch, dist = R.torch, R.dist
    ok = 1
    try:
        allh = R.all_gather_bytes(handle_fn())
    except Exception:
        ok = 0
    okt = torch.tensor([ok], device=R.dev)
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    if not int(okt.item()):
        return False
    try:
        enable_fn(allh)
    except Exception as e:  # cannot map peer memory here
        ok = 0
        print(f"[rank {R.rank}] peer mapping failed: {e}", file=sys.stderr)
    okt = torch.tensor([ok], device=R.dev)
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    if not int(okt.item()):
        raise SystemExit("peer mapping succeeded on some ranks only; rerun with --exchange nccl")
    return True


def check_full_size_step(R, lib, agg, shapes, bits, grads, refresh, stream):
    """One more step of the aggregator that was just timed, with a seeded sample of columns of every tensor captured before
    and after and replayed on the CPU checker from ALL ranks' inputs (tests/parity_util.py)."""
    import numpy as np
    import parity_util as pu
    from oracle import backend
    torch, K = R.torch, R.K
    be = backend.OracleBackend()
    cols = pu.pick_columns(shapes, K, seed=4242)
    cap = pu.RankCapture(lib, agg, R.rank, K, shapes, bits, cols)
    refresh(10007)
    torch.cuda.synchronize()
    cap.before(grads)
    agg.step_header([g.data_ptr() for g in grads], [1.0, 2.0, 3.0], stream)
    torch.cuda.synchronize()
    cap.after(grads)
    flat = torch.from_numpy(cap.flat_inputs()).to(R.dev)
    if K > 1:
        out = [torch.zeros_like(flat) for _ in range(K)]
        R.dist.all_gather(out, flat)
        inputs = [cap.inputs_from_flat(t.cpu().numpy()) for t in out]
    else:
        inputs = [cap.inp]
    n = pu.verify(be, cap, inputs)
    hdr = agg.header_result(3, stream)
    assert hdr == [1.0 * K, 2.0 * K, 3.0 * K], f"header sum {hdr}"
    return n


def time_steps(R, agg, ptrs, refresh, steps, warmup, stream, header):
    torch = R.torch
    for s in range(warmup):
        refresh(s)
        agg.step_header(ptrs, header, stream)
    torch.cuda.synchronize()
    agg.set_profiling(True)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    R.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for s in range(steps):
        refresh(warmup + s)
        ev[s][0].record()
        agg.step_header(ptrs, header, stream)
        ev[s][1].record()
    torch.cuda.synchronize()
    R.barrier()
    wall = time.perf_counter() - t0
    step_ms = [a.elapsed_time(b) for a, b in ev]
    phases = agg.phase_ms()
    agg.set_profiling(False)
    vals = R.max_over_ranks([sum(step_ms) / len(step_ms)] + phases)
    return vals[0], vals[1:], wall / steps * 1e3


def run_ours(args):
    import torch
    from cntk_b200 import lib, workloads

    R = Ranks()
    rank, K, dev = R.rank, R.K, R.dev
    if K != args.gpus and not (K == 1 and args.gpus == 1):
        raise SystemExit("launch with torch.distributed.run for --gpus > 1 (WORLD_SIZE must equal --gpus)")
    affinity = bind_near_gpu(R.local)
    shapes, bits = get_shapes(args.workload)
    V = workloads.total_values(shapes)
    comm = lib.Comm.create(R.unique_id(lib), rank, K, R.local)
    agg = lib.Aggregator(comm, shapes, bits)
    exchange = "none (1 rank)"
    if K > 1:
        exchange = "nccl send/recv + all-gather"
        if args.exchange == "p2p" and enable_peer(R, agg, agg.peer_handle, agg.enable_peer):
            exchange = "peer-memory stores over NVLink + flag hand-shake (no collective)"

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
    sampler = ClockSampler(R.local)
    sampler.start()
    header = [0.25 * (rank + 1), 256.0, 256.0, 0.5, 128.0]  # criterion, numSamples, numSamplesWithLabel, one evaluation pair
    t_step, phases, wall_ms = time_steps(R, agg, ptrs, refresh, args.steps, args.warmup, stream, header)

    # end to end through the host-buffer entry point: pinned host gradients in, aggregated gradients back out, column chunks
    # pipelined over streams inside the library (upload / kernels / download of different chunks overlap)
    hagg = lib.HostAggregator(comm, shapes, bits, chunks=args.e2e_chunks)
    if K > 1 and exchange.startswith("peer"):
        hagg.enable_peer(R.all_gather_bytes(hagg.peer_handles()))
    hpool = [torch.empty((n, m), dtype=torch.float32).normal_(0, 1e-3).pin_memory() for (m, n) in shapes]
    hgrads = [torch.empty((n, m), dtype=torch.float32).pin_memory() for (m, n) in shapes]
    hptrs = [h.data_ptr() for h in hgrads]
    e2e_steps = max(3, min(args.steps, 10))

    def timed_host_loop(fn):
        ts = []
        for s in range(2 + e2e_steps):
            for h, p in zip(hgrads, hpool):
                h.copy_(p)
            R.barrier()
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            fn()
            dt = time.perf_counter() - t1
            if s >= 2:
                ts.append(dt)
        return R.max_over_ranks([sum(ts) / len(ts) * 1e3])[0]

    e2e_ms = timed_host_loop(lambda: hagg.step(hptrs))  # returns after the results are back in host memory
    copy_floor_ms = timed_host_loop(lambda: hagg.copy_only(hptrs))  # the same uploads and downloads, no kernels
    clocks = sampler.stop()
    hagg.check()
    e2e_launches = e2e_steps * hagg.chunks * agg.launches_per_step
    R.barrier()
    hagg.destroy()

    # ---- parity, outside every timed region ----
    parity = {"checked": False}
    if not args.no_parity:
        cols = check_full_size_step(R, lib, agg, shapes, bits, grads, refresh, stream)
        small = 0
        if K > 1:
            import multi_gpu_check
            small = multi_gpu_check.run_checks(comm, rank, K, dev)
        agg.check(stream)
        counts = R.max_over_ranks([float(cols), float(small)])
        parity = {"checked": True, "ranks": K, "columns": int(counts[0]),
                  "what": "sampled columns of every tensor of one full-size step (aggregate, residual, stripe residual, gathered packed "
                          "column, header sum) bit-identical to the CPU checker on every rank"
                          + ("; plus the small multi-rank set (NCCL and peer paths, 1 bit zero/mean threshold, 4 bits, raw own stripe, "
                             "host-buffer aggregator), 4 steps each" if K > 1 else ""),
                  "small_set_steps": int(counts[1])}

    # ---- CPU baseline in the same run (rank 0; the other ranks wait without spinning) ----
    cpu = None
    if not args.no_cpu_baseline:
        R.quiet_barrier()
        if rank == 0:
            r = cpu_reference_run(shapes, bits, K, 2 if K > 1 else 3, 1)
            cpu = {"value": r["gbs_total"], "unit": UNIT, "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]}
        R.quiet_barrier()

    if rank == 0:
        peak, peak_kind = load_peaks()
        alg = workloads.algorithmic_bytes(shapes, bits, K)

        def roof(name, kernel, ms, extra=None):
            gbs = alg[name] / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
            d = {"kernel": kernel, "achieved": gbs, "frac": gbs / peak, "algorithmic_bytes_per_launch": alg[name], "ms": ms}
            if extra:
                d.update(extra)
            return d

        k1 = roof("quantize", "k_stream1 (quantize: level sums + pack + deferred residual)", phases[0])
        kern_ms = phases[0] + phases[2] + phases[4]
        roofline = {"bound": "hbm", "kernel": k1["kernel"], "achieved": k1["achieved"], "peak": peak, "unit": "GB/s", "frac": k1["frac"],
                    "peak_kind": peak_kind, "traffic": NCU_TRAFFIC_BYTES.get((args.workload, K)),
                    "algorithmic_bytes_per_launch": alg["quantize"],
                    "unquantize": roof("unquantize", "k_unquantize", phases[4]),
                    "all_kernels": {"algorithmic_bytes": alg["total"], "ms": kern_ms,
                                    "frac": alg["total"] / (kern_ms * 1e-3) / 1e9 / peak if kern_ms > 0 else None}}
        if K > 1:
            roofline["reduce_requantize"] = roof("reduce_requantize", "k_owner_form + k_owner_walk (owner: sum of stripes, requantize)", phases[2],
                                                 {"note": "two launches; the walk is an ordered fp32 add chain over the tallest owned column, "
                                                          "a latency floor of about 4.6 cycles per row whatever the bytes"})
        line = {
            "metric": METRIC, "value": 4.0 * V * K / (t_step * 1e-3) / 1e9, "unit": UNIT,
            "per_gpu_value": 4.0 * V / (t_step * 1e-3) / 1e9,
            "n_gpus": K, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.workload, shapes, V, bits, K),
            "arm": {"exchange": exchange,
                    "header": "a 5-value DistGradHeader is summed over the ranks inside every timed step",
                    "l2_refresh": "gradients are re-copied from a pre-generated pool between steps, outside the per-step events",
                    "timing": "CUDA events around each step on the launch stream, mean over steps, max over ranks",
                    "host": affinity},
            "phases_ms": {"quantize": phases[0], "scatter": phases[1], "reduce_requantize": phases[2], "all_gather": phases[3],
                          "unquantize": phases[4]},
            "roofline": roofline,
            "wire": {"bytes_per_step_per_gpu_each_way": agg.wire_bytes,
                     "nvlink_frac_of_770GBs": (agg.wire_bytes / ((phases[1] + phases[3]) * 1e-3) / 770e9) if K > 1 and (phases[1] + phases[3]) > 0 else None},
            "e2e": {"value": 4.0 * V * K / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": 4 * V, "d2h_bytes_per_step": 4 * V, "steps": e2e_steps,
                    "chunks": hagg.chunks, "copy_floor_ms": copy_floor_ms,
                    "api": "qagg_hagg_step (pinned host buffers, column chunks pipelined over three streams)"},
            "gpu_launches": agg.launches_per_step * args.steps, "gpu_launches_e2e": e2e_launches,
            "parity": parity, "clocks": clocks, "wall_ms_per_step_including_refresh": wall_ms,
        }
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    agg.check(stream)
    R.barrier()
    agg.destroy()
    comm.destroy()
    R.close()


def run_sweep(args):
    """BASELINE config 5: one 1024-row matrix of 1 Mi .. 1 Gi values; 1 bit, 2 bits and the unquantized 32-bit arm; at the
    launched number of ranks.  One JSON line with the table under "sweep"."""
    import torch
    from cntk_b200 import lib, workloads

    R = Ranks()
    rank, K, dev = R.rank, R.K, R.dev
    comm = lib.Comm.create(R.unique_id(lib), rank, K, R.local)
    peak, peak_kind = load_peaks()
    stream = torch.cuda.current_stream().cuda_stream
    rows = []
    for k in range(args.sweep_max_k + 1):
        shapes = workloads.sweep(k)
        V = workloads.total_values(shapes)
        g = torch.empty((shapes[0][1], shapes[0][0]), device=dev, dtype=torch.float32)
        src = torch.randn(g.shape, device=dev, dtype=torch.float32) * 1e-3
        for bits in (1, 2, 32):
            if bits == 32:
                agg = lib.DenseAggregator(comm, shapes)
                peer_ok = K > 1 and enable_peer(R, agg, agg.peer_handle, agg.enable_peer)
                step = lambda: agg.step([g.data_ptr()], stream)
                alg_bytes = workloads.dense_algorithmic_bytes(shapes, K)
                wire = agg.wire_bytes
            else:
                agg = lib.Aggregator(comm, shapes, bits)
                peer_ok = K > 1 and enable_peer(R, agg, agg.peer_handle, agg.enable_peer)
                step = lambda: agg.step([g.data_ptr()], stream)
                alg_bytes = workloads.algorithmic_bytes(shapes, bits, K)["total"]
                wire = agg.wire_bytes
            steps = max(3, min(args.steps, 10))
            for s in range(3):
                g.copy_(src)
                step()
            torch.cuda.synchronize()
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            R.barrier()
            for s in range(steps):
                g.copy_(src)
                ev[s][0].record()
                step()
                ev[s][1].record()
            torch.cuda.synchronize()
            ms = R.max_over_ranks([sum(a.elapsed_time(b) for a, b in ev) / steps])[0]
            agg.check(stream)
            R.barrier()
            agg.destroy()
            rows.append({"values": V, "bits": bits, "ms_per_step": ms, "gbs_per_gpu": 4.0 * V / (ms * 1e-3) / 1e9,
                         "hbm_frac": alg_bytes / (ms * 1e-3) / 1e9 / peak,
                         "wire_bytes_each_way": wire, "nvlink_frac_of_770GBs_if_only_wire": (wire / (ms * 1e-3) / 770e9) if K > 1 else None,
                         "peer": bool(peer_ok)})
        del g, src
        torch.cuda.empty_cache()
    if rank == 0:
        best = max(r["gbs_per_gpu"] for r in rows if r["bits"] == 1)
        print(json.dumps({"metric": METRIC, "value": best * K, "unit": UNIT, "per_gpu_value": best, "n_gpus": K, "steps": args.steps, "warmup": 3,
                          "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                          "config": {"workload": "sweep", "rows": 1024, "note": "value = the best 1-bit row of the table"},
                          "peak": peak, "peak_kind": peak_kind, "sweep": rows}), flush=True)
    comm.destroy()
    R.close()


def run_local_group(args):
    """K simulated ranks on ONE GPU (qagg_comm_create_local_group): every rank's quantize / reduce-requantize / unquantize
    kernel time from the aggregator's phase events, mean over the timed steps.  The ranks run one after the other on one
    device, so the step time of the group is meaningless; the per-rank kernel times are what a rank would spend."""
    import torch
    from cntk_b200 import lib, workloads
    K = args.local_ranks
    shapes, bits = get_shapes(args.workload)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    comms = lib.Comm.local_group(K, 0)
    aggs = [lib.Aggregator(c, shapes, bits) for c in comms]
    if K > 1 and args.exchange == "p2p":
        hs = [a.peer_handle() for a in aggs]
        for a in aggs:
            a.enable_peer(hs)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234)
    pool = [torch.randn((n, m), generator=gen, device=dev, dtype=torch.float32) * 1e-3 for (m, n) in shapes]  # shared by the ranks
    grads = [[torch.empty_like(t) for t in pool] for _ in range(K)]
    ptrs = [[t.data_ptr() for t in grads[r]] for r in range(K)]

    def refresh():
        for r in range(K):
            for g, p_ in zip(grads[r], pool):
                g.copy_(p_)

    def timed(steps):
        for a in aggs:
            a.set_profiling(True)
        for _ in range(steps):
            refresh()
            lib.step_group(aggs, ptrs)
        torch.cuda.synchronize()
        ph = [a.phase_ms() for a in aggs]
        for a in aggs:
            a.set_profiling(False)
        return ph

    for _ in range(args.warmup):
        refresh()
        lib.step_group(aggs, ptrs)
    torch.cuda.synchronize()
    ph = timed(args.steps)
    V = workloads.total_values(shapes)
    P = workloads.packed_bytes(shapes, bits)
    peak, peak_kind = load_peaks()
    us = lambda k: [round(p_[k] * 1e3, 1) for p_ in ph]
    k1, k2, k3 = us(0), us(2), us(4)
    out = {"mode": "local_group", "note": "kernel times of K simulated ranks on one GPU; not a bench value", "simulated_ranks": K,
           "workload": args.workload, "bits": bits, "steps": args.steps, "warmup": args.warmup,
           "quantize_us": k1, "reduce_requantize_us": k2, "unquantize_us": k3,
           "roofline_frac_of_" + peak_kind: {
               "quantize": round((12 * V + P) / (max(k1) * 1e-6) / (peak * 1e9), 3),
               "reduce_requantize": round((8 * V / K + P * (1 + 1.0 / K)) / (max(k2) * 1e-6) / (peak * 1e9), 3) if K > 1 else None,
               "unquantize": round((4 * V + P) / (max(k3) * 1e-6) / (peak * 1e9), 3)}}
    if args.fused_update:
        w = [[torch.randn_like(t) for t in pool] for _ in range(K)]
        sm = [[torch.zeros_like(t) for t in pool] for _ in range(K)]
        for r in range(K):
            aggs[r].bind_update([t.data_ptr() for t in w[r]], [t.data_ptr() for t in sm[r]])
        lr, mom, ug = 0.05, 0.9, 0.1

        def rank_update_ms(fused):
            # one rank's unquantize kernel (+ its separate update launches when not fused), from events around them
            for a in aggs:
                a.set_update(fused, lr, mom, ug)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            tot = 0.0
            for it in range(args.warmup + args.steps):
                refresh()
                lib.step_group(aggs, ptrs)
                e0.record()
                if not fused:
                    for i, (m, n) in enumerate(shapes):
                        lib.sgd_update(w[0][i].data_ptr(), grads[0][i].data_ptr(), sm[0][i].data_ptr(), m * n, lr, mom, ug)
                e1.record()
                torch.cuda.synchronize()
                if it >= args.warmup:
                    tot += e0.elapsed_time(e1)
            return tot / args.steps

        unf = rank_update_ms(False)
        k3_plain = max(k3) * 1e-3
        rank_update_ms(True)  # switches the fused step on (and warms it up)
        ph_f = timed(args.steps)
        k3_fused = max(p_[4] for p_ in ph_f)
        out["consumer_fusion"] = {"rule": "momentum SGD (Matrix::MomentumSGDUpdate)", "unfused_ms": round(k3_plain + unf, 4),
                                  "unfused_parts_ms": {"unquantize": round(k3_plain, 4), "update_kernels": round(unf, 4)},
                                  "fused_ms": round(k3_fused, 4),
                                  "bytes_unfused": 24 * V + P, "bytes_fused": 16 * V + P,
                                  "fused_frac_of_" + peak_kind: round((16 * V + P) / (k3_fused * 1e-3) / (peak * 1e9), 3)}
    for a in aggs:
        a.check()
        a.destroy()
    for c in comms:
        c.destroy()
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="speech_dnn", choices=["speech_dnn", "resnet50", "lstm_lm", "round_trip_2048", "sweep"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--e2e-chunks", type=int, default=6, help="column chunks pipelined by the host-buffer entry point")
    ap.add_argument("--sweep-max-k", type=int, default=5, help="largest matrix of the sweep: 1024 x 1024 * 4^k values")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"], help="multi-GPU transport of the packed stripes")
    ap.add_argument("--local-ranks", type=int, default=0, help="one GPU: kernel times of this many simulated ranks (not a bench value)")
    ap.add_argument("--fused-update", action="store_true", help="with --local-ranks: time the learner step fused into the last kernel")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.local_ranks > 0:
        run_local_group(args)
    elif args.workload == "sweep":
        run_sweep(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
