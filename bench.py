"""Benchmark of the trace post-processing hot path.

    python bench.py --gpus N --steps K --warmup W [--workload W --size N]   # this library (CUDA, sm_100a)
    python bench.py --impl reference --gpus N --steps K ...               # the reference's CPU path on host cores

Workloads (seeded synthetic traces that stand in for real captures; `--size` is the generator's size argument
per GPU):

    mixed             (default, n = 10 000 000)  10 M mixed activities per GPU: 60 % kernels, 20 % memcpy (HtoD /
                      DtoH / DtoD / PtoP), 5 % memset, 15 % runtime-only calls, each with its launching runtime
                      record, EXTERNAL_CORRELATION record and CPU op; 50 000 names of 20-400 bytes, 2 % with JSON
                      escapes; 5 % orphaned correlation ids
    kernel_launches   n Kernel9 + n cudaLaunchKernel + n EXTERNAL_CORRELATION records + n CPU ops, correlation ids
                      shuffled by a seeded permutation, 4096 names
    op_tree           a CPU op tree of n nested record_function spans with shape strings, flows, 2 n kernel launches
    distributed_rank  one rank of a distributed job: n launches, 20 % NCCL collectives with metadata, events sorted
                      by start time; with N GPUs every GPU formats its own rank's trace (no exchange)
    memory_events     kernel_launches plus n / 2 cpu_instant_event rows
    generic           n GenericTraceActivity kernel records fed straight to the JSON logger

With N > 1 the mixed and kernel_launches traces are N times as long and sharded by contiguous record range, one
shard per GPU (weak scaling); the shards exchange their EXTERNAL_CORRELATION records and CPU-op ids with NCCL so
that the join covers the whole trace.

One "step" = one pass of the path over the shard.  `value` counts input records (CUPTI records + CPU ops) per
second with the inputs already resident in HBM; `e2e` is the same through the C ABI with pinned HOST buffers:
host->device copies of every input and the slab-by-slab device->host copy of the text inside the timed region.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "trace_records_per_sec"
UNIT = "records/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one emit launch (k_events<true, false>) divided by the JSON bytes it
# wrote, from ncu captures of whole launches at size argument 1 000 000 (1.5 and 1.9 GB of text, far beyond the L2;
# profiles/emit_kernel_dram_traffic.txt).  Traffic grows in proportion to the text, so the line scales it to the
# launch it timed; workloads without a capture report null.
EMIT_TRAFFIC_PER_OUT_BYTE = {"mixed": 2254.8 / 1510.1, "kernel_launches": 2637.2 / 1858.1}
SLAB_BYTES = 256 << 20

DEFAULT_N = {"mixed": 10_000_000, "kernel_launches": 1_000_000, "op_tree": 2_000_000, "distributed_rank": 2_000_000,
             "memory_events": 1_000_000, "generic": 2_000_000}
SHARDED = ("mixed", "kernel_launches")      # one trace, cut by record range, join keys exchanged
REPLICATED = ("distributed_rank",)          # one independent trace per GPU


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mixed", choices=sorted(DEFAULT_N))
    ap.add_argument("--size", dest="n", type=int, default=0, help="size argument of the generator per GPU (0: the workload's default)")
    ap.add_argument("--launches", type=int, default=0, help="same as --workload kernel_launches --size LAUNCHES")
    ap.add_argument("--cpu-sample", type=int, default=250_000, help="size argument of the CPU-baseline / parity sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--no-save-e2e", action="store_true", help="skip the save() comparison through the reference's logger factory")
    ap.add_argument("--exchange", default="auto", choices=["auto", "wanted", "all"],
                    help="sharded runs: all-gather only the join keys another shard can want (three small collectives and a host "
                         "round trip: pays from four shards on, the default there), or all of them")
    ap.add_argument("--parity-full", action="store_true",
                    help="also run the reference on the WHOLE benchmark trace and compare sha256 (minutes of CPU time)")
    a = ap.parse_args()
    if a.launches:
        a.workload, a.n = "kernel_launches", a.launches
    if not a.n:
        a.n = DEFAULT_N[a.workload]
    return a


def generate(workload, n, rank=0, world=1):
    from kineto_b200 import synth
    if workload == "mixed":
        return synth.gen_mixed(n, seed=3, shard=(rank, world))
    if workload == "kernel_launches":
        return synth.gen_kernel_launches(n, seed=2, shard=(rank, world))
    if workload == "op_tree":
        return synth.gen_op_tree(n, seed=4 + rank)
    if workload == "distributed_rank":
        t = synth.gen_distributed_rank(n, rank=rank, seed=5)
        t.params["flags"] |= 2  # events in order of their start time (64-bit radix sort)
        return t
    if workload == "memory_events":
        return synth.gen_kernel_launches(n, seed=2 + rank, memory_events=0.5)
    return synth.gen_generic_kernels(n, seed=1 + rank)


def config(args, world, n):
    what = {"mixed": "mixed: per GPU %d activities (60%% kernels, 20%% memcpy, 5%% memset, 15%% runtime-only), each with runtime + "
                     "EXTERNAL_CORRELATION record + CPU op, 50k names of 20-400 B (2%% JSON escapes), 5%% orphans",
            "kernel_launches": "kernel_launches: per GPU %d Kernel9 + cudaLaunchKernel + EXTERNAL_CORRELATION records + CPU ops, "
                               "shuffled correlation ids, 8 devices x 32 streams, 4096 names of 20-400 B",
            "op_tree": "op_tree: %d nested record_function spans with shape strings and flows, 2 launches per op",
            "distributed_rank": "distributed_rank: per GPU one rank's trace, %d launches, 20%% collectives with metadata, sorted by start",
            "memory_events": "memory_events: %d launches + half as many cpu_instant_event rows",
            "generic": "generic: %d GenericTraceActivity kernel records"}[args.workload] % n
    return {"workload": what, "name": args.workload, "n_per_gpu": n,
            "sharding": ("contiguous record range, %d shard(s), join keys exchanged (%s)" % (world, "all" if args.exchange == "all" or (args.exchange == "auto" and world < 4) else "those another shard can want")) if args.workload in SHARDED
            else ("%d independent trace(s)" % world),
            "l2": "inputs and output of one step exceed the 126 MB L2 many times over; no flush needed", "seed": "fixed"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only queries) while the timed region runs."""

    def __init__(self, index):
        self.index, self.sm, self.reasons, self.max_sm = index, [], set(), None
        self._stop = threading.Event()
        self.t = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                import torch
                self.h = pynvml.nvmlDeviceGetHandleByUUID("GPU-" + str(torch.cuda.get_device_properties(self.index).uuid))
            except Exception:  # noqa: BLE001
                self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # noqa: BLE001
            self.err = repr(e)
            return
        self.t = threading.Thread(target=self._loop, daemon=True)
        self.t.start()

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.002)

    def stop(self):
        if self.t is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["NVML unavailable: " + getattr(self, "err", "")]}
        self._stop.set()
        self.t.join(timeout=2)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_sm,
                "reasons": sorted(self.reasons), "samples": len(self.sm)}


def activities_span(doc: bytes) -> bytes:
    """The events of a file written through ActivityTrace::save(): one run between the metadata rows and the trace span."""
    a = doc.find(b'\n  {\n    "ph": "X",')
    b = doc.rfind(b'\n  {\n    "ph": "X",\n    "cat": "Trace",')
    return doc[a:b]


# ------------------------------------------------------------------------------------------------
# the reference's own CPU code (oracle/_ref/ref_driver), or our CPU restatement where it is absent
# ------------------------------------------------------------------------------------------------
def run_reference_once(trace, procs, keep_output=False):
    """`procs` concurrent single-threaded reference processes, each over its own copy of `trace`.  Returns
    (aggregate records/s, seconds, records per process, kind, sha256 of the activities text or None)."""
    ref = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
    with tempfile.TemporaryDirectory(dir="/dev/shm" if os.path.isdir("/dev/shm") else None) as d:
        path = os.path.join(d, "sample.k2jt")
        trace.write(path)
        if os.path.exists(ref):
            cmds = [[ref, path, os.path.join(d, "out%d.json" % i)] for i in range(procs)]
            ps = [subprocess.Popen(c, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True) for c in cmds]
            outs = [p.communicate()[0] for p in ps]
            if any(p.returncode for p in ps):
                raise RuntimeError("ref_driver failed")
            secs = max(json.loads(o.strip().splitlines()[-1])["seconds_mean"] for o in outs)
            digest = None
            if keep_output:
                doc = open(os.path.join(d, "out0.json"), "rb").read()
                span = activities_span(doc) if int(trace.params["mode"][0]) == 1 else None
                digest = (hashlib.sha256(span).hexdigest(), len(span)) if span is not None else None
            kind = "reference"
        else:  # the reference binary is not present: our CPU restatement (one core)
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            import helpers
            t0 = time.perf_counter()
            data, _ = helpers.run_port(trace, path=path)
            secs = time.perf_counter() - t0
            digest = (hashlib.sha256(data).hexdigest(), len(data))
            kind, procs = "port", 1
    return secs, kind, procs, digest


def cupti_record_count(trace):
    """Number of CUPTI records of a generated trace (the generators pack whole records back to back)."""
    from kineto_b200 import tracefile as tf
    view, pos, n, total = memoryview(trace.cupti), 0, 0, len(trace.cupti)
    while pos < total:
        kind = int.from_bytes(view[pos:pos + 4], "little")
        if kind not in tf.RECORD_SIZE:
            break
        pos += (tf.RECORD_SIZE[kind] + 7) & ~7
        n += 1
    return n


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    procs = max(1, min(cores, 32))
    sample_n = min(args.n, max(1000, args.cpu_sample))   # per process: the size the cpu_baseline sample has
    trace = generate(args.workload, sample_n)
    n_rec = cupti_record_count(trace) + len(trace.op_start)
    vals, secs_all = [], []
    kind = "reference"
    for i in range(args.warmup + args.steps):
        secs, kind, used, _ = run_reference_once(trace, procs)
        if i >= args.warmup:
            vals.append(n_rec * used / secs)
            secs_all.append(secs)
    value = statistics.mean(vals)
    cfg = config(args, args.gpus, args.n)
    cfg["reference_sample"] = ("every step: %d concurrent single-threaded reference processes, each over a %s trace of size "
                               "argument %d (%d records), processTrace + save to tmpfs; the reference has no multi-threaded "
                               "path, so its throughput does not depend on the trace's length beyond its hash maps"
                               % (procs, args.workload, sample_n, n_rec))
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(secs_all),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": cfg,
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": procs if kind == "reference" else 1, "kind": kind,
                             "sample": cfg["reference_sample"]},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def fit_n(args, world):
    """Per-GPU size argument, reduced when the host cannot hold the traces and the pinned copies of all ranks."""
    try:
        import psutil
        avail = psutil.virtual_memory().available
    except Exception:  # noqa: BLE001
        return args.n, None
    per_unit = {"mixed": 2300, "kernel_launches": 2700, "op_tree": 3500, "distributed_rank": 2500, "memory_events": 3000,
                "generic": 700}[args.workload]  # host bytes per unit of n: trace + pinned inputs + pinned text (one lane)
    lanes_extra = 1600 if world == 1 else 0     # the second pinned text buffer of the end-to-end leg
    need = world * args.n * (per_unit + lanes_extra)
    if need <= 0.7 * avail:
        return args.n, None
    n = int(0.7 * avail / (world * (per_unit + lanes_extra)))
    return max(n, 10_000), "size argument reduced from %d to fit %.0f GB of free host memory" % (args.n, avail / 1e9)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from kineto_b200 import api, sharding

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n, n_note = fit_n(args, world)
    exchange = world > 1 and args.workload in SHARDED
    depth = 2 if world == 1 else 1  # contexts alternating in the end-to-end leg

    trace = generate(args.workload, n, rank, world if args.workload in SHARDED else 1)
    # one stream for the context's kernels, torch's copies, the NCCL exchange (ordered with the current stream) and the
    # timing events
    stream = torch.cuda.Stream(dev)
    torch.cuda.set_stream(stream)
    ctx = api.K2J(local, stream.cuda_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    exchange_events = []
    exchanges = {}
    kept_fraction = [None]  # filtered exchange: the largest share of its join keys a shard had to send

    def prepare(c, s):
        """segment -> (all-gather join keys): everything before the emit step."""
        if not exchange:
            c.segment(sync=False)
            return
        info = c.segment()
        n_ext, n_ops = int(info.n_external), int(info.n_ops)
        ext_local = api.device_view(info.external_records, n_ext * 2, "<i8", dev)
        ops_local = api.device_view(info.op_ids, n_ops, "<i4", dev)
        x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        x0.record(s)
        if args.exchange == "all" or (args.exchange == "auto" and world < 4):
            ex = exchanges.setdefault(id(c), sharding.JoinExchange(rank, world, dist, dev))
            rows, ext_stride, ops_stride, counts = ex.gather(ext_local, ops_local)
        else:  # only the records another shard can want travel
            ex = exchanges.setdefault(id(c), sharding.FilteredJoinExchange(rank, world, dist, dev))
            ex.exchange(c, info)
            kept_fraction[0] = max(ex.kept_counts) / max(1, ex.ext_stride)
            x1.record(s)
            exchange_events.append((x0, x1))
            return
        x1.record(s)
        exchange_events.append((x0, x1))
        c.set_global_join_rows(rows, ext_stride, ops_stride, counts, world, rank)

    # ---- resident: inputs already in HBM, the text stays in HBM ----
    dev_arrays = api.device_arrays(trace, dev)
    ctx.load(trace, dev_arrays)
    for _ in range(args.warmup):
        prepare(ctx, stream)
        res = ctx.emit()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # before the barrier: its set-up must not delay rank 0 inside the other ranks' timed region
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    stage = {k: 0.0 for k in ("ms_segment", "ms_join", "ms_size", "ms_scan", "ms_emit")}
    launches = 0
    for _ in range(args.steps):
        prepare(ctx, stream)
        res = ctx.emit()
        for k in stage:
            stage[k] += res[k]
        launches += res["kernel_launches"]
    e1.record(stream)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1)
    ms_exchange = sum(a.elapsed_time(b) for a, b in exchange_events[-args.steps:]) / args.steps if exchange else 0.0
    n_records = res["n_records"] + len(trace.op_start)
    out_bytes = res["out_bytes"]
    resident_ptr, _ = ctx.output_ptr()
    resident_text = api.device_view(resident_ptr, out_bytes, "|u1", dev) if out_bytes else None

    # ---- end to end: pinned host buffers in, one pinned host buffer out ----
    # Every step uploads all of its inputs and downloads all of its text inside the timed region; inside a step the
    # text leaves slab by slab while the next slab is written (k2j_emit_to_host).  On one GPU two contexts on two
    # streams alternate, so that one step's download also overlaps the next step's upload.
    ms_e2e, h2d, e2e_equal = None, 0, None
    if not args.no_e2e:
        host = {}
        for k in api.K2J.ARRAYS:
            a = np.ascontiguousarray(getattr(trace, k))
            a = a.view(np.uint8) if a.dtype.fields is not None else a
            a = a.view(np.int64) if a.dtype == np.uint64 else (a.view(np.int32) if a.dtype == np.uint32 else a)
            host[k] = torch.from_numpy(a).pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in host.values())
        lanes = []
        for i in range(depth):
            s_i = stream if i == 0 else torch.cuda.Stream(dev)
            c_i = ctx if i == 0 else api.K2J(local, s_i.cuda_stream)
            lanes.append((c_i, s_i, torch.empty(out_bytes + 4096, dtype=torch.uint8).pin_memory()))

        def e2e_step(i):
            c_i, s_i, out_i = lanes[i % depth]
            with torch.cuda.stream(s_i):
                c_i.load(trace, host)
                prepare(c_i, s_i)
                return c_i.emit_to_host(out_i, SLAB_BYTES)  # returns when the whole text has arrived

        # with two lanes the steps of the two contexts run on two host threads, so that their copies overlap
        def run_e2e(count):
            if depth == 1:
                for i in range(count):
                    e2e_step(i)
                return
            def worker(lane):
                torch.cuda.set_device(local)
                for i in range(lane, count, depth):
                    e2e_step(i)
            ts = [threading.Thread(target=worker, args=(lane,)) for lane in range(depth)]
            for t in ts:
                t.start()
            for t in ts:
                t.join()

        run_e2e(max(depth, min(args.warmup, 3)))
        barrier()
        t0 = time.perf_counter()
        run_e2e(args.steps)
        torch.cuda.synchronize()
        ms_e2e = 1e3 * (time.perf_counter() - t0)  # several streams and threads: host clock around fully drained work
        barrier()
        # the text that arrived on the host is the text of the resident run: length and every byte (checked on the GPU)
        e2e_equal = True
        for _, _, out_i in lanes[:min(depth, args.steps)]:
            chunk = 1 << 30
            for b in range(0, out_bytes, chunk):
                e = min(out_bytes, b + chunk)
                if not torch.equal(out_i[b:e].to(dev, non_blocking=False), resident_text[b:e]):
                    e2e_equal = False
        for c_i, _, _ in lanes[1:]:
            c_i.close()
        del lanes, host

    # ---- max over ranks ----
    if world > 1:
        t = torch.tensor([ms, ms_e2e or 0.0], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e_max = float(t[0]), float(t[1])
        ms_e2e = ms_e2e_max if ms_e2e is not None else None
        tot = torch.tensor([n_records, out_bytes, h2d, int(bool(e2e_equal)) if e2e_equal is not None else 1], dtype=torch.int64, device=dev)
        dist.all_reduce(tot)
        total_records, total_out, total_h2d = int(tot[0]), int(tot[1]), int(tot[2])
        if e2e_equal is not None:
            e2e_equal = int(tot[3]) == world
    else:
        total_records, total_out, total_h2d = n_records, out_bytes, h2d

    if rank == 0:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(peaks_path):
            peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        else:
            peak, peak_src = FALLBACK_HBM_GBS, "fallback"
        emit_ms = stage["ms_emit"] / args.steps
        ops_bytes_in = sum(getattr(trace, k).nbytes for k in ("op_start", "op_end", "op_id", "op_device", "op_resource",
                                                             "op_type", "op_name", "op_flow", "op_flowt", "op_mdoff", "md"))
        ext_bytes = 24 * (res["n_records"] - (res["x_events"] - len(trace.op_start))) if args.workload == "kernel_launches" else 0
        alg_emit = (res["in_bytes"] - ext_bytes) + ops_bytes_in + res["name_bytes"] + out_bytes
        alg_all = res["in_bytes"] + ops_bytes_in + res["name_bytes"] + out_bytes
        achieved = alg_emit / (emit_ms * 1e-3) / 1e9
        value = total_records * args.steps / (ms * 1e-3)
        cfg = config(args, world, n)
        if n_note:
            cfg["note"] = n_note
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u8", "data": "synthetic", "config": cfg, "clocks": clocks,
            "gpu_launches": launches,
            "records_per_step": total_records,
            "output_gb_per_s": total_out * args.steps / (ms * 1e-3) / 1e9,
            "output_bytes_per_step": total_out,
            "roofline": {"bound": "hbm", "kernel": "k_events<true, false> (emit pass)", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": alg_emit, "ms_per_launch": emit_ms,
                         "traffic": (EMIT_TRAFFIC_PER_OUT_BYTE[args.workload] * out_bytes) if args.workload in EMIT_TRAFFIC_PER_OUT_BYTE else None,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch at size argument 1000000, scaled by the text bytes",
                         "pipeline_frac": alg_all / (sum(stage.values()) / args.steps * 1e-3) / 1e9 / peak},
            "stage_ms_per_step": dict({k: v / args.steps for k, v in stage.items()}, ms_exchange=ms_exchange),
            "exchange_keys_sent_fraction": kept_fraction[0],
        }
        if ms_e2e is not None:
            line["e2e"] = {"value": total_records * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                           "h2d_bytes_per_step": total_h2d, "d2h_bytes_per_step": total_out,
                           "output_gb_per_s": total_out * args.steps / (ms_e2e * 1e-3) / 1e9,
                           "contexts": depth, "slab_bytes": SLAB_BYTES, "text_equals_resident_run": e2e_equal,
                           "note": "k2j_emit_to_host: the text leaves the GPU slab by slab while the next slab is written; "
                                   "%d context(s) per GPU; every step moves all of its bytes; host clock around the drained region" % depth}
        if world == 1 and not args.no_cpu_baseline:
            line.update(cpu_baseline_and_parity(args, api, local))
        if args.parity_full and world == 1:
            secs, kind, _, digest = run_reference_once(trace, 1, keep_output=True)
            text = resident_text.cpu().numpy().tobytes()
            line["parity_full"] = {"sha256_match": digest is not None and digest[0] == hashlib.sha256(text).hexdigest(),
                                   "bytes": len(text), "reference_bytes": digest[1] if digest else None,
                                   "reference_seconds": secs, "kind": kind, "trace": "the benchmark trace itself"}
        print(json.dumps(line))
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def save_through_the_reference(args):
    """ActivityTrace::save() of the unmodified reference, once with its own ChromeTraceLogger and once with the
    B200TraceLogger registered in its logger factory, on 250 000 kernel launches (the reference's own replayed
    processTrace() feeds both): seconds of each save() on the third replay of one process, and whether the two files
    are the same bytes.  None when the driver was not built."""
    shim = os.path.join(ROOT, "oracle", "_ref", "shim_driver")
    if not os.path.exists(shim) or args.no_save_e2e:
        return None
    from kineto_b200 import synth
    trace = synth.gen_kernel_launches(250_000, seed=11)
    with tempfile.TemporaryDirectory(dir="/dev/shm" if os.path.isdir("/dev/shm") else None) as d:
        path, ref, mine = (os.path.join(d, f) for f in ("t.k2jt", "ref.json", "b200.json"))
        trace.write(path)
        r = subprocess.run([shim, path, ref, mine, "--repeat", "3"], capture_output=True, text=True)
        if r.returncode:
            return {"error": r.stderr[-300:]}
        info = json.loads(r.stdout.strip().splitlines()[-1])
        a = open(ref, "rb").read().replace(ref.encode(), b"<trace>")
        b = open(mine, "rb").read().replace(mine.encode(), b"<trace>")
    return {"workload": "kernel_launches, size argument 250000", "save_reference_s": info["save_reference_s"],
            "save_b200_s": info["save_b200_s"], "files_equal": a == b, "bytes": len(b), "skipped": info["skipped"]}


def cpu_baseline_and_parity(args, api, device):
    """The reference on one host core over a bounded sample of the same workload, and the same sample through the
    CUDA path: throughput of the former, sha256 of both texts."""
    sample_n = min(args.n, args.cpu_sample)
    sample = generate(args.workload, sample_n)
    unsorted = bool(int(sample.params["flags"][0]) & 2)
    if unsorted:  # the reference has no ordering option: the sample is formatted in buffer order by both sides
        sample.params["flags"] &= ~2
    secs, kind, _, digest = run_reference_once(sample, 1, keep_output=True)
    text, r = api.process(sample, device=device)
    n_rec = r["n_records"] + len(sample.op_start)
    out = {"cpu_baseline": {"value": n_rec / secs, "unit": UNIT, "cores": 1, "kind": kind,
                            "sample": "%s trace of size argument %d (%d records, %d bytes of text), one single-threaded process "
                                      "(the reference path is single-threaded), %.1f s, output on tmpfs"
                                      % (args.workload, sample_n, n_rec, len(text), secs)}}
    out["cpu_baseline"]["save_e2e"] = save_through_the_reference(args)
    if digest is not None:
        out["parity"] = {"sha256_match": digest[0] == hashlib.sha256(text).hexdigest(), "bytes": len(text),
                         "reference_bytes": digest[1],
                         "sample": "the cpu_baseline sample (same generator, size argument %d%s)"
                                   % (sample_n, ", without the ordering option, which the reference does not have" if unsorted else ""),
                         "checker": kind}
    return out


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
