"""Benchmark of the trace post-processing hot path.

    python bench.py --gpus N --steps K --warmup W            # this library (CUDA, sm_100a)
    python bench.py --impl reference --gpus N --steps K ...   # the reference's CPU path on host cores

Workload (config.workload): the "kernel launches" configuration — per GPU 1 000 000 CUpti_ActivityKernel9
records + 1 000 000 cudaLaunchKernel runtime records + 1 000 000 EXTERNAL_CORRELATION records +
1 000 000 CPU ops, correlation ids shuffled by a seeded permutation, 8 devices x 32 streams, a pool
of 4096 kernel names of 20-400 bytes; full join + timestamp handling + Chrome-trace JSON.  Seeded
synthetic data stands in for a real capture.  With N > 1 the trace is N times as long and sharded by
contiguous record range, one shard per GPU (weak scaling); the shards exchange their
EXTERNAL_CORRELATION records and CPU-op ids with NCCL so the join covers the whole trace.

One "step" = one pass of the path over the shard.  `value` counts input records (CUPTI records + CPU
ops) per second with the inputs already resident in HBM; `e2e` is the same through the C ABI with
pinned HOST buffers, host->device and device->host copies inside the timed region.
"""
from __future__ import annotations

import argparse
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
# dram__bytes_read.sum + dram__bytes_write.sum of one k_events<true> launch divided by the JSON bytes
# it wrote, from the ncu capture summarised in profiles/ (None until a capture exists).
EMIT_TRAFFIC_PER_OUT_BYTE = 1.036  # dram read+write of the emit launch per output byte (ncu, profiles/event_kernels_kernel_launches_100k.txt)


E2E_DEPTH = 2  # contexts alternating in the end-to-end leg


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--launches", type=int, default=1_000_000, help="kernel launches per GPU")
    ap.add_argument("--cpu-sample", type=int, default=250_000, help="launches in the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def config(args, world):
    return {"workload": "kernel_launches: per GPU %d Kernel9 + %d cudaLaunchKernel + %d EXTERNAL_CORRELATION records"
                        " + %d CPU ops, shuffled correlation ids, 8 devices x 32 streams, 4096 names of 20-400 B"
                        % ((args.launches,) * 4),
            "launches_per_gpu": args.launches, "sharding": "contiguous record range, %d shard(s)" % world,
            "l2": "inputs (272 MB/GPU) and output (1.86 GB/GPU) exceed the 126 MB L2; no flush needed",
            "seed": 2}


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


def make_shard(args, rank, world):
    from kineto_b200 import synth
    return synth.gen_kernel_launches(args.launches, seed=2, shard=(rank, world))


# ------------------------------------------------------------------------------------------------
# reference arm: the reference's own CPU code (oracle/_ref/ref_driver), all host cores
# ------------------------------------------------------------------------------------------------
def reference_records_per_sec(sample_launches, procs, repeat=1):
    """Runs `procs` concurrent reference processes, each over its own copy of a sample trace of the
    workload; returns (aggregate records/s, seconds, records per process, kind)."""
    from kineto_b200 import synth
    ref = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
    trace = synth.gen_kernel_launches(sample_launches, seed=2)
    n_rec = sample_launches * 4
    with tempfile.TemporaryDirectory(dir="/dev/shm" if os.path.isdir("/dev/shm") else None) as d:
        path = os.path.join(d, "sample.k2jt")
        trace.write(path)
        if os.path.exists(ref):
            cmds = [[ref, path, os.path.join(d, "out%d.json" % i), "--repeat", str(repeat)] for i in range(procs)]
            ps = [subprocess.Popen(c, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True) for c in cmds]
            outs = [p.communicate()[0] for p in ps]
            if any(p.returncode for p in ps):
                raise RuntimeError("ref_driver failed")
            secs = max(json.loads(o.strip().splitlines()[-1])["seconds_mean"] for o in outs)
            return n_rec * procs / secs, secs, n_rec, "reference"
        # the reference binary is not present: time our CPU restatement instead (one core)
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import helpers
        t0 = time.perf_counter()
        helpers.run_port(trace, path=path)
        secs = time.perf_counter() - t0
        return n_rec / secs, secs, n_rec, "port"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    procs = max(1, min(cores, 32))
    sample = min(args.launches, 50_000)
    vals, secs_all = [], []
    kind = "reference"
    for i in range(args.warmup + args.steps):
        v, secs, n_rec, kind = reference_records_per_sec(sample, procs)
        if i >= args.warmup:
            vals.append(v)
            secs_all.append(secs)
    value = statistics.mean(vals)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(secs_all),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": config(args, args.gpus),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": procs if kind == "reference" else 1, "kind": kind,
                             "sample": "%d concurrent single-threaded reference processes, each %d launches "
                                       "(%d records) of the workload, processTrace + save to tmpfs" % (procs, sample, sample * 4)},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
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

    trace = make_shard(args, rank, world)
    stream = torch.cuda.current_stream()
    ctx = api.K2J(local, stream.cuda_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    exchange_events = []

    def exchange_and_emit(ctx=ctx, stream=stream):
        """segment -> (all-gather join keys) -> emit; returns the result dict."""
        if world == 1:
            return ctx.run()
        info = ctx.segment()
        n_ext, n_ops = int(info.n_external), int(info.n_ops)
        ext_local = api.device_view(info.external_records, n_ext * 2, "<i8", dev)
        ops_local = api.device_view(info.op_ids, n_ops, "<i4", dev)
        x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        x0.record(stream)
        ext_all, ops_all, own_begin = sharding.gather_join_keys(ext_local, ops_local, rank, world, dist)
        x1.record(stream)
        exchange_events.append((x0, x1))
        ctx.set_global_join(ext_all, ext_all.numel() // 2, own_begin, ops_all, ops_all.numel())
        return ctx.emit()

    # ---- resident: inputs already in HBM ----
    dev_arrays = api.device_arrays(trace, dev)
    ctx.load(trace, dev_arrays)
    for _ in range(args.warmup):
        res = exchange_and_emit()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # before the barrier: its set-up must not delay rank 0 inside the other ranks' timed region
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    stage = {k: 0.0 for k in ("ms_segment", "ms_join", "ms_size", "ms_scan", "ms_emit")}
    launches = 0
    for _ in range(args.steps):
        res = exchange_and_emit()
        for k in stage:
            stage[k] += res[k]
        launches += res["kernel_launches"]
    e1.record(stream)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1)
    ms_exchange = sum(a.elapsed_time(b) for a, b in exchange_events[-args.steps:]) / args.steps if world > 1 else 0.0
    n_records = res["n_records"] + len(trace.op_start)

    # ---- end to end: pinned host buffers in, pinned host buffers out ----
    # Two contexts on two streams alternate: while the text of one step travels to the host, the next
    # step's inputs travel to the device and are formatted.  Every step still uploads all of its
    # inputs and downloads all of its output inside the timed region.
    host = {}
    for k in api.K2J.ARRAYS:
        a = np.ascontiguousarray(getattr(trace, k))
        a = a.view(np.uint8) if a.dtype.fields is not None else a
        a = a.view(np.int64) if a.dtype == np.uint64 else (a.view(np.int32) if a.dtype == np.uint32 else a)
        host[k] = torch.from_numpy(a).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    lanes = []
    for i in range(E2E_DEPTH):
        s_i = stream if i == 0 else torch.cuda.Stream(dev)
        c_i = ctx if i == 0 else api.K2J(local, s_i.cuda_stream)
        lanes.append((c_i, s_i, torch.empty(res["out_bytes"] + 4096, dtype=torch.uint8).pin_memory()))

    def e2e_step(i):
        c_i, s_i, out_i = lanes[i % E2E_DEPTH]
        with torch.cuda.stream(s_i):
            c_i.synchronize()  # the copy this lane started E2E_DEPTH steps ago has landed
            c_i.load(trace, host)
            r = exchange_and_emit(c_i, s_i)
            c_i.copy_output_async(out_i)
        return r

    def e2e_drain():
        for c_i, _, _ in lanes:
            c_i.synchronize()

    for i in range(max(E2E_DEPTH, args.warmup - 1)):
        e2e_step(i)
    e2e_drain()
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        r2 = e2e_step(i)
    e2e_drain()
    torch.cuda.synchronize()
    ms_e2e = 1e3 * (time.perf_counter() - t0)  # several streams: host clock around fully drained work
    barrier()
    for _, _, out_i in lanes[:min(E2E_DEPTH, args.steps)]:
        assert bytes(out_i[:64].numpy().tobytes()).startswith(b'\n  {\n    "ph": "X"')
    for c_i, _, _ in lanes[1:]:
        c_i.close()

    # ---- max over ranks ----
    if world > 1:
        t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
        tot = torch.tensor([n_records, res["out_bytes"], h2d], dtype=torch.int64, device=dev)
        dist.all_reduce(tot)
        total_records, total_out, total_h2d = int(tot[0]), int(tot[1]), int(tot[2])
    else:
        total_records, total_out, total_h2d = n_records, res["out_bytes"], h2d

    if rank == 0:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(peaks_path):
            peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        else:
            peak, peak_src = FALLBACK_HBM_GBS, "fallback"
        emit_ms = stage["ms_emit"] / args.steps
        ops_bytes_in = sum(getattr(trace, k).nbytes for k in ("op_start", "op_end", "op_id", "op_device", "op_resource",
                                                             "op_type", "op_name", "op_flow", "op_flowt", "op_mdoff", "md"))
        ext_bytes = 24 * (res["n_records"] - (res["x_events"] - len(trace.op_start)))
        alg_emit = (res["in_bytes"] - ext_bytes) + ops_bytes_in + res["name_bytes"] + res["out_bytes"]
        alg_all = res["in_bytes"] + ops_bytes_in + res["name_bytes"] + res["out_bytes"]
        achieved = alg_emit / (emit_ms * 1e-3) / 1e9
        value = total_records * args.steps / (ms * 1e-3)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u8", "data": "synthetic", "config": config(args, world), "clocks": clocks,
            "e2e": {"value": total_records * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": total_h2d, "d2h_bytes_per_step": total_out,
                    "output_gb_per_s": total_out * args.steps / (ms_e2e * 1e-3) / 1e9,
                    "contexts": E2E_DEPTH,
                    "note": "%d contexts alternate so that one step's download overlaps the next step's upload and "
                            "kernels; every step moves all of its bytes; host clock around the drained region" % E2E_DEPTH},
            "gpu_launches": launches,
            "output_gb_per_s": total_out * args.steps / (ms * 1e-3) / 1e9,
            "output_bytes_per_step": total_out,
            "roofline": {"bound": "hbm", "kernel": "k_events<true> (emit pass)", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": alg_emit, "ms_per_launch": emit_ms,
                         "traffic": (EMIT_TRAFFIC_PER_OUT_BYTE * res["out_bytes"]) if EMIT_TRAFFIC_PER_OUT_BYTE else None,
                         "pipeline_frac": alg_all / (sum(stage.values()) / args.steps * 1e-3) / 1e9 / peak},
            "stage_ms_per_step": dict({k: v / args.steps for k, v in stage.items()}, ms_exchange=ms_exchange),
        }
        if world == 1 and not args.no_cpu_baseline:
            v, secs, n_rec, kind = reference_records_per_sec(min(args.cpu_sample, args.launches), 1)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": 1, "kind": kind,
                                    "sample": "%d launches (%d records) of the same workload, one single-threaded "
                                              "process (the reference path is single-threaded), %.1f s, output on tmpfs"
                                              % (min(args.cpu_sample, args.launches), n_rec, secs)}
        print(json.dumps(line))
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
