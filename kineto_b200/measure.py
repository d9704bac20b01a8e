"""Stage times of the CUDA path on the other synthetic workloads (the benchmark itself, bench.py, times the
kernel-launches workload only).  One GPU, inputs resident in HBM, best of a few runs:

    python -m kineto_b200.measure --workload mixed --n 3000000
"""
from __future__ import annotations

import argparse
import json

from . import api, synth

WORKLOADS = {
    "mixed": lambda n: synth.gen_mixed(n, seed=3),
    "op_tree": lambda n: synth.gen_op_tree(n, seed=4),
    "distributed_rank": lambda n: synth.gen_distributed_rank(n, rank=0, seed=5),
    "memory_events": lambda n: synth.gen_kernel_launches(n, seed=2, memory_events=0.5),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", choices=sorted(WORKLOADS), required=True)
    ap.add_argument("--n", type=int, default=1_000_000, help="size argument of the generator")
    ap.add_argument("--runs", type=int, default=5)
    args = ap.parse_args()
    trace = WORKLOADS[args.workload](args.n)
    ctx = api.K2J(0)
    try:
        ctx.load(trace, api.device_arrays(trace, "cuda:0"))
        best = None
        for _ in range(args.runs):
            res = ctx.run()
            if best is None or res["ms_total"] < best["ms_total"]:
                best = res
    finally:
        ctx.close()
    records = best["n_records"] + len(trace.op_start)
    out = {"workload": args.workload, "n": args.n, "records": records, "out_bytes": best["out_bytes"],
           "records_per_s": records / (best["ms_total"] * 1e-3), "out_gb_per_s": best["out_bytes"] / (best["ms_total"] * 1e6),
           "kernel_launches": best["kernel_launches"]}
    out.update({k: round(best[k], 4) for k in ("ms_segment", "ms_join", "ms_size", "ms_scan", "ms_emit", "ms_total")})
    print(json.dumps(out))


if __name__ == "__main__":
    main()
