"""Drop-in check of the C++ logger shim: the unmodified reference's processTrace + ActivityTrace::save()
with B200TraceLogger registered in its ActivityLoggerFactory must write the same FILE, byte for byte,
as with the reference's own ChromeTraceLogger (only the trace name, which is the path, differs)."""
import json
import os
import subprocess

import pytest

import cases
import helpers
from kineto_b200 import synth

pytestmark = pytest.mark.gpu
SHIM = os.path.join(helpers.ROOT, "oracle", "_ref", "shim_driver")


@pytest.mark.skipif(not os.path.exists(SHIM), reason="oracle/_ref/shim_driver not built (needs the reference tree)")
@pytest.mark.parametrize("gen", [
    lambda: synth.gen_kernel_launches(3000, seed=401, pool_size=100, user_annotations=12),
    lambda: synth.gen_mixed(8000, seed=402, pool_size=300, escape_fraction=0.1),
    lambda: cases.edge_trace(flags=1),
    cases.annotation_trace,
    lambda: cases.tsc_trace(1500),
    cases.sync_trace,
    lambda: cases.sync_mix_trace(6000, seed=48),
    lambda: cases.collective_trace(300, seed=55),
    lambda: cases.without_flags(synth.gen_distributed_rank(5000, rank=1, seed=403, pool_size=100)),
    cases.instant_trace,
    # more than 50 000 wrappers: the logger packs them on several threads and merges the pieces in order
    lambda: synth.gen_mixed(150_000, seed=404, pool_size=800, escape_fraction=0.05),
    lambda: cases.sync_mix_trace(90_000, seed=49),
    lambda: cases.without_flags(synth.gen_distributed_rank(60_000, rank=3, seed=405, pool_size=300)),
], ids=["launches_annot", "mixed", "edge", "annotations", "tsc", "sync", "sync_mix", "collectives", "distributed_rank", "instant",
        "mixed_threads", "sync_mix_threads", "distributed_rank_threads"])
def test_logger_shim_writes_the_reference_file(gen, tmp_path):
    trace = gen()
    p = str(tmp_path / "t.k2jt")
    trace.write(p)
    ref, mine = str(tmp_path / "ref.json"), str(tmp_path / "b200.json")
    r = subprocess.run([SHIM, p, ref, mine], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    info = json.loads(r.stdout.strip().splitlines()[-1])
    assert info["skipped"] == 0
    a = open(ref, "rb").read().replace(ref.encode(), b"<trace>")
    b = open(mine, "rb").read().replace(mine.encode(), b"<trace>")
    assert len(a) > 1000
    assert a == b, helpers.first_diff(a, b)
