"""Parity of the CUDA path (through the C ABI) with the CPU checkers, on a real GPU."""
import hashlib
import os

import numpy as np
import pytest

import cases
import helpers
from kineto_b200 import synth
from kineto_b200 import tracefile as tf

pytestmark = pytest.mark.gpu

GOLDEN = sorted(f[:-5] for f in os.listdir(helpers.GOLDEN) if f.endswith(".k2jt"))
UNSUPPORTED_ON_GPU = set()


def gpu_run(trace, **kw):
    from kineto_b200 import api
    return api.process(trace, **kw)


def check_counters(res, stats, trace):
    assert res["x_events"] == stats["x_events"]
    assert res["flow_events"] == stats["flow_events"]
    assert res["n_records"] == stats["records"]
    assert res["out_of_range_events"] == stats["out_of_range"]
    assert res["blocklisted_runtime_events"] == stats["blocklisted_runtime"]
    assert res["invalid_external_correlation_events"] == stats["invalid_external_correlation"]
    assert res["unexpected_cuda_events"] == stats["unexpected"]
    assert res["ops_bytes"] == stats["ops_end"]
    assert res["out_bytes"] - res["annotation_bytes"] == stats["gpu_end"]
    assert res["kernel_launches"] > 0


@pytest.mark.parametrize("name", [g for g in GOLDEN if g not in UNSUPPORTED_ON_GPU])
def test_gpu_matches_reference_golden(name):
    trace = tf.Trace.read(os.path.join(helpers.GOLDEN, name + ".k2jt"))
    want = open(os.path.join(helpers.GOLDEN, name + ".ref.json"), "rb").read()
    got, res = gpu_run(trace)
    assert got == want, helpers.first_diff(want, got)
    _, stats = helpers.run_port(trace)
    check_counters(res, stats, trace)


@pytest.mark.parametrize("gen", [
    lambda: synth.gen_generic_kernels(50_000, seed=201),
    lambda: synth.gen_kernel_launches(100_000, seed=202, pool_size=1000, orphan_fraction=0.05),
    lambda: synth.gen_kernel_launches(30_000, seed=203, pool_size=300, shard=(2, 4)),
    lambda: synth.gen_mixed(200_000, seed=204, pool_size=5000, escape_fraction=0.05),
    lambda: synth.gen_mixed(50_000, seed=205, pool_size=500, buffer_bytes=4096 + 64),
    lambda: cases.tsc_trace(40_000),
    cases.edge_trace,
    lambda: cases.edge_trace(flags=1),
    cases.annotation_trace,
    lambda: cases.overhead_mix_trace(60_000, seed=42),
    lambda: cases.with_flags(cases.overhead_mix_trace(20_000, seed=43), tf.FLAG_SORT_BY_START),
    lambda: synth.gen_kernel_launches(60_000, seed=206, pool_size=300, user_annotations=40),
    lambda: cases.with_flags(synth.gen_kernel_launches(70_000, seed=207, pool_size=300), tf.FLAG_SORT_BY_START),
    lambda: cases.with_flags(synth.gen_mixed(120_000, seed=208, pool_size=900), tf.FLAG_SORT_BY_START),
    lambda: cases.with_flags(synth.gen_kernel_launches(20_000, seed=209, pool_size=100, user_annotations=15), tf.FLAG_SORT_BY_START),
    lambda: cases.with_flags(cases.tsc_trace(9_000), tf.FLAG_SORT_BY_START),
    lambda: cases.with_flags(cases.annotation_trace(), tf.FLAG_SORT_BY_START),
    cases.sync_trace,
    lambda: cases.sync_mix_trace(40_000, seed=45),
    lambda: cases.sync_mix_trace(9_000, seed=46, flags=1),
    lambda: cases.with_flags(cases.sync_trace(), tf.FLAG_SORT_BY_START),
    lambda: cases.with_flags(cases.sync_mix_trace(30_000, seed=47), tf.FLAG_SORT_BY_START),
    lambda: synth.gen_op_tree(60_000, seed=210, pool_size=500, n_shapes=256),
    lambda: cases.collective_trace(3000, seed=53),
    lambda: cases.with_flags(cases.collective_trace(500, seed=54), tf.FLAG_SORT_BY_START),
    lambda: synth.gen_distributed_rank(80_000, rank=2, seed=211, pool_size=500),
    lambda: cases.without_flags(synth.gen_distributed_rank(30_000, rank=7, seed=212, pool_size=300)),
    cases.instant_trace,
    lambda: synth.gen_kernel_launches(20_000, seed=213, pool_size=100, memory_events=0.5),
], ids=["generic", "launches", "shard", "mixed", "mixed_small_buffers", "tsc", "edge", "edge_annot", "annotations",
        "overhead_mix", "sorted_overhead_mix", "launches_annot", "sorted_launches", "sorted_mixed", "sorted_annot", "sorted_tsc", "sorted_small",
        "sync", "sync_mix", "sync_mix_annot", "sorted_sync", "sorted_sync_mix", "op_tree", "collectives", "sorted_collectives", "distributed_rank_sorted", "distributed_rank", "instant", "launches_memory_events"])
def test_gpu_matches_port(gen):
    trace = gen()
    want, stats = helpers.run_port(trace)
    got, res = gpu_run(trace)
    assert got == want, helpers.first_diff(want, got)
    check_counters(res, stats, trace)


def test_device_resident_inputs_and_context_reuse():
    """Inputs already in HBM give the same bytes as host inputs; a context can be reused."""
    from kineto_b200 import api
    t1 = synth.gen_mixed(30_000, seed=301, pool_size=300)
    t2 = synth.gen_kernel_launches(8_000, seed=302, pool_size=100)
    want1, _ = helpers.run_port(t1)
    want2, _ = helpers.run_port(t2)
    ctx = api.K2J(0)
    try:
        ctx.load(t1)
        ctx.run()
        assert ctx.copy_output().tobytes() == want1
        ctx.load(t2, api.device_arrays(t2, "cuda:0"))
        for _ in range(2):
            ctx.run()
            assert ctx.copy_output().tobytes() == want2
        ctx.load(t1, api.device_arrays(t1, "cuda:0"))
        ctx.run()
        assert ctx.copy_output().tobytes() == want1
    finally:
        ctx.close()


def test_write_output_streams_the_same_bytes(tmp_path):
    """k2j_write_output: text larger than its staging chunks, a small one and an empty one arrive in the file as
    copy_output returns them, appended at the descriptor's position; a bad descriptor is an I/O error."""
    from kineto_b200 import api
    ctx = api.K2J(0)
    try:
        path = str(tmp_path / "out.json")
        want = b"header"
        with open(path, "wb") as f:
            f.write(b"header")
            f.flush()
            for trace in (synth.gen_kernel_launches(30_000, seed=303, pool_size=200), cases.edge_trace(), synth.TraceBuilder().build()):
                ctx.load(trace)
                ctx.run()
                text = ctx.copy_output().tobytes()
                assert ctx.write_output(f.fileno()) == len(text)
                want += text
        assert len(want) > (48 << 20)   # several 16 MiB chunks
        assert open(path, "rb").read() == want
        # positioned range writes: the text's two halves, second half first, behind a gap
        ctx.load(synth.gen_kernel_launches(30_000, seed=304, pool_size=200))
        res = ctx.run()
        text = ctx.copy_output().tobytes()
        cut = res["ops_bytes"]
        p2 = str(tmp_path / "at.json")
        fd = os.open(p2, os.O_WRONLY | os.O_CREAT)
        ctx.write_output_at(fd, 100 + cut, cut, len(text) - cut)
        ctx.write_output_at(fd, 100, 0, cut)
        ctx.write_output_at(fd, 0, 0, 0)
        os.close(fd)
        assert open(p2, "rb").read() == bytes(100) + text
        with pytest.raises(api.K2JError):
            ctx.write_output_at(1, 0, len(text), 1)   # range outside the output
        r, w = os.pipe()
        os.close(w); os.close(r)
        ctx.load(cases.edge_trace())
        ctx.run()
        with pytest.raises(api.K2JError) as e:
            ctx.write_output(r)
        assert e.value.status == 6
    finally:
        ctx.close()


def test_bench_runs_another_workload():
    """bench.py --workload: one JSON line with the contract's keys for a workload other than the default, small
    enough for a test, with the text that travelled to the host equal to the resident run's and the sha256 of the
    sample equal to the reference's (or, without the reference build, to the CPU restatement's)."""
    import json
    import subprocess
    import sys
    r = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "bench.py"), "--workload", "distributed_rank", "--size", "20000",
                        "--steps", "2", "--warmup", "3", "--cpu-sample", "5000"], capture_output=True, text=True, cwd=helpers.ROOT)
    assert r.returncode == 0, r.stderr[-1000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["records_per_step"] == 80_000 and line["stage_ms_per_step"]["ms_emit"] > 0 and line["output_bytes_per_step"] > 10_000_000
    assert line["e2e"]["text_equals_resident_run"] is True and line["e2e"]["d2h_bytes_per_step"] == line["output_bytes_per_step"]
    assert line["parity"]["sha256_match"] is True and line["cpu_baseline"]["value"] > 0
    assert line["roofline"]["frac"] > 0 and line["gpu_launches"] > 0


def test_empty_and_degenerate_inputs():
    from kineto_b200 import api
    b = synth.TraceBuilder()
    out, res = api.process(b.build())                      # nothing at all
    assert out == b"" and res["out_bytes"] == 0
    b = synth.TraceBuilder()
    b.op(b.t0 + 1, b.t0 + 2, 1, "only an op")
    t = b.build()
    assert api.process(t)[0] == helpers.run_port(t)[0]
    b = synth.TraceBuilder()
    b.extcorr(1, 1)                                        # records that emit nothing
    b.runtime(b.t0 + 1, b.t0 + 2, 1, cbid=synth.CBID_cudaGetLastError)
    t = b.build()
    out, res = api.process(t)
    assert out == b"" and res["blocklisted_runtime_events"] == 1
    b = synth.TraceBuilder()
    b.raw_record(99, 64)                                   # a buffer that starts with an unknown kind
    t = b.build()
    out, res = api.process(t)
    assert out == b"" and res["unexpected_cuda_events"] == 1


def test_error_behaviour():
    from kineto_b200 import api
    ctx = api.K2J(0)
    try:
        with pytest.raises(api.K2JError) as e:
            ctx.run()
        assert e.value.status == 4                         # STATE: no params yet
        t = synth.gen_kernel_launches(100, seed=1, pool_size=10)
        bad = t.buftab.copy()
        bad[0] = 4                                         # misaligned buffer offset
        ctx.set_params(t)
        a = {k: np.ascontiguousarray(getattr(t, k)) for k in api.K2J.ARRAYS}
        with pytest.raises(api.K2JError) as e:
            ctx.set_arrays(a, bad, t.tidmap)
        assert e.value.status == 1
        bad = t.buftab.copy()
        bad[1] = len(t.cupti) + 8                          # buffer past the end
        with pytest.raises(api.K2JError) as e:
            ctx.set_arrays(a, bad, t.tidmap)
        assert e.value.status == 1
        # string id out of range -> the kernels' own check trips, the context stays usable
        k = t.cupti.copy()
        k[64 + 104:64 + 112].view(np.uint64)[0] = 1 << 20  # name field of the first kernel record (after 24 + 40 bytes)
        a2 = dict(a, cupti=k)
        ctx.set_arrays(a2, t.buftab, t.tidmap)
        with pytest.raises(api.K2JError) as e:
            ctx.run()
        assert e.value.status == 5
        # a CPU activity type libkineto does not define
        a3 = dict(a, op_type=np.full(len(t.op_type), 40, np.int32))
        ctx.set_arrays(a3, t.buftab, t.tidmap)
        with pytest.raises(api.K2JError) as e:
            ctx.run()
        assert e.value.status == 5
        ctx.set_arrays(a, t.buftab, t.tidmap)
        ctx.run()
        assert ctx.copy_output().tobytes() == helpers.run_port(t)[0]
    finally:
        ctx.close()


def test_error_behaviour_of_the_sharding_entry_points():
    """Call order and argument checks of the entry points for sharded traces: a status, never a fault."""
    import torch
    from kineto_b200 import api
    t = synth.gen_kernel_launches(2000, seed=3, pool_size=20)
    ctx = api.K2J(0)
    try:
        ctx.load(t)
        bits = torch.zeros(1 << 17, dtype=torch.uint8, device="cuda:0")
        torch.cuda.synchronize()
        for call in (lambda: ctx.export_lookup_records(), lambda: ctx.join_need_bits(bits),
                     lambda: ctx.op_id_bits(0, torch.zeros(64, dtype=torch.int64, device="cuda:0"))):
            with pytest.raises(api.K2JError) as e:
                call()
            assert e.value.status == 4                     # STATE: not segmented yet
        with pytest.raises(api.K2JError) as e:
            ctx.partial_spans()
        assert e.value.status == 4                         # STATE: no run yet
        info = ctx.segment()
        with pytest.raises(api.K2JError) as e:
            ctx.join_need_bits(bits[:1000])                # not a power of two
        assert e.value.status == 1
        for front, back in ((4, len(t.cupti)), (len(t.cupti), 8), (0, len(t.cupti) + 8), (8, len(t.cupti))):
            with pytest.raises(api.K2JError) as e:
                ctx.set_guest_ranges(front, back)          # misaligned, crossing, past the end, through a buffer
            assert e.value.status == 1
        with pytest.raises(api.K2JError) as e:
            ctx.set_guest_ops(t.n_ops + 1)
        assert e.value.status == 1
        with pytest.raises(api.K2JError) as e:
            ctx.set_global_op_bits(bits.data_ptr(), 64, torch.zeros(2, dtype=torch.int64, device="cuda:0"))
        assert e.value.status == 4                         # STATE: no gathered rows yet
        ptr, n = ctx.export_lookup_records()               # no synchronisation records: the first writers of contexts and streams only
        assert n > 0 and n % 8 == 0
        with pytest.raises(api.K2JError) as e:
            ctx.append_spans(np.zeros(0, api.SPAN))
        assert e.value.status == 4                         # STATE: nothing emitted yet
        ctx.emit()                                         # still one shard: k2j_run's result
        bad = np.zeros(1, api.SPAN)
        bad["op_row"] = t.n_ops
        with pytest.raises(api.K2JError) as e:
            ctx.append_spans(bad)
        assert e.value.status == 1
        assert ctx.append_spans(np.zeros(0, api.SPAN)) == 0
        assert ctx.copy_output().tobytes() == helpers.run_port(t)[0] and int(info.n_ops) == t.n_ops
    finally:
        ctx.close()


@pytest.mark.parametrize("n", [1, 255, 2048, 2049, 1_000_003])
def test_exclusive_scan_entry_point(n):
    import torch
    from kineto_b200 import api
    rng = np.random.default_rng(n)
    sizes = rng.integers(0, 5000, n).astype(np.int32)
    sizes[rng.integers(0, n, max(1, n // 50))] = 0
    ctx = api.K2J(0)
    try:
        d_sizes = torch.from_numpy(sizes).cuda()
        d_off = torch.empty(n, dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()  # the context scans on its own stream: its inputs must be complete first
        total = ctx.exclusive_scan(d_sizes, d_off)
        want = np.concatenate([[0], np.cumsum(sizes.astype(np.int64))])
        assert total == want[-1]
        assert (d_off.cpu().numpy() == want[:-1]).all()
    finally:
        ctx.close()


@pytest.mark.parametrize("n_shards", [3, 5])
def test_sharded_runs_concatenate_to_the_whole(n_shards):
    """Size-independent property at the benchmark's full size: processing contiguous buffer ranges
    separately, with the join arrays gathered from all of them, gives exactly the bytes of one run
    over the whole trace (events are emitted in record order and depend only on the record and the
    join).  With five shards the gathered keys pass through the per-shard key filter."""
    import torch
    from kineto_b200 import api
    n = 1_000_000
    t = synth.gen_kernel_launches(n, seed=2)
    ctx = api.K2J(0)
    try:
        ctx.load(t, api.device_arrays(t, "cuda:0"))
        res = ctx.run()
        assert res["x_events"] == 3 * n and res["flow_events"] == 2 * n and res["n_records"] == 3 * n
        whole = ctx.copy_output()
        h_whole = hashlib.sha256(whole.tobytes()).hexdigest()
        # closed-form check of the first events against the CPU checker on a prefix of the trace
        nb = t.n_buffers
        parts = []
        bt = t.buftab.reshape(-1, 2)
        cuts = [nb * i // n_shards for i in range(n_shards + 1)]
        op_cuts = [0] + [n * (i + 1) // (n_shards + 1) for i in range(n_shards - 1)] + [n]
        infos = []
        ctxs = [api.K2J(0) for _ in range(n_shards)]
        try:
            for i, c in enumerate(ctxs):
                sub = tf.Trace(**{attr: getattr(t, attr) for _, attr, _ in tf._SECTIONS})
                sub.buftab = bt[cuts[i]:cuts[i + 1]].reshape(-1).copy()
                lo, hi = op_cuts[i], op_cuts[i + 1]
                for col in ("op_start", "op_end", "op_id", "op_device", "op_resource", "op_thread", "op_type", "op_name",
                            "op_flow", "op_flowt"):
                    setattr(sub, col, getattr(t, col)[lo:hi].copy())
                mo = t.op_mdoff[lo:hi + 1]
                sub.md = t.md[mo[0]:mo[-1]].copy()
                sub.op_mdoff = (mo - mo[0]).astype(np.uint32)
                c.load(sub)
                infos.append(c.segment())
            def view(ptr, n_items, ts):
                return api.device_view(ptr, n_items, ts).clone()
            ext = torch.cat([view(i.external_records, int(i.n_external) * 2, "<i8") for i in infos])
            ops = torch.cat([view(i.op_ids, int(i.n_ops), "<i4") for i in infos])
            torch.cuda.synchronize()  # the gathered arrays were built on torch's stream; the contexts read them on theirs
            begin = 0
            for c, i in zip(ctxs, infos):
                c.set_global_join(ext, ext.numel() // 2, begin, ops, ops.numel())
                begin += int(i.n_external)
                c.emit()
                parts.append(c.copy_output().tobytes())
            # the same join keys as the equal-sized rows an all-gather leaves (sharding.JoinExchange), read in place
            ext_stride = max(int(i.n_external) for i in infos) + 7
            ops_stride = (max(int(i.n_ops) for i in infos) + 9) & ~1
            words = ext_stride * 2 + ops_stride // 2
            rows = torch.zeros(words * n_shards, dtype=torch.int64, device="cuda:0")
            counts = torch.zeros(2 * n_shards, dtype=torch.int64, device="cuda:0")
            pos_e = pos_o = 0
            for r, i in enumerate(infos):
                ne, no = int(i.n_external), int(i.n_ops)
                row = rows[r * words:(r + 1) * words]
                row[:ne * 2] = ext[pos_e * 2:(pos_e + ne) * 2]
                row[ext_stride * 2:].view(torch.int32)[:no] = ops[pos_o:pos_o + no]
                counts[2 * r], counts[2 * r + 1] = ne, no
                pos_e += ne
                pos_o += no
            torch.cuda.synchronize()
            for r, c in enumerate(ctxs):
                c.segment()
                c.set_global_join_rows(rows, ext_stride, ops_stride, counts, n_shards, r)
                res_rows = c.emit()
                assert c.copy_output().tobytes() == parts[r], "rows of shard %d" % r
                assert res_rows["invalid_external_correlation_events"] == 0
            # and with rows that hold, per shard, only the records another shard can want (k2j_join_need_bits,
            # k2j_filter_join_keys; sharding.FilteredJoinExchange does this with collectives)
            n_bits = 1 << 24
            need = torch.empty(n_bits // 8 * n_shards, dtype=torch.uint8, device="cuda:0")
            for r, c in enumerate(ctxs):
                c.segment()
                c.join_need_bits(need[r * (n_bits // 8):(r + 1) * (n_bits // 8)])
            kept, n_kept = [], []
            for r, (c, i) in enumerate(zip(ctxs, infos)):
                out = torch.empty(max(1, int(i.n_external)) * 2, dtype=torch.int64, device="cuda:0")
                n_out = torch.zeros(1, dtype=torch.int64, device="cuda:0")
                c.filter_join_keys(need, n_shards, r, out, n_out)
                c.synchronize()
                kept.append(out)
                n_kept.append(int(n_out.item()))
            assert all(0 < k <= int(i.n_external) for k, i in zip(n_kept, infos))
            cap = max(n_kept) + 3
            words = cap * 2 + ops_stride // 2
            rows = torch.zeros(words * n_shards, dtype=torch.int64, device="cuda:0")
            pos_o = 0
            for r, i in enumerate(infos):
                no = int(i.n_ops)
                row = rows[r * words:(r + 1) * words]
                row[:n_kept[r] * 2] = kept[r][:n_kept[r] * 2]
                row[cap * 2:].view(torch.int32)[:no] = ops[pos_o:pos_o + no]
                counts[2 * r], counts[2 * r + 1] = n_kept[r], no
                pos_o += no
            saved = rows[0:8].clone()
            rows[0:8] = -1  # a shard's own row is never read: what it holds does not matter
            torch.cuda.synchronize()
            for r, c in enumerate(ctxs):
                if r == 0:
                    c.set_global_join_rows(rows, ext_stride, ops_stride, counts, n_shards, r, ext_capacity=cap)
                    assert c.emit()["x_events"] == c.result["x_events"] and c.copy_output().tobytes() == parts[0], "filtered rows of shard 0"
            rows[0:8] = saved
            torch.cuda.synchronize()
            for r, c in enumerate(ctxs):
                if r > 0:
                    c.set_global_join_rows(rows, ext_stride, ops_stride, counts, n_shards, r, ext_capacity=cap)
                    c.emit()
                    assert c.copy_output().tobytes() == parts[r], "filtered rows of shard %d" % r
            # and with the other shards' CPU-op ids as bitmaps of their id ranges (k2j_op_id_bits, k2j_set_global_op_bits)
            ids = [api.device_view(i.op_ids, int(i.n_ops), "<i4").clone() for i in infos]
            firsts = [int(v.min()) for v in ids]
            tail = max((int(v.max()) - f + 64) // 64 for v, f in zip(ids, firsts))
            bit_rows = torch.zeros(n_shards * tail, dtype=torch.int64, device="cuda:0")
            meta = torch.tensor([v for f in firsts for v in (f, tail * 64)], dtype=torch.int64, device="cuda:0")
            for r, c in enumerate(ctxs):
                c.op_id_bits(firsts[r], bit_rows[r * tail:(r + 1) * tail])
            with pytest.raises(api.K2JError, match="outside"):
                ctxs[0].op_id_bits(firsts[0] + 1, bit_rows[:tail].clone())
            rows.view(torch.int32)[:] = torch.where(torch.arange(rows.numel() * 2, device="cuda:0") % (words * 2) >= cap * 4,
                                                    torch.full((1,), 0x7FFFFFF0, dtype=torch.int32, device="cuda:0"),
                                                    rows.view(torch.int32))   # the id lists are not read any more
            torch.cuda.synchronize()
            for r, c in enumerate(ctxs):
                c.set_global_join_rows(rows, ext_stride, ops_stride, counts, n_shards, r, ext_capacity=cap)
                c.set_global_op_bits(bit_rows.data_ptr(), tail * 8, meta)
                c.set_join_user_records(False)   # no shard holds CUSTOM1 records: nothing to clear or fill for spans
                c.emit()
                assert c.copy_output().tobytes() == parts[r], "op id bitmaps, shard %d" % r
        finally:
            for c in ctxs:
                c.close()
        # CPU-op events come first in every shard: reorder to [all ops][all gpu events]
        ops_txt = b"".join(p[:c.result["ops_bytes"]] for p, c in zip(parts, ctxs))
        gpu_txt = b"".join(p[c.result["ops_bytes"]:] for p, c in zip(parts, ctxs))
        assert hashlib.sha256(ops_txt + gpu_txt).hexdigest() == h_whole
    finally:
        ctx.close()


@pytest.mark.parametrize("n_shards,seed", [(2, 61), (3, 62), (5, 63)])
def test_sharded_synchronisation_records_concatenate_to_the_whole(n_shards, seed):
    """Synchronisation and CUDA event records look things up in maps the reference fills from the whole trace
    (contexts' devices, CUDA event records, streams with GPU work, the first stream synchronisation of a row).  With
    every shard given the other shards' lookup records as guests (k2j_export_lookup_records, k2j_set_guest_ranges)
    the shards' texts concatenate to the text of one run over the whole trace, and the counts add up."""
    import torch
    from kineto_b200 import api, sharding
    t = cases.sync_mix_trace(60_000, seed=seed)
    whole, res = gpu_run(t)
    subs = helpers.cut_into_shards(t, n_shards)
    ctxs = [api.K2J(0) for _ in subs]
    try:
        cupti_dev = torch.from_numpy(np.ascontiguousarray(t.cupti)).to("cuda:0")
        blobs = []
        for c, sub in zip(ctxs, subs):
            c.load(sub)
            c.segment()
            ptr, n = c.export_lookup_records()
            blobs.append(api.device_view(ptr, n, "|u1").clone())
        assert sum(b.numel() for b in blobs) > 0
        torch.cuda.synchronize()
        # without the guests a sharded run with such records is refused
        info = ctxs[0].segment()
        e0 = api.device_view(info.external_records, int(info.n_external) * 2, "<i8").clone()
        o0 = api.device_view(info.op_ids, int(info.n_ops), "<i4").clone()
        torch.cuda.synchronize()
        ctxs[0].set_global_join(e0, e0.numel() // 2, 0, o0, o0.numel())
        with pytest.raises(api.K2JError, match="UNSUPPORTED|lookup records"):
            ctxs[0].emit()
        infos = []
        for r, (c, sub) in enumerate(zip(ctxs, subs)):
            data, table, front_end, back_begin = sharding.with_guest_records(cupti_dev, sub.buftab, blobs, r)
            torch.cuda.synchronize()
            c.set_cupti(data, table)
            c.set_guest_ranges(front_end, back_begin)
            infos.append(c.segment())
        ext = torch.cat([api.device_view(i.external_records, int(i.n_external) * 2, "<i8").clone() for i in infos])
        ops = torch.cat([api.device_view(i.op_ids, int(i.n_ops), "<i4").clone() for i in infos])
        torch.cuda.synchronize()
        parts, results, begin = [], [], 0
        for c, i in zip(ctxs, infos):
            c.set_global_join(ext, ext.numel() // 2, begin, ops, ops.numel())
            begin += int(i.n_external)
            results.append(c.emit())
            parts.append(c.copy_output().tobytes())
    finally:
        for c in ctxs:
            c.close()
    ops_txt = b"".join(p[:r["ops_bytes"]] for p, r in zip(parts, results))
    gpu_txt = b"".join(p[r["ops_bytes"]:] for p, r in zip(parts, results))
    got = ops_txt + gpu_txt
    assert got == whole, helpers.first_diff(whole, got)
    for k in ("x_events", "flow_events", "n_records", "out_of_range_events", "blocklisted_runtime_events",
              "invalid_external_correlation_events", "unexpected_cuda_events"):
        assert sum(r[k] for r in results) == res[k], k


@pytest.mark.parametrize("n_shards", [2, 4])
def test_sharded_collectives_concatenate_to_the_whole(n_shards):
    """A kernel prints the collective metadata of the record_param_comms op that launched it, and that op may belong
    to another shard: with the other shards' collective ops appended as guest rows (k2j_set_guest_ops) the shards'
    texts concatenate to the text of one run over the whole trace."""
    import torch
    from kineto_b200 import api, sharding
    t = helpers.rebuffer(cases.collective_trace(300, seed=56), 37)
    whole, res = gpu_run(t)
    assert whole.count(b'"Collective name"') > 200
    subs = helpers.cut_into_shards(t, n_shards)
    colls = [sharding.collective_ops(sub) for sub in subs]
    assert all(colls)
    ctxs = [api.K2J(0) for _ in subs]
    try:
        infos = []
        for r, (c, sub) in enumerate(zip(ctxs, subs)):
            guests = [g for q, ops in enumerate(colls) if q != r for g in ops]
            shard, n_guests = sharding.with_guest_ops(sub, guests)
            c.load(shard)
            c.set_guest_ops(n_guests)
            infos.append(c.segment())
            assert int(infos[-1].n_ops) == sub.n_ops
        ext = torch.cat([api.device_view(i.external_records, int(i.n_external) * 2, "<i8").clone() for i in infos])
        ops = torch.cat([api.device_view(i.op_ids, int(i.n_ops), "<i4").clone() for i in infos])
        torch.cuda.synchronize()
        parts, results, begin = [], [], 0
        for c, i in zip(ctxs, infos):
            c.set_global_join(ext, ext.numel() // 2, begin, ops, ops.numel())
            begin += int(i.n_external)
            results.append(c.emit())
            parts.append(c.copy_output().tobytes())
    finally:
        for c in ctxs:
            c.close()
    got = b"".join(p[:r["ops_bytes"]] for p, r in zip(parts, results)) + b"".join(p[r["ops_bytes"]:] for p, r in zip(parts, results))
    assert got == whole, helpers.first_diff(whole, got)
    assert sum(r["x_events"] for r in results) == res["x_events"]


@pytest.mark.parametrize("gen,n_shards", [
    (lambda: synth.gen_kernel_launches(60_000, seed=305, pool_size=300, user_annotations=40, buffer_bytes=1 << 20), 3),
    (lambda: helpers.rebuffer(cases.annotation_trace(), 5), 2),
], ids=["launches", "annotation_fixture"])
def test_sharded_user_annotations_concatenate_to_the_whole(gen, n_shards):
    """A gpu_user_annotation span covers the GPU activities correlated to its annotation op wherever they are in the
    trace.  Every shard reports its part of every span, the parts are merged, and the last shard writes the merged
    spans behind its text (k2j_partial_spans, k2j_append_spans): the texts concatenate to the whole trace's text."""
    import torch
    from kineto_b200 import api, sharding
    t = gen()
    whole, res = gpu_run(t)
    assert whole.count(b'"gpu_user_annotation"') > 3
    subs = helpers.cut_into_shards(t, n_shards)
    guests_of = [sharding.annotation_ops(sub) for sub in subs]
    ctxs = [api.K2J(0) for _ in subs]
    try:
        infos, shards = [], []
        for r, (c, sub) in enumerate(zip(ctxs, subs)):
            shard, n_guests = sharding.with_guest_ops(sub, [g for q, ops in enumerate(guests_of) if q != r for g in ops])
            shards.append(shard)
            c.load(shard)
            c.set_guest_ops(n_guests)
            infos.append(c.segment())
        ext = torch.cat([api.device_view(i.external_records, int(i.n_external) * 2, "<i8").clone() for i in infos])
        ops = torch.cat([api.device_view(i.op_ids, int(i.n_ops), "<i4").clone() for i in infos])
        torch.cuda.synchronize()
        parts, results, spans, begin = [], [], [], 0
        for c, i in zip(ctxs, infos):
            c.set_global_join(ext, ext.numel() // 2, begin, ops, ops.numel())
            begin += int(i.n_external)
            results.append(c.emit())
            spans.append(c.partial_spans())
            parts.append(c.copy_output().tobytes())
        assert sum(len(p) for p in spans) > 3
        # told that no shard holds CUSTOM1 records, a run keeps no span tables: the same text, no parts
        ctxs[0].set_global_join(ext, ext.numel() // 2, 0, ops, ops.numel())
        ctxs[0].set_join_user_records(False)
        assert ctxs[0].emit()["x_events"] == results[0]["x_events"] and len(ctxs[0].partial_spans()) == 0
        assert ctxs[0].copy_output().tobytes() == parts[0]
        merged = sharding.merge_spans(spans, shards[-1].op_id)
        added = ctxs[-1].append_spans(merged)
        last = ctxs[-1].copy_output().tobytes()
        assert len(last) == len(parts[-1]) + added and last[:len(parts[-1])] == parts[-1]
        parts[-1] = last
    finally:
        for c in ctxs:
            c.close()
    got = b"".join(p[:r["ops_bytes"]] for p, r in zip(parts, results)) + b"".join(p[r["ops_bytes"]:] for p, r in zip(parts, results))
    assert got == whole, helpers.first_diff(whole, got)
    assert sum(r["x_events"] for r in results) + len(merged) == res["x_events"]


@pytest.mark.skipif(not helpers.have_ref(), reason="reference build (oracle/_ref) not present")
def test_full_size_against_reference():
    """The benchmark workload at a quarter of its size, byte for byte against the unmodified reference."""
    t = synth.gen_kernel_launches(250_000, seed=2)
    doc, _ = helpers.run_ref(t)
    want = helpers.activities_span(doc)
    got, res = gpu_run(t)
    assert len(got) == len(want)
    assert got == want, helpers.first_diff(want, got)


@pytest.mark.parametrize("gen", [
    lambda: synth.gen_mixed(120_000, seed=301, pool_size=3000, escape_fraction=0.05),
    lambda: synth.gen_kernel_launches(60_000, seed=302, pool_size=300, user_annotations=40),
    lambda: cases.with_flags(synth.gen_mixed(90_000, seed=303, pool_size=2000), tf.FLAG_SORT_BY_START),
    lambda: cases.sync_mix_trace(60_000, seed=304),
    lambda: synth.gen_distributed_rank(40_000, rank=1, seed=305),
    lambda: synth.gen_kernel_launches(30_000, seed=306, pool_size=300, memory_events=0.5),
    lambda: synth.gen_op_tree(30_000, seed=307),
    cases.edge_trace,
])
def test_tiled_emit_equals_resident_emit(gen, tmp_path):
    """The text produced slab by slab (to host memory, and to a file descriptor) is the text of a run that keeps it
    whole on the device: slabs of 4 MiB (the smallest), so that every trace here spans several slabs, the user
    annotation spans leave as a slab of their own, and classes start and end inside slabs."""
    import torch
    from kineto_b200 import api
    trace = gen()
    want, res0 = gpu_run(trace)
    ctx = api.K2J(0)
    try:
        ctx.load(trace)
        ctx.segment()
        dst = torch.empty(len(want) + 64, dtype=torch.uint8).pin_memory()
        dst.fill_(0x55)
        res = ctx.emit_to_host(dst, 4 << 20)
        assert res["out_bytes"] == len(want)
        got = dst[:len(want)].numpy().tobytes()
        assert got == want, helpers.first_diff(want, got)
        assert bytes(dst[len(want):].numpy().tobytes()) == b"\x55" * 64   # nothing past the text
        for k in ("x_events", "flow_events", "out_of_range_events", "ops_bytes", "annotation_bytes"):
            assert res[k] == res0[k], k
        with pytest.raises(api.K2JError):   # no text stays in the context
            ctx.output_ptr()
        path = tmp_path / "tiled.json"
        fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_TRUNC)
        try:
            os.write(fd, b"HEADER")
            ctx.segment()
            res2 = ctx.emit_to_fd(fd, 4 << 20)
        finally:
            os.close(fd)
        assert res2["out_bytes"] == len(want)
        assert path.read_bytes() == b"HEADER" + want
        small = torch.empty(max(1, len(want) // 2), dtype=torch.uint8).pin_memory()
        ctx.segment()
        with pytest.raises(api.K2JError) as e:
            ctx.emit_to_host(small, 4 << 20)
        assert e.value.status == 1
        # and the context still serves an ordinary run afterwards
        assert ctx.run()["out_bytes"] == len(want)
        assert ctx.copy_output().tobytes() == want
    finally:
        ctx.close()
