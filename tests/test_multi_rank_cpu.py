"""The N > 1 path on CPUs: two gloo ranks exchange their join keys with kineto_b200.sharding, each
runs the CPU checker on its shard with the gathered keys, and the shard outputs must concatenate to
the output of the whole trace processed at once."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import helpers
from kineto_b200 import sharding, synth
from kineto_b200 import tracefile as tf

WORLD = 2
N = 1500


def ext_records(trace):
    """The EXTERNAL_CORRELATION records of a launches trace as (external id, corr | kind << 32) pairs."""
    group = trace.cupti.reshape(-1, 272)            # 24 (ext) + 40 (api) + 208 (kernel) bytes per launch
    ext = np.ascontiguousarray(group[:, :24]).view(tf.EXTCORR).reshape(-1)
    out = np.zeros((len(ext), 2), np.uint64)
    out[:, 0] = ext["externalId"]
    out[:, 1] = ext["correlationId"].astype(np.uint64) | (ext["externalKind"].astype(np.uint64) << np.uint64(32))
    return out.reshape(-1)


def _rank_main(rank, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(WORLD))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    shard = synth.gen_kernel_launches(N, seed=77, pool_size=60, shard=(rank, WORLD))
    ext_local = torch.from_numpy(ext_records(shard).view(np.int64).copy())
    ops_local = torch.from_numpy(shard.op_id.copy())
    ext_all, ops_all, own_begin = sharding.gather_join_keys(ext_local, ops_local, rank, WORLD, dist)
    assert own_begin == rank * N
    shard.g_ext = ext_all.numpy().view(np.uint64)
    shard.g_ops = ops_all.numpy()
    out, stats = helpers.run_port(shard)
    base, total = sharding.output_bases(len(out), rank, WORLD, dist, "cpu")
    # both ranks fill one file: CPU-op events of all ranks first, then the GPU-side events
    path = os.path.join(tmp, "whole.json")
    if rank == 0:
        open(path, "wb").write(b"HEAD")
    dist.barrier()
    fd = os.open(path, os.O_WRONLY)
    total2 = sharding.write_shared_file(lambda f, off, b, n: os.pwrite(f, out[b:b + n], off), fd, 4, stats["ops_end"], len(out),
                                        rank, WORLD, dist, "cpu")
    os.close(fd)
    assert total2 == total
    summed = sharding.reduce_counters(dict(x_events=stats["x_events"], flow_events=stats["flow_events"], n_records=stats["records"],
                                           out_of_range_events=stats["out_of_range"], blocklisted_runtime_events=0,
                                           invalid_external_correlation_events=0, unexpected_cuda_events=0, out_bytes=len(out)),
                                      dist, "cpu")
    assert summed["out_bytes"] == total and summed["x_events"] == 3 * N * WORLD and summed["n_records"] == 3 * N * WORLD
    np.save(os.path.join(tmp, "out%d.npy" % rank), np.frombuffer(out, np.uint8))
    np.save(os.path.join(tmp, "meta%d.npy" % rank), np.array([stats["ops_end"], base, total, len(out)]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_whole_trace(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_rank_main, args=(port, str(tmp_path)), nprocs=WORLD, join=True)
    shards = [synth.gen_kernel_launches(N, seed=77, pool_size=60, shard=(r, WORLD)) for r in range(WORLD)]
    whole = tf.Trace(**{attr: getattr(shards[0], attr) for _, attr, _ in tf._SECTIONS})
    for col in ("op_start", "op_end", "op_id", "op_device", "op_resource", "op_thread", "op_type", "op_name", "op_flow",
                "op_flowt", "md"):
        setattr(whole, col, np.concatenate([getattr(s, col) for s in shards]))
    whole.op_mdoff = np.concatenate([shards[0].op_mdoff, shards[1].op_mdoff[1:] + shards[0].op_mdoff[-1]]).astype(np.uint32)
    whole.cupti = np.concatenate([s.cupti for s in shards])
    bt1 = shards[1].buftab.copy()
    bt1[0::2] += np.uint64(len(shards[0].cupti))
    whole.buftab = np.concatenate([shards[0].buftab, bt1])
    want, stats = helpers.run_port(whole)
    outs = [np.load(str(tmp_path / ("out%d.npy" % r))).tobytes() for r in range(WORLD)]
    metas = [np.load(str(tmp_path / ("meta%d.npy" % r))) for r in range(WORLD)]
    ops_txt = b"".join(o[:int(m[0])] for o, m in zip(outs, metas))
    gpu_txt = b"".join(o[int(m[0]):] for o, m in zip(outs, metas))
    assert ops_txt + gpu_txt == want, helpers.first_diff(want, ops_txt + gpu_txt)
    assert int(metas[1][1]) == len(outs[0]) and int(metas[0][2]) == len(outs[0]) + len(outs[1])
    assert open(str(tmp_path / "whole.json"), "rb").read() == b"HEAD" + want   # the ranks' positioned writes
    # the join really crosses shards: most kernels of shard 0 are linked to ops of shard 1 and vice versa
    alone, _ = helpers.run_port(shards[0])
    assert alone != outs[0]


def _uneven_main(rank, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(WORLD))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    n_ext, n_ops = (5, 0) if rank == 0 else (8, 7)   # ragged: different record counts, an odd id count, an empty side
    ext = torch.arange(n_ext * 2, dtype=torch.int64) + 1000 * rank
    ops = torch.arange(n_ops, dtype=torch.int32) + 100 * rank
    ext_all, ops_all, own_begin = sharding.gather_join_keys(ext, ops, rank, WORLD, dist)
    want_ext = torch.cat([torch.arange(10, dtype=torch.int64), torch.arange(16, dtype=torch.int64) + 1000])
    want_ops = torch.arange(7, dtype=torch.int32) + 100
    ok = torch.equal(ext_all, want_ext) and torch.equal(ops_all, want_ops) and own_begin == (0 if rank == 0 else 5)
    np.save(os.path.join(tmp, "ok%d.npy" % rank), np.array([int(ok)]))
    dist.barrier()
    dist.destroy_process_group()


def test_join_key_exchange_with_ragged_shards(tmp_path):
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_uneven_main, args=(port, str(tmp_path)), nprocs=WORLD, join=True)
    assert all(int(np.load(str(tmp_path / ("ok%d.npy" % r)))[0]) == 1 for r in range(WORLD))


def _guest_rank_main(rank, port, tmp):
    """Two gloo ranks exchange what the cross-shard record families need beyond the join keys."""
    import cases
    from kineto_b200 import api
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(WORLD))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        whole = helpers.rebuffer(cases.collective_trace(60, seed=57), 11)
        sub = helpers.cut_into_shards(whole, WORLD)[rank]
        guests = sharding.gather_guest_ops(sub, rank, WORLD, dist)
        other = helpers.cut_into_shards(whole, WORLD)[1 - rank]
        assert guests == sharding.collective_ops(other) + sharding.annotation_ops(other) and guests
        shard, n = sharding.with_guest_ops(sub, guests)
        assert n == len(guests) and shard.n_ops == sub.n_ops + n and len(shard.op_mdoff) == shard.n_ops + 1
        pool = shard.pool()
        for k, (op_id, name, entries) in enumerate(guests):
            row = sub.n_ops + k
            assert int(shard.op_id[row]) == op_id and pool[int(shard.op_name[row])] == name
            got = shard.md[int(shard.op_mdoff[row]):int(shard.op_mdoff[row + 1])]
            assert [(pool[int(e["key"])], int(e["type"])) for e in got] == [(key, typ) for key, typ, _ in entries]
            for e, (_, typ, value) in zip(got, entries):
                assert (pool[int(e["value"])] if typ in (tf.MD_STRING, tf.MD_RAWJSON) else int(e["value"])) == value
        # the shard's own rows and strings are untouched
        assert np.array_equal(shard.op_id[:sub.n_ops], sub.op_id) and np.array_equal(shard.md[:len(sub.md)], sub.md)
        assert np.array_equal(shard.pool_data[:len(sub.pool_data)], sub.pool_data)
        # spans: every rank reports parts, the merge is the same on every rank
        part = np.zeros(2, api.SPAN)
        part[0] = (100 + rank, 500 + 10 * rank, 7 - rank, 0, 20, 900, 0)
        part[1] = (50, 60, 3, rank, 21, 901 + rank, 0)
        everyone = [None] * WORLD
        dist.all_gather_object(everyone, part)
        merged = sharding.merge_spans(everyone, np.array([5, 900, 901, 900], np.int32))
        by_key = {(int(m["device"]), int(m["stream"]), int(m["op_id"])): m for m in merged}
        assert len(merged) == 3
        m = by_key[(0, 20, 900)]
        assert (int(m["start_ns"]), int(m["end_ns"]), int(m["first_event"]), int(m["op_row"])) == (100, 510, 7, 3)
        assert int(by_key[(0, 21, 901)]["op_row"]) == 2 and int(by_key[(1, 21, 902)]["op_row"]) == 0xFFFFFFFF
        assert int(by_key[(1, 21, 902)]["first_event"]) == (1 << 40) | 3
        open(os.path.join(tmp, "guest_ok%d" % rank), "w").write("1")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_exchange_guest_ops_and_spans(tmp_path):
    port = 29300 + (os.getpid() % 500)
    mp.spawn(_guest_rank_main, args=(port, str(tmp_path)), nprocs=WORLD, join=True)
    assert all(os.path.exists(str(tmp_path / ("guest_ok%d" % r))) for r in range(WORLD))


def test_guest_records_are_laid_out_around_the_shards_own_buffers():
    """sharding.with_guest_records: lower shards' lookup records in front, higher shards' behind, the shard's own
    buffers moved by the bytes in front, and the two boundaries for k2j_set_guest_ranges."""
    own = torch.arange(64, dtype=torch.uint8)
    blobs = [torch.full((16,), 1, dtype=torch.uint8), torch.zeros(0, dtype=torch.uint8), torch.full((8,), 3, dtype=torch.uint8),
             torch.full((24,), 4, dtype=torch.uint8)]
    data, table, front_end, back_begin = sharding.with_guest_records(own, np.array([8, 16, 40, 24], np.uint64), blobs, 1)
    assert (front_end, back_begin) == (16, 80) and data.numel() == 16 + 64 + 8 + 24
    assert table.tolist() == [0, 16, 24, 16, 56, 24, 80, 8, 88, 24]
    assert data[:16].eq(1).all() and torch.equal(data[16:80], own) and data[80:88].eq(3).all() and data[88:].eq(4).all()
    data, table, front_end, back_begin = sharding.with_guest_records(own, np.array([0, 64], np.uint64), [blobs[1], blobs[1]], 0)
    assert data is own and table.tolist() == [0, 64] and (front_end, back_begin) == (0, 64)


class _FakeContext:
    """Stands in for api.K2J in the exchange's control flow: records the calls, fills what the library would fill."""

    def __init__(self, n_ext, kept):
        self.n_ext, self.kept, self.calls = n_ext, kept, []

    def join_need_bits(self, bits):
        bits.zero_()
        self.calls.append(("need", bits.numel() * 8))

    def filter_join_keys(self, need, world, rank, out, n_out):
        out[:self.kept * 2] = torch.arange(self.kept * 2, dtype=torch.int64) + 1000 * rank
        n_out[0] = self.kept
        self.calls.append(("filter", need.numel(), world, rank))

    def op_id_bits(self, first, bits):
        bits.zero_()
        bits[0] = 1
        self.calls.append(("op_bits", first, bits.numel() * 64))

    def set_global_join_rows(self, rows, ext_stride, ops_stride, counts, world, rank, ext_capacity=None):
        self.calls.append(("rows", rows.numel(), ext_stride, ops_stride, counts.tolist(), world, rank, ext_capacity))

    def set_global_op_bits(self, ptr, pitch, meta):
        self.calls.append(("op_rows", pitch, meta.tolist()))

    def set_join_user_records(self, any_records):
        self.calls.append(("user", any_records))


def _filtered_rank_main(rank, port, tmp):
    from kineto_b200 import api
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(WORLD))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        ids = torch.arange(100 * rank + 5, 100 * rank + 5 + 40 + rank, dtype=torch.int32)
        api_view = api.device_view
        api.device_view = lambda ptr, n, typestr, device="cpu": ids[:n]       # the library's id array, on the host here

        class Info:
            n_external, n_ops, n_records, op_ids, n_user_external = 300 + rank, len(ids), 1000, 0, 3 * rank
        for bitmaps in (True, False):
            fx = sharding.FilteredJoinExchange(rank, WORLD, dist, "cpu", op_bitmaps=bitmaps)
            for step in range(2):
                ctx = _FakeContext(300 + rank, kept=20 + 7 * rank + step)
                fx.exchange(ctx, Info)
                names = [c[0] for c in ctx.calls]
                assert names == (["need", "filter", "op_bits", "rows", "op_rows", "user"] if bitmaps else ["need", "filter", "rows", "user"])
                rows = dict((c[0], c) for c in ctx.calls)["rows"]
                assert rows[4] == [20 + step, 40, 27 + step, 41] and rows[5:7] == (WORLD, rank) and rows[7] == fx.cap >= 27 + step
                assert rows[2] >= 301 and rows[3] >= 41 and rows[1] == fx.row_words * WORLD
                assert dict((c[0], c) for c in ctx.calls)["user"][1] is True       # rank 1 holds CUSTOM1 records
                assert fx.kept_counts == [20 + step, 27 + step] and fx.dense == bitmaps
                # what travelled: every rank's kept records in front of its row, then its ids (as bits or as a list)
                for r in range(WORLD):
                    row = fx.rows[r * fx.row_words:(r + 1) * fx.row_words]
                    assert row[:fx.kept_counts[r] * 2].tolist() == [1000 * r + k for k in range(fx.kept_counts[r] * 2)]
                    if bitmaps:
                        assert int(row[fx.cap * 2]) == 1
                    else:
                        assert row[fx.cap * 2:].view(torch.int32)[:40 + r].tolist() == list(range(100 * r + 5, 100 * r + 45 + r))
                if bitmaps:
                    meta = dict((c[0], c) for c in ctx.calls)["op_rows"]
                    assert meta[1] == fx.row_words * 8 and meta[2][0::2] == [5, 105] and meta[2][1] == meta[2][3] >= 41
        api.device_view = api_view
        open(os.path.join(tmp, "filtered_ok%d" % rank), "w").write("1")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_run_the_filtered_exchange(tmp_path):
    """The control flow of sharding.FilteredJoinExchange over two gloo ranks with a stand-in for the context: the
    collectives, the sizes agreed in the one host round trip, the rows' layout and the calls the library receives."""
    port = 29400 + (os.getpid() % 500)
    mp.spawn(_filtered_rank_main, args=(port, str(tmp_path)), nprocs=WORLD, join=True)
    assert all(os.path.exists(str(tmp_path / ("filtered_ok%d" % r))) for r in range(WORLD))
