"""Two ranks on two GPUs: segment -> NCCL all-gather of the join keys -> emit, compared per shard with
the CPU checker given the same gathered keys.  Skipped on boxes with one GPU."""
import datetime
import os

import numpy as np
import pytest
import torch

import helpers
from kineto_b200 import synth

pytestmark = pytest.mark.gpu
WORLD = 2
N = 40_000


def _rank_main(rank, port, tmp):
    import torch.distributed as dist
    from kineto_b200 import api, sharding
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(WORLD),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=WORLD, device_id=dev, timeout=datetime.timedelta(seconds=90))  # a rank that failed ends the other soon
    shard = synth.gen_kernel_launches(N, seed=91, pool_size=500, shard=(rank, WORLD))
    stream = torch.cuda.Stream(dev)   # the context, torch's copies and the collectives share it
    torch.cuda.set_stream(stream)
    ctx = api.K2J(rank, stream.cuda_stream)
    try:
        ctx.load(shard)
        info = ctx.segment()
        ext_local = api.device_view(info.external_records, int(info.n_external) * 2, "<i8", dev)
        ops_local = api.device_view(info.op_ids, int(info.n_ops), "<i4", dev)
        ext_all, ops_all, own_begin = sharding.gather_join_keys(ext_local, ops_local, rank, WORLD, dist)
        ctx.set_global_join(ext_all, ext_all.numel() // 2, own_begin, ops_all, ops_all.numel())
        res = ctx.emit()
        got = ctx.copy_output().tobytes()
        # the same through the exchange that leaves the rows of the all-gather where they are
        info2 = ctx.segment()
        ex = sharding.JoinExchange(rank, WORLD, dist, dev)
        rows, ext_stride, ops_stride, counts = ex.gather(api.device_view(info2.external_records, int(info2.n_external) * 2, "<i8", dev),
                                                         api.device_view(info2.op_ids, int(info2.n_ops), "<i4", dev))
        ctx.set_global_join_rows(rows, ext_stride, ops_stride, counts, WORLD, rank)
        res_rows = ctx.emit()
        got_rows = ctx.copy_output().tobytes()
        assert got_rows == got and res_rows["x_events"] == res["x_events"] and res_rows["invalid_external_correlation_events"] == res["invalid_external_correlation_events"]
        # and with rows that hold only the records another shard can want
        for bitmaps in (True, False):   # the CPU-op ids as bitmaps of the shards' id ranges, or as lists
            fx = sharding.FilteredJoinExchange(rank, WORLD, dist, dev, op_bitmaps=bitmaps)
            for _ in range(2):
                info3 = ctx.segment()
                fx.exchange(ctx, info3)
                res_f = ctx.emit()
                assert ctx.copy_output().tobytes() == got and res_f["x_events"] == res["x_events"]
                assert fx.kept_counts[rank] <= int(info3.n_external) and fx.dense == bitmaps
        shard.g_ext = ext_all.cpu().numpy().view(np.uint64)
        shard.g_ops = ops_all.cpu().numpy()
        want, stats = helpers.run_port(shard)
        ok = got == want and res["x_events"] == stats["x_events"] and res["ops_bytes"] == stats["ops_end"]
        # both ranks stream their two parts into one file (k2j_write_output_at)
        path = os.path.join(tmp, "whole.json")
        if rank == 0:
            open(path, "wb").close()
        dist.barrier()
        fd = os.open(path, os.O_WRONLY)
        total = sharding.write_shared_file(ctx.write_output_at, fd, 0, res["ops_bytes"], res["out_bytes"], rank, WORLD, dist, dev)
        os.close(fd)
        np.save(os.path.join(tmp, "part%d.npy" % rank), np.frombuffer(got, np.uint8))
        open(os.path.join(tmp, "meta%d" % rank), "w").write("%d %d" % (res["ops_bytes"], total))
        alone, _ = helpers.run_port(synth.gen_kernel_launches(N, seed=91, pool_size=500, shard=(rank, WORLD)))
        open(os.path.join(tmp, "ok%d" % rank), "w").write("%d %d" % (int(ok), int(alone != want)))
        dist.barrier()
    except BaseException:
        # a rank that failed says why and leaves at once: waiting in destroy_process_group for a peer that sits in a
        # collective would hide the failure behind the peer's timeout
        import traceback
        open(os.path.join(tmp, "err%d" % rank), "w").write(traceback.format_exc())
        os._exit(1)
    ctx.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_ranks_match_checker(tmp_path):
    import torch.multiprocessing as mp
    port = 29700 + (os.getpid() % 2000)
    try:
        mp.spawn(_rank_main, args=(port, str(tmp_path)), nprocs=WORLD, join=True)
    except Exception as e:  # noqa: BLE001
        errs = [open(str(f)).read() for f in sorted(tmp_path.glob("err*"))]
        pytest.fail("a rank failed: %s\n%s" % (e, "\n".join(errs)))
    for r in range(WORLD):
        ok, crosses = open(str(tmp_path / ("ok%d" % r))).read().split()
        assert ok == "1", "rank %d output differs from the checker" % r
        assert crosses == "1"   # the join does reach into the other shard
    parts = [np.load(str(tmp_path / ("part%d.npy" % r))).tobytes() for r in range(WORLD)]
    metas = [[int(x) for x in open(str(tmp_path / ("meta%d" % r))).read().split()] for r in range(WORLD)]
    want = b"".join(p[:m[0]] for p, m in zip(parts, metas)) + b"".join(p[m[0]:] for p, m in zip(parts, metas))
    assert metas[0][1] == len(want)
    assert open(str(tmp_path / "whole.json"), "rb").read() == want


def _sync_rank_main(rank, port, tmp):
    import torch.distributed as dist
    import cases
    from kineto_b200 import api, sharding
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(WORLD),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    try:
        dist.init_process_group("nccl", rank=rank, world_size=WORLD, device_id=dev, timeout=datetime.timedelta(seconds=90))
        stream = torch.cuda.Stream(dev)
        torch.cuda.set_stream(stream)
        sub = helpers.cut_into_shards(cases.sync_mix_trace(40_000, seed=71), WORLD)[rank]
        ctx = api.K2J(rank, stream.cuda_stream)
        ctx.load(sub)
        ctx.segment()
        blobs = sharding.gather_lookup_records(ctx, rank, WORLD, dist, dev)
        own = torch.from_numpy(np.ascontiguousarray(sub.cupti)).to(dev)
        data, table, front_end, back_begin = sharding.with_guest_records(own, sub.buftab, blobs, rank)
        torch.cuda.synchronize()
        ctx.set_cupti(data, table)
        ctx.set_guest_ranges(front_end, back_begin)
        info = ctx.segment()
        ex = sharding.JoinExchange(rank, WORLD, dist, dev)
        rows, ext_stride, ops_stride, counts = ex.gather(api.device_view(info.external_records, int(info.n_external) * 2, "<i8", dev),
                                                         api.device_view(info.op_ids, int(info.n_ops), "<i4", dev))
        ctx.set_global_join_rows(rows, ext_stride, ops_stride, counts, WORLD, rank)
        res = ctx.emit()
        got = ctx.copy_output().tobytes()
        total = sharding.reduce_counters(res, dist, dev)
        np.save(os.path.join(tmp, "sync_part%d.npy" % rank), np.frombuffer(got, np.uint8))
        open(os.path.join(tmp, "sync_meta%d" % rank), "w").write("%d %d %d" % (res["ops_bytes"], total["x_events"], total["n_records"]))
        dist.barrier()
    except BaseException:
        import traceback
        open(os.path.join(tmp, "err%d" % rank), "w").write(traceback.format_exc())
        os._exit(1)
    ctx.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_ranks_with_synchronisation_records(tmp_path):
    """A trace with synchronisation and CUDA event records on two GPUs: the ranks all-gather their lookup records
    (NCCL), run with the other rank's as guests, and their texts concatenate to the text of the whole trace."""
    import torch.multiprocessing as mp
    import cases
    from kineto_b200 import api
    port = 29700 + ((os.getpid() + 7) % 2000)
    try:
        mp.spawn(_sync_rank_main, args=(port, str(tmp_path)), nprocs=WORLD, join=True)
    except Exception as e:  # noqa: BLE001
        errs = [open(str(f)).read() for f in sorted(tmp_path.glob("err*"))]
        pytest.fail("a rank failed: %s\n%s" % (e, "\n".join(errs)))
    whole, res = api.process(cases.sync_mix_trace(40_000, seed=71))
    parts = [np.load(str(tmp_path / ("sync_part%d.npy" % r))).tobytes() for r in range(WORLD)]
    metas = [[int(x) for x in open(str(tmp_path / ("sync_meta%d" % r))).read().split()] for r in range(WORLD)]
    got = b"".join(p[:m[0]] for p, m in zip(parts, metas)) + b"".join(p[m[0]:] for p, m in zip(parts, metas))
    assert got == whole, helpers.first_diff(whole, got)
    assert metas[0][1] == res["x_events"] and metas[0][2] == res["n_records"]
