"""Host-side plumbing for traces sharded by contiguous record range over several ranks.

Each rank owns whole CUPTI buffers and a contiguous range of CPU ops.  The event text of a record
depends on its own bytes, scalars, and the correlation join, so the only data that must cross ranks is
the join keys: every rank's EXTERNAL_CORRELATION records (16 bytes each, processing order) and CPU-op
ids (4 bytes each).  `gather_join_keys` all-gathers both in rank order, which is global processing
order, so "last writer wins" (libkineto/src/CuptiActivityProfiler.cpp:293-296) is decided by position
in the gathered array exactly as in a single-process run.  Works with any torch.distributed backend
(NCCL on GPUs, gloo on CPUs).
"""
from __future__ import annotations

import numpy as np


def gather_join_keys(ext_local, ops_local, rank: int, world: int, dist):
    """ext_local: int64 tensor with 2 words per record; ops_local: int32 tensor.
    Returns (ext_all, ops_all, own_begin): the gathered arrays in rank order and the index of this
    rank's first EXTERNAL_CORRELATION record in ext_all.  Two collectives: the counts, then one
    packed payload (records and ids in one buffer, padded to the largest shard)."""
    import torch

    dev = ext_local.device
    n_ext, n_ops = ext_local.numel() // 2, ops_local.numel()
    counts = torch.tensor([n_ext, n_ops], dtype=torch.int64, device=dev)
    all_counts = torch.empty(world * 2, dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(all_counts, counts)
    all_counts = all_counts.view(world, 2).tolist()
    max_ext = max(1, max(c[0] for c in all_counts))
    max_ops = max(1, max(c[1] for c in all_counts))
    ops_words = (max_ops + 1) // 2                       # op ids packed two per 64-bit word
    stride = max_ext * 2 + ops_words
    pack = torch.empty(stride, dtype=torch.int64, device=dev)
    pack[:n_ext * 2] = ext_local
    pack[max_ext * 2:].view(torch.int32)[:n_ops] = ops_local
    gathered = torch.empty(world * stride, dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(gathered, pack)
    g = gathered.view(world, stride)
    if all(c[0] == max_ext for c in all_counts):
        ext_all = g[:, :max_ext * 2].reshape(-1)
    else:
        ext_all = torch.cat([g[r, :all_counts[r][0] * 2] for r in range(world)])
    gi = g[:, max_ext * 2:].view(torch.int32)
    if all(c[1] == max_ops for c in all_counts) and max_ops % 2 == 0:
        ops_all = gi.reshape(-1)
    else:
        ops_all = torch.cat([gi[r, :all_counts[r][1]] for r in range(world)])
    own_begin = sum(c[0] for c in all_counts[:rank])
    return ext_all.contiguous(), ops_all.contiguous(), own_begin


class JoinExchange:
    """The same exchange without a host round trip per step.  Every rank sends one row: room for `ext_stride`
    records and `ops_stride` ids (the largest shard's counts; agreed once, with a little head room, when the exchange
    is created or has to grow), the rows are all-gathered as they are, and the library reads them in place
    (k2j_set_global_join_rows) together with the all-gathered counts, which never leave the device."""

    def __init__(self, rank: int, world: int, dist, device):
        self.rank, self.world, self.dist, self.device = rank, world, dist, device
        self.ext_stride = self.ops_stride = 0

    def _agree(self, n_ext: int, n_ops: int):
        import torch
        t = torch.tensor([n_ext, n_ops], dtype=torch.int64, device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        m = t.tolist()
        self.ext_stride = max(1, int(m[0] * 1.02) + 16)
        self.ops_stride = (max(1, int(m[1] * 1.02) + 16) + 1) & ~1      # two ids per 64-bit word
        words = self.ext_stride * 2 + self.ops_stride // 2
        self.row = torch.zeros(words, dtype=torch.int64, device=self.device)
        self.rows = torch.empty(words * self.world, dtype=torch.int64, device=self.device)
        self.counts = torch.empty(2 * self.world, dtype=torch.int64, device=self.device)
        self.mine = torch.empty(2, dtype=torch.int64, device=self.device)

    def gather(self, ext_local, ops_local):
        """ext_local: int64 tensor, 2 words per record; ops_local: int32 tensor (both on the device).  Returns
        (rows, ext_stride, ops_stride, counts) for K2J.set_global_join_rows."""
        n_ext, n_ops = ext_local.numel() // 2, ops_local.numel()
        if self.ext_stride == 0:
            self._agree(n_ext, n_ops)   # first call, on every rank
        elif n_ext > self.ext_stride or n_ops > self.ops_stride:
            raise ValueError("this shard outgrew the row size the ranks agreed on: create a new JoinExchange on every rank")
        self.row[:n_ext * 2] = ext_local
        self.row[self.ext_stride * 2:].view(ops_local.dtype)[:n_ops] = ops_local
        self.mine[0], self.mine[1] = n_ext, n_ops
        self.dist.all_gather_into_tensor(self.counts, self.mine)
        self.dist.all_gather_into_tensor(self.rows, self.row)
        return self.rows, self.ext_stride, self.ops_stride, self.counts


USER_ANNOTATION = 1  # libkineto::ActivityType::USER_ANNOTATION


def annotation_ops(trace):
    """The user-annotation ops of a shard as guests that carry only their name: (id, name bytes, [])."""
    pool = trace.pool()
    return [(int(trace.op_id[r]), pool[int(trace.op_name[r])], []) for r in np.flatnonzero(trace.op_type == USER_ANNOTATION)]


def merge_spans(parts, op_ids, n_own_rows=None):
    """Merges the shards' parts of the user-annotation spans (`parts[r]`: K2J.partial_spans() of shard r): per
    (device, stream, op id) the smallest start, the largest end and the first event in (shard, event number) order.
    `op_ids`: the id column of the LAST shard's CPU-side activities, guest rows included; every span gets the row of
    the last activity with its id (0xFFFFFFFF when there is none).  Returns an array for K2J.append_spans."""
    from . import api
    merged = {}
    for r, part in enumerate(parts):
        for s in part:
            key = (int(s["device"]), int(s["stream"]), int(s["op_id"]))
            first = (r << 40) | int(s["first_event"])
            m = merged.get(key)
            if m is None:
                merged[key] = [int(s["start_ns"]), int(s["end_ns"]), first]
            else:
                m[0], m[1], m[2] = min(m[0], int(s["start_ns"])), max(m[1], int(s["end_ns"])), min(m[2], first)
    row_of = {int(v): i for i, v in enumerate(np.asarray(op_ids))}   # the last row with an id stays
    out = np.zeros(len(merged), api.SPAN)
    for k, ((dev, stream, op_id), (start, end, first)) in enumerate(merged.items()):
        out[k] = (start, end, first, dev, stream, op_id, row_of.get(op_id, 0xFFFFFFFF))
    return out


def collective_ops(trace):
    """The record_param_comms ops of a shard in a form that travels: (id, name, [(key bytes, type, value or bytes)])."""
    from . import tracefile as tf
    pool = trace.pool()
    want = [i for i in range(len(pool)) if pool[i] == b"record_param_comms"]
    if not want:
        return []
    out = []
    for row in np.flatnonzero(np.isin(trace.op_name, np.array(want, dtype=np.uint32))):
        entries = []
        for e in trace.md[int(trace.op_mdoff[row]):int(trace.op_mdoff[row + 1])]:
            text = e["type"] in (tf.MD_STRING, tf.MD_RAWJSON)
            entries.append((pool[int(e["key"])], int(e["type"]), pool[int(e["value"])] if text else int(e["value"])))
        out.append((int(trace.op_id[row]), b"record_param_comms", entries))
    return out


def with_guest_ops(trace, guests):
    """A copy of the shard with other shards' ops (`collective_ops`, `annotation_ops` of those shards) appended as
    guest rows behind its own; returns (trace, number of guest rows) for K2J.load and K2J.set_guest_ops."""
    import copy
    from . import tracefile as tf
    if not guests:
        return trace, 0
    t = copy.copy(trace)
    pool = trace.pool()
    md, mdoff = [trace.md], [trace.op_mdoff]
    rows, at = [], int(trace.op_mdoff[-1])
    for _, _, entries in guests:
        e = np.zeros(len(entries), tf.MD_ENTRY)
        for k, (key, typ, value) in enumerate(entries):
            e[k] = (pool.add(key), typ, pool.add(value) if typ in (tf.MD_STRING, tf.MD_RAWJSON) else value)
        rows.append(e)
        at += len(entries)
        mdoff.append(np.array([at], np.uint32))
    n = len(guests)
    t.md = np.concatenate(md + rows)
    t.op_mdoff = np.concatenate(mdoff).astype(np.uint32)
    z = lambda a, fill=0: np.concatenate([a, np.full(n, fill, a.dtype)])  # noqa: E731
    t.op_start, t.op_end, t.op_device, t.op_resource, t.op_thread = z(trace.op_start), z(trace.op_end), z(trace.op_device), z(trace.op_resource), z(trace.op_thread)
    t.op_type, t.op_flow, t.op_flowt = z(trace.op_type), z(trace.op_flow), z(trace.op_flowt)
    t.op_id = np.concatenate([trace.op_id, np.array([g[0] for g in guests], trace.op_id.dtype)])
    t.op_name = np.concatenate([trace.op_name, np.array([pool.add(g[1]) for g in guests], trace.op_name.dtype)])
    t.set_pool(pool)
    return t, n


def gather_guest_ops(trace, rank: int, world: int, dist):
    """All shards' record_param_comms and user-annotation ops except this shard's own, in shard order (host-side
    collective of pickled lists: such ops are few)."""
    everyone = [None] * world
    dist.all_gather_object(everyone, collective_ops(trace) + annotation_ops(trace))
    return [g for r, ops in enumerate(everyone) if r != rank for g in ops]


def with_guest_records(own_cupti, own_buftab, blobs, rank: int):
    """The CUPTI bytes a shard runs on when the trace has synchronisation or CUDA event records: the lookup records
    of the lower shards (`blobs[:rank]`, uint8 device tensors from k2j_export_lookup_records) in front of the shard's
    own bytes, those of the higher shards behind them.  Returns (bytes tensor, buffer table, front_end_bytes,
    back_begin_bytes) for K2J.set_cupti and K2J.set_guest_ranges."""
    import numpy as np
    import torch
    front = [b for b in blobs[:rank] if b.numel()]
    back = [b for b in blobs[rank + 1:] if b.numel()]
    n_front = sum(b.numel() for b in front)
    n_own = own_cupti.numel()
    whole = torch.cat(front + [own_cupti] + back) if front or back else own_cupti
    table, at = [], 0
    for b in front:
        table += [at, b.numel()]
        at += b.numel()
    own = np.asarray(own_buftab, dtype=np.uint64).reshape(-1, 2)
    for off, valid in own:
        table += [n_front + int(off), int(valid)]
    at = n_front + n_own
    for b in back:
        table += [at, b.numel()]
        at += b.numel()
    return whole, np.array(table, dtype=np.uint64), n_front, n_front + n_own


def gather_lookup_records(ctx, rank: int, world: int, dist, device):
    """All-gathers the shards' lookup records (K2J.export_lookup_records): one collective for the sizes (with a host
    round trip: the buffers are laid out on the host), one for the padded records.  Returns the list of per-shard
    uint8 device tensors for `with_guest_records`."""
    import torch
    from . import api
    ptr, n = ctx.export_lookup_records()
    sizes = torch.empty(world, dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(sizes, torch.tensor([n], dtype=torch.int64, device=device))
    sizes = [int(v) for v in sizes.cpu()]
    pad = max(8, max(sizes))
    mine = torch.zeros(pad, dtype=torch.uint8, device=device)
    if n:
        mine[:n] = api.device_view(ptr, n, "|u1", device)
    everyone = torch.empty(pad * world, dtype=torch.uint8, device=device)
    dist.all_gather_into_tensor(everyone, mine)
    return [everyone[r * pad:r * pad + sizes[r]] for r in range(world)]


class FilteredJoinExchange:
    """The exchange that sends join keys only where they can be wanted.  Per step: every rank all-gathers the filter
    of the correlation ids its events carry (K2J.join_need_bits, a few bits per event), keeps of its own
    EXTERNAL_CORRELATION records those that hit another rank's filter (K2J.filter_join_keys, in order), and the
    ranks all-gather rows of [kept records | CPU-op ids] sized by the largest kept count (one host round trip for
    the sizes).  The CPU-op ids travel as bitmaps of the shards' id ranges when every shard's ids are dense
    (K2J.op_id_bits: the join only asks whether an id exists), else as lists.  The library reads a rank's own records
    and ids from the rank's own arrays, so nothing else is needed."""

    def __init__(self, rank: int, world: int, dist, device, op_bitmaps: bool = True):
        self.rank, self.world, self.dist, self.device = rank, world, dist, device
        self.op_bitmaps = op_bitmaps
        self.ext_stride = 0
        self.cap = self.tail = self.row_words = 0

    def _agree(self, n_ext: int, n_ops: int, n_records: int):
        import torch
        t = torch.tensor([n_ext, n_ops, n_records], dtype=torch.int64, device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        m = t.tolist()
        self.ext_stride = max(1, int(m[0] * 1.02) + 16)                 # index stride: room for a shard's own records
        self.ops_stride = (max(1, int(m[1] * 1.02) + 16) + 1) & ~1
        n_bits = 1 << 20
        while n_bits < 3 * m[2] and n_bits < (1 << 32):   # records walked, of which about three quarters own an event
            n_bits *= 2
        self.bits = torch.empty(n_bits // 8, dtype=torch.uint8, device=self.device)
        self.need = torch.empty(n_bits // 8 * self.world, dtype=torch.uint8, device=self.device)
        self.kept = torch.empty(self.ext_stride * 2, dtype=torch.int64, device=self.device)
        self.mine = torch.zeros(5, dtype=torch.int64, device=self.device)
        self.all5 = torch.empty(5 * self.world, dtype=torch.int64, device=self.device)

    def exchange(self, ctx, info):
        """`info`: what K2J.segment() returned.  Leaves the context ready for K2J.emit()."""
        import torch
        from . import api
        n_ext, n_ops = int(info.n_external), int(info.n_ops)
        if self.ext_stride == 0:
            self._agree(n_ext, n_ops, int(info.n_records))
        elif n_ext > self.ext_stride or n_ops > self.ops_stride:
            raise ValueError("this shard outgrew the sizes the ranks agreed on: create a new FilteredJoinExchange on every rank")
        ctx.join_need_bits(self.bits)
        self.dist.all_gather_into_tensor(self.need, self.bits)
        ctx.filter_join_keys(self.need, self.world, self.rank, self.kept, self.mine[:1])
        ops_local = api.device_view(info.op_ids, n_ops, "<i4", self.device)
        self.mine[1] = n_ops
        if n_ops:
            lo, hi = torch.aminmax(ops_local)
            self.mine[2], self.mine[3] = lo, hi
        else:
            self.mine[2], self.mine[3] = 0, -1
        self.mine[4] = int(info.n_user_external)
        self.dist.all_gather_into_tensor(self.all5, self.mine)
        sizes = self.all5.cpu().view(self.world, 5)                     # the one host round trip of the exchange
        cap = max(1, int(sizes[:, 0].max()))
        spans = [(int(r[2]), int(r[3]) - int(r[2]) + 1, int(r[1])) for r in sizes]   # (first id, ids spanned, ids held)
        dense = self.op_bitmaps and all(n == 0 or span <= 64 * n + 4096 for _, span, n in spans)
        tail = max(1, max((span + 63) // 64 for _, span, _ in spans)) if dense else self.ops_stride // 2
        if cap > self.cap or tail > self.tail:                          # grow-only row buffers
            self.cap, self.tail = max(self.cap, int(cap * 1.25) + 16), max(self.tail, tail)
            self.row_words = self.cap * 2 + self.tail
            self.row = torch.zeros(self.row_words, dtype=torch.int64, device=self.device)
            self.rows = torch.empty(self.row_words * self.world, dtype=torch.int64, device=self.device)
        n_kept = int(sizes[self.rank, 0])
        self.row[:n_kept * 2] = self.kept[:n_kept * 2]
        if dense:
            ctx.op_id_bits(spans[self.rank][0], self.row[self.cap * 2:])
        else:
            self.row[self.cap * 2:].view(ops_local.dtype)[:n_ops] = ops_local
        self.dist.all_gather_into_tensor(self.rows, self.row)
        self.counts = self.all5.view(self.world, 5)[:, :2].contiguous().view(-1)
        ctx.set_global_join_rows(self.rows, self.ext_stride, self.ops_stride, self.counts, self.world, self.rank, ext_capacity=self.cap)
        if dense:
            self.meta = torch.tensor([v for first, _, _ in spans for v in (first, self.tail * 64)], dtype=torch.int64, device=self.device)
            ctx.set_global_op_bits(self.rows.data_ptr() + self.cap * 16, self.row_words * 8, self.meta)
        ctx.set_join_user_records(bool(int(sizes[:, 4].sum())))         # no CUSTOM1 records anywhere: no span tables to clear
        self.kept_counts, self.dense = [int(v) for v in sizes[:, 0]], dense


def output_bases(out_bytes: int, rank: int, world: int, dist, device):
    """All-gathers the per-shard text sizes; returns (this shard's byte offset in the whole file's
    activities section, total bytes).  CPU-op events of all shards precede GPU events in the
    reference's file; callers that need that exact order place the two parts separately."""
    import torch

    mine = torch.tensor([out_bytes], dtype=torch.int64, device=device)
    sizes = torch.empty(world, dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(sizes, mine)
    sizes = sizes.cpu()
    return int(sizes[:rank].sum()), int(sizes.sum())


def shared_file_layout(ops_bytes: int, out_bytes: int, rank: int, world: int, dist, device):
    """Where this shard's text goes in the whole trace's activities text.  The reference writes every CPU-side
    activity before the first GPU-side one (libkineto/src/output_membuf.h:91-107), and a shard's text is its own
    CPU-op events followed by its GPU-side events, so a shard has two destinations: its CPU-op events after those
    of the lower ranks, its GPU-side events after ALL CPU-op events and the lower ranks' GPU-side events.
    One collective of two numbers per rank.  Returns (ops_offset, gpu_offset, total_bytes); also sums nothing
    else: counters are reduced by `reduce_counters`."""
    import torch

    mine = torch.tensor([ops_bytes, out_bytes - ops_bytes], dtype=torch.int64, device=device)
    sizes = torch.empty(world * 2, dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(sizes, mine)
    sizes = sizes.cpu().view(world, 2)
    all_ops = int(sizes[:, 0].sum())
    return int(sizes[:rank, 0].sum()), all_ops + int(sizes[:rank, 1].sum()), all_ops + int(sizes[:, 1].sum())


def write_shared_file(write_at, fd: int, base: int, ops_bytes: int, out_bytes: int, rank: int, world: int, dist, device):
    """Every rank writes its two parts into the one file open as `fd` (each rank opens the file itself), the
    activities text starting at file offset `base`.  `write_at(fd, file_offset, begin, n_bytes)` writes bytes
    [begin, begin + n_bytes) of the shard's text: `K2J.write_output_at` on a GPU.  Returns the total length of
    the activities text; the caller adds header and trailer and renames the file."""
    ops_off, gpu_off, total = shared_file_layout(ops_bytes, out_bytes, rank, world, dist, device)
    write_at(fd, base + ops_off, 0, ops_bytes)
    write_at(fd, base + gpu_off, ops_bytes, out_bytes - ops_bytes)
    return total


_COUNTERS = ("x_events", "flow_events", "n_records", "out_of_range_events", "blocklisted_runtime_events",
             "invalid_external_correlation_events", "unexpected_cuda_events", "out_bytes")


def reduce_counters(result: dict, dist, device) -> dict:
    """Sums the per-shard event and error counts over the ranks (the reference keeps one set per trace:
    GenericActivityProfiler::ErrorCounts, libkineto/src/GenericActivityProfiler.h:528-535)."""
    import torch

    t = torch.tensor([int(result[k]) for k in _COUNTERS], dtype=torch.int64, device=device)
    dist.all_reduce(t)
    return dict(zip(_COUNTERS, (int(v) for v in t.cpu())))
