"""Named parity cases shared by the CPU and GPU test suites."""
from __future__ import annotations

import numpy as np

from kineto_b200 import synth
from kineto_b200 import tracefile as tf

I64_MIN = -(1 << 63)


def edge_trace(flags=0) -> tf.Trace:
    """Hand-built trace that walks the reference's special cases one by one."""
    b = synth.TraceBuilder(n_devices=2, flags=flags, buffer_bytes=1 << 20)
    t0 = b.t0
    b.window = (t0, t0 + 1_000_000)
    b.thread(1001, 5001)
    b.thread(1001, 6001)          # duplicate thread id: the first pair wins
    b.thread(-7, -5002)           # negative system tid prints as its absolute value
    # ---- CPU-side activities ----
    b.op(t0 + 100, t0 + 900, 1, "aten::add", md=[("Sequence number", tf.MD_INT64, 7),
                                                 ("Input Dims", tf.MD_RAWJSON, "[[2, 3], []]")])
    b.op(t0 + 1000, t0 + 1900, 2, 'aten::"mul"\\x', flow_id=5, flow_type=1, flow_start=1)
    b.op(t0 + 2000, t0 + 2100, 3, "kernel", type=synth.USER_ANNOTATION, resource=-77)
    b.op(t0 + 2200, t0 + 2300, 0, "no external id", resource=I64_MIN, flow_id=9, flow_type=2, flow_start=0)
    b.op(t0 + 2400, t0 + 2500, -4, "negative\nid\ttab", type=synth.PYTHON_FUNCTION, flow_id=11, flow_type=3)
    b.op(t0 + 2600, t0 + 2600, 5, "", md=[("d1", tf.MD_DOUBLE, 1.5), ("d2", tf.MD_DOUBLE, float("inf")),
                                          ("d3", tf.MD_DOUBLE, -0.0), ("d4", tf.MD_DOUBLE, 1e22),
                                          ("d5", tf.MD_DOUBLE, float("nan")), ("b", tf.MD_BOOL, 1),
                                          ("s", tf.MD_STRING, 'C:\\path\n"q"'), ("u", tf.MD_UINT64, (1 << 64) - 1),
                                          ("i", tf.MD_INT64, I64_MIN), ("k\\ey\n", tf.MD_BOOL, 0)])
    b.op(t0 + 2700, t0 + 2800, 6, "gpu annotation", type=synth.GPU_USER_ANNOTATION, device=0, resource=7)
    b.op(b.base - 50, t0 + 10, 7, "starts before base time")
    b.op(t0 + 3000, t0 + 3100, 2, "duplicate id 2: last one wins")
    b.op(t0 + 3200, t0 + 3300, 8, "é utf8 name", type=synth.CONCURRENT_KERNEL, device=1, resource=3)
    # ---- first buffer ----
    b.extcorr(100, 1)
    b.runtime(t0 + 200, t0 + 300, 100)
    b.kernel(t0 + 500, t0 + 1500, 100, "void foo<int>(float*)", device=1, stream=9, grid=(100, 2, 1),
             block=(256, 1, 1), regs=40, ssmem=1024, dsmem=2048, queued=t0 + 400, graph=3, graph_node=77,
             channel=4, channel_type=2)
    b.extcorr(101, 99)             # first writer for correlation 101 ...
    b.extcorr(101, 2)              # ... replaced by the last writer
    b.runtime(t0 + 1200, t0 + 1300, 101, cbid=synth.CBID_cudaMemcpyAsync)
    b.memcpy(t0 + 1500, t0 + 2500, 101, 1 << 20)
    b.runtime(t0 + 1400, t0 + 1450, 102, cbid=synth.CBID_cudaMemsetAsync, tid=-7 & 0xFFFFFFFF)
    b.memset(t0 + 2600, t0 + 2700, 102, 4096, value=7)
    b.memcpy_p2p(t0 + 2800, t0 + 2900, 103, 12345)
    b.runtime(t0 + 3000, t0 + 3100, 104, cbid=synth.CBID_cudaGetLastError)   # blocklisted
    b.runtime(t0 + 3000, t0 + 3100, 104, cbid=16)                            # blocklisted
    b.runtime(t0 + 3000, t0 + 3100, 104, cbid=20, tid=4242)                  # no flow start: "f" event
    b.runtime(t0 + 3000, t0 + 3100, 0, cbid=200)                             # correlation 0: no flow
    b.runtime(t0 + 3000, t0 + 3100, 106, cbid=5000)                          # past the name table
    b.driver(t0 + 3200, t0 + 3300, 105)
    b.driver(t0 + 3200, t0 + 3300, 105, cbid=549)                            # tracked, no flow start
    b.driver(t0 + 3200, t0 + 3300, 105, cbid=1)                              # untracked driver call
    b.kernel(t0 + 3500, t0 + 3600, 105, "k\tbad")                            # non-printable: "unknown"
    b.kernel(t0 + 3500, t0 + 3600, 107, "kernel")                            # legacy rename
    b.kernel(t0 + 3500, t0 + 3600, 108, 'quo"te\\back\nslash')
    b.kernel(t0 + 3500, t0 + 3600, 109, "del\x7f")
    b.kernel(t0 + 3500, t0 + 3600, 110, "")
    b.new_buffer()
    # ---- second buffer: join and window corner cases ----
    b.extcorr(0x80000005, 1)
    b.kernel(t0 + 4000, t0 + 4100, 0x80000005, "corr above 2^31 never links")
    b.extcorr(120, (1 << 32) + 1)
    b.kernel(t0 + 4000, t0 + 4100, 120, "external id does not fit an int")
    b.extcorr(121, 55)
    b.kernel(t0 + 4000, t0 + 4100, 121, "external id without a CPU op")
    b.extcorr(122, 1, ext_kind=7)                                            # invalid external kind
    b.extcorr(123, 0)
    b.kernel(t0 + 4000, t0 + 4100, 123, "linked op with id 0")
    b.extcorr(124, 0xFFFFFFFFFFFFFFFC)                                       # -4 as uint64
    b.kernel(t0 + 4000, t0 + 4100, 124, "negative external id links to op -4")
    b.kernel(t0 - 1, t0 + 50, 125, "starts before the window")
    b.kernel(t0 + 999_000, t0 + 1_000_001, 126, "ends after the window")
    b.kernel(t0 + 999_000, t0 + 1_000_000, 127, "ends exactly at the window end")
    b.runtime(t0 - 5, t0 + 5, 128)
    b.memcpy(t0 + 5000, t0 + 5000, 129, 100)                                 # zero duration: no bandwidth
    b.memcpy(t0 + 5000, t0 + 4990, 130, 100)                                 # negative duration
    b.memcpy(t0 + 5000, t0 + 5003, 131, (1 << 64) - 1, copy_kind=0, src_kind=9, dst_kind=0)
    b.memcpy(t0 + 5000, t0 + 5007, 132, 1, copy_kind=9, src_kind=7, dst_kind=6)
    b.memset(t0 + 5000, t0 + 5003, 133, 10, memory_kind=9)
    b.memset(t0 + 5000, t0 + 5003, 134, 10, memory_kind=0, device=5, stream=0xFFFFFFFF)
    b.kernel(t0 + 6000, t0 + 6100, 135, "device out of range", device=2)
    b.kernel(t0 + 6000, t0 + 6100, 136, "zero block", block=(0, 1, 1))
    b.kernel(t0 + 6000, t0 + 6100, 137, "grid product wraps", grid=(65536, 65536, 2), block=(1024, 1, 1))
    b.kernel(t0 + 6000, t0 + 6100, 138, "negative grid", grid=(-3, 1, 1), block=(33, 3, 1), regs=255,
             ssmem=0x7FFFFFFF, dsmem=1)
    b.kernel(t0 + 6000, t0 + 6100, 139, "too much smem", block=(128, 1, 1), ssmem=100_000, dsmem=200_000)
    b.kernel(t0 + 6000, t0 + 6100, 140, "regs limited", block=(1024, 1, 1), regs=128)
    b.kernel(t0 + 6000, t0 + 6100, 141, "big ids", queued=(1 << 64) - 1, graph=0xFFFFFFFF, graph_node=(1 << 64) - 1,
             channel=0xFFFFFFFF, channel_type=0x7FFFFFFF, context=0xFFFFFFFF, stream=0xFFFFFFFF)
    # overhead records (CUPTI_ACTIVITY_KIND_OVERHEAD): every named kind, an unknown kind, window corner cases
    for i, k in enumerate([0, 1, 1 << 16, 2 << 16, 3 << 16, 4 << 16, 5 << 16, 6 << 16, 7 << 16, 0x7FFFFFFF, 12345]):
        b.overhead(t0 + 6500 + i, t0 + 6600 + 3 * i, overhead_kind=k, corr=100 if i == 2 else 0, pid=77, tid=88)
    b.overhead(t0 + 6700, t0 + 6690)                                         # negative duration
    b.overhead(0, 0)                                                         # no timestamps: outside the window
    b.overhead(t0 + 999_990, t0 + 1_000_001)                                 # ends after the window
    b.new_buffer()
    # ---- third buffer: an unknown kind ends the walk of this buffer ----
    b.kernel(t0 + 7000, t0 + 7100, 150, "before the unknown record")
    b.raw_record(77, 48)
    b.kernel(t0 + 7000, t0 + 7100, 151, "never reached")
    b.new_buffer()
    # ---- fourth buffer ----
    b.kernel(t0 + 8000, t0 + 8100, 152, "after the broken buffer")
    return b.build()


def annotation_trace() -> tf.Trace:
    """User annotations: CUSTOM1 correlation records extend per-(device, stream) spans."""
    b = synth.TraceBuilder(n_devices=2, flags=tf.FLAG_USER_ANNOTATIONS)
    t0 = b.t0
    b.op(t0 + 100, t0 + 5000, 1, "aten::add")
    b.op(t0 + 50, t0 + 9000, 20, "ProfilerStep#3", type=synth.USER_ANNOTATION)
    b.op(t0 + 60, t0 + 8000, 21, 'anno "two"', type=synth.USER_ANNOTATION)
    for i in range(12):
        corr = 300 + i
        b.extcorr(corr, 1)
        b.extcorr(corr, 20 + (i % 2), ext_kind=tf.EXTERNAL_KIND_CUSTOM1)
        b.runtime(t0 + 200 + 10 * i, t0 + 205 + 10 * i, corr)
        b.kernel(t0 + 1000 + 100 * i, t0 + 1050 + 100 * i, corr, "k%d" % i, device=i % 2, stream=7 + (i % 3))
    b.extcorr(400, 999, ext_kind=tf.EXTERNAL_KIND_CUSTOM1)   # annotation op unknown
    b.memcpy(t0 + 3000, t0 + 3100, 400, 64)
    b.extcorr(401, 20, ext_kind=tf.EXTERNAL_KIND_CUSTOM1)
    b.memset(t0 + 10, t0 + 20, 401, 64, stream=7)            # earliest start on (0, 7)
    b.extcorr(402, 21, ext_kind=tf.EXTERNAL_KIND_CUSTOM1)
    b.kernel(t0 - 100, t0 + 20, 402, "out of window, no span")
    return b.build()


def tsc_trace(n=3000) -> tf.Trace:
    return synth.gen_kernel_launches(n, seed=21, pool_size=64, ts_mode=1)


def overhead_mix_trace(n=3000, seed=41, flags=0) -> tf.Trace:
    """Random mixture of every record kind the path formats, overhead records included, packed into
    small buffers so that records of every size straddle chunk and buffer boundaries."""
    rng = np.random.default_rng(seed)
    b = synth.TraceBuilder(n_devices=4, flags=flags, buffer_bytes=1 << 20)
    t0 = b.t0
    b.window = (t0, t0 + 50_000_000)
    b.thread(1001, 5001)
    for i in range(n // 10):
        b.op(t0 + 100 * i, t0 + 100 * i + 60, i + 1, "aten::op%d" % (i % 7))
    kinds = [0, 1 << 16, 2 << 16, 3 << 16, 5 << 16, 99]
    for i in range(n):
        ts = t0 + 1000 + 37 * i
        k = int(rng.integers(0, 8))
        corr = 1000 + i
        if k == 0:
            b.extcorr(corr, int(rng.integers(1, n // 10 + 5)))
        elif k == 1:
            b.runtime(ts, ts + 20, corr - int(rng.integers(0, 3)))
        elif k == 2:
            b.kernel(ts, ts + int(rng.integers(1, 5000)), corr - int(rng.integers(0, 3)), "k%d" % (i % 13), device=i % 4,
                     stream=7 + i % 5, grid=(int(rng.integers(1, 500)), 1, 1), block=(int(rng.integers(1, 1025)), 1, 1))
        elif k == 3:
            b.memcpy(ts, ts + int(rng.integers(0, 900)), corr - 1, int(rng.integers(1, 1 << 30)))
        elif k == 4:
            b.memset(ts, ts + 5, corr - 1, int(rng.integers(1, 1 << 20)))
        elif k == 5:
            b.memcpy_p2p(ts, ts + 7, corr - 2, int(rng.integers(1, 1 << 24)))
        else:
            b.overhead(ts, ts + int(rng.integers(0, 300)), overhead_kind=kinds[int(rng.integers(0, len(kinds)))])
        if rng.random() < 0.004:
            b.new_buffer()
    return b.build()


def sync_trace(flags=0) -> tf.Trace:
    """CUDA synchronisation and CUDA event records (CUPTI_ACTIVITY_KIND_SYNCHRONIZATION / CUDA_EVENT): the
    context -> device map, the (context, event) -> record lookup, deferred stream-wait events, the
    dedicated row of stream syncs and its once-per-row metadata."""
    NO = 0xFFFFFFFF
    b = synth.TraceBuilder(n_devices=4, flags=flags, buffer_bytes=1 << 20)
    t0 = b.t0
    b.window = (t0, t0 + 1_000_000)
    b.op(t0 + 100, t0 + 900, 1, "aten::sync_user")
    b.op(t0 + 100, t0 + 900, 2, "aten::other")
    # a sync before any record names its context: device 0
    b.sync(t0 + 10, t0 + 20, 200, type=tf.SYNC_TYPE_CONTEXT_SYNCHRONIZE, context=5, stream=NO)
    b.kernel(t0 + 100, t0 + 200, 201, "on device 1", device=1, context=5, stream=9)
    b.kernel(t0 + 100, t0 + 200, 202, "second writer of context 5", device=3, context=5, stream=9)
    b.memcpy(t0 + 100, t0 + 110, 203, 64, device=2, context=6, stream=11)
    b.memset(t0 + 100, t0 + 110, 204, 64, device=3, context=7, stream=12)
    b.memcpy_p2p(t0 + 100, t0 + 110, 205, 64, device=0, context=1, stream=7, src_device=2, src_context=8,
                 dst_device=3, dst_context=9)
    b.memcpy_p2p(t0 + 100, t0 + 110, 206, 64, device=0, context=1, stream=7, src_device=1, src_context=10,
                 dst_device=2, dst_context=10)
    b.kernel(t0 - 500, t0 - 400, 207, "out of window: still names context 11", device=2, context=11, stream=13)
    # CUDA events: several records per (context, event)
    b.extcorr(300, 1)
    b.cuda_event(t0 + 300, 300, event=70, context=5, stream=9)
    b.cuda_event(t0 + 310, 310, event=70, context=5, stream=10)
    b.cuda_event(t0 + 320, 320, event=70, context=5, stream=NO)
    b.cuda_event(t0 + 330, 310, event=70, context=5, stream=14)     # same correlation id as an earlier record
    b.cuda_event(t0 + 340, 305, event=70, context=6, stream=15)     # other context
    b.cuda_event(t0 + 350, 0, event=71, context=5, stream=16)       # correlation 0: no flow
    b.cuda_event(t0 - 5, 301, event=72, context=5, stream=9)        # before the window
    b.cuda_event(t0 + 1_000_000, 302, event=72, context=5, stream=9)  # ts + 1 ns ends after the window
    b.cuda_event(0, 303, event=73, context=12, stream=9)            # unknown context
    b.new_buffer()
    # synchronisation records
    b.extcorr(400, 2)
    b.sync(t0 + 400, t0 + 450, 400, type=tf.SYNC_TYPE_EVENT_SYNCHRONIZE, context=5, stream=NO, event=70)  # before every record
    b.sync(t0 + 400, t0 + 450, 309, type=tf.SYNC_TYPE_EVENT_SYNCHRONIZE, context=5, stream=9, event=70)   # -> record 300
    b.sync(t0 + 400, t0 + 450, 310, type=tf.SYNC_TYPE_EVENT_SYNCHRONIZE, context=5, stream=9, event=70)   # equal id
    b.sync(t0 + 400, t0 + 450, 315, type=tf.SYNC_TYPE_EVENT_SYNCHRONIZE, context=5, stream=9, event=70)
    b.sync(t0 + 400, t0 + 450, 1000, type=tf.SYNC_TYPE_EVENT_SYNCHRONIZE, context=5, stream=9, event=70)  # -> stream -1
    b.sync(t0 + 400, t0 + 450, 299, type=tf.SYNC_TYPE_EVENT_SYNCHRONIZE, context=5, stream=9, event=70)   # none precedes
    b.sync(t0 + 400, t0 + 450, 500, type=tf.SYNC_TYPE_EVENT_SYNCHRONIZE, context=6, stream=11, event=70)
    b.sync(t0 + 400, t0 + 450, 500, type=tf.SYNC_TYPE_EVENT_SYNCHRONIZE, context=6, stream=11, event=99)  # unknown event
    b.sync(t0 + 500, t0 + 560, 501, type=tf.SYNC_TYPE_STREAM_SYNCHRONIZE, context=5, stream=9)
    b.sync(t0 + 510, t0 + 570, 0, type=tf.SYNC_TYPE_STREAM_SYNCHRONIZE, context=5, stream=9)             # same row: no metadata
    b.sync(t0 + 520, t0 + 580, 502, type=tf.SYNC_TYPE_STREAM_SYNCHRONIZE, context=6, stream=9)            # other device
    b.sync(t0 - 50, t0 + 10, 503, type=tf.SYNC_TYPE_STREAM_SYNCHRONIZE, context=7, stream=12)             # out of window ...
    b.sync(t0 + 530, t0 + 531, 504, type=tf.SYNC_TYPE_STREAM_SYNCHRONIZE, context=7, stream=12)           # ... so this one is first
    b.sync(t0 + 540, t0 + 541, 505, type=tf.SYNC_TYPE_STREAM_SYNCHRONIZE, context=7, stream=NO)
    b.sync(t0 + 550, t0 + 540, 506, type=tf.SYNC_TYPE_STREAM_SYNCHRONIZE, context=77, stream=3)           # negative duration
    b.sync(t0 + 560, t0 + 565, 507, type=tf.SYNC_TYPE_CONTEXT_SYNCHRONIZE, context=9, stream=NO)
    b.sync(t0 + 570, t0 + 575, 508, type=0, context=8, stream=4)
    b.sync(t0 + 580, t0 + 585, 509, type=99, context=10, stream=4, event=70)
    # stream-wait events: deferred to the end, dropped on streams without GPU work in the window
    b.sync(t0 + 600, t0 + 605, 320, type=tf.SYNC_TYPE_STREAM_WAIT_EVENT, context=5, stream=9, event=70)    # (1, 9) seen
    b.sync(t0 + 610, t0 + 615, 321, type=tf.SYNC_TYPE_STREAM_WAIT_EVENT, context=5, stream=10, event=70)   # (1, 10) never
    b.sync(t0 + 620, t0 + 625, 322, type=tf.SYNC_TYPE_STREAM_WAIT_EVENT, context=11, stream=13, event=1)   # only out of window
    b.sync(t0 + 630, t0 + 635, 323, type=tf.SYNC_TYPE_STREAM_WAIT_EVENT, context=6, stream=21, event=70)   # seen later
    b.sync(t0 - 30, t0 + 635, 324, type=tf.SYNC_TYPE_STREAM_WAIT_EVENT, context=5, stream=9, event=70)     # out of window
    b.sync(t0 + 640, t0 + 645, 400, type=tf.SYNC_TYPE_STREAM_WAIT_EVENT, context=6, stream=11, event=70)   # linked
    b.sync(t0 + 650, t0 + 655, 325, type=tf.SYNC_TYPE_STREAM_WAIT_EVENT, context=5, stream=NO, event=70)
    b.new_buffer()
    b.kernel(t0 + 700, t0 + 800, 600, "makes (2, 21) a seen stream", device=2, context=6, stream=21)
    b.kernel(t0 + 700, t0 + 800, 601, "after the deferred records", device=1, context=5, stream=NO)
    b.runtime(t0 + 700, t0 + 710, 602)
    return b.build()


def sync_mix_trace(n=3000, seed=43, flags=0) -> tf.Trace:
    """Random mixture with synchronisation and CUDA event records: few contexts, events and streams, so that
    lookups hit records with equal and neighbouring correlation ids and stream-wait events meet both seen
    and unseen streams; small buffers."""
    rng = np.random.default_rng(seed)
    b = synth.TraceBuilder(n_devices=4, flags=flags, buffer_bytes=1 << 20)
    t0 = b.t0
    b.window = (t0, t0 + 100_000)
    for i in range(n // 20):
        b.op(t0 + 100 * i, t0 + 100 * i + 60, i + 1, "aten::op%d" % (i % 7))
    for i in range(n):
        ts = t0 - 2000 + 37 * i            # the first and the last records fall outside the window
        k = int(rng.integers(0, 10))
        corr = 1000 + int(rng.integers(0, n // 4))
        ctx = int(rng.integers(1, 7))
        stream = int(rng.choice([7, 8, 9, 20, 0xFFFFFFFF]))
        if k == 0:
            b.extcorr(corr, int(rng.integers(1, n // 20 + 5)))
        elif k == 1:
            b.runtime(ts, ts + 20, corr)
        elif k == 2:
            b.kernel(ts, ts + int(rng.integers(1, 500)), corr, "k%d" % (i % 13), device=int(rng.integers(0, 4)), context=ctx,
                     stream=stream)
        elif k == 3:
            b.memcpy(ts, ts + int(rng.integers(0, 90)), corr, 4096, device=int(rng.integers(0, 4)), context=ctx, stream=stream)
        elif k == 4:
            b.memcpy_p2p(ts, ts + 7, corr, 64, device=0, context=ctx, stream=stream, src_device=int(rng.integers(0, 4)),
                         src_context=int(rng.integers(1, 9)), dst_device=int(rng.integers(0, 4)), dst_context=int(rng.integers(1, 9)))
        elif k in (5, 6):
            b.cuda_event(ts, corr, event=int(rng.integers(1, 6)), context=ctx, stream=stream)
        else:
            b.sync(ts, ts + int(rng.integers(0, 60)), corr, type=int(rng.integers(0, 6)), context=int(rng.integers(1, 9)),
                   stream=stream, event=int(rng.integers(1, 7)))
        if rng.random() < 0.004:
            b.new_buffer()
    return b.build()


def collective_trace(n=40, seed=51) -> tf.Trace:
    """Kernels launched from record_param_comms CPU ops: the logger copies the op's collective metadata onto the
    kernel event (libkineto/src/output_json.cpp:718-801, :900-906).  Covers complete and incomplete key sets,
    quoted and unquoted strings, every value type, and ops that are not collectives."""
    rng = np.random.default_rng(seed)
    b = synth.TraceBuilder(n_devices=8)
    t0 = b.t0
    colls = ["allreduce", "allgather", "reduce_scatter", "all_to_all"]
    S, R, I, U, D, B = tf.MD_STRING, tf.MD_RAWJSON, tf.MD_INT64, tf.MD_UINT64, tf.MD_DOUBLE, tf.MD_BOOL
    for i in range(n):
        name = colls[i % 4]
        size = int(np.exp(rng.uniform(np.log(1 << 10), np.log(1 << 32))))
        ranks = list(range(int(rng.integers(2, 9))))
        md = [("Collective name", S if i % 3 else R, name if i % 3 else '"%s"' % name),
              ("In msg nelems", I, size), ("Out msg nelems", I, size * (len(ranks) if name == "allgather" else 1)),
              ("Group size", I, len(ranks)), ("dtype", S, "BFloat16" if i % 2 else '"Float"'),
              ("Process Group Name", S, str(i % 3)), ("Process Group Description", S, "default_pg" if i % 3 == 0 else "tp\\group"),
              ("Process Group Ranks", R, str(ranks)), ("Rank", I, 3), ("Seq", I, i), ("Comms Id", U, (1 << 63) + i)]
        if name == "all_to_all":
            md += [("In split size", R, str([size // len(ranks)] * len(ranks))), ("Out split size", R, "[]" if i % 8 == 3 else str(ranks))]
        if i % 5 == 1:
            md += [("Input Tensors start", R, "[139800000000000]"), ("Output Tensors start", S, "[1, 2]")]
        if i % 7 == 2:
            md += [("Src Rank", I, 1), ("Dst Rank", I, -1)]
        if i % 9 == 4:
            md = [m for m in md if m[0] != "Group size"]             # incomplete: the first five keys are dropped together
        if i % 11 == 5:
            md = [m for m in md if m[0] != "dtype"] + [("dtype", S, '""')]   # a quoted empty string counts as absent
        if i % 13 == 6:
            md += [("Dst Rank", D, 2.5), ("Src Rank", B, 1)] if i % 7 != 2 else []
        if i % 17 == 8:   # non-finite doubles print as plain text here ("inf", "-nan"), quoted only where the key is
            md = [m for m in md if m[0] not in ("Seq", "Comms Id", "Process Group Name")] + [
                ("Seq", D, float("inf")), ("Comms Id", D, -float("nan")), ("Process Group Name", D, -float("inf"))]
        while len({m[0] for m in md}) > 13:   # one bucket generation of the reference's metadata map
            md.pop()
        b.op(t0 + 1000 * i, t0 + 1000 * i + 800, 100 + i, "record_param_comms", md=md)
        b.extcorr(500 + i, 100 + i)
        b.runtime(t0 + 1000 * i + 10, t0 + 1000 * i + 20, 500 + i)
        b.kernel(t0 + 1000 * i + 300, t0 + 1000 * i + 700, 500 + i, "ncclDevKernel_%s_RING_LL(ncclDevKernelArgs)" % name,
                 device=i % 8, stream=20 + i % 3)
    # not collectives: another op name, a copy launched by a collective op, a kernel without a link
    b.op(t0 + 90_000, t0 + 90_500, 900, "aten::add", md=[("Collective name", S, "allreduce")])
    b.extcorr(901, 900)
    b.kernel(t0 + 90_100, t0 + 90_200, 901, "linked to an ordinary op")
    b.extcorr(902, 100)
    b.memcpy(t0 + 90_300, t0 + 90_400, 902, 4096)
    b.kernel(t0 + 90_500, t0 + 90_600, 903, "no link")
    b.op(t0 + 91_000, t0 + 91_500, 950, "record_param_comms")                      # no metadata at all
    b.extcorr(951, 950)
    b.kernel(t0 + 91_100, t0 + 91_200, 951, "collective op without metadata")
    return b.build()


def instant_trace() -> tf.Trace:
    """CPU instant events (PyTorch's memory events): their own event shape, no sanitising of name or metadata."""
    b = synth.TraceBuilder(n_devices=2)
    t0 = b.t0
    I, S, R, D = tf.MD_INT64, tf.MD_STRING, tf.MD_RAWJSON, tf.MD_DOUBLE
    b.op(t0 + 100, t0 + 900, 1, "aten::empty")
    b.op(t0 + 150, t0 + 150, 0, "[memory]", type=synth.CPU_INSTANT_EVENT, md=[("Total Reserved", I, 1 << 33), ("Total Allocated", I, 123456789),
                                                                               ("Bytes", I, -4096), ("Addr", I, 139800000000000),
                                                                               ("Device Id", I, 0), ("Device Type", I, 1)])
    b.op(t0 + 160, t0 + 999, 7, 'back\\slash "quoted"\nname', type=synth.CPU_INSTANT_EVENT, resource=-77,
         md=[("k\\ey", S, 'C:\\dir\n"x"'), ("raw", R, "[1, 2]"), ("d", D, 0.5)])
    b.op(t0 + 170, t0 + 170, 8, "no metadata", type=synth.CPU_INSTANT_EVENT, device=0, flow_id=5, flow_type=1, flow_start=1)
    b.op(b.base - 5, t0, 9, "before the base time", type=synth.CPU_INSTANT_EVENT, device=1, resource=I64_MIN)
    b.op(t0 + 180, t0 + 190, 9, "op after instants, same id as one of them")
    b.extcorr(300, 9)
    b.kernel(t0 + 500, t0 + 600, 300, "linked to id 9")
    b.extcorr(301, 7)
    b.kernel(t0 + 500, t0 + 600, 301, "linked to an instant event")
    return b.build()


def gaps_trace(mode=1) -> tf.Trace:
    """Behaviour of the reference that rarely shows: activities that had not ended when the trace stopped
    (processCpuTrace ends them at the window's end and adds "finished": false), records of kinds the profiler only
    counts (stepped over), a kind no header defines (ends the walk of its buffer), correlation id 0 with and
    without a link next to keys that hash to the same table slot, and counter events."""
    b = synth.TraceBuilder(mode=mode, n_devices=2, buffer_bytes=1 << 20)
    t0 = b.t0
    b.window = (t0, t0 + 5_000_000)
    I, S, R, D, C = tf.MD_INT64, tf.MD_STRING, tf.MD_RAWJSON, tf.MD_DOUBLE, tf.MD_COUNTER
    fin = ("finished", R, "false")
    # ---- unfinished activities: end < start ----
    b.op(t0 + 100, t0 + 50, 1, "aten::unfinished", md=[("Sequence number", I, 7), ("Input Dims", R, "[[2, 3], []]"), fin])
    b.op(t0 + 200, 0, 2, "aten::end zero", md=[fin])
    b.op(t0 + 300, t0 + 299, 3, "annotation that never closed", type=synth.USER_ANNOTATION,
         md=[("a", I, 1), ("b", I, 2), ("c", I, 3), ("d", I, 4), ("e", S, "x"), fin], flow_id=4, flow_type=1, flow_start=1)
    b.op(t0 + 6_000_000, t0 + 5_999_999, 4, "starts after the window's end", md=[fin])
    b.op(t0 + 400, t0 + 500, 5, "finished in time", md=[("finished", R, "true")])
    b.op(t0 + 600, t0 + 100, 0, "id 0, unfinished", md=[fin])
    # ---- counter events ----
    b.op(t0 + 700, t0 + 700, 11, "mtia counters", type=17, device=3, resource=-9,
         md=[("ignored", I, 5), ("hbm_read_bw", C, 1.5), ("cache \"hit\"", C, 0.25), ("big", C, 1e22), ("nan", C, float("nan")),
             ("neg inf", C, float("-inf")), ("zero", C, 0.0)])
    b.op(t0 + 710, t0 + 715, 12, "mtia, no values", type=17)
    if mode == 0:  # these two types are not in the profiler's default selection; a logger driven directly writes them
        b.op(t0 + 720, t0 + 720, 13, "xpu scope", type=26, device=0, resource=I64_MIN, md=[("metric.a", C, 3.0), ("metric.b", C, 1e-7)])
        b.op(t0 + 730, t0 + 730, 14, "hw counters", type=28, device=1, resource=42,
             md=[("sm__cycles_active.avg", C, 123456.75), ("dram__bytes_read.sum", C, 1.8446744073709552e19), ("q\"uote", C, -2.5)])
        b.op(t0 + 740, t0 + 740, 15, "hw counters without values", type=28, device=1, resource=42, md=[("x", I, 1)])
        b.op(b.base - 10, t0, 16, "hw counter before the base time", type=28, device=0, resource=-3, md=[("c", C, 2.0)])
    if mode == 0:  # a logger driven directly sees no CUPTI records
        return b.build()
    # ---- first buffer: kinds that are only counted ----
    b.other(9, 32)                     # CONTEXT
    b.extcorr(100, 1)
    b.other(12, 56)                    # MARKER
    b.runtime(t0 + 200, t0 + 300, 100)
    b.other(49, 128)                   # MEMORY2
    b.other(8, 184)                    # DEVICE
    b.kernel(t0 + 500, t0 + 1500, 100, "after four skipped records", device=1, stream=9)
    b.other(3, 208)                    # KERNEL (the serialised-kernel kind, same structure as CONCURRENT_KERNEL)
    b.other(48, 40)                    # INTERNAL_LAUNCH_API: 40 bytes, like a runtime record
    b.other(37, 24)                    # STREAM
    b.memcpy(t0 + 1500, t0 + 2500, 100, 1 << 20)
    for k in (6, 7, 11, 13, 14, 21, 23, 27, 28, 31, 32, 41, 45, 50, 52, 54):
        b.other(k, 8 * [0, 12, 11, 26, 5, 5, 3, 3, 23, 4, 26, 4, 7, 4, 3, 7, 5, 7, 18, 5, 5, 4, 12, 4, 6, 13, 4, 3, 3, 7, 5, 4, 3, 19,
                        19, 15, 7, 3, 7, 3, 17, 4, 4, 4, 4, 10, 21, 5, 5, 16, 9, 7, 8, 7, 8][k])
    b.kernel(t0 + 1600, t0 + 1700, 100, "after sixteen more")
    b.new_buffer()
    # ---- second buffer: correlation id 0 ----
    b.extcorr(0, 5)                    # correlation id 0, linked to op 5
    b.kernel(t0 + 2000, t0 + 2100, 0, "correlation 0 (no flow), linked")
    b.memset(t0 + 2000, t0 + 2100, 0, 64)
    for corr, ext in ((2654435769, 3), (1, 2), (2, 1), (3, 99)):
        b.extcorr(corr, ext)
        b.kernel(t0 + 2200, t0 + 2300, corr, "corr %d" % corr)
    b.new_buffer()
    # ---- third buffer: a kind no header defines ends the walk; the records behind it are lost, as in a walk that
    # cannot size the record ----
    b.kernel(t0 + 3000, t0 + 3100, 1, "before the undefined kind")
    b.other(60, 16)
    b.kernel(t0 + 3200, t0 + 3300, 2, "never reached")
    b.new_buffer()
    b.kernel(t0 + 3400, t0 + 3500, 3, "next buffer is walked again")
    b.other(0, 8)                      # kind 0 (INVALID): undefined as well
    return b.build()


def corr_zero_unlinked_trace() -> tf.Trace:
    """Correlation id 0 whose external id names no CPU op, in front of keys that probe past the slot id 0 hashes to."""
    b = synth.TraceBuilder(n_devices=1)
    t0 = b.t0
    b.op(t0 + 100, t0 + 200, 1, "op 1")
    b.op(t0 + 100, t0 + 200, 0, "op 0")
    b.extcorr(0, 77)                   # no op 77: correlation 0 stays unlinked
    for corr in range(1, 40):
        b.extcorr(corr, corr & 1)
        b.kernel(t0 + 300 + corr, t0 + 400 + corr, corr, "k%d" % corr)
    b.kernel(t0 + 500, t0 + 600, 0, "correlation 0, unlinked")
    b.sync(t0 + 700, t0 + 800, 0, stream=7)            # a synchronisation record prints its own correlation id when unlinked
    return b.build()


CASES = {
    "edge": edge_trace,
    "generic_300": lambda: synth.gen_generic_kernels(300, seed=31, pool_size=40),
    "launches_150": lambda: synth.gen_kernel_launches(150, seed=32, pool_size=50),
    "mixed_400": lambda: synth.gen_mixed(400, seed=33, pool_size=100, escape_fraction=0.2),
    "tsc_100": lambda: tsc_trace(100),
    "sync": sync_trace,
    "collectives": collective_trace,
    "instant": instant_trace,
    "gaps": gaps_trace,
    "gaps_direct": lambda: gaps_trace(mode=0),
    "corr_zero": corr_zero_unlinked_trace,
}


def without_flags(trace: tf.Trace) -> tf.Trace:
    """Copy of `trace` with every flag bit cleared (the reference itself never sorts)."""
    import copy
    t = copy.copy(trace)
    t.params = trace.params.copy()
    t.params["flags"] = 0
    return t


def with_flags(trace: tf.Trace, extra: int) -> tf.Trace:
    """Copy of `trace` with extra flag bits set."""
    import copy
    t = copy.copy(trace)
    t.params = trace.params.copy()
    t.params["flags"] = int(trace.params["flags"][0]) | extra
    return t


def presorted_launches(trace: tf.Trace) -> tf.Trace:
    """The same launches trace with its runtime and kernel records moved into stable order of their
    start timestamps (EXTERNAL_CORRELATION records first): what the sort option must reproduce."""
    import copy
    g = trace.cupti.reshape(-1, 272)
    ext = np.ascontiguousarray(g[:, :24]).view(tf.EXTCORR).reshape(-1)
    api = np.ascontiguousarray(g[:, 24:64]).view(tf.API).reshape(-1)
    ker = np.ascontiguousarray(g[:, 64:]).view(tf.KERNEL9).reshape(-1)
    starts = np.concatenate([api["start"].astype(np.int64), ker["start"].astype(np.int64)])
    kind = np.concatenate([np.zeros(len(api), np.int8), np.ones(len(ker), np.int8)])
    orig = np.concatenate([np.arange(len(api)) * 3 + 1, np.arange(len(ker)) * 3 + 2])
    o = np.lexsort((orig, starts))
    order = np.concatenate([np.zeros(len(ext), np.int8), kind[o] + 1])

    def by_start(a):
        raw = np.ascontiguousarray(a).view(np.uint8).reshape(len(a), -1)
        return raw[np.argsort(a["start"], kind="stable")].reshape(-1).view(a.dtype)

    t = copy.copy(trace)
    t.cupti, offs = tf.interleave([ext, by_start(api), by_start(ker)], order)
    t.buftab = tf.make_buftab(offs)
    return t
