"""Seeded synthetic traces with the shapes of the benchmark configurations.

These stand in for real profiler captures (no public dataset is involved): every generator is a
pure function of its arguments and seed.  `TraceBuilder` assembles small hand-written traces for
edge cases; `gen_generic_kernels`, `gen_kernel_launches` and `gen_mixed` are the vectorised
generators behind the named configurations.
"""
from __future__ import annotations

import os
import re

import numpy as np

from . import tracefile as tf
from .md_order import md_visit_order

# ActivityType values (libkineto/include/ActivityType.h:19-47)
CPU_OP, USER_ANNOTATION, GPU_USER_ANNOTATION, GPU_MEMCPY, GPU_MEMSET, CONCURRENT_KERNEL = range(6)
CUDA_RUNTIME, CUDA_DRIVER, CPU_INSTANT_EVENT = 7, 8, 9
PYTHON_FUNCTION = 10
LINK_FWD_BWD, LINK_ASYNC_CPU_GPU = 1, 2

DEFAULT_BASE_TIME = 227 * tf.BASE_PERIOD_NS  # a period boundary in late 2026
DEFAULT_PID = 424242

# Runtime callback ids used by the generators (cupti_runtime_cbid.h)
CBID_cudaGetLastError = 10
CBID_cudaMemcpy = 31
CBID_cudaMemcpyAsync = 41
CBID_cudaMemsetAsync = 51
CBID_cudaStreamSynchronize = 131
CBID_cudaEventCreate = 133
CBID_cudaLaunchKernel = 211
CBID_cuLaunchKernel = 307  # driver domain


def cbid_names(domain: str, cuda_home: str | None = None) -> list[str]:
    """Callback names per id for the runtime ('R') or driver ('D') domain, parsed from the CUDA
    toolkit's public cupti_*_cbid.h enum and stripped of the `_vNNNN` CUDA-version suffix the way
    the reference does (libkineto/src/cupti_strings.cpp:106-128); ids the enum does not name map to
    "INVALID"."""
    cuda_home = cuda_home or os.environ.get("CUDA_HOME", "/usr/local/cuda")
    fn = "cupti_runtime_cbid.h" if domain == "R" else "cupti_driver_cbid.h"
    prefix = "CUPTI_RUNTIME_TRACE_CBID_" if domain == "R" else "CUPTI_DRIVER_TRACE_CBID_"
    path = None
    for d in ("include", "extras/CUPTI/include", "targets/x86_64-linux/include"):
        cand = os.path.join(cuda_home, d, fn)
        if os.path.exists(cand):
            path = cand
            break
    if path is None:
        raise FileNotFoundError(fn)
    names: dict[int, str] = {}
    size = 0
    for m in re.finditer(prefix + r"(\w+)\s*=\s*(\d+)", open(path).read()):
        name, val = m.group(1), int(m.group(2))
        if name == "SIZE":
            size = val
            continue
        if name in ("INVALID", "FORCE_INT"):
            continue
        mm = re.match(r"^(.*)_v(\d{4,})$", name)
        names[val] = mm.group(1) if mm else name
    size = size or (max(names) + 1)
    return [names.get(i, "INVALID") for i in range(size)]


def _ident(rng: np.random.Generator, length: int) -> str:
    first = "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXY"  # never '_' or 'Z' first: not a mangled name
    rest = "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789_:<>, ()*&"
    s = first[rng.integers(len(first))] + "".join(rest[i] for i in rng.integers(len(rest), size=length - 1))
    return s


_cxa = None


def demangles(name: bytes) -> bool:
    """Does abi::__cxa_demangle accept `name`?  The reference shows kernel names through it
    (libkineto/src/Demangle.cpp:30-50), and it accepts more than `_Z...` symbols: any string that parses as a
    mangled TYPE demangles too ("G77" + 77 characters is an imaginary type of that name).  The library takes names
    that are already demangled, so the generators only hand out names the demangler leaves alone."""
    global _cxa
    if _cxa is None:
        import ctypes
        import ctypes.util
        lib = ctypes.CDLL(ctypes.util.find_library("stdc++") or "libstdc++.so.6")
        libc = ctypes.CDLL(ctypes.util.find_library("c") or "libc.so.6")
        lib.__cxa_demangle.restype = ctypes.c_void_p
        lib.__cxa_demangle.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
        libc.free.argtypes = [ctypes.c_void_p]
        _cxa = (ctypes, lib, libc)
    ctypes, lib, libc = _cxa
    if b"\0" in name:
        name = name.split(b"\0")[0]
    status = ctypes.c_int(0)
    p = lib.__cxa_demangle(name, None, None, ctypes.byref(status))
    if p:
        libc.free(p)
    return status.value == 0


def demangled(name: bytes) -> bytes:
    """What the reference's demangle() shows for `name` (libkineto/src/Demangle.cpp:33-53)."""
    if len(name) > 8192 or not demangles(name):
        return name
    ctypes, lib, libc = _cxa
    status = ctypes.c_int(0)
    p = lib.__cxa_demangle(name, None, None, ctypes.byref(status))
    out = ctypes.string_at(p)
    libc.free(p)
    return out


def name_pool(rng, count: int, lo: int, hi: int, escape_fraction: float = 0.0) -> list[bytes]:
    """`count` distinct ASCII identifiers of length uniform in [lo, hi].  A fraction carries bytes
    the JSON writer treats specially: quote, backslash, newline, TAB/control, UTF-8 multibyte."""
    out, seen = [], set()
    specials = [b'"', b"\\", b"\n", b"\t", b"\x01", "é".encode(), "核".encode(), b'""', b'\\"', b"\x7f"]
    while len(out) < count:
        n = int(rng.integers(lo, hi + 1))
        s = _ident(rng, n).encode()
        if rng.random() < escape_fraction:
            k = int(rng.integers(1, 4))
            b = bytearray(s)
            for _ in range(k):
                sp = specials[int(rng.integers(len(specials)))]
                pos = int(rng.integers(1, len(b)))
                b[pos:pos] = sp
            s = bytes(b[:max(n, 2)]) if len(b) > hi else bytes(b)
        if s not in seen and not demangles(s):
            seen.add(s)
            out.append(s)
    return out


def _params(mode: int, window: tuple[int, int], n_devices: int, base=DEFAULT_BASE_TIME, pid=DEFAULT_PID,
            flags=tf.FLAG_USER_ANNOTATIONS, ts_mode=0, conv=None):
    p = np.zeros(1, tf.PARAMS)
    p["base_time_ns"], p["window_start_ns"], p["window_end_ns"] = base, window[0], window[1]
    p["pid"], p["mode"], p["ts_mode"], p["flags"], p["n_devices"] = pid, mode, ts_mode, flags, n_devices
    if conv is not None:
        p["conv_t0"], p["conv_t0_approx"], p["conv_scale_mant"], p["conv_scale_exp"] = conv
    else:
        p["conv_scale_mant"], p["conv_scale_exp"] = 1 << 63, 0
    return p


def _ordered_md(keys: list[str]) -> list[int]:
    """Positions of `keys` in the order the reference visits them."""
    order = md_visit_order(tuple(keys))
    return [keys.index(k) for k in order]


class TraceBuilder:
    """Hand-assembled traces: records are appended in buffer order."""

    def __init__(self, mode=1, window=None, n_devices=8, base=DEFAULT_BASE_TIME, pid=DEFAULT_PID,
                 flags=tf.FLAG_USER_ANNOTATIONS, ts_mode=0, conv=None, buffer_bytes=4 << 20):
        self.base = base
        self.t0 = base + 1_000_000_000  # default window start: 1 s after base
        self.window = window or (self.t0, self.t0 + 10_000_000_000)
        self.pool = tf.StringPool()
        self.records: list[np.ndarray] = []
        self.ops: list[dict] = []
        self.tidmap: list[tuple[int, int]] = []
        self.kw = dict(mode=mode, n_devices=n_devices, base=base, pid=pid, flags=flags, ts_mode=ts_mode, conv=conv)
        self.pid = pid
        self.buffer_bytes = buffer_bytes
        self.buffer_breaks: list[int] = []

    def _rec(self, kind, **kw):
        r = np.zeros(1, tf.RECORD_DTYPE[kind])
        r["kind"] = kind
        for k, v in kw.items():
            r[k] = v
        self.records.append(r)
        return r

    def other(self, kind: int, nbytes: int, fill: int = 0xAB):
        """A record of a kind the path does not format: `nbytes` (a multiple of 8) of which the first four hold the kind."""
        assert nbytes % 8 == 0 and nbytes >= 8
        r = np.full(nbytes, fill, np.uint8)
        r[:4] = np.array([kind], "<u4").view(np.uint8)
        self.records.append(r)
        return r

    def kernel(self, start, end, corr, name="kernel", device=0, context=1, stream=7, grid=(1, 1, 1),
               block=(32, 1, 1), regs=32, ssmem=0, dsmem=0, queued=0, graph=0, graph_node=0, channel=0,
               channel_type=0):
        return self._rec(tf.KIND_CONCURRENT_KERNEL, start=start, end=end, correlationId=corr,
                         name=self.pool.add(name), deviceId=device, contextId=context, streamId=stream,
                         gridX=grid[0], gridY=grid[1], gridZ=grid[2], blockX=block[0], blockY=block[1],
                         blockZ=block[2], registersPerThread=regs, staticSharedMemory=ssmem,
                         dynamicSharedMemory=dsmem, queued=queued, graphId=graph, graphNodeId=graph_node,
                         channelID=channel, channelType=channel_type)

    def runtime(self, start, end, corr, cbid=CBID_cudaLaunchKernel, tid=1001, kind=tf.KIND_RUNTIME):
        return self._rec(kind, start=start, end=end, correlationId=corr, cbid=cbid, threadId=tid,
                         processId=self.pid)

    def driver(self, start, end, corr, cbid=CBID_cuLaunchKernel, tid=1001):
        return self.runtime(start, end, corr, cbid, tid, kind=tf.KIND_DRIVER)

    def extcorr(self, corr, ext_id, ext_kind=tf.EXTERNAL_KIND_CUSTOM0):
        return self._rec(tf.KIND_EXTERNAL_CORRELATION, correlationId=corr, externalId=ext_id, externalKind=ext_kind)

    def memcpy(self, start, end, corr, nbytes, copy_kind=1, src_kind=1, dst_kind=3, device=0, context=1,
               stream=7, graph=0, graph_node=0, channel=0, channel_type=0):
        return self._rec(tf.KIND_MEMCPY, start=start, end=end, correlationId=corr, bytes=nbytes,
                         copyKind=copy_kind, srcKind=src_kind, dstKind=dst_kind, deviceId=device,
                         contextId=context, streamId=stream, graphId=graph, graphNodeId=graph_node,
                         channelID=channel, channelType=channel_type)

    def memcpy_p2p(self, start, end, corr, nbytes, device=0, context=1, stream=7, src_device=0, src_context=1,
                   dst_device=1, dst_context=2, copy_kind=10, src_kind=3, dst_kind=3, graph=0, graph_node=0,
                   channel=0, channel_type=0):
        return self._rec(tf.KIND_MEMCPY2, start=start, end=end, correlationId=corr, bytes=nbytes,
                         copyKind=copy_kind, srcKind=src_kind, dstKind=dst_kind, deviceId=device,
                         contextId=context, streamId=stream, srcDeviceId=src_device, srcContextId=src_context,
                         dstDeviceId=dst_device, dstContextId=dst_context, graphId=graph,
                         graphNodeId=graph_node, channelID=channel, channelType=channel_type)

    def memset(self, start, end, corr, nbytes, value=0, memory_kind=3, device=0, context=1, stream=7, graph=0,
               graph_node=0, channel=0, channel_type=0):
        return self._rec(tf.KIND_MEMSET, start=start, end=end, correlationId=corr, bytes=nbytes, value=value,
                         memoryKind=memory_kind, deviceId=device, contextId=context, streamId=stream,
                         graphId=graph, graphNodeId=graph_node, channelID=channel, channelType=channel_type)

    def overhead(self, start, end, overhead_kind=1 << 16, corr=0, object_kind=1, pid=0, tid=0):
        """CUpti_ActivityOverhead (CUPTI_ACTIVITY_KIND_OVERHEAD); `overhead_kind` is the CUPTI enum value."""
        return self._rec(tf.KIND_OVERHEAD, start=start, end=end, overheadKind=overhead_kind, objectKind=object_kind,
                         objectId0=pid, objectId1=tid, correlationId=corr)

    def sync(self, start, end, corr, type=tf.SYNC_TYPE_STREAM_SYNCHRONIZE, context=1, stream=7, event=0):
        """CUpti_ActivitySynchronization; `stream` 0xFFFFFFFF means "no stream applies"."""
        return self._rec(tf.KIND_SYNCHRONIZATION, type=type, start=start, end=end, correlationId=corr,
                         contextId=context, streamId=stream, cudaEventId=event)

    def cuda_event(self, ts, corr, event, context=1, stream=7):
        """CUpti_ActivityCudaEvent2 (a cudaEventRecord as seen by the device)."""
        return self._rec(tf.KIND_CUDA_EVENT, correlationId=corr, contextId=context, streamId=stream, eventId=event,
                         deviceTimestamp=ts)

    def raw_record(self, kind: int, size: int):
        """A record of a kind the path does not know, `size` bytes (multiple of 8)."""
        r = np.zeros(size // 4, np.uint32)
        r[0] = kind
        self.records.append(r.view(np.dtype((np.void, size))))

    def new_buffer(self):
        """Ends the current CUPTI buffer here."""
        self.buffer_breaks.append(len(self.records))

    def thread(self, tid: int, sys_tid: int):
        self.tidmap.append((tid, sys_tid))

    def op(self, start, end, id, name="aten::op", type=CPU_OP, device=None, resource=5001, thread=1001,
           flow_id=0, flow_type=0, flow_start=0, md=None):
        """`md`: list of (key, type, value) in insertion order; strings are interned here."""
        self.ops.append(dict(start=start, end=end, id=id, name=name, type=type,
                             device=self.pid if device is None else device, resource=resource, thread=thread,
                             flow_id=flow_id, flow_type=flow_type, flow_start=flow_start, md=md or []))

    def build(self) -> tf.Trace:
        t = tf.Trace()
        n = len(self.ops)
        t.op_start = np.array([o["start"] for o in self.ops], np.int64)
        t.op_end = np.array([o["end"] for o in self.ops], np.int64)
        t.op_id = np.array([o["id"] for o in self.ops], np.int64).astype(np.int32)
        t.op_device = np.array([o["device"] for o in self.ops], np.int32)
        t.op_resource = np.array([o["resource"] for o in self.ops], np.int64)
        t.op_thread = np.array([o["thread"] for o in self.ops], np.int32)
        t.op_type = np.array([o["type"] for o in self.ops], np.int32)
        t.op_name = np.array([self.pool.add(o["name"]) for o in self.ops], np.uint32)
        t.op_flow = np.array([o["flow_id"] for o in self.ops], np.uint32)
        t.op_flowt = np.array([o["flow_type"] | (o["flow_start"] << 4) for o in self.ops], np.uint8)
        mdoff, ents = [0], []
        for o in self.ops:
            md = o["md"]
            counters = [m for m in md if m[1] == tf.MD_COUNTER]   # counter values are a list: they keep their order
            md = [m for m in md if m[1] != tf.MD_COUNTER]
            keys = [k for k, _, _ in md]
            for k, ty, v in [md[j] for j in (_ordered_md(keys) if len(keys) > 1 else range(len(keys)))] + counters:
                if ty in (tf.MD_STRING, tf.MD_RAWJSON):
                    v = self.pool.add(v)
                elif ty in (tf.MD_DOUBLE, tf.MD_COUNTER):
                    v = int(np.array([v], np.float64).view(np.uint64)[0])
                elif ty == tf.MD_INT64:
                    v = int(np.array([v], np.int64).view(np.uint64)[0])
                ents.append((self.pool.add(k), ty, int(v)))
            mdoff.append(len(ents))
        t.op_mdoff = np.array(mdoff, np.uint32)
        t.md = np.array(ents, tf.MD_ENTRY) if ents else np.zeros(0, tf.MD_ENTRY)
        # records -> buffers
        raws = [np.ascontiguousarray(r).tobytes() for r in self.records]
        offs = np.concatenate([[0], np.cumsum([len(r) for r in raws])]).astype(np.int64)
        t.cupti = np.frombuffer(b"".join(raws), np.uint8).copy()
        breaks = sorted(set(self.buffer_breaks) | {0, len(raws)})
        tabs = []
        for a, b in zip(breaks[:-1], breaks[1:]):
            if b > a:
                sub = tf.make_buftab(offs[a:b + 1], self.buffer_bytes)
                tabs.append(sub)
        t.buftab = np.concatenate(tabs) if tabs else np.zeros(0, np.uint64)
        t.tidmap = np.array(self.tidmap, np.int32).reshape(-1)
        rt, dr = cbid_names("R"), cbid_names("D")
        t.rt_names = np.array([self.pool.add(s) for s in rt], np.uint32)
        t.dr_names = np.array([self.pool.add(s) for s in dr], np.uint32)
        t.set_pool(self.pool)
        t.devprops = tf.b200_device_props(self.kw["n_devices"])
        t.params = _params(self.kw["mode"], self.window, self.kw["n_devices"], self.kw["base"], self.kw["pid"],
                           self.kw["flags"], self.kw["ts_mode"], self.kw["conv"])
        return t


def _finish(t: tf.Trace, pool: tf.StringPool, mode, window, n_devices, **kw):
    rt, dr = cbid_names("R"), cbid_names("D")
    t.rt_names = np.array([pool.add(s) for s in rt], np.uint32)
    t.dr_names = np.array([pool.add(s) for s in dr], np.uint32)
    t.set_pool(pool)
    t.devprops = tf.b200_device_props(n_devices)
    t.params = _params(mode, window, n_devices, **kw)
    return t


def _monotone_starts(rng, n, t0, mean_gap_ns=2000.0):
    gaps = rng.exponential(mean_gap_ns, n).astype(np.int64) + 1
    return t0 + np.cumsum(gaps)


def _lognormal_dur(rng, n, median_ns=10_000.0, sigma=1.5):
    return np.maximum(1, rng.lognormal(np.log(median_ns), sigma, n)).astype(np.int64)


def gen_generic_kernels(n=100_000, seed=1, pool_size=512, name_len=(20, 200)) -> tf.Trace:
    """json_output_benchmark-style input: `n` GenericTraceActivity GPU-kernel records fed straight to
    the JSON logger (reference generator: benchmarks/json_output_benchmark.cpp:140-214): device 0,
    stream ids uniform in 7..38, monotone starts with Exp(2 us) gaps, lognormal durations,
    correlation id = index+1, names from a pool of ASCII identifiers, grid/block metadata."""
    rng = np.random.default_rng(seed)
    pool = tf.StringPool()
    names = np.array([pool.add(s) for s in name_pool(rng, pool_size, *name_len)], np.uint32)
    t = tf.Trace()
    t0 = DEFAULT_BASE_TIME + 1_000_000_000
    t.op_start = _monotone_starts(rng, n, t0)
    t.op_end = t.op_start + _lognormal_dur(rng, n)
    t.op_id = np.arange(1, n + 1, dtype=np.int32)
    t.op_device = np.zeros(n, np.int32)
    t.op_resource = rng.integers(7, 39, n).astype(np.int64)
    t.op_thread = np.zeros(n, np.int32)
    t.op_type = np.full(n, CONCURRENT_KERNEL, np.int32)
    t.op_name = names[rng.integers(0, pool_size, n)]
    t.op_flow = np.zeros(n, np.uint32)
    t.op_flowt = np.zeros(n, np.uint8)
    keys = ["grid", "block"]
    vals = {"grid": rng.integers(1, 65536, n), "block": rng.integers(32, 1025, n)}
    order = md_visit_order(tuple(keys))
    md = np.zeros(n * 2, tf.MD_ENTRY)
    for j, k in enumerate(order):
        md["key"][j::2] = pool.add(k)
        md["type"][j::2] = tf.MD_INT64
        md["value"][j::2] = vals[k].astype(np.uint64)
    t.md = md
    t.op_mdoff = (np.arange(n + 1, dtype=np.uint32) * 2).astype(np.uint32)
    window = (t0, int(t.op_end.max()) + 1000)
    return _finish(t, pool, 0, window, 1)


_ATEN = ["aten::add", "aten::mul", "aten::mm", "aten::addmm", "aten::conv2d", "aten::linear", "aten::relu",
         "aten::layer_norm", "aten::softmax", "aten::embedding", "aten::gelu", "aten::dropout", "aten::matmul",
         "aten::bmm", "aten::cat", "aten::copy_", "aten::to", "aten::empty", "aten::zeros", "aten::sum",
         "aten::mean", "aten::div", "aten::sub", "aten::transpose", "aten::view", "aten::reshape",
         "aten::native_layer_norm", "aten::_softmax", "aten::scaled_dot_product_attention", "aten::index_select",
         "autograd::engine::evaluate_function: AddmmBackward0", "Optimizer.step#AdamW.step"]


def _cpu_ops(rng, pool, n, starts, pid, n_threads=16, with_md=True, id_base=0):
    """`n` cpu_op rows with ids id_base+1..id_base+n on `n_threads` host threads."""
    t = tf.Trace()
    t.op_start = starts
    t.op_end = starts + rng.integers(2_000, 60_000, n)
    t.op_id = np.arange(id_base + 1, id_base + n + 1, dtype=np.int32)
    t.op_device = np.full(n, pid, np.int32)
    thr = rng.integers(0, n_threads, n)
    t.op_resource = (50_000 + thr).astype(np.int64)  # system tid
    t.op_thread = (1_000_000 + 7 * thr).astype(np.int32)  # low 32 bits of the pthread id
    t.op_type = np.full(n, CPU_OP, np.int32)
    aten = np.array([pool.add(s) for s in _ATEN], np.uint32)
    t.op_name = aten[rng.integers(0, len(aten), n)]
    t.op_flow = np.zeros(n, np.uint32)
    t.op_flowt = np.zeros(n, np.uint8)
    if with_md:
        keys = ["Sequence number", "Fwd thread id", "Input Dims"]
        order = md_visit_order(tuple(keys))
        dims = np.array([pool.add(s) for s in ["[[32, 64, 28, 28], [64, 64, 3, 3]]", "[[8, 1024], [1024, 4096]]",
                                               "[[], [128]]", "[[4, 16, 512, 64], [4, 16, 512, 64], []]"]], np.uint64)
        cols = {"Sequence number": (tf.MD_INT64, (id_base + np.arange(n)).astype(np.uint64)),
                "Fwd thread id": (tf.MD_INT64, (thr % 3).astype(np.uint64)),
                "Input Dims": (tf.MD_RAWJSON, dims[rng.integers(0, len(dims), n)])}
        md = np.zeros(n * 3, tf.MD_ENTRY)
        for j, k in enumerate(order):
            md["key"][j::3] = pool.add(k)
            md["type"][j::3] = cols[k][0]
            md["value"][j::3] = cols[k][1]
        t.md = md
        t.op_mdoff = (np.arange(n + 1, dtype=np.uint32) * 3).astype(np.uint32)
    else:
        t.op_mdoff = np.zeros(n + 1, np.uint32)
    tidmap = np.stack([1_000_000 + 7 * np.arange(n_threads), 50_000 + np.arange(n_threads)], 1).astype(np.int32)
    t.tidmap = tidmap.reshape(-1)
    return t, thr


def _kernel_records(rng, n, names, starts, durs, corr, n_devices, n_streams):
    k = np.zeros(n, tf.KERNEL9)
    k["kind"] = tf.KIND_CONCURRENT_KERNEL
    k["start"], k["end"] = starts, starts + durs
    dev = rng.integers(0, n_devices, n)
    k["deviceId"], k["contextId"] = dev, dev + 1
    k["streamId"] = rng.integers(7, 7 + n_streams, n)
    k["gridX"] = rng.integers(1, 65536, n)
    k["gridY"] = np.where(rng.random(n) < 0.2, rng.integers(1, 64, n), 1)
    k["gridZ"] = np.where(rng.random(n) < 0.05, rng.integers(1, 8, n), 1)
    k["blockX"] = rng.choice([32, 64, 96, 128, 192, 256, 384, 512, 768, 1024], n)
    k["blockY"] = np.where((k["blockX"] <= 128) & (rng.random(n) < 0.15), rng.integers(1, 5, n), 1)
    k["blockZ"] = 1
    k["registersPerThread"] = rng.choice([16, 24, 32, 40, 48, 64, 80, 96, 128, 168, 255], n)
    k["staticSharedMemory"] = rng.choice([0, 0, 0, 1024, 4096, 16384, 32768, 49152], n)
    k["dynamicSharedMemory"] = rng.choice([0, 0, 0, 0, 8192, 65536, 98304, 200000], n)
    k["correlationId"] = corr
    k["name"] = names[rng.integers(0, len(names), n)]
    k["queued"] = np.where(rng.random(n) < 0.1, starts - rng.integers(100, 5000, n), 0)
    k["graphId"] = np.where(rng.random(n) < 0.1, rng.integers(1, 50, n), 0)
    k["graphNodeId"] = np.where(k["graphId"] > 0, rng.integers(1, 1 << 40, n), 0)
    k["channelID"] = rng.integers(0, 16, n)
    k["channelType"] = rng.integers(0, 3, n)
    return k


def gen_kernel_launches(n=1_000_000, seed=2, n_devices=8, n_streams=32, pool_size=4096, name_len=(20, 400),
                        orphan_fraction=0.0, buffer_bytes=4 << 20, ts_mode=0, shard=(0, 1), user_annotations=0,
                        memory_events=0.0) -> tf.Trace:
    """`n` kernel launches: per launch one EXTERNAL_CORRELATION(CUSTOM0) record, one cudaLaunchKernel
    runtime record and one CUpti_ActivityKernel9, plus `n` CPU ops.  Kernel records carry the
    correlation ids in a seeded permutation, so the join is not positional.

    `shard=(r, w)`: the trace has w*n launches and this call returns the r-th contiguous record range
    (n launches, n kernel records, n CPU ops).  The permutation is global, so a kernel's
    EXTERNAL_CORRELATION record and CPU op usually live in another shard."""
    r, w = shard
    total = n * w
    g = np.random.default_rng(seed)  # global draws: identical in every shard
    pool = tf.StringPool()
    names = np.array([pool.add(s) for s in name_pool(g, pool_size, *name_len)], np.uint64)
    t0 = DEFAULT_BASE_TIME + 1_000_000_000
    op_starts_all = _monotone_starts(g, total, t0, 3000.0)
    api_start_all = op_starts_all + g.integers(200, 1500, total)
    perm_all = g.permutation(total)
    kdelay_all = g.integers(3000, 200_000, total)
    window = (t0 - 1000, int(api_start_all.max()) + 200_000 + 10_000_000_000)
    rng = np.random.default_rng([seed, r])  # shard-local draws
    lo, hi = r * n, (r + 1) * n
    ops, thr = _cpu_ops(rng, pool, n, op_starts_all[lo:hi], DEFAULT_PID, id_base=lo)
    corr_all_base = 1000
    corr = (np.arange(lo, hi, dtype=np.int64) + corr_all_base).astype(np.uint32)

    ext = np.zeros(n, tf.EXTCORR)
    ext["kind"], ext["externalKind"] = tf.KIND_EXTERNAL_CORRELATION, tf.EXTERNAL_KIND_CUSTOM0
    ext["externalId"], ext["correlationId"] = ops.op_id.astype(np.uint64), corr
    if orphan_fraction > 0:  # launches whose CPU op is unknown
        orphan = rng.random(n) < orphan_fraction
        ext["externalId"] = np.where(orphan, ext["externalId"] + np.uint64(1 << 30), ext["externalId"])

    api = np.zeros(n, tf.API)
    api["kind"], api["cbid"] = tf.KIND_RUNTIME, CBID_cudaLaunchKernel
    api["start"] = api_start_all[lo:hi]
    api["end"] = api["start"] + rng.integers(1500, 9000, n)
    api["processId"], api["threadId"] = DEFAULT_PID, ops.op_thread.astype(np.uint32)
    api["correlationId"] = corr

    perm = perm_all[lo:hi]
    kstart = api_start_all[perm].astype(np.int64) + kdelay_all[lo:hi]
    kcorr = (perm + corr_all_base).astype(np.uint32)
    kern = _kernel_records(rng, n, names, kstart, _lognormal_dur(rng, n), kcorr, n_devices, n_streams)

    conv = None
    if ts_mode == 1:
        conv = tsc_converter_for(window)
        for rec in (api, kern):
            rec["start"], rec["end"] = ns_to_ticks(rec["start"], conv), ns_to_ticks(rec["end"], conv)
    t = ops
    if memory_events > 0:
        # PyTorch memory events: `memory_events * n` cpu_instant_event rows named "[memory]" with six integer entries
        m = int(memory_events * n)
        at = np.sort(rng.integers(0, n, m))
        keys = ["Device Type", "Device Id", "Addr", "Bytes", "Total Allocated", "Total Reserved"]
        vals = {"Device Type": np.ones(m, np.uint64), "Device Id": rng.integers(0, n_devices, m).astype(np.uint64),
                "Addr": (139_800_000_000_000 + 512 * rng.integers(0, 1 << 30, m)).astype(np.uint64),
                "Bytes": (rng.integers(-(1 << 28), 1 << 28, m)).astype(np.int64).view(np.uint64),
                "Total Allocated": rng.integers(0, 1 << 36, m).astype(np.uint64), "Total Reserved": rng.integers(0, 1 << 37, m).astype(np.uint64)}
        md = np.zeros(m * 6, tf.MD_ENTRY)
        for j, k in enumerate(md_visit_order(tuple(keys))):
            md["key"][j::6] = pool.add(k)
            md["type"][j::6] = tf.MD_INT64
            md["value"][j::6] = vals[k]
        add = dict(op_start=t.op_start[at] + 7, op_end=t.op_start[at] + 7, op_id=np.zeros(m, np.int32),
                   op_device=np.full(m, DEFAULT_PID, np.int32), op_resource=t.op_resource[at], op_thread=t.op_thread[at],
                   op_type=np.full(m, CPU_INSTANT_EVENT, np.int32), op_name=np.full(m, pool.add("[memory]"), np.uint32),
                   op_flow=np.zeros(m, np.uint32), op_flowt=np.zeros(m, np.uint8))
        for col, v in add.items():
            setattr(t, col, np.concatenate([getattr(t, col), v.astype(getattr(t, col).dtype)]))
        t.op_mdoff = np.concatenate([t.op_mdoff, t.op_mdoff[-1] + 6 * np.arange(1, m + 1, dtype=np.uint32)]).astype(np.uint32)
        t.md = np.concatenate([t.md, md])
    if user_annotations:
        # `user_annotations` user_annotation ops (ids above every cpu_op id), each covering a contiguous
        # run of launches through a CUSTOM1 correlation record per launch
        k = user_annotations
        ann_id = (total + 1 + (np.arange(lo, hi) * k // total)).astype(np.int32)
        extu = np.zeros(n, tf.EXTCORR)
        extu["kind"], extu["externalKind"] = tf.KIND_EXTERNAL_CORRELATION, tf.EXTERNAL_KIND_CUSTOM1
        extu["externalId"], extu["correlationId"] = ann_id.astype(np.uint64), corr
        ids = np.unique(ann_id)
        m = len(ids)
        first = np.array([np.argmax(ann_id == i) for i in ids])
        add = dict(op_start=op_starts_all[lo:hi][first] - 50, op_end=op_starts_all[lo:hi][first] + 5_000_000,
                   op_id=ids, op_device=np.full(m, DEFAULT_PID, np.int32), op_resource=t.op_resource[first],
                   op_thread=t.op_thread[first], op_type=np.full(m, USER_ANNOTATION, np.int32),
                   op_name=np.array([pool.add("ProfilerStep#%d" % i) for i in ids], np.uint32),
                   op_flow=np.zeros(m, np.uint32), op_flowt=np.zeros(m, np.uint8))
        for col, v in add.items():
            setattr(t, col, np.concatenate([getattr(t, col), v.astype(getattr(t, col).dtype)]))
        t.op_mdoff = np.concatenate([t.op_mdoff, np.full(m, t.op_mdoff[-1], np.uint32)])
        order = np.tile(np.array([0, 3, 1, 2], np.int8), n)
        t.cupti, offs = tf.interleave([ext, api, kern, extu], order)
    else:
        order = np.tile(np.array([0, 1, 2], np.int8), n)
        t.cupti, offs = tf.interleave([ext, api, kern], order)
    t.buftab = tf.make_buftab(offs, buffer_bytes)
    return _finish(t, pool, 1, window, n_devices, ts_mode=ts_mode, conv=conv)


def scale_to_x87(scale: float) -> tuple[int, int]:
    """(64-bit significand, unbiased exponent) of `scale` as an x87 extended value."""
    from fractions import Fraction
    f = Fraction(scale)
    e = 0
    while f >= 2:
        f /= 2
        e += 1
    while f < 1:
        f *= 2
        e -= 1
    mant = int(f * (1 << 63))
    return mant | (1 << 63), e


TSC_SCALE = 0.5208333134651184  # ns per tick of a 1.92 GHz counter (exactly representable in float32)
TSC_T0_APPROX = 123_456_789_012


def tsc_converter_for(window):
    """Fixed converter constants (t0, t0_approx, 64-bit significand, exponent) for ts_mode 1."""
    mant, exp = scale_to_x87(TSC_SCALE)
    mant |= 0x5A5  # use the low significand bits a double cannot hold
    return (int(window[0]) - 5_000_000, TSC_T0_APPROX, mant, exp)


def ns_to_ticks(ns, conv):
    """Inverse of the converter (to within a tick) for building ts_mode 1 traces."""
    t0, t0a, mant, exp = conv
    scale = mant * 2.0 ** (exp - 63)
    return (t0a + np.round((np.asarray(ns, np.float64) - t0) / scale)).astype(np.uint64)


def gen_mixed(n=10_000_000, seed=3, n_devices=8, n_streams=32, pool_size=50_000, name_len=(20, 400),
              escape_fraction=0.02, orphan_fraction=0.05, buffer_bytes=4 << 20, shard=(0, 1), cross_fraction=0.05) -> tf.Trace:
    """Mixed trace: 60 % kernels, 20 % memcpy (bytes log-uniform 4 B..1 GB; HtoD/DtoH/DtoD/PtoP
    uniform, PtoP as MEMCPY2 records), 5 % memset, 15 % runtime-only calls; every GPU activity has a
    launching runtime record and an EXTERNAL_CORRELATION record; `orphan_fraction` of the
    correlation ids have no CPU op; `escape_fraction` of the names carry JSON-special bytes.

    `shard=(r, w)`: the trace has w*n activities and this call returns the r-th contiguous record range (string
    pool, window and id ranges are those of the whole trace).  `cross_fraction` of a shard's kernel records belong
    to launches at the end of the shard before it (GPU records arrive after their launch), so their
    EXTERNAL_CORRELATION record and CPU op live in that shard."""
    r, w = shard
    lo = r * n
    t0 = DEFAULT_BASE_TIME + 1_000_000_000
    if w == 1:
        rng = np.random.default_rng(seed)
        pool = tf.StringPool()
        names = np.array([pool.add(s) for s in name_pool(rng, pool_size, *name_len, escape_fraction=escape_fraction)], np.uint64)
        first_start = t0
    else:
        g = np.random.default_rng(seed)  # global draws: identical in every shard
        pool = tf.StringPool()
        names = np.array([pool.add(s) for s in name_pool(g, pool_size, *name_len, escape_fraction=escape_fraction)], np.uint64)
        rng = np.random.default_rng([seed, r])
        first_start = t0 + lo * 3002  # shards follow each other in time (mean gap between launches: 3001 ns)
    cls = rng.choice(4, n, p=[0.60, 0.20, 0.05, 0.15])  # 0 kernel 1 memcpy 2 memset 3 runtime-only
    op_starts = _monotone_starts(rng, n, first_start, 3000.0)
    ops, thr = _cpu_ops(rng, pool, n, op_starts, DEFAULT_PID, id_base=lo)
    corr = (np.arange(lo, lo + n, dtype=np.int64) + 1000).astype(np.uint32)

    gpu = cls < 3
    ext = np.zeros(n, tf.EXTCORR)
    ext["kind"], ext["externalKind"] = tf.KIND_EXTERNAL_CORRELATION, tf.EXTERNAL_KIND_CUSTOM0
    orphan = rng.random(n) < orphan_fraction
    ext["externalId"] = np.where(orphan, ops.op_id.astype(np.uint64) + np.uint64(1 << 30), ops.op_id.astype(np.uint64))
    ext["correlationId"] = corr

    api = np.zeros(n, tf.API)
    api["kind"] = tf.KIND_RUNTIME
    misc = rng.choice([CBID_cudaStreamSynchronize, CBID_cudaGetLastError, CBID_cudaEventCreate, 22, 200, 9], n)
    api["cbid"] = np.select([cls == 0, cls == 1, cls == 2], [CBID_cudaLaunchKernel, CBID_cudaMemcpyAsync, CBID_cudaMemsetAsync], misc)
    api["start"] = op_starts + rng.integers(200, 1500, n)
    api["end"] = api["start"] + rng.integers(1500, 9000, n)
    api["processId"], api["threadId"] = DEFAULT_PID, ops.op_thread.astype(np.uint32)
    api["correlationId"] = corr

    gstart = api["start"].astype(np.int64) + rng.integers(3000, 200_000, n)
    ik, im, iset = np.nonzero(cls == 0)[0], np.nonzero(cls == 1)[0], np.nonzero(cls == 2)[0]
    kcorr = corr[ik]
    if r > 0 and cross_fraction > 0:  # late arrivals: GPU records of launches near the end of the previous shard
        late = np.random.default_rng([seed, r, 1]).random(len(ik)) < cross_fraction
        back = np.random.default_rng([seed, r, 2]).integers(1, min(n, 50_000) + 1, len(ik))
        kcorr = np.where(late, (lo - back + 1000).astype(np.uint32), kcorr)
    kern = _kernel_records(rng, len(ik), names, gstart[ik], _lognormal_dur(rng, len(ik)), kcorr, n_devices, n_streams)

    nbytes = np.exp(rng.uniform(np.log(4), np.log(1 << 30), len(im))).astype(np.uint64)
    mkind = rng.integers(0, 4, len(im))  # HtoD DtoH DtoD PtoP
    mdur = np.maximum(0, (nbytes / 25.0).astype(np.int64) + rng.integers(-2, 2000, len(im)))
    mdur = np.where(rng.random(len(im)) < 0.01, 0, mdur)  # zero durations: no bandwidth field
    p2p = mkind == 3
    i1, i2 = np.nonzero(~p2p)[0], np.nonzero(p2p)[0]
    mc = np.zeros(len(i1), tf.MEMCPY5)
    mc["kind"] = tf.KIND_MEMCPY
    mc["copyKind"] = np.array([1, 2, 8])[mkind[i1]]  # CUPTI_ACTIVITY_MEMCPY_KIND_HTOD/DTOH/DTOD
    mc["srcKind"] = np.where(mkind[i1] == 0, rng.choice([1, 2], len(i1)), 3)
    mc["dstKind"] = np.where(mkind[i1] == 1, rng.choice([1, 2], len(i1)), 3)
    mc["bytes"], mc["start"] = nbytes[i1], gstart[im][i1]
    mc["end"] = mc["start"] + mdur[i1].astype(np.uint64)
    d = rng.integers(0, n_devices, len(i1))
    mc["deviceId"], mc["contextId"] = d, d + 1
    mc["streamId"] = rng.integers(7, 7 + n_streams, len(i1))
    mc["correlationId"] = corr[im][i1]
    mc["channelID"], mc["channelType"] = rng.integers(0, 16, len(i1)), 2
    pp = np.zeros(len(i2), tf.MEMCPYP2P4)
    pp["kind"], pp["copyKind"], pp["srcKind"], pp["dstKind"] = tf.KIND_MEMCPY2, 10, 3, 3
    pp["bytes"], pp["start"] = nbytes[i2], gstart[im][i2]
    pp["end"] = pp["start"] + mdur[i2].astype(np.uint64)
    d = rng.integers(0, n_devices, len(i2))
    d2 = (d + rng.integers(1, n_devices, len(i2))) % n_devices
    pp["deviceId"], pp["contextId"], pp["srcDeviceId"], pp["srcContextId"] = d, d + 1, d, d + 1
    pp["dstDeviceId"], pp["dstContextId"] = d2, d2 + 1
    pp["streamId"] = rng.integers(7, 7 + n_streams, len(i2))
    pp["correlationId"] = corr[im][i2]
    pp["channelID"], pp["channelType"] = rng.integers(0, 16, len(i2)), 2

    ms = np.zeros(len(iset), tf.MEMSET4)
    ms["kind"] = tf.KIND_MEMSET
    ms["bytes"] = np.exp(rng.uniform(np.log(4), np.log(1 << 28), len(iset))).astype(np.uint64)
    ms["start"] = gstart[iset]
    ms["end"] = ms["start"] + np.maximum(1, (ms["bytes"] / 1500.0)).astype(np.uint64) + rng.integers(0, 900, len(iset)).astype(np.uint64)
    d = rng.integers(0, n_devices, len(iset))
    ms["deviceId"], ms["contextId"] = d, d + 1
    ms["streamId"] = rng.integers(7, 7 + n_streams, len(iset))
    ms["correlationId"] = corr[iset]
    ms["memoryKind"] = rng.choice([3, 3, 3, 5, 2], len(iset))
    ms["value"] = rng.integers(0, 256, len(iset))
    ms["channelID"], ms["channelType"] = rng.integers(0, 16, len(iset)), 1

    # Buffer order: CPU-side records (ext, api) in launch order; each GPU record lands a random lag
    # after its launch, which shuffles GPU records relative to the launches.
    ngpu = int(gpu.sum())
    lag = rng.integers(1, 5000, ngpu)
    gpu_idx = np.nonzero(gpu)[0]
    key_cpu = np.repeat(np.arange(n, dtype=np.float64), 2) + np.tile([0.0, 0.25], n)
    key_gpu = gpu_idx + lag + 0.5
    keys = np.concatenate([key_cpu, key_gpu])
    # stream ids: 0 ext, 1 api, 2 kernel, 3 memcpy, 4 p2p, 5 memset
    gcls = np.full(n, -1, np.int8)
    gcls[ik] = 2
    gcls[im[i1]] = 3
    gcls[im[i2]] = 4
    gcls[iset] = 5
    sid = np.concatenate([np.tile(np.array([0, 1], np.int8), n), gcls[gpu_idx]])
    o = np.argsort(keys, kind="stable")
    order = sid[o]
    # Each stream's records must be listed in the order they appear: GPU streams appear sorted by key.
    gorder = np.argsort(key_gpu, kind="stable")
    g_sorted_idx = gpu_idx[gorder]

    def _reorder(recs, members):
        rank = np.full(n, -1, np.int64)
        rank[members] = np.arange(len(members))
        sel = g_sorted_idx[np.isin(g_sorted_idx, members)] if len(members) else np.zeros(0, np.int64)
        # index the raw bytes: field-wise copies of a padded struct dtype leave the padding undefined
        raw = np.ascontiguousarray(recs).view(np.uint8).reshape(len(recs), -1)
        return raw[rank[sel]].reshape(-1).view(recs.dtype)

    kern = _reorder(kern, ik)
    mc = _reorder(mc, im[i1])
    pp = _reorder(pp, im[i2])
    ms = _reorder(ms, iset)
    t = ops
    t.cupti, offs = tf.interleave([ext, api, kern, mc, pp, ms], order)
    t.buftab = tf.make_buftab(offs, buffer_bytes)
    if w == 1:
        last = max(int(kern["end"].max()) if len(kern) else 0, int(api["end"].max()))
        window = (t0 - 1000, last + 1_000_000)
    else:  # one window for the whole trace, the same in every shard
        window = (t0 - 1000, t0 + w * n * 3002 + 200 * n + 100_000_000_000)
    return _finish(t, pool, 1, window, n_devices)


def _shape_strings(rng, pool, count, max_len=256):
    """`count` (Input Dims, Input type) string-id pairs: nested lists of tensor shapes and the matching dtype
    lists, as PyTorch's profiler renders them, up to `max_len` bytes."""
    dtypes = ["float", "c10::Half", "c10::BFloat16", "long int", "int", "bool", "Scalar", ""]
    dims, types = [], []
    for _ in range(count):
        while True:
            n_in = int(rng.integers(1, 9))
            shapes = [[int(x) for x in rng.integers(1, 65536, int(rng.integers(0, 5)))] for _ in range(n_in)]
            d = "[" + ", ".join("[" + ", ".join(map(str, s)) + "]" for s in shapes) + "]"
            ty = "[" + ", ".join('"%s"' % dtypes[int(rng.integers(0, len(dtypes)))] for _ in range(n_in)) + "]"
            if len(d) <= max_len and len(ty) <= max_len:
                break
        dims.append(pool.add(d))
        types.append(pool.add(ty))
    return np.array(dims, np.uint64), np.array(types, np.uint64)


def _span_tree(rng, n_ops, t0, root_ns=20_000_000, max_depth=(1, 16), children_mean=3.0):
    """Nested spans, level by level: roots follow one another; a node below its root's depth limit (uniform in
    `max_depth`) and wide enough to hold them gets Poisson(`children_mean`) children that split its interior.
    Every root's tree is grown in full; the first `n_ops` nodes in order of their start time are returned as
    (start, end, depth, root)."""
    starts, ends, depths, roots = [], [], [], []
    total, next_t, root_id = 0, t0, 0
    while total < n_ops:
        n_roots = max(1, (n_ops - total) // 100_000)
        s = next_t + np.arange(n_roots, dtype=np.int64) * (root_ns + 1000)
        e = s + root_ns
        next_t = int(e[-1]) + 1000
        limit = rng.integers(max_depth[0], max_depth[1] + 1, n_roots)
        root = root_id + np.arange(n_roots)
        root_id += n_roots
        depth = 1
        while len(s):
            starts.append(s); ends.append(e); depths.append(np.full(len(s), depth, np.int32)); roots.append(root)
            total += len(s)
            k = rng.poisson(children_mean, len(s))
            k = np.where((depth < limit) & (e - s >= 64 * (k + 1)), k, 0)
            par = np.repeat(np.arange(len(s)), k)
            if len(par) == 0:
                break
            idx = np.arange(len(par)) - np.repeat(np.cumsum(k) - k, k)   # child number within its parent
            w = (e[par] - s[par] - 16) // k[par]
            cs = s[par] + 8 + idx * w
            s, e, limit, root = cs, cs + w - 4, limit[par], root[par]
            depth += 1
    s, e, d, r = (np.concatenate(x) for x in (starts, ends, depths, roots))
    o = np.argsort(s, kind="stable")[:n_ops]
    return s[o], e[o], d[o], r[o]


def gen_op_tree(n_ops=200_000, launches_per_op=2.0, seed=4, n_devices=8, n_streams=32, pool_size=4096,
                name_len=(20, 400), n_shapes=2048, buffer_bytes=4 << 20) -> tf.Trace:
    """A CPU op tree of nested record_function spans (depth limit uniform 1-16 per root, Poisson(3) children)
    whose ops carry `Input Dims` / `Input type` strings of up to 256 bytes, forward-backward flow pairs between
    ops, and `launches_per_op * n_ops` kernel launches (EXTERNAL_CORRELATION + cudaLaunchKernel + Kernel9
    records: two GPU-side activities each) issued by random ops of the tree."""
    rng = np.random.default_rng(seed)
    pool = tf.StringPool()
    names = np.array([pool.add(s) for s in name_pool(rng, pool_size, *name_len)], np.uint64)
    t0 = DEFAULT_BASE_TIME + 1_000_000_000
    s, e, depth, _ = _span_tree(rng, n_ops, t0)
    n = len(s)
    t = tf.Trace()
    t.op_start, t.op_end = s, e
    t.op_id = np.arange(1, n + 1, dtype=np.int32)
    t.op_device = np.full(n, DEFAULT_PID, np.int32)
    thr = rng.integers(0, 16, n)
    t.op_resource = (50_000 + thr).astype(np.int64)
    t.op_thread = (1_000_000 + 7 * thr).astype(np.int32)
    t.op_type = np.full(n, CPU_OP, np.int32)
    aten = np.array([pool.add(x) for x in _ATEN], np.uint32)
    t.op_name = aten[rng.integers(0, len(aten), n)]
    # forward-backward links: every 16th op starts a flow that the op 8 places later ends
    t.op_flow = np.zeros(n, np.uint32)
    t.op_flowt = np.zeros(n, np.uint8)
    src = np.arange(0, n - 8, 16)
    t.op_flow[src] = t.op_flow[src + 8] = (src // 16 + 1).astype(np.uint32)
    t.op_flowt[src], t.op_flowt[src + 8] = 1 | (1 << 4), 1
    keys = ["Sequence number", "Input Dims", "Input type", "Record function id"]
    order = md_visit_order(tuple(keys))
    dims, types = _shape_strings(rng, pool, n_shapes)
    pick = rng.integers(0, n_shapes, n)
    cols = {"Sequence number": (tf.MD_INT64, np.arange(n).astype(np.uint64)),
            "Input Dims": (tf.MD_RAWJSON, dims[pick]), "Input type": (tf.MD_RAWJSON, types[pick]),
            "Record function id": (tf.MD_INT64, depth.astype(np.uint64))}
    nk = len(keys)
    md = np.zeros(n * nk, tf.MD_ENTRY)
    for j, k in enumerate(order):
        md["key"][j::nk] = pool.add(k)
        md["type"][j::nk] = cols[k][0]
        md["value"][j::nk] = cols[k][1]
    t.md = md
    t.op_mdoff = (np.arange(n + 1, dtype=np.uint32) * nk).astype(np.uint32)
    t.tidmap = np.stack([1_000_000 + 7 * np.arange(16), 50_000 + np.arange(16)], 1).astype(np.int32).reshape(-1)
    # launches
    m = int(launches_per_op * n)
    owner = np.sort(rng.integers(0, n, m))
    corr = (np.arange(m, dtype=np.int64) + 1000).astype(np.uint32)
    ext = np.zeros(m, tf.EXTCORR)
    ext["kind"], ext["externalKind"] = tf.KIND_EXTERNAL_CORRELATION, tf.EXTERNAL_KIND_CUSTOM0
    ext["externalId"], ext["correlationId"] = t.op_id[owner].astype(np.uint64), corr
    api = np.zeros(m, tf.API)
    api["kind"], api["cbid"] = tf.KIND_RUNTIME, CBID_cudaLaunchKernel
    api["start"] = s[owner] + rng.integers(0, 8, m)
    api["end"] = api["start"] + rng.integers(1500, 9000, m)
    api["processId"], api["threadId"] = DEFAULT_PID, t.op_thread[owner].astype(np.uint32)
    api["correlationId"] = corr
    perm = rng.permutation(m)
    kstart = api["start"][perm].astype(np.int64) + rng.integers(3000, 200_000, m)
    kern = _kernel_records(rng, m, names, kstart, _lognormal_dur(rng, m), corr[perm], n_devices, n_streams)
    window = (t0 - 1000, int(max(e.max(), kstart.max())) + 10_000_000_000)
    t.cupti, offs = tf.interleave([ext, api, kern], np.tile(np.array([0, 1, 2], np.int8), m))
    t.buftab = tf.make_buftab(offs, buffer_bytes)
    return _finish(t, pool, 1, window, n_devices)


def gen_distributed_rank(n=200_000, rank=0, world=8, seed=5, coll_fraction=0.2, n_devices=8, n_streams=32,
                         pool_size=4096, name_len=(20, 400), buffer_bytes=4 << 20) -> tf.Trace:
    """One rank's trace of a distributed job: `n` kernel launches of which `coll_fraction` are NCCL collectives
    issued by record_param_comms ops that carry the collective metadata (type among allreduce / allgather /
    reduce_scatter / all_to_all, message size log-uniform 1 KB - 4 GB, process groups of 2-8 ranks).  Ranks differ
    by their seed stream and by the `Rank` value; each rank's trace is processed on its own."""
    rng = np.random.default_rng([seed, rank])
    pool = tf.StringPool()
    names = np.array([pool.add(s) for s in name_pool(rng, pool_size, *name_len)], np.uint64)
    t0 = DEFAULT_BASE_TIME + 1_000_000_000
    op_starts = _monotone_starts(rng, n, t0, 3000.0)
    ops, thr = _cpu_ops(rng, pool, n, op_starts, DEFAULT_PID, with_md=False)
    is_coll = rng.random(n) < coll_fraction
    nc = int(is_coll.sum())
    colls = ["allreduce", "allgather", "reduce_scatter", "all_to_all"]
    ops.op_name = np.where(is_coll, np.uint32(pool.add("record_param_comms")), ops.op_name).astype(np.uint32)
    # metadata: three entries for ordinary ops, ten for collectives (one key set each, so one visit order each)
    keys_n = ["Sequence number", "Fwd thread id", "Input Dims"]
    keys_c = ["Collective name", "In msg nelems", "Out msg nelems", "Group size", "dtype", "Process Group Name",
              "Process Group Description", "Process Group Ranks", "Rank", "Seq"]
    dims = np.array([pool.add(s) for s in ["[[32, 64, 28, 28], [64, 64, 3, 3]]", "[[8, 1024], [1024, 4096]]", "[[], [128]]"]], np.uint64)
    groups = [list(range(k)) for k in range(2, world + 1)]
    group_ids = np.array([pool.add(str(g)) for g in groups], np.uint64)
    gpick = rng.integers(0, len(groups), n)
    size = np.exp(rng.uniform(np.log(1 << 10), np.log(1 << 32), n)).astype(np.uint64)
    kind = rng.integers(0, 4, n)
    gsize = np.array([len(g) for g in groups], np.uint64)[gpick]
    cols_n = {"Sequence number": (tf.MD_INT64, np.arange(n).astype(np.uint64)), "Fwd thread id": (tf.MD_INT64, (thr % 3).astype(np.uint64)),
              "Input Dims": (tf.MD_RAWJSON, dims[rng.integers(0, len(dims), n)])}
    cols_c = {"Collective name": (tf.MD_STRING, np.array([pool.add(c) for c in colls], np.uint64)[kind]),
              "In msg nelems": (tf.MD_INT64, size), "Out msg nelems": (tf.MD_INT64, np.where(kind == 1, size * gsize, size)),
              "Group size": (tf.MD_INT64, gsize), "dtype": (tf.MD_STRING, np.array([pool.add(x) for x in ["Float", "BFloat16", "Half"]], np.uint64)[rng.integers(0, 3, n)]),
              "Process Group Name": (tf.MD_STRING, np.array([pool.add(str(i)) for i in range(len(groups))], np.uint64)[gpick]),
              "Process Group Description": (tf.MD_STRING, np.where(gpick == len(groups) - 1, np.uint64(pool.add("default_pg")), np.uint64(pool.add("model_parallel")))),
              "Process Group Ranks": (tf.MD_RAWJSON, group_ids[gpick]), "Rank": (tf.MD_INT64, np.full(n, rank, np.uint64)),
              "Seq": (tf.MD_INT64, np.cumsum(is_coll).astype(np.uint64))}
    cnt = np.where(is_coll, len(keys_c), len(keys_n)).astype(np.uint32)
    mdoff = np.concatenate([[0], np.cumsum(cnt)]).astype(np.uint32)
    md = np.zeros(int(mdoff[-1]), tf.MD_ENTRY)
    for sel, keys, cols in ((~is_coll, keys_n, cols_n), (is_coll, keys_c, cols_c)):
        base = mdoff[:-1][sel]
        for j, k in enumerate(md_visit_order(tuple(keys))):
            md["key"][base + j] = pool.add(k)
            md["type"][base + j] = cols[k][0]
            md["value"][base + j] = cols[k][1][sel]
    ops.md, ops.op_mdoff = md, mdoff
    # launches: every op launches one kernel; collective kernels carry NCCL names
    corr = (np.arange(n, dtype=np.int64) + 1000).astype(np.uint32)
    ext = np.zeros(n, tf.EXTCORR)
    ext["kind"], ext["externalKind"] = tf.KIND_EXTERNAL_CORRELATION, tf.EXTERNAL_KIND_CUSTOM0
    ext["externalId"], ext["correlationId"] = ops.op_id.astype(np.uint64), corr
    api = np.zeros(n, tf.API)
    api["kind"], api["cbid"] = tf.KIND_RUNTIME, CBID_cudaLaunchKernel
    api["start"] = op_starts + rng.integers(200, 1500, n)
    api["end"] = api["start"] + rng.integers(1500, 9000, n)
    api["processId"], api["threadId"] = DEFAULT_PID, ops.op_thread.astype(np.uint32)
    api["correlationId"] = corr
    perm = rng.permutation(n)
    kstart = api["start"][perm].astype(np.int64) + rng.integers(3000, 200_000, n)
    kern = _kernel_records(rng, n, names, kstart, _lognormal_dur(rng, n), corr[perm], n_devices, n_streams)
    nccl = np.array([pool.add("ncclDevKernel_%s_RING_LL(ncclDevKernelArgsStorage<4096ul>)" % c) for c in
                     ["AllReduce_Sum_bf16", "AllGather", "ReduceScatter_Sum_bf16", "SendRecv"]], np.uint64)
    kern["name"] = np.where(is_coll[perm], nccl[kind[perm]], kern["name"])
    kern["deviceId"], kern["contextId"] = rank % n_devices, rank % n_devices + 1      # one GPU per rank
    window = (t0 - 1000, int(kstart.max()) + 10_000_000_000)
    t = ops
    t.cupti, offs = tf.interleave([ext, api, kern], np.tile(np.array([0, 1, 2], np.int8), n))
    t.buftab = tf.make_buftab(offs, buffer_bytes)
    return _finish(t, pool, 1, window, n_devices, flags=tf.FLAG_SORT_BY_START)
