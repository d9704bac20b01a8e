"""Shared test plumbing: run the CPU checkers (oracle/) on a synthetic trace and cut the
"activities" part out of a Chrome-trace file."""
from __future__ import annotations

import ctypes
import json
import os
import re
import subprocess
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DRIVER = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
PORT_LIB = os.path.join(ROOT, "oracle", "_build", "libk2j_oracle.so")
GOLDEN = os.path.join(ROOT, "tests", "golden")

_EVENT_START = b"\n  {\n"


def have_ref() -> bool:
    return os.path.exists(REF_DRIVER)


def build_port():
    if not os.path.exists(PORT_LIB) or os.path.getmtime(PORT_LIB) < os.path.getmtime(
            os.path.join(ROOT, "oracle", "k2j_oracle.cpp")):
        subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "port"], check=True)
    return PORT_LIB


_port = None


def port_lib():
    global _port
    if _port is None:
        _port = ctypes.CDLL(build_port())
        _port.k2j_oracle_run_file.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p),
                                              ctypes.POINTER(ctypes.c_uint64)]
        _port.k2j_oracle_free.argtypes = [ctypes.c_void_p]
        _port.k2j_oracle_fmt_double.argtypes = [ctypes.c_double, ctypes.c_char_p, ctypes.c_int]
    return _port


STAT_NAMES = ["out_bytes", "ops_end", "gpu_end", "x_events", "flow_events", "records", "out_of_range",
              "blocklisted_runtime", "invalid_external_correlation", "unexpected"]


def run_port(trace, path=None):
    """Runs the CPU restatement; returns (activities bytes, stats dict)."""
    lib = port_lib()
    with tempfile.TemporaryDirectory() as d:
        p = path or os.path.join(d, "t.k2jt")
        if path is None:
            trace.write(p)
        out = ctypes.c_void_p()
        stats = (ctypes.c_uint64 * 10)()
        rc = lib.k2j_oracle_run_file(p.encode(), ctypes.byref(out), stats)
        assert rc == 0
        data = ctypes.string_at(out, stats[0])
        lib.k2j_oracle_free(out)
    return data, dict(zip(STAT_NAMES, [int(x) for x in stats]))


def port_fmt_double(v: float) -> str:
    buf = ctypes.create_string_buffer(64)
    n = port_lib().k2j_oracle_fmt_double(v, buf, 64)
    assert n >= 0
    return buf.value.decode()


def run_ref(trace, repeat=1, path=None):
    """Runs the unmodified reference; returns (full JSON bytes, timing dict)."""
    with tempfile.TemporaryDirectory() as d:
        p = path or os.path.join(d, "t.k2jt")
        if path is None:
            trace.write(p)
        out = os.path.join(d, "out.json")
        r = subprocess.run([REF_DRIVER, p, out, "--repeat", str(repeat)], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        timing = json.loads(r.stdout.strip().splitlines()[-1])
        return open(out, "rb").read(), timing


def split_events(doc: bytes):
    """Splits a Chrome-trace file written by the reference logger into (header, events, trailer).
    Every event starts with "\\n  {\\n" (names and args have newlines stripped, so the marker cannot
    occur inside an event)."""
    first = doc.find(_EVENT_START)
    end = doc.rfind(b"\n  ],")
    body = doc[first:end]
    parts = body.split(_EVENT_START)
    assert parts[0] == b""
    return doc[:first], [_EVENT_START + p for p in parts[1:]], doc[end:]


_ACT = re.compile(rb'\n  \{\n    ("ph": "(X|s|f|C)",\n    "(cat|id)": |"name": "thread_(name|sort_index)", "ph": "M", "ts": |"ph": "i",\n    \n    "cat": "cpu_instant_event",)')


def activities_segment(doc: bytes) -> bytes:
    """The events the device pipeline is responsible for: every X / flow / counter event except the
    host-written "Trace" spans, plus the metadata rows the logger writes in line before the first
    stream sync of a row (libkineto/src/output_json.cpp:921-938; the header's metadata rows start with "ph") and the
    instant events of CPU-side activities (the host-written instant events have no category)."""
    _, events, _ = split_events(doc)
    keep = []
    for e in events:
        if not _ACT.match(e):
            continue
        if e.startswith(b'\n  {\n    "ph": "X",\n    "cat": "Trace",'):
            continue
        keep.append(e)
    return b"".join(keep)


def first_diff(a: bytes, b: bytes, ctx=120) -> str:
    n = min(len(a), len(b))
    aa = np.frombuffer(a[:n], np.uint8)
    bb = np.frombuffer(b[:n], np.uint8)
    d = np.nonzero(aa != bb)[0]
    i = int(d[0]) if len(d) else n
    return (f"len {len(a)} vs {len(b)}, first difference at {i}:\n--- a\n{a[max(0, i - ctx):i + ctx]!r}\n"
            f"--- b\n{b[max(0, i - ctx):i + ctx]!r}")


def activities_span(doc: bytes) -> bytes:
    """Fast cut for large mode-1 files: the activities are one contiguous run between the metadata
    rows and the CPU trace span."""
    a = doc.find(b'\n  {\n    "ph": "X",')
    b = doc.rfind(b'\n  {\n    "ph": "X",\n    "cat": "Trace",')
    return doc[a:b]


MANGLED = [b"_Z3fooIiEvT_", b"_ZN2at6native12_GLOBAL__N_110sum_kernelIfLi4EEEvPT_PKS3_l", b"_Z10saxpy_halfiPK6__halfPS_",
           b"_ZN7cutlass6KernelINS_4gemm6kernel4GemmIfEEEEvNT_6ParamsE", b"_Z", b"_Znot_a_symbol", b"G3abc", b"x" * 9000]


def with_raw_kernel_names(trace, extra_names=()):
    """A copy of `trace`'s CUPTI bytes as CUPTI would have written them: every kernel record's `name` field holds the
    address of a NUL-terminated string instead of a string id.  `extra_names` (mangled symbols, say) replace the
    names of the first kernels, in turn.  Returns (bytes array, keep-alive object, expected name per kernel record)."""
    import ctypes
    import numpy as np
    from kineto_b200 import tracefile as tf
    pool = trace.pool()
    strings = [pool[i] for i in range(len(pool))]
    texts = list(strings) + list(extra_names)
    blob = b"\0".join(texts) + b"\0"
    buf = ctypes.create_string_buffer(blob, len(blob))
    base = ctypes.addressof(buf)
    addr, pos = [], 0
    for t in texts:
        addr.append(base + pos)
        pos += len(t) + 1
    raw = np.array(trace.cupti, dtype=np.uint8, copy=True)
    expected, k = [], 0
    for b in range(trace.n_buffers):
        at, valid = int(trace.buftab[2 * b]), int(trace.buftab[2 * b + 1])
        end = at + valid
        while at + 8 <= end:
            kind = int(raw[at:at + 4].view(np.uint32)[0])
            size = (tf.RECORD_SIZE[kind] + 7) & ~7
            if kind == tf.KIND_CONCURRENT_KERNEL:
                field = raw[at + 104:at + 112].view(np.uint64)
                which = len(strings) + k if k < len(extra_names) else int(field[0])
                field[0] = addr[which]
                expected.append(texts[which])
                k += 1
            at += size
    return raw, buf, expected


def cut_into_shards(t, n_shards):
    import numpy as np
    from kineto_b200 import tracefile as tf
    """Contiguous shards of a trace: whole buffers and a contiguous range of CPU-side activities each."""
    bt = t.buftab.reshape(-1, 2)
    nb, n = t.n_buffers, t.n_ops
    cuts = [nb * i // n_shards for i in range(n_shards + 1)]
    op_cuts = [0] + [n * (i + 1) // (n_shards + 1) for i in range(n_shards - 1)] + [n]
    subs = []
    for i in range(n_shards):
        sub = tf.Trace(**{attr: getattr(t, attr) for _, attr, _ in tf._SECTIONS})
        sub.buftab = bt[cuts[i]:cuts[i + 1]].reshape(-1).copy()
        lo, hi = op_cuts[i], op_cuts[i + 1]
        for col in ("op_start", "op_end", "op_id", "op_device", "op_resource", "op_thread", "op_type", "op_name", "op_flow", "op_flowt"):
            setattr(sub, col, getattr(t, col)[lo:hi].copy())
        mo = t.op_mdoff[lo:hi + 1]
        sub.md = t.md[mo[0]:mo[-1]].copy()
        sub.op_mdoff = (mo - mo[0]).astype(np.uint32)
        subs.append(sub)
    return subs


def rebuffer(trace, records_per_buffer):
    """The same records in buffers of at most `records_per_buffer` records each (cut at record boundaries)."""
    import copy
    import numpy as np
    from kineto_b200 import tracefile as tf
    table = []
    for b in range(trace.n_buffers):
        at, end = int(trace.buftab[2 * b]), int(trace.buftab[2 * b]) + int(trace.buftab[2 * b + 1])
        start, n = at, 0
        while at + 8 <= end:
            kind = int(trace.cupti[at:at + 4].view(np.uint32)[0])
            at += (tf.RECORD_SIZE[kind] + 7) & ~7
            n += 1
            if n == records_per_buffer:
                table += [start, at - start]
                start, n = at, 0
        if at > start:
            table += [start, at - start]
    t = copy.copy(trace)
    t.buftab = np.array(table, np.uint64)
    return t
