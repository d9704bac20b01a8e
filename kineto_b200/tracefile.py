"""Synthetic-trace container: the inputs of the trace post-processing path as flat arrays.

One `Trace` holds exactly what the C ABI in include/k2j.h takes (raw CUPTI record bytes, the buffer
table, the string pool, CPU-op columns, typed metadata entries, scalars) and can be written to a
single file so the CPU checkers under oracle/ read the same bytes.  Record layouts are those of
CUDA 12.9's cupti_activity.h (CUpti_ActivityKernel9 / Memcpy5 / MemcpyPtoP4 / Memset4 /
CUpti_ActivityAPI / CUpti_ActivityExternalCorrelation), the types the reference selects in
libkineto/src/DeviceProperties.h:30-46.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

# ---- CUPTI activity kinds (cupti_activity.h, CUpti_ActivityKind) -------------------------------
KIND_MEMCPY = 1
KIND_MEMSET = 2
KIND_DRIVER = 4
KIND_RUNTIME = 5
KIND_CONCURRENT_KERNEL = 10
KIND_OVERHEAD = 17
KIND_MEMCPY2 = 22
KIND_CUDA_EVENT = 36
KIND_SYNCHRONIZATION = 38
KIND_EXTERNAL_CORRELATION = 39
EXTERNAL_KIND_CUSTOM0 = 3  # CPU-op correlation  (libkineto/src/CuptiActivityProfiler.cpp:292)
EXTERNAL_KIND_CUSTOM1 = 4  # user-annotation correlation (:295)

RECORD_SIZE = {
    KIND_CONCURRENT_KERNEL: 208,
    KIND_MEMCPY: 88,
    KIND_MEMCPY2: 96,
    KIND_MEMSET: 88,
    KIND_RUNTIME: 40,
    KIND_DRIVER: 40,
    KIND_EXTERNAL_CORRELATION: 24,
    KIND_OVERHEAD: 56,
    KIND_SYNCHRONIZATION: 40,
    KIND_CUDA_EVENT: 56,
}


def _dt(size, fields):
    return np.dtype({"names": [f[0] for f in fields], "formats": [f[1] for f in fields],
                     "offsets": [f[2] for f in fields], "itemsize": size})


KERNEL9 = _dt(208, [
    ("kind", "<u4", 0), ("cacheConfig", "u1", 4), ("sharedMemoryConfig", "u1", 5),
    ("registersPerThread", "<u2", 6), ("start", "<u8", 16), ("end", "<u8", 24),
    ("deviceId", "<u4", 40), ("contextId", "<u4", 44), ("streamId", "<u4", 48),
    ("gridX", "<i4", 52), ("gridY", "<i4", 56), ("gridZ", "<i4", 60),
    ("blockX", "<i4", 64), ("blockY", "<i4", 68), ("blockZ", "<i4", 72),
    ("staticSharedMemory", "<i4", 76), ("dynamicSharedMemory", "<i4", 80),
    ("correlationId", "<u4", 92), ("name", "<u8", 104), ("queued", "<u8", 120),
    ("graphNodeId", "<u8", 144), ("graphId", "<u4", 156), ("channelID", "<u4", 168),
    ("channelType", "<u4", 172)])
MEMCPY5 = _dt(88, [
    ("kind", "<u4", 0), ("copyKind", "u1", 4), ("srcKind", "u1", 5), ("dstKind", "u1", 6),
    ("bytes", "<u8", 8), ("start", "<u8", 16), ("end", "<u8", 24), ("deviceId", "<u4", 32),
    ("contextId", "<u4", 36), ("streamId", "<u4", 40), ("correlationId", "<u4", 44),
    ("graphNodeId", "<u8", 64), ("graphId", "<u4", 72), ("channelID", "<u4", 76),
    ("channelType", "<u4", 80)])
MEMCPYP2P4 = _dt(96, [
    ("kind", "<u4", 0), ("copyKind", "u1", 4), ("srcKind", "u1", 5), ("dstKind", "u1", 6),
    ("bytes", "<u8", 8), ("start", "<u8", 16), ("end", "<u8", 24), ("deviceId", "<u4", 32),
    ("contextId", "<u4", 36), ("streamId", "<u4", 40), ("srcDeviceId", "<u4", 44),
    ("srcContextId", "<u4", 48), ("dstDeviceId", "<u4", 52), ("dstContextId", "<u4", 56),
    ("correlationId", "<u4", 60), ("graphNodeId", "<u8", 72), ("graphId", "<u4", 80),
    ("channelID", "<u4", 84), ("channelType", "<u4", 88)])
MEMSET4 = _dt(88, [
    ("kind", "<u4", 0), ("value", "<u4", 4), ("bytes", "<u8", 8), ("start", "<u8", 16),
    ("end", "<u8", 24), ("deviceId", "<u4", 32), ("contextId", "<u4", 36), ("streamId", "<u4", 40),
    ("correlationId", "<u4", 44), ("flags", "<u2", 48), ("memoryKind", "<u2", 50),
    ("graphNodeId", "<u8", 64), ("graphId", "<u4", 72), ("channelID", "<u4", 76),
    ("channelType", "<u4", 80)])
API = _dt(40, [
    ("kind", "<u4", 0), ("cbid", "<u4", 4), ("start", "<u8", 8), ("end", "<u8", 16),
    ("processId", "<u4", 24), ("threadId", "<u4", 28), ("correlationId", "<u4", 32),
    ("returnValue", "<u4", 36)])
EXTCORR = _dt(24, [
    ("kind", "<u4", 0), ("externalKind", "<u4", 4), ("externalId", "<u8", 8),
    ("correlationId", "<u4", 16)])
OVERHEAD = _dt(56, [  # CUpti_ActivityOverhead3; the reference reads its 40-byte prefix (CUpti_ActivityOverhead)
    ("kind", "<u4", 0), ("overheadKind", "<u4", 4), ("objectKind", "<u4", 8), ("objectId0", "<u4", 12),
    ("objectId1", "<u4", 16), ("objectId2", "<u4", 20), ("start", "<u8", 24), ("end", "<u8", 32),
    ("correlationId", "<u4", 40), ("overheadData", "<u8", 48)])
SYNC = _dt(40, [  # CUpti_ActivitySynchronization
    ("kind", "<u4", 0), ("type", "<u4", 4), ("start", "<u8", 8), ("end", "<u8", 16),
    ("correlationId", "<u4", 24), ("contextId", "<u4", 28), ("streamId", "<u4", 32), ("cudaEventId", "<u4", 36)])
CUDA_EVENT2 = _dt(56, [  # CUpti_ActivityCudaEvent2 (CUDA 12.8+)
    ("kind", "<u4", 0), ("correlationId", "<u4", 4), ("contextId", "<u4", 8), ("streamId", "<u4", 12),
    ("eventId", "<u4", 16), ("deviceTimestamp", "<u8", 40)])
SYNC_TYPE_EVENT_SYNCHRONIZE, SYNC_TYPE_STREAM_WAIT_EVENT, SYNC_TYPE_STREAM_SYNCHRONIZE, SYNC_TYPE_CONTEXT_SYNCHRONIZE = 1, 2, 3, 4
RECORD_DTYPE = {KIND_OVERHEAD: OVERHEAD, KIND_SYNCHRONIZATION: SYNC, KIND_CUDA_EVENT: CUDA_EVENT2, KIND_CONCURRENT_KERNEL: KERNEL9, KIND_MEMCPY: MEMCPY5, KIND_MEMCPY2: MEMCPYP2P4,
                KIND_MEMSET: MEMSET4, KIND_RUNTIME: API, KIND_DRIVER: API,
                KIND_EXTERNAL_CORRELATION: EXTCORR}

# ---- scalar blocks -------------------------------------------------------------------------------
PARAMS = np.dtype([
    ("base_time_ns", "<i8"), ("window_start_ns", "<i8"), ("window_end_ns", "<i8"),
    ("pid", "<i4"), ("mode", "<i4"), ("ts_mode", "<i4"), ("flags", "<i4"),
    ("conv_t0", "<i8"), ("conv_t0_approx", "<u8"), ("conv_scale_mant", "<u8"),
    ("conv_scale_exp", "<i4"), ("n_devices", "<i4")])
DEVICE_PROPS = np.dtype([
    ("major", "<i4"), ("minor", "<i4"), ("max_threads_per_block", "<i4"),
    ("max_threads_per_sm", "<i4"), ("regs_per_block", "<i4"), ("regs_per_sm", "<i4"),
    ("warp_size", "<i4"), ("num_sms", "<i4"), ("smem_per_block", "<u8"),
    ("smem_per_block_optin", "<u8"), ("smem_per_sm", "<u8"), ("reserved_smem_per_block", "<u8"),
    ("total_global_mem", "<u8"), ("name", "S64")])
MD_ENTRY = np.dtype([("key", "<u4"), ("type", "<u4"), ("value", "<u8")])
MD_INT64, MD_UINT64, MD_DOUBLE, MD_BOOL, MD_STRING, MD_RAWJSON, MD_COUNTER = range(7)  # MD_COUNTER: a counter value (name, double)

FLAG_USER_ANNOTATIONS = 1
FLAG_SORT_BY_START = 2

# The reference floors "now" to 7 889 238 s periods for its base time
# (libkineto/src/output_json.h:262-277).
BASE_PERIOD_NS = 7_889_238 * 1_000_000_000


def b200_device_props(n: int) -> np.ndarray:
    """Device properties of a B200 as cudaGetDeviceProperties reports them (compute 10.0)."""
    p = np.zeros(n, DEVICE_PROPS)
    p["major"], p["minor"] = 10, 0
    p["max_threads_per_block"], p["max_threads_per_sm"] = 1024, 2048
    p["regs_per_block"], p["regs_per_sm"] = 65536, 65536
    p["warp_size"], p["num_sms"] = 32, 148
    p["smem_per_block"], p["smem_per_block_optin"] = 49152, 232448
    p["smem_per_sm"], p["reserved_smem_per_block"] = 233472, 1024
    p["total_global_mem"] = 191_000_000_000
    p["name"] = b"NVIDIA B200"
    return p


class StringPool:
    """Interned byte strings; ids index POOLOFF/POOLDATA."""

    def __init__(self):
        self._ids: dict[bytes, int] = {}
        self._strs: list[bytes] = []

    def add(self, s) -> int:
        b = s.encode() if isinstance(s, str) else bytes(s)
        i = self._ids.get(b)
        if i is None:
            i = len(self._strs)
            self._ids[b] = i
            self._strs.append(b)
        return i

    def __len__(self):
        return len(self._strs)

    def __getitem__(self, i) -> bytes:
        return self._strs[i]

    def arrays(self):
        off = np.zeros(len(self._strs) + 1, np.uint64)
        if self._strs:
            off[1:] = np.cumsum([len(s) for s in self._strs], dtype=np.uint64)
        data = np.frombuffer(b"".join(self._strs), np.uint8).copy()
        return off, data

    @classmethod
    def from_arrays(cls, off, data):
        p = cls()
        raw = data.tobytes()
        for i in range(len(off) - 1):
            p._strs.append(raw[int(off[i]):int(off[i + 1])])
            p._ids.setdefault(p._strs[-1], i)
        return p


_SECTIONS = [  # (tag, attribute, dtype)
    ("PARAMS", "params", PARAMS), ("DEVPROPS", "devprops", DEVICE_PROPS),
    ("POOLOFF", "pool_off", np.uint64), ("POOLDATA", "pool_data", np.uint8),
    ("CUPTI", "cupti", np.uint8), ("BUFTAB", "buftab", np.uint64), ("TIDMAP", "tidmap", np.int32),
    ("RTNAME", "rt_names", np.uint32), ("DRNAME", "dr_names", np.uint32),
    ("OPSTART", "op_start", np.int64), ("OPEND", "op_end", np.int64), ("OPID", "op_id", np.int32),
    ("OPDEV", "op_device", np.int32), ("OPRES", "op_resource", np.int64),
    ("OPTHR", "op_thread", np.int32), ("OPTYPE", "op_type", np.int32),
    ("OPNAME", "op_name", np.uint32), ("OPFLOW", "op_flow", np.uint32),
    ("OPFLOWT", "op_flowt", np.uint8), ("OPMDOFF", "op_mdoff", np.uint32),
    ("MDENT", "md", MD_ENTRY),
    # optional: join keys gathered from all shards of a sharded trace (see kineto_b200/sharding.py)
    ("GEXT", "g_ext", np.uint64), ("GOPS", "g_ops", np.int32),
]


def _empty(dt):
    return np.zeros(0, dt)


@dataclass
class Trace:
    params: np.ndarray = field(default_factory=lambda: np.zeros(1, PARAMS))
    devprops: np.ndarray = field(default_factory=lambda: _empty(DEVICE_PROPS))
    pool_off: np.ndarray = field(default_factory=lambda: np.zeros(1, np.uint64))
    pool_data: np.ndarray = field(default_factory=lambda: _empty(np.uint8))
    cupti: np.ndarray = field(default_factory=lambda: _empty(np.uint8))
    buftab: np.ndarray = field(default_factory=lambda: _empty(np.uint64))
    tidmap: np.ndarray = field(default_factory=lambda: _empty(np.int32))
    rt_names: np.ndarray = field(default_factory=lambda: _empty(np.uint32))
    dr_names: np.ndarray = field(default_factory=lambda: _empty(np.uint32))
    op_start: np.ndarray = field(default_factory=lambda: _empty(np.int64))
    op_end: np.ndarray = field(default_factory=lambda: _empty(np.int64))
    op_id: np.ndarray = field(default_factory=lambda: _empty(np.int32))
    op_device: np.ndarray = field(default_factory=lambda: _empty(np.int32))
    op_resource: np.ndarray = field(default_factory=lambda: _empty(np.int64))
    op_thread: np.ndarray = field(default_factory=lambda: _empty(np.int32))
    op_type: np.ndarray = field(default_factory=lambda: _empty(np.int32))
    op_name: np.ndarray = field(default_factory=lambda: _empty(np.uint32))
    op_flow: np.ndarray = field(default_factory=lambda: _empty(np.uint32))
    op_flowt: np.ndarray = field(default_factory=lambda: _empty(np.uint8))
    op_mdoff: np.ndarray = field(default_factory=lambda: np.zeros(1, np.uint32))
    md: np.ndarray = field(default_factory=lambda: _empty(MD_ENTRY))
    g_ext: np.ndarray = field(default_factory=lambda: _empty(np.uint64))
    g_ops: np.ndarray = field(default_factory=lambda: _empty(np.int32))

    @property
    def n_ops(self) -> int:
        return len(self.op_start)

    @property
    def n_buffers(self) -> int:
        return len(self.buftab) // 2

    def set_pool(self, pool: StringPool):
        self.pool_off, self.pool_data = pool.arrays()

    def pool(self) -> StringPool:
        return StringPool.from_arrays(self.pool_off, self.pool_data)

    def write(self, path: str):
        secs = []
        for tag, attr, dt in _SECTIONS:
            a = np.ascontiguousarray(getattr(self, attr), dtype=dt)
            if tag in ("GEXT", "GOPS") and a.size == 0:
                continue
            secs.append((tag, a.tobytes()))
        table_end = 16 + 24 * len(secs)
        pos = (table_end + 63) // 64 * 64
        table, offs = b"", []
        for tag, raw in secs:
            table += tag.encode().ljust(8, b"\0") + struct.pack("<QQ", pos, len(raw))
            offs.append(pos)
            pos = (pos + len(raw) + 63) // 64 * 64
        with open(path, "wb") as f:
            f.write(b"K2JTRACE" + struct.pack("<II", 1, len(secs)) + table)
            for off, (_, raw) in zip(offs, secs):
                f.seek(off)
                f.write(raw)
            f.truncate(pos)

    @classmethod
    def read(cls, path: str) -> "Trace":
        raw = open(path, "rb").read()
        assert raw[:8] == b"K2JTRACE"
        ver, n = struct.unpack_from("<II", raw, 8)
        assert ver == 1
        dts = {tag: (attr, dt) for tag, attr, dt in _SECTIONS}
        t = cls()
        for i in range(n):
            tag = raw[16 + 24 * i:24 + 24 * i].rstrip(b"\0").decode()
            off, size = struct.unpack_from("<QQ", raw, 24 + 24 * i)
            attr, dt = dts[tag]
            setattr(t, attr, np.frombuffer(raw, dt, count=size // np.dtype(dt).itemsize, offset=off).copy())
        return t


def make_buftab(offs: np.ndarray, buffer_bytes: int = 4 << 20) -> np.ndarray:
    """Splits packed records into CUPTI-style buffers of at most `buffer_bytes` (the reference's
    buffer size, libkineto/src/CuptiActivityApi.cpp:27); a record never straddles a buffer.
    `offs` are the n+1 record byte offsets.  Returns the flat (offset, valid size) table."""
    buftab, i, n = [], 0, len(offs) - 1
    while i < n:
        base = int(offs[i])
        j = int(np.searchsorted(offs, base + buffer_bytes, side="right")) - 1
        j = max(j, i + 1)
        buftab += [base, int(offs[j]) - base]
        i = j
    return np.array(buftab, np.uint64)


def interleave(parts: list[np.ndarray], order: np.ndarray):
    """Serialises records of several kinds in a given global order.  `parts[k]` holds the records of
    stream k in their own order; `order` is an array of stream indices, one per output record.
    Returns (bytes, offsets[n+1])."""
    sizes = np.array([p.dtype.itemsize for p in parts], np.int64)
    rec_size = sizes[order] if len(order) else np.zeros(0, np.int64)
    offs = np.concatenate([[0], np.cumsum(rec_size)]).astype(np.int64)
    out = np.zeros(int(offs[-1]) // 8, np.uint64)
    for k, p in enumerate(parts):
        idx = np.nonzero(order == k)[0]
        assert len(idx) == len(p), (k, len(idx), len(p))
        if len(idx) == 0:
            continue
        src = np.ascontiguousarray(p).view(np.uint64).reshape(len(p), -1)
        base = offs[idx] // 8
        for w in range(src.shape[1]):
            out[base + w] = src[:, w]
    return out.view(np.uint8), offs
