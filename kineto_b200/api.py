"""ctypes binding of libk2j.so (C ABI in include/k2j.h).

There is no CPU implementation behind this module: if the CUDA library is missing or no GPU is
present, constructing a `K2J` context raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import tracefile as tf

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("K2J_LIBRARY") or os.path.join(_HERE, "libk2j.so")  # K2J_LIBRARY: another build of the same ABI

STATUS = {0: "OK", 1: "INVALID_ARGUMENT", 2: "CUDA", 3: "UNSUPPORTED", 4: "STATE", 5: "DEVICE_CHECK", 6: "IO"}


class K2JError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"k2j: {STATUS.get(status, status)}: {msg}")
        self.status = status


class Params(C.Structure):
    _fields_ = [("base_time_ns", C.c_int64), ("window_start_ns", C.c_int64), ("window_end_ns", C.c_int64),
                ("pid", C.c_int32), ("ts_mode", C.c_int32), ("flags", C.c_int32), ("n_devices", C.c_int32),
                ("conv_t0", C.c_int64), ("conv_t0_approx", C.c_uint64), ("conv_scale_mant", C.c_uint64),
                ("conv_scale_exp", C.c_int32), ("activity_type_mask", C.c_uint32)]


class DeviceProps(C.Structure):
    _fields_ = [("major", C.c_int32), ("minor", C.c_int32), ("max_threads_per_block", C.c_int32),
                ("max_threads_per_sm", C.c_int32), ("regs_per_block", C.c_int32), ("regs_per_sm", C.c_int32),
                ("warp_size", C.c_int32), ("num_sms", C.c_int32), ("smem_per_block", C.c_uint64),
                ("smem_per_block_optin", C.c_uint64), ("smem_per_sm", C.c_uint64),
                ("reserved_smem_per_block", C.c_uint64)]


class Ops(C.Structure):
    _fields_ = [("n_ops", C.c_uint64), ("start_ns", C.c_void_p), ("end_ns", C.c_void_p), ("id", C.c_void_p),
                ("device", C.c_void_p), ("resource", C.c_void_p), ("thread", C.c_void_p), ("type", C.c_void_p),
                ("name", C.c_void_p), ("flow_id", C.c_void_p), ("flow_info", C.c_void_p), ("md_off", C.c_void_p),
                ("md", C.c_void_p)]


class Result(C.Structure):
    _fields_ = [("out_bytes", C.c_uint64), ("ops_bytes", C.c_uint64), ("n_records", C.c_uint64),
                ("x_events", C.c_uint64), ("flow_events", C.c_uint64), ("out_of_range_events", C.c_uint64),
                ("blocklisted_runtime_events", C.c_uint64), ("invalid_external_correlation_events", C.c_uint64),
                ("unexpected_cuda_events", C.c_uint64), ("in_bytes", C.c_uint64), ("name_bytes", C.c_uint64), ("annotation_bytes", C.c_uint64),
                ("kernel_launches", C.c_uint32), ("reserved", C.c_uint32), ("ms_segment", C.c_float),
                ("ms_join", C.c_float), ("ms_size", C.c_float), ("ms_scan", C.c_float), ("ms_emit", C.c_float),
                ("ms_total", C.c_float)]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_ if n != "reserved"}


class SegmentInfo(C.Structure):
    _fields_ = [("n_records", C.c_uint64), ("n_external", C.c_uint64), ("external_records", C.c_void_p),
                ("n_ops", C.c_uint64), ("op_ids", C.c_void_p), ("n_user_external", C.c_uint64)]


SPAN = np.dtype([("start_ns", "<i8"), ("end_ns", "<i8"), ("first_event", "<u8"), ("device", "<u4"), ("stream", "<u4"),
                 ("op_id", "<i4"), ("op_row", "<u4")])  # k2j_span

EXPORTS = ["k2j_set_global_join_rows", "k2j_join_need_bits", "k2j_filter_join_keys", "k2j_op_id_bits", "k2j_set_global_op_bits", "k2j_set_join_user_records", "k2j_emit_to_host", "k2j_emit_to_fd", "k2j_exclusive_scan_u32", "k2j_exclusive_scan_u32_noalloc", "k2j_segment", "k2j_set_global_join", "k2j_emit", "k2j_create", "k2j_destroy", "k2j_last_error", "k2j_set_params", "k2j_set_strings",
           "k2j_set_cbid_names", "k2j_set_thread_map", "k2j_set_ops", "k2j_set_cupti", "k2j_run", "k2j_output",
           "k2j_copy_output", "k2j_copy_output_async", "k2j_write_output", "k2j_write_output_at", "k2j_synchronize", "k2j_version",
           "k2j_export_lookup_records", "k2j_set_guest_ranges", "k2j_set_guest_ops", "k2j_partial_spans", "k2j_append_spans", "k2j_names_create", "k2j_names_destroy", "k2j_names_intern", "k2j_names_pool", "k2j_intern_kernel_names"]

_lib = None


def load_library():
    """Loads libk2j.so; raises if it has not been built (python -m kineto_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m kineto_b200.build`")
    lib = C.CDLL(LIB_PATH)
    vp = C.c_void_p
    lib.k2j_create.argtypes = [C.c_int, vp, C.POINTER(vp)]
    lib.k2j_destroy.argtypes = [vp]
    lib.k2j_destroy.restype = None
    lib.k2j_last_error.argtypes = [vp]
    lib.k2j_last_error.restype = C.c_char_p
    lib.k2j_set_params.argtypes = [vp, C.POINTER(Params), C.POINTER(DeviceProps)]
    lib.k2j_set_strings.argtypes = [vp, vp, vp, C.c_uint64]
    lib.k2j_set_cbid_names.argtypes = [vp, vp, C.c_uint32, vp, C.c_uint32]
    lib.k2j_set_thread_map.argtypes = [vp, vp, C.c_uint32]
    lib.k2j_set_ops.argtypes = [vp, C.POINTER(Ops)]
    lib.k2j_set_cupti.argtypes = [vp, vp, C.c_uint64, vp, C.c_uint32]
    lib.k2j_run.argtypes = [vp, C.POINTER(Result)]
    lib.k2j_segment.argtypes = [vp, C.POINTER(SegmentInfo)]
    lib.k2j_set_global_join.argtypes = [vp, vp, C.c_uint64, C.c_uint64, vp, C.c_uint64]
    lib.k2j_set_global_join_rows.argtypes = [vp, vp, C.c_uint64, vp, C.c_uint64, C.c_uint64, vp, C.c_uint32, C.c_uint32]
    lib.k2j_join_need_bits.argtypes = [vp, vp, C.c_uint64]
    lib.k2j_op_id_bits.argtypes = [vp, C.c_int64, C.c_uint64, vp]
    lib.k2j_set_global_op_bits.argtypes = [vp, vp, C.c_uint64, vp]
    lib.k2j_set_join_user_records.argtypes = [vp, C.c_int]
    lib.k2j_filter_join_keys.argtypes = [vp, vp, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, vp, C.c_uint64, vp]
    lib.k2j_emit.argtypes = [vp, C.POINTER(Result)]
    lib.k2j_emit_to_host.argtypes = [vp, vp, C.c_uint64, C.c_uint64, C.POINTER(Result)]
    lib.k2j_emit_to_fd.argtypes = [vp, C.c_int, C.c_uint64, C.POINTER(Result)]
    lib.k2j_exclusive_scan_u32.argtypes = [vp, vp, C.c_uint64, vp, C.POINTER(C.c_uint64)]
    lib.k2j_exclusive_scan_u32_noalloc.argtypes = [C.c_int, vp, vp, C.c_uint64, vp, vp]
    lib.k2j_output.argtypes = [vp, C.POINTER(vp), C.POINTER(C.c_uint64)]
    lib.k2j_copy_output.argtypes = [vp, vp, C.c_uint64]
    lib.k2j_copy_output_async.argtypes = [vp, vp, C.c_uint64]
    lib.k2j_write_output.argtypes = [vp, C.c_int, C.POINTER(C.c_uint64)]
    lib.k2j_write_output_at.argtypes = [vp, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64]
    lib.k2j_synchronize.argtypes = [vp]
    lib.k2j_export_lookup_records.argtypes = [vp, C.POINTER(vp), C.POINTER(C.c_uint64)]
    lib.k2j_set_guest_ranges.argtypes = [vp, C.c_uint64, C.c_uint64]
    lib.k2j_set_guest_ops.argtypes = [vp, C.c_uint64]
    lib.k2j_partial_spans.argtypes = [vp, C.POINTER(vp), C.POINTER(C.c_uint64)]
    lib.k2j_append_spans.argtypes = [vp, vp, C.c_uint64, C.POINTER(C.c_uint64)]
    lib.k2j_names_create.argtypes = [C.POINTER(vp)]
    lib.k2j_names_destroy.argtypes = [vp]
    lib.k2j_names_destroy.restype = None
    lib.k2j_names_intern.argtypes = [vp, C.c_char_p, C.c_uint64, C.POINTER(C.c_uint32)]
    lib.k2j_names_pool.argtypes = [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(C.c_uint64)]
    lib.k2j_intern_kernel_names.argtypes = [vp, vp, C.c_uint64, vp, C.c_uint32, C.c_int, C.POINTER(C.c_uint64)]
    lib.k2j_version.restype = C.c_char_p
    _lib = lib
    return lib


def activity_type_mask(mode: int, flags: int) -> int:
    """Selected CPU-side activity types: everything when the logger is driven directly (mode 0);
    otherwise libkineto's default selection (types 0..17), GPU_USER_ANNOTATION by flag bit 0."""
    if mode == 0:
        return 0xFFFFFFFF
    m = (1 << 18) - 1
    return m if flags & 1 else m & ~(1 << 2)


def _ptr(a):
    """Address of a numpy array or a torch tensor (host or device)."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data if a.size else None
    return a.data_ptr() if a.numel() else None  # torch tensor


class K2J:
    """One processing context on one GPU."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self.lib = load_library()
        h = C.c_void_p()
        # None: a stream owned by the context.  0 is the handle torch reports for the default stream: the context then
        # runs on the legacy default stream (cudaStreamLegacy, handle 1), NOT on a stream of its own (which is what a
        # NULL handle means to k2j_create), so that it stays ordered with the caller's work on that stream.
        handle = None if stream is None else C.c_void_p(stream if stream != 0 else 1)
        st = self.lib.k2j_create(device, handle, C.byref(h))
        if st != 0:
            raise K2JError(st, "k2j_create failed (is a CUDA device present?)")
        self.h = h
        self._keep = {}

    def close(self):
        if self.h:
            self.lib.k2j_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st):
        if st != 0:
            raise K2JError(st, self.lib.k2j_last_error(self.h).decode())

    # -- inputs ------------------------------------------------------------------------------
    def set_params(self, trace: tf.Trace):
        p = trace.params[0]
        cp = Params(int(p["base_time_ns"]), int(p["window_start_ns"]), int(p["window_end_ns"]), int(p["pid"]),
                    int(p["ts_mode"]), int(p["flags"]) | (12 if int(p["mode"]) == 1 else 0), int(p["n_devices"]), int(p["conv_t0"]),
                    int(p["conv_t0_approx"]), int(p["conv_scale_mant"]), int(p["conv_scale_exp"]),
                    activity_type_mask(int(p["mode"]), int(p["flags"])))
        n = int(p["n_devices"])
        props = (DeviceProps * max(n, 1))()
        for i in range(n):
            d = trace.devprops[i]
            for name, _ in DeviceProps._fields_:
                setattr(props[i], name, int(d[name]))
        self._check(self.lib.k2j_set_params(self.h, C.byref(cp), props))

    def set_arrays(self, a: dict, buftab: np.ndarray, tidmap: np.ndarray):
        """`a` maps Trace attribute names to numpy arrays (host) or torch tensors (host or device)."""
        self._keep = dict(a, buftab=buftab, tidmap=tidmap)
        n_str = len(a["pool_off"]) - 1
        self._check(self.lib.k2j_set_strings(self.h, _ptr(a["pool_off"]), _ptr(a["pool_data"]), n_str))
        self._check(self.lib.k2j_set_cbid_names(self.h, _ptr(a["rt_names"]), len(a["rt_names"]), _ptr(a["dr_names"]),
                                                len(a["dr_names"])))
        self._check(self.lib.k2j_set_thread_map(self.h, _ptr(tidmap), len(tidmap) // 2))
        n_ops = len(a["op_start"])
        ops = Ops(n_ops, _ptr(a["op_start"]), _ptr(a["op_end"]), _ptr(a["op_id"]), _ptr(a["op_device"]),
                  _ptr(a["op_resource"]), _ptr(a["op_thread"]), _ptr(a["op_type"]), _ptr(a["op_name"]),
                  _ptr(a["op_flow"]), _ptr(a["op_flowt"]), _ptr(a["op_mdoff"]), _ptr(a["md"]))
        self._check(self.lib.k2j_set_ops(self.h, C.byref(ops)))
        nbytes = a["cupti"].nbytes if isinstance(a["cupti"], np.ndarray) else a["cupti"].numel()
        self._check(self.lib.k2j_set_cupti(self.h, _ptr(a["cupti"]), nbytes, _ptr(buftab), len(buftab) // 2))

    ARRAYS = ["pool_off", "pool_data", "rt_names", "dr_names", "op_start", "op_end", "op_id", "op_device",
              "op_resource", "op_thread", "op_type", "op_name", "op_flow", "op_flowt", "op_mdoff", "md", "cupti"]

    def load(self, trace: tf.Trace, arrays: dict | None = None):
        """Stages a whole trace.  `arrays` overrides the numpy arrays of `trace` (e.g. device tensors)."""
        self.set_params(trace)
        a = {k: np.ascontiguousarray(getattr(trace, k)) for k in self.ARRAYS}
        if arrays:
            a.update(arrays)
        self.set_arrays(a, np.ascontiguousarray(trace.buftab), np.ascontiguousarray(trace.tidmap))

    # -- run ----------------------------------------------------------------------------------
    def run(self) -> dict:
        r = Result()
        st = self.lib.k2j_run(self.h, C.byref(r))
        self.result = r.as_dict()
        self._check(st)
        return self.result

    def segment(self, sync: bool = True):
        """k2j_segment.  `sync=False`: no shard information is wanted, the call only enqueues the work."""
        if not sync:
            self._check(self.lib.k2j_segment(self.h, None))
            return None
        info = SegmentInfo()
        self._check(self.lib.k2j_segment(self.h, C.byref(info)))
        return info

    def export_lookup_records(self) -> tuple[int, int]:
        """(device address, byte count) of this shard's lookup records: one CUPTI buffer in the context's device
        memory, valid until the context's next call (k2j_export_lookup_records)."""
        ptr, n = C.c_void_p(), C.c_uint64()
        self._check(self.lib.k2j_export_lookup_records(self.h, C.byref(ptr), C.byref(n)))
        return ptr.value or 0, n.value

    def set_cupti(self, cupti, buftab: np.ndarray):
        """The CUPTI bytes alone (uint8 numpy array or device tensor) with their (offset, valid bytes) table."""
        bt = np.ascontiguousarray(buftab, dtype=np.uint64)
        self._keep["cupti"], self._keep["buftab"] = cupti, bt
        n = cupti.nbytes if isinstance(cupti, np.ndarray) else cupti.numel()
        self._check(self.lib.k2j_set_cupti(self.h, _ptr(cupti), n, _ptr(bt), bt.size // 2))

    def partial_spans(self) -> np.ndarray:
        """This shard's parts of the user-annotation spans after a sharded emit (a copy; dtype SPAN)."""
        ptr, n = C.c_void_p(), C.c_uint64()
        self._check(self.lib.k2j_partial_spans(self.h, C.byref(ptr), C.byref(n)))
        if n.value == 0:
            return np.zeros(0, SPAN)
        raw = C.string_at(ptr.value, n.value * SPAN.itemsize)
        return np.frombuffer(raw, SPAN).copy()

    def append_spans(self, spans: np.ndarray) -> int:
        """Formats merged spans behind the text of the last emit (k2j_append_spans); returns the bytes added."""
        a = np.ascontiguousarray(spans, dtype=SPAN)
        n = C.c_uint64()
        self._check(self.lib.k2j_append_spans(self.h, _ptr(a), a.size, C.byref(n)))
        self.result["out_bytes"] += n.value
        return n.value

    def set_guest_ops(self, n_guest_ops: int):
        self._check(self.lib.k2j_set_guest_ops(self.h, n_guest_ops))

    def set_guest_ranges(self, front_end_bytes: int, back_begin_bytes: int):
        self._check(self.lib.k2j_set_guest_ranges(self.h, front_end_bytes, back_begin_bytes))

    def set_global_join(self, ext_all, n_ext_all: int, own_begin: int, op_ids_all, n_ops_all: int):
        """`ext_all`: device tensor of 16-byte external-correlation records of all shards in shard
        order; `op_ids_all`: device tensor of all shards' CPU-activity ids."""
        self._keep["g_ext"], self._keep["g_ops"] = ext_all, op_ids_all
        self._check(self.lib.k2j_set_global_join(self.h, _ptr(ext_all), n_ext_all, own_begin, _ptr(op_ids_all),
                                                 n_ops_all))

    def set_global_join_rows(self, rows, ext_stride: int, ops_stride: int, counts, world: int, rank: int, ext_capacity: int | None = None):
        """`rows`: the int64 device tensor an all-gather of per-shard rows produced (sharding.JoinExchange): every row
        holds room for `ext_capacity` 16-byte records (default: ext_stride, the index stride) followed by ops_stride
        ids; `counts`: int64 device tensor, 2 per shard."""
        self._keep["g_rows"], self._keep["g_counts"] = rows, counts
        pitch = rows.numel() * 8 // world
        cap = ext_stride if ext_capacity is None else ext_capacity
        self._check(self.lib.k2j_set_global_join_rows(self.h, rows.data_ptr(), ext_stride, rows.data_ptr() + cap * 16,
                                                      ops_stride, pitch, counts.data_ptr(), world, rank))

    def op_id_bits(self, min_id: int, bits):
        """Sets, in the int64 device tensor `bits`, bit id - min_id for every CPU-side activity of this shard."""
        self._check(self.lib.k2j_op_id_bits(self.h, min_id, bits.numel() * 64, bits.data_ptr()))

    def set_global_op_bits(self, bit_rows_ptr: int, row_pitch_bytes: int, meta):
        """`meta`: int64 device tensor, (min_id, n_bits) per shard; `bit_rows_ptr`: address of shard 0's bitmap."""
        self._keep["g_op_meta"] = meta
        self._check(self.lib.k2j_set_global_op_bits(self.h, bit_rows_ptr, row_pitch_bytes, meta.data_ptr()))

    def set_join_user_records(self, any_records: bool):
        """Sharded runs: whether any shard holds CUSTOM1 correlation records (k2j_set_join_user_records)."""
        self._check(self.lib.k2j_set_join_user_records(self.h, 1 if any_records else 0))

    def join_need_bits(self, bits):
        """Fills the uint8 device tensor `bits` (a power-of-two number of bits) with this shard's filter."""
        self._check(self.lib.k2j_join_need_bits(self.h, bits.data_ptr(), bits.numel() * 8))

    def filter_join_keys(self, need_rows, world: int, rank: int, out_records, n_out):
        """`need_rows`: uint8 device tensor, the shards' filters one after the other; `out_records`: int64 device tensor
        with room for this shard's records (2 words each); `n_out`: int64 device tensor of one element."""
        pitch = need_rows.numel() // world
        self._check(self.lib.k2j_filter_join_keys(self.h, need_rows.data_ptr(), pitch, pitch * 8, world, rank, out_records.data_ptr(),
                                                  out_records.numel() // 2, n_out.data_ptr()))

    def emit(self) -> dict:
        r = Result()
        st = self.lib.k2j_emit(self.h, C.byref(r))
        self.result = r.as_dict()
        self._check(st)
        return self.result

    def emit_to_host(self, dst, slab_bytes: int = 0) -> dict:
        """Tiled emit: the text goes to `dst` (uint8 numpy array or pinned torch tensor) slab by slab."""
        r = Result()
        cap = dst.nbytes if isinstance(dst, np.ndarray) else dst.numel()
        st = self.lib.k2j_emit_to_host(self.h, _ptr(dst) or 0, cap, slab_bytes, C.byref(r))
        self.result = r.as_dict()
        self._check(st)
        return self.result

    def emit_to_fd(self, fd: int, slab_bytes: int = 0) -> dict:
        """Tiled emit: the text is written to the open file descriptor `fd` slab by slab."""
        r = Result()
        st = self.lib.k2j_emit_to_fd(self.h, fd, slab_bytes, C.byref(r))
        self.result = r.as_dict()
        self._check(st)
        return self.result

    def exclusive_scan(self, sizes, offsets) -> int:
        """`sizes`: int32/uint32 device tensor, `offsets`: int64 device tensor of the same length; returns the total."""
        total = C.c_uint64()
        self._check(self.lib.k2j_exclusive_scan_u32(self.h, _ptr(sizes), sizes.numel(), _ptr(offsets), C.byref(total)))
        return total.value

    def output_ptr(self):
        p, n = C.c_void_p(), C.c_uint64()
        self._check(self.lib.k2j_output(self.h, C.byref(p), C.byref(n)))
        return p.value, n.value

    def copy_output(self, dst=None) -> np.ndarray:
        """Copies the produced text to host memory (`dst`: uint8 numpy array or pinned torch tensor)."""
        n = self.result["out_bytes"]
        if dst is None:
            dst = np.empty(n, np.uint8)
        cap = dst.nbytes if isinstance(dst, np.ndarray) else dst.numel()
        self._check(self.lib.k2j_copy_output(self.h, _ptr(dst) or 0, cap))
        return dst

    def copy_output_async(self, dst):
        """Enqueues the copy on the context's stream and returns; `synchronize()` completes it."""
        cap = dst.nbytes if isinstance(dst, np.ndarray) else dst.numel()
        self._check(self.lib.k2j_copy_output_async(self.h, _ptr(dst) or 0, cap))
        return dst

    def write_output(self, fd: int) -> int:
        """Streams the produced text to the open file descriptor `fd` (chunked copy overlapped with the writes)."""
        n = C.c_uint64()
        self._check(self.lib.k2j_write_output(self.h, fd, C.byref(n)))
        return n.value

    def write_output_at(self, fd: int, file_offset: int, begin: int, n_bytes: int):
        """Writes bytes [begin, begin + n_bytes) of the text at `file_offset` of `fd` (pwrite)."""
        self._check(self.lib.k2j_write_output_at(self.h, fd, file_offset, begin, n_bytes))

    def synchronize(self):
        self._check(self.lib.k2j_synchronize(self.h))


def device_arrays(trace: tf.Trace, device="cuda:0") -> dict:
    """Uploads the large arrays of a trace with torch and returns them as device tensors, so a context
    can use them in place (inputs resident in HBM)."""
    import torch

    out = {}
    for k in K2J.ARRAYS:
        a = np.ascontiguousarray(getattr(trace, k))
        if a.dtype.fields is not None:  # structured (metadata entries): ship as bytes
            a = a.view(np.uint8)
        if a.dtype == np.uint64:
            a = a.view(np.int64)
        elif a.dtype == np.uint32:
            a = a.view(np.int32)
        out[k] = torch.from_numpy(a).to(device)
    # the copies ran on torch's current stream; a context reads the arrays on its own stream (see include/k2j.h on
    # device memory handed to the library), so they are made complete here
    torch.cuda.synchronize(device)
    return out


class Names:
    """Host-side string table (k2j_names): ids for the strings of a trace and, for drained CUPTI buffers that still
    hold `const char*` kernel names, the in-place replacement of those pointers by ids.  No GPU is needed."""

    def __init__(self):
        self.lib = load_library()
        self.h = C.c_void_p()
        if self.lib.k2j_names_create(C.byref(self.h)) != 0:
            raise RuntimeError("k2j_names_create failed")

    def close(self):
        if self.h:
            self.lib.k2j_names_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        self.close()

    def intern(self, s: bytes) -> int:
        out = C.c_uint32()
        st = self.lib.k2j_names_intern(self.h, s, len(s), C.byref(out))
        if st != 0:
            raise RuntimeError("k2j_names_intern: %s" % STATUS.get(st, st))
        return out.value

    def intern_kernel_names(self, cupti: np.ndarray, buftab: np.ndarray, demangle: bool = True) -> int:
        """`cupti` (writable uint8 array) is changed in place; returns the number of kernel records seen."""
        assert cupti.dtype == np.uint8 and cupti.flags.writeable and cupti.flags.c_contiguous
        bt = np.ascontiguousarray(buftab, dtype=np.uint64)
        n = C.c_uint64()
        st = self.lib.k2j_intern_kernel_names(self.h, _ptr(cupti), cupti.size, _ptr(bt), bt.size // 2, int(demangle), C.byref(n))
        if st != 0:
            raise RuntimeError("k2j_intern_kernel_names: %s" % STATUS.get(st, st))
        return n.value

    def pool(self) -> tuple[np.ndarray, np.ndarray]:
        """(offsets, bytes) as k2j_set_strings takes them (copies)."""
        off, data, n = C.c_void_p(), C.c_void_p(), C.c_uint64()
        st = self.lib.k2j_names_pool(self.h, C.byref(off), C.byref(data), C.byref(n))
        if st != 0:
            raise RuntimeError("k2j_names_pool: %s" % STATUS.get(st, st))
        offs = np.ctypeslib.as_array(C.cast(off, C.POINTER(C.c_uint64)), shape=(n.value + 1,)).copy()
        total = int(offs[-1])
        blob = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(total,)).copy() if total else np.zeros(0, np.uint8)
        return offs, blob


def process(trace: tf.Trace, device: int = 0) -> tuple[bytes, dict]:
    """Convenience: run one trace from host arrays, return (activities text, result dict)."""
    ctx = K2J(device)
    try:
        ctx.load(trace)
        res = ctx.run()
        out = ctx.copy_output().tobytes()
    finally:
        ctx.close()
    return out, res


class _DeviceMemory:
    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}


def device_view(ptr: int, n: int, typestr: str, device="cuda:0"):
    """A torch tensor over `n` elements of device memory at address `ptr` (no copy).  The memory
    belongs to the context that returned the address and is valid until its next call."""
    import torch

    if n == 0:
        return torch.empty(0, dtype={"<i8": torch.int64, "<i4": torch.int32, "|u1": torch.uint8}[typestr], device=device)
    return torch.as_tensor(_DeviceMemory(ptr, n, typestr), device=device)
