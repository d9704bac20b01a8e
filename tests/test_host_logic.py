"""CPU tests of the host-side pieces: container round trip, metadata visit order, callback names,
the C ABI surface, and the CPU build of the formatting routines."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

import helpers
from kineto_b200 import md_order, synth
from kineto_b200 import tracefile as tf

ROOT = helpers.ROOT


def test_container_round_trip(tmp_path):
    t = synth.gen_mixed(500, seed=9, pool_size=50)
    p = str(tmp_path / "t.k2jt")
    t.write(p)
    u = tf.Trace.read(p)
    for _, attr, _ in tf._SECTIONS:
        assert getattr(t, attr).tobytes() == getattr(u, attr).tobytes(), attr


def test_record_layouts_match_cupti_header_sizes():
    assert {k: v.itemsize for k, v in tf.RECORD_DTYPE.items()} == tf.RECORD_SIZE


def test_buffers_never_split_records():
    t = synth.gen_kernel_launches(2000, seed=4, pool_size=30, buffer_bytes=8192)
    bt = t.buftab.reshape(-1, 2)
    assert (bt[:, 1] <= 8192).all() and bt[:, 1].sum() == len(t.cupti)
    for off, valid in bt:
        pos, end = int(off), int(off + valid)
        while pos < end:
            kind = int(t.cupti[pos:pos + 4].view(np.uint32)[0])
            pos += tf.RECORD_SIZE[kind]
        assert pos == end


def test_md_order_known():
    assert md_order.md_visit_order(("grid", "block")) == ("block", "grid")


@pytest.mark.skipif(not helpers.have_ref(), reason="reference build not present")
def test_md_order_matches_libstdcpp():
    rng = np.random.default_rng(3)
    words = ["grid", "block", "Sequence number", "Fwd thread id", "Input Dims", "Input type", "External id",
             "Python id", "a", "bb", "finished", "Collective name", "dtype", "In msg nelems", "Rank", "kwinputs"]
    for _ in range(40):
        k = [words[i] for i in rng.permutation(len(words))[:int(rng.integers(1, 13))]]
        ref = subprocess.run([helpers.REF_DRIVER, "--md-order", *k], capture_output=True, text=True).stdout.split("\n")[:-1]
        assert list(md_order.md_visit_order(tuple(k))) == ref
    # more than 13 keys: the container moves to 29, then 59 buckets and re-links its nodes
    many = words + ["key%d" % i for i in range(50)]
    for _ in range(30):
        k = [many[i] for i in rng.permutation(len(many))[:int(rng.integers(14, 62))]]
        ref = subprocess.run([helpers.REF_DRIVER, "--md-order", *k], capture_output=True, text=True).stdout.split("\n")[:-1]
        assert list(md_order.md_visit_order(tuple(k))) == ref


@pytest.mark.skipif(not helpers.have_ref(), reason="reference build not present")
def test_cbid_names_match_reference(tmp_path):
    out = str(tmp_path / "cbid.txt")
    subprocess.run([helpers.REF_DRIVER, "--cbid-names", out], check=True)
    ref = {"R": {}, "D": {}}
    for line in open(out):
        d, c, name = line.rstrip("\n").split(" ", 2)
        ref[d][int(c)] = name
    for d in "RD":
        mine = synth.cbid_names(d)
        assert len(mine) == len(ref[d])
        # id 0 is the enum's INVALID entry, which CUPTI names itself
        bad = [(i, mine[i], ref[d][i]) for i in range(1, len(mine)) if mine[i] != ref[d][i]]
        assert not bad, bad[:5]


def test_cbid_known_answers():
    """libkineto/test/CuptiStringsTest.cpp:15-78"""
    rt = synth.cbid_names("R")
    assert rt[211] == "cudaLaunchKernel" and rt[31] == "cudaMemcpy" and rt[131] == "cudaStreamSynchronize"
    assert synth.cbid_names("D")[307] == "cuLaunchKernel"


def test_library_exports_every_declared_symbol():
    """The shared library loads without a GPU and exports exactly what include/k2j.h declares."""
    from kineto_b200 import api
    header = open(os.path.join(ROOT, "include", "k2j.h")).read()
    declared = set(re.findall(r"\b(k2j_[a-z0-9_]+)\s*\(", header))
    lib = ctypes.CDLL(api.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert declared == set(api.EXPORTS)
    assert b"k2j" in ctypes.cast(ctypes.CDLL(api.LIB_PATH).k2j_version, ctypes.CFUNCTYPE(ctypes.c_char_p))()


def test_context_creation_fails_loudly_without_gpu():
    import torch
    from kineto_b200 import api
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(api.K2JError):
        api.K2J(0)


@pytest.fixture(scope="module")
def fc(tmp_path_factory):
    so = str(tmp_path_factory.mktemp("fc") / "libfc.so")
    subprocess.run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-I" + os.path.join(ROOT, "kineto_b200", "csrc"),
                    os.path.join(ROOT, "tests", "native", "format_check.cpp"), "-o", so], check=True)
    return ctypes.CDLL(so)


def _batch(fc, fn, arr, stride=40):
    out = np.zeros((len(arr), stride), np.uint8)
    getattr(fc, fn)(arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(len(arr)), out.ctypes.data_as(ctypes.c_void_p),
                    ctypes.c_int(stride))
    return [bytes(r).split(b"\0")[0].decode() for r in out]


def test_integer_formatting(fc):
    rng = np.random.default_rng(0)
    v = np.concatenate([rng.integers(0, 2 ** 63, 20000, dtype=np.uint64) >> rng.integers(0, 64, 20000).astype(np.uint64),
                        np.array([0, 1, 9, 10, 2 ** 64 - 1], np.uint64)] +
                       [np.array([10 ** k - 1, 10 ** k, 10 ** k + 1], np.uint64) for k in range(1, 20)])
    assert _batch(fc, "fc_u64", v) == [str(int(x)) for x in v]
    vi = v.view(np.int64)
    assert _batch(fc, "fc_i64", vi) == [str(int(x)) for x in vi]
    ts = np.abs(vi) >> 1
    assert _batch(fc, "fc_ts", ts) == ["%d.%03d" % (int(x) // 1000, int(x) % 1000) for x in ts]


def test_double_formatting_against_port(fc):
    rng = np.random.default_rng(1)
    d = np.concatenate([rng.integers(0, 2 ** 63, 30000, dtype=np.uint64).view(np.float64), rng.random(5000),
                        rng.random(5000) * 1e6, (rng.integers(1, 2 ** 24, 10000) / 148.0).astype(np.float32).astype(np.float64),
                        np.array([0.0, -0.0, 1.0, 2.0, 1e16, 1e15, 9.999999999999999e15, 1e-4, 1e-5, 5e-324,
                                  1.7976931348623157e308, 2.2250738585072014e-308, np.inf, -np.inf, 0.1, 1 / 3, 1e22, 1e23,
                                  9007199254740993.0, 4.35, 1048.576])])
    d = d[~np.isnan(d)]
    got = _batch(fc, "fc_doubles", d)
    for g, x in zip(got, d):
        want = helpers.port_fmt_double(float(x))
        if not np.isfinite(x):
            want = '"' + want + '"'
        assert g == want, (x, g, want)


def test_tsc_conversion_matches_x87(fc):
    if fc.fc_long_double_mant_dig() != 64:
        pytest.skip("host long double is not the x87 80-bit format")
    rng = np.random.default_rng(2)
    for mant, exp in [((1 << 63) + 123456789123, 0), (synth.scale_to_x87(synth.TSC_SCALE)[0] | 0x5A5, -1),
                      ((1 << 64) - 1, 0), (0xC000000000000001, -1), (0x8000000000000001, 3)]:
        t = rng.integers(1, 2 ** 62, 50000, dtype=np.uint64) >> rng.integers(0, 40, 50000).astype(np.uint64)
        o1, o2 = np.zeros(len(t), np.int64), np.zeros(len(t), np.int64)
        for fn, o in (("fc_tsc", o1), ("fc_tsc_native", o2)):
            getattr(fc, fn)(t.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(len(t)), ctypes.c_uint64(1000),
                            ctypes.c_int64(17 * 10 ** 17), ctypes.c_uint64(mant), ctypes.c_int(exp),
                            o.ctypes.data_as(ctypes.c_void_p))
        assert (o1 == o2).all()


def test_window_sink_on_cpu(tmp_path):
    """The emit pass's output sink, compiled for the host: random events through every append primitive, written in
    random order at every alignment, give the plain concatenation of their texts (windows flush, the open block
    moves, neighbours share their boundary words)."""
    so = str(tmp_path / "libsc.so")
    subprocess.run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-I" + os.path.join(ROOT, "kineto_b200", "csrc"),
                    os.path.join(ROOT, "tests", "native", "sink_check.cpp"), "-o", so], check=True)
    sc = ctypes.CDLL(so)
    sc.sc_fuzz.restype = ctypes.c_int64
    sc.sc_fuzz.argtypes = [ctypes.c_uint64, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    for seed in range(1, 121):
        assert sc.sc_fuzz(seed, 300, seed % 40, (seed * 7) % 400) == 0, seed
    assert sc.sc_fuzz(1000, 2000, 0, 0) == 0      # shortest events only
    assert sc.sc_fuzz(1001, 50, 6, 5000) == 0     # copies far longer than a window


def kernel_name_ids(cupti, buftab):
    from kineto_b200 import tracefile as tf
    out = []
    for b in range(len(buftab) // 2):
        at, end = int(buftab[2 * b]), int(buftab[2 * b]) + int(buftab[2 * b + 1])
        while at + 8 <= end:
            kind = int(cupti[at:at + 4].view(np.uint32)[0])
            if kind == tf.KIND_CONCURRENT_KERNEL:
                out.append(int(cupti[at + 104:at + 112].view(np.uint64)[0]))
            at += (tf.RECORD_SIZE[kind] + 7) & ~7
    return out


@pytest.mark.parametrize("n,demangle", [(3000, True), (3000, False), (120_000, True)], ids=["small", "kept_mangled", "threads"])
def test_intern_kernel_names_replaces_pointers_by_ids_of_demangled_names(n, demangle):
    """Buffers as CUPTI writes them (kernel names are pointers) become buffers for k2j_set_cupti: every kernel record
    names the id of demangle(name) as libkineto/src/Demangle.cpp:33-53 gives it, each distinct string once in the
    pool, ids in order of first sight whatever the number of threads (the large case is walked on several)."""
    from kineto_b200 import api, synth
    trace = synth.gen_mixed(n, seed=77, pool_size=300, escape_fraction=0.1)
    raw, keep, expected = helpers.with_raw_kernel_names(trace, helpers.MANGLED)
    names = api.Names()
    pre = names.intern(b"cudaLaunchKernel")
    assert pre == 0 and names.intern(b"cudaLaunchKernel") == 0 and names.intern(b"") == 1
    seen = names.intern_kernel_names(raw, trace.buftab, demangle=demangle)
    assert seen == len(expected) > len(helpers.MANGLED)
    off, data = names.pool()
    blob = data.tobytes()
    strings = [blob[int(off[i]):int(off[i + 1])] for i in range(len(off) - 1)]
    assert len(set(strings)) == len(strings)
    want = [synth.demangled(e) if demangle else e for e in expected]
    ids = kernel_name_ids(raw, trace.buftab)
    assert [strings[i] for i in ids] == want
    if demangle:
        assert strings[ids[0]] == b"void foo<int>(int)" and strings[ids[4]] == b"_Z" and strings[ids[7]] == b"x" * 9000
    first_sight = list(dict.fromkeys(want))
    assert [s for s in strings[2:]] == [s for s in first_sight if s not in (b"cudaLaunchKernel", b"")]
    # everything that is not a kernel name is untouched
    a, b = np.array(trace.cupti, copy=True), raw.copy()
    for arr in (a, b):
        for at in kernel_offsets(arr, trace.buftab):
            arr[at + 104:at + 112] = 0
    assert np.array_equal(a, b)
    del keep


def kernel_offsets(cupti, buftab):
    from kineto_b200 import tracefile as tf
    for b in range(len(buftab) // 2):
        at, end = int(buftab[2 * b]), int(buftab[2 * b]) + int(buftab[2 * b + 1])
        while at + 8 <= end:
            kind = int(cupti[at:at + 4].view(np.uint32)[0])
            if kind == tf.KIND_CONCURRENT_KERNEL:
                yield at
            at += (tf.RECORD_SIZE[kind] + 7) & ~7


def test_intern_kernel_names_rejects_bad_tables():
    from kineto_b200 import api
    names = api.Names()
    buf = np.zeros(64, np.uint8)
    for tab in ([4, 8], [0, 72], [128, 0]):
        with pytest.raises(RuntimeError, match="INVALID_ARGUMENT"):
            names.intern_kernel_names(buf, np.array(tab, np.uint64))
    assert names.intern_kernel_names(buf, np.array([0, 64], np.uint64)) == 0  # kind 0: ends the walk
    assert names.intern_kernel_names(np.zeros(0, np.uint8), np.zeros(0, np.uint64)) == 0


def test_intern_kernel_names_round_trip_gives_the_generated_buffers():
    """With the trace's own strings interned first (ids 0..n-1 in pool order), replacing the pointers gives back the
    generated buffers bit for bit: the bytes k2j_set_cupti is tested with everywhere else."""
    from kineto_b200 import api, synth
    trace = synth.gen_kernel_launches(20_000, seed=79, pool_size=500, user_annotations=5)
    raw, keep, _ = helpers.with_raw_kernel_names(trace)
    assert not np.array_equal(raw, trace.cupti)
    names = api.Names()
    pool = trace.pool()
    assert [names.intern(pool[i]) for i in range(len(pool))] == list(range(len(pool)))
    names.intern_kernel_names(raw, trace.buftab)
    assert np.array_equal(raw, trace.cupti)
    off, data = names.pool()
    assert np.array_equal(off, trace.pool_off) and np.array_equal(data, trace.pool_data)
