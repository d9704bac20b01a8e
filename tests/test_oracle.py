"""CPU checks of the oracle itself: the restatement (oracle/k2j_oracle.cpp) against the committed
reference outputs, and — where the reference build is present — against the live reference."""
import os

import pytest

import cases
import helpers
from kineto_b200 import synth
from kineto_b200 import tracefile as tf

GOLDEN = sorted(f[:-5] for f in os.listdir(helpers.GOLDEN) if f.endswith(".k2jt"))


@pytest.mark.parametrize("name", GOLDEN)
def test_port_matches_golden(name):
    path = os.path.join(helpers.GOLDEN, name + ".k2jt")
    want = open(os.path.join(helpers.GOLDEN, name + ".ref.json"), "rb").read()
    got, stats = helpers.run_port(None, path=path)
    assert got == want, helpers.first_diff(want, got)
    assert stats["out_bytes"] == len(want)


@pytest.mark.parametrize("name", GOLDEN)
def test_golden_container_is_reproducible(name):
    """The committed containers are exactly what the seeded generators produce today."""
    gen = dict(cases.CASES, annotations=cases.annotation_trace)[name]
    want = tf.Trace.read(os.path.join(helpers.GOLDEN, name + ".k2jt"))
    got = gen()
    for _, attr, _ in tf._SECTIONS:
        a, b = getattr(want, attr), getattr(got, attr)
        assert a.tobytes() == b.tobytes(), attr


@pytest.mark.skipif(not helpers.have_ref(), reason="reference build (oracle/_ref) not present")
@pytest.mark.parametrize("gen", [
    lambda: synth.gen_generic_kernels(4000, seed=101),
    lambda: synth.gen_kernel_launches(3000, seed=102, pool_size=200, orphan_fraction=0.1),
    lambda: synth.gen_kernel_launches(1500, seed=103, pool_size=80, shard=(1, 3)),
    lambda: synth.gen_mixed(6000, seed=104, pool_size=400, escape_fraction=0.1),
    lambda: cases.tsc_trace(2000),
    cases.edge_trace,
    lambda: cases.edge_trace(flags=1),
    cases.annotation_trace,
    cases.overhead_mix_trace,
    lambda: synth.gen_kernel_launches(4000, seed=105, pool_size=100, user_annotations=25),
    cases.sync_trace,
    cases.sync_mix_trace,
    lambda: cases.sync_mix_trace(5000, seed=44, flags=1),
    lambda: synth.gen_op_tree(3000, seed=106, pool_size=100, n_shapes=64),
    cases.collective_trace,
    lambda: cases.collective_trace(400, seed=52),
    lambda: cases.without_flags(synth.gen_distributed_rank(3000, rank=5, seed=107, pool_size=100)),
    cases.instant_trace,
], ids=["generic", "launches", "shard", "mixed", "tsc", "edge", "edge_annot", "annotations", "overhead_mix", "launches_annot",
        "sync", "sync_mix", "sync_mix_annot", "op_tree", "collectives", "collectives_400", "distributed_rank", "instant"])
def test_port_matches_live_reference(gen):
    trace = gen()
    doc, _ = helpers.run_ref(trace)
    want = helpers.activities_segment(doc)
    got, stats = helpers.run_port(trace)
    assert got == want, helpers.first_diff(want, got)


@pytest.mark.skipif(not helpers.have_ref(), reason="reference build (oracle/_ref) not present")
def test_sort_option_equals_reference_on_presorted_buffers():
    """The reference never sorts; ordering by start timestamp is defined as what the reference writes
    for buffers that were sorted beforehand."""
    trace = synth.gen_kernel_launches(3000, seed=55, pool_size=100)
    got, _ = helpers.run_port(cases.with_flags(trace, tf.FLAG_SORT_BY_START))
    doc, _ = helpers.run_ref(cases.presorted_launches(trace))
    want = helpers.activities_segment(doc)
    assert got == want, helpers.first_diff(want, got)
    plain, _ = helpers.run_port(trace)
    assert plain != got


def test_reference_known_answers_in_port_output():
    """Known-answer strings the reference's own tests pin (libkineto/test/CuptiActivityProfilerTest.cpp:564-582,
    libkineto/test/OutputJsonTest.cpp:145-152, libkineto/test/TypedMetadataTest.cpp:164-178)."""
    b = synth.TraceBuilder()
    t0 = b.t0
    b.op(t0 + 10, t0 + 20, 1, 'op "quoted"', md=[("count", tf.MD_INT64, 5), ("ratio", tf.MD_DOUBLE, 1.5),
                                                 ("big", tf.MD_UINT64, 18446744073709551615)])
    b.runtime(t0 + 30, t0 + 40, 7, cbid=synth.CBID_cudaMemcpy)
    b.memcpy(t0 + 50, t0 + 60, 7, 128, copy_kind=1, src_kind=2, dst_kind=3)
    b.kernel(t0 + 70, t0 + 80, 8, "kernel")
    out, _ = helpers.run_port(b.build())
    assert b'"name": "op \\"quoted\\""' in out
    assert b'"count": 5' in out and b'"ratio": 1.5' in out and b'"big": 18446744073709551615' in out
    assert b'"name": "Memcpy HtoD (Pinned -> Device)"' in out
    assert b'"name": "cudaMemcpy"' in out
    assert b'"name": "Kernel"' in out


def test_reference_sync_known_answers_in_port_output():
    """The out-of-order case of the reference's own test (libkineto/test/CuptiActivityProfilerTest.cpp:660-740):
    a stream-wait event and an event sync come before the CUDA event record and the kernel they refer to; both
    must name the record's correlation id and stream, and the wait event shows because its stream has a kernel."""
    b = synth.TraceBuilder(n_devices=4)
    t0 = b.t0
    for name, s, e, i in [("op1", 10, 50, 1), ("op_record", 60, 80, 100), ("op_wait", 90, 110, 200), ("op_evt_sync", 120, 140, 300)]:
        b.op(t0 + s, t0 + e, i, name)
    b.runtime(t0 + 10, t0 + 20, 1)
    b.sync(t0 + 100, t0 + 110, 200, type=tf.SYNC_TYPE_STREAM_WAIT_EVENT, context=7, stream=13, event=7777)
    b.sync(t0 + 120, t0 + 140, 300, type=tf.SYNC_TYPE_EVENT_SYNCHRONIZE, context=7, stream=0xFFFFFFFF, event=7777)
    b.cuda_event(t0 + 25, 100, event=7777, context=7, stream=11)
    b.kernel(t0 + 30, t0 + 50, 1, "k", device=3, context=7, stream=13)
    out, _ = helpers.run_port(b.build())
    want = b'"wait_on_stream": 11, "wait_on_cuda_event_record_corr_id": 100, "wait_on_cuda_event_id": 7777'
    assert out.count(b'"cuda_sync_kind": "Stream Wait Event", ' + want) == 1
    assert out.count(b'"cuda_sync_kind": "Event Sync", ' + want) == 1
    assert out.rfind(b'"name": "Stream Wait Event"') > out.rfind(b'"cat": "kernel"')   # deferred to the end of the pass


def test_port_double_formatting_known_answers():
    for v, s in [(2.0, "2"), (1e16, "1e+16"), (1e-5, "1e-05"), (174.76266666666666, "174.76266666666666"),
                 (1.5, "1.5"), (0.1, "0.1"), (1e15, "1000000000000000"), (1e-4, "0.0001"), (123456.789, "123456.789"),
                 (5e-324, "5e-324"), (1.7976931348623157e308, "1.7976931348623157e+308"), (-0.0, "-0")]:
        assert helpers.port_fmt_double(v) == s
