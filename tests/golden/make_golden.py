"""Regenerates the golden fixtures: for every named case in tests/cases.py the synthetic trace
container (<case>.k2jt) and the activities text the UNMODIFIED reference produced for it
(<case>.ref.json, cut out of the reference's trace file by tests/helpers.activities_segment).

Needs the reference build (make -C oracle ref).  Run from the repository root:
    python tests/golden/make_golden.py
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import cases  # noqa: E402
import helpers  # noqa: E402


def main():
    assert helpers.have_ref(), "build the reference first: make -C oracle ref"
    for name, gen in list(cases.CASES.items()) + [("annotations", cases.annotation_trace)]:
        trace = gen()
        trace.write(os.path.join(HERE, name + ".k2jt"))
        doc, _ = helpers.run_ref(trace)
        seg = helpers.activities_segment(doc)
        open(os.path.join(HERE, name + ".ref.json"), "wb").write(seg)
        print(name, len(seg), "bytes")


if __name__ == "__main__":
    main()
