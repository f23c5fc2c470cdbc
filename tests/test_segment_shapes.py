"""tests/golden/segment_shapes.json (made by tests/golden/make_segment_shapes.py from the reference's cell-exact cost model):
the recorded components must add up to the recorded totals, and the numbers the benchmark's decode-step mode quotes must be the
fixture's."""
import json
import os

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def segments():
    return json.load(open(os.path.join(HERE, "golden", "segment_shapes.json")))["segments"]


def test_components_add_up_to_the_recorded_cells(segments):
    assert set(segments) == {"layer_8b_s32_c2048", "head_8b_s32_c2048", "micro_s32_c128"}
    for name, seg in segments.items():
        base = sum(c["repeat"] * (c["base_cols"] << c["log_rows"]) for c in seg["components"])
        inter = sum(c["repeat"] * (c["interaction_cols"] << c["log_rows"]) for c in seg["components"])
        boundary = sum(b["cols"] << b["log_rows"] for b in seg["boundary_cols"])
        assert (base, inter, boundary) == (seg["cells"]["base"], seg["cells"]["interaction"], seg["cells"]["boundary"]), name
        assert base + inter + boundary == seg["cells"]["fresh"], name
        assert all(4 <= c["log_rows"] <= 26 for c in seg["components"]), name


def test_recorded_microbenchmark_total(segments):
    # the reference's recorded run of this segment committed 28,387,616 cells (harness/costmodel/exact_chunks.json, first point)
    assert segments["micro_s32_c128"]["cells"]["fresh"] == 28387616


def test_decode_step_cell_count_matches_the_fixture(segments):
    import re

    src = open(os.path.join(os.path.dirname(HERE), "bench.py")).read()
    m = re.search(r"cells = 32 \* (\d+) \+ (\d+)", src)
    assert m and int(m.group(1)) == segments["layer_8b_s32_c2048"]["cells"]["fresh"]
    assert int(m.group(2)) == segments["head_8b_s32_c2048"]["cells"]["fresh"]
