"""Route-trace lines follow the reference's SP_MOE_TRACE_FILE format
(src/backends/cuda/cuda_forward.cu:8561-8588): R <fwd> <P|D> <L> <t> <us> e:w:h,..."""
import os
import re
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kairos_engine_b200 import trace  # noqa: E402


def test_line_format_and_phase():
    sel = np.array([[[5, 1, 9]], [[2, 0, 7]]], np.int32)          # 2 layers, 1 token, NU = 3
    wts = np.array([[[0.5, 0.3, 0.2]], [[0.4, 0.35, 0.25]]], np.float32)
    lines = trace.format_lines(7, sel, wts, layer_first=3, us=1234)
    assert lines == ["R 7 D 3 0 1234 5:0.5000:1,1:0.3000:1,9:0.2000:1", "R 7 D 4 0 1234 2:0.4000:1,0:0.3500:1,7:0.2500:1"]
    batched = trace.format_lines(1, np.repeat(sel, 2, axis=1), np.repeat(wts, 2, axis=1), 0, 5)
    assert len(batched) == 4 and all(l.split()[2] == "P" for l in batched)
    pat = re.compile(r"^R \d+ [PD] \d+ \d+ \d+ (\d+:\d\.\d{4}:-?[01],?)+$")
    assert all(pat.match(l) for l in lines + batched)


def test_file_trace_counts_forwards(tmp_path):
    f = tmp_path / "route.txt"
    tr = trace.RouteTrace({"SP_MOE_TRACE": "1", "SP_MOE_TRACE_FILE": str(f)})
    sel = np.zeros((1, 1, 2), np.int32); wts = np.full((1, 1, 2), 0.5, np.float32)
    tr.record(sel, wts); tr.record(sel, wts)
    tr.close()
    rows = f.read_text().strip().split("\n")
    assert [r.split()[1] for r in rows] == ["1", "2"]
    off = trace.RouteTrace({})
    off.record(sel, wts)            # not armed: nothing happens
    assert not off.on
