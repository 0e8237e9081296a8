"""Timeline arithmetic of benchmarks/step_profile.py on a hand-made trace."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load():
    spec = importlib.util.spec_from_file_location("step_profile", os.path.join(ROOT, "benchmarks", "step_profile.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_union_busy_time_gaps_and_ranking():
    sp = _load()
    k = lambda name, ts, dur, stream, cat="kernel": {"ph": "X", "cat": cat, "name": name, "ts": ts,  # noqa: E731
                                                     "dur": dur, "args": {"stream": stream}}
    events = [
        k("gemm", 1000, 400, 7),                 # [1000, 1400)
        k("copy", 1200, 500, 9, "gpu_memcpy"),   # overlaps the gemm: union [1000, 1700)
        k("gemm", 1800, 400, 7),                 # gap of 100 us, then [1800, 2200)
        k("norm", 2200, 50, 7),                  # back to back: no gap
        k("adam", 2300, 100, 11),                # gap of 50 us
        {"ph": "X", "cat": "cpu_op", "name": "aten::mm", "ts": 0, "dur": 5000},      # not device work
        {"ph": "i", "cat": "kernel", "name": "marker", "ts": 10},
    ]
    s = sp.summarize_trace(events, top=2, gaps=5)
    assert s["kernels"] == 5
    assert abs(s["span_ms"] - 1.4) < 1e-9                      # 1000 .. 2400 us
    assert abs(s["busy_union_ms"] - 1.25) < 1e-9               # 700 + 450 + 100
    assert abs(s["idle_ms"] - 0.15) < 1e-9
    assert s["busiest_stream"] == "7" and abs(s["per_stream_busy_ms"]["7"] - 0.85) < 1e-9
    assert [t["name"] for t in s["top_kernels"]] == ["gemm", "copy"]
    assert s["top_kernels"][0]["count"] == 2 and abs(s["top_kernels"][0]["mean_us"] - 400) < 1e-9
    gaps = s["idle_gaps"]
    assert [g["gap_us"] for g in gaps] == [100, 50]
    assert gaps[0]["after"] == "copy" and gaps[0]["before"] == "gemm"
    assert gaps[1]["after"] == "norm" and gaps[1]["before"] == "adam"
    assert abs(s["idle_in_gaps_over_50us_ms"] - 0.1) < 1e-9
    # the first gemm shares the GPU with the copy for half of its time, the second runs alone
    g = s["top_kernels"][0]
    assert (g["alone"], g["shared"]) == (1, 1) and g["alone_median_us"] == 400 and g["shared_median_us"] == 400
    c = s["top_kernels"][1]
    assert (c["alone"], c["shared"]) == (0, 1) and c["alone_median_us"] is None
    text = sp.format_summary(s)
    assert "alone x1" in text and "shared x1" in text
    assert "idle 0.1" in text or "idle 0.2" in text
    assert sp.summarize_trace([]) == {"kernels": 0}
    assert "no device activity" in sp.format_summary({"kernels": 0})
