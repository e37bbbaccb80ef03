"""Stage timer, metrics structs, memory monitor and the offline benchmark's report."""
import json
import os
import time

from tensorrt_edge_llm_b200 import profiling as prof
from tensorrt_edge_llm_b200.benchmarks import llm_bench


def test_stage_timer_and_switch():
    t = prof.StageTimer()
    prof.set_profiling_enabled(False)
    with t.stage("A"):
        pass
    assert t.samples() == []
    prof.set_profiling_enabled(True)
    try:
        for _ in range(3):
            with t.stage("A", batch=2, tokens=10):
                time.sleep(0.002)
        h = t.begin("B")
        t.end(h)
        s = t.summary()
        assert s["A"]["count"] == 3 and s["A"]["tokens"] == 30 and s["A"]["total_ms"] >= 5.0 and s["B"]["count"] == 1
        assert "A" in t.format() and prof.timer() is prof.timer()
        t.reset()
        assert t.samples() == []
    finally:
        prof.set_profiling_enabled(False)
    m = prof.SpecDecodeMetrics(rounds=2, acceptance_lengths=[3, 4])
    assert prof.metrics_dict(m)["mean_acceptance_length"] == 3.5
    assert prof.PrefillMetrics(computed_tokens=100, time_ms=50.0).tokens_per_second == 2000.0


def test_memory_monitor_with_a_scripted_probe():
    vals = iter([10, 50, 30] + [20] * 1000)
    mon = prof.MemoryMonitor(interval_s=0.001, probe=lambda: next(vals))
    with mon:
        time.sleep(0.05)
    assert mon.peak_bytes == 50 and mon.samples >= 3


def test_llm_bench_report(tmp_path):
    out = str(tmp_path / "rep")
    assert llm_bench.main(["--shape", "tiny", "--layers", "2", "--dtype", "float32", "--input-len", "24", "--batch-size", "2", "--osl", "5",
                           "--warmup", "1", "--iterations", "2", "--device", "cpu", "--output-dir", out]) == 0
    rep = json.load(open(os.path.join(out, "report.json")))
    assert rep["schema_version"] == 2 and rep["status"] == "complete" and len(rep["samples"]) == 2
    assert rep["samples"][0]["output_tokens"] == 10 and rep["statistics"]["total_ms"]["count"] == 2
    assert "LLM_PREFILL" in rep["samples"][0]["stages"] and "VANILLA_DECODING" in rep["samples"][0]["stages"]
    assert len(rep["fingerprints"]["output_tokens"]) == 16
    assert llm_bench.summarize([3.0, 1.0, 2.0, 4.0])["median"] == 3.0          # upper median
    assert llm_bench.fnv1a64(b"") == "cbf29ce484222325"
