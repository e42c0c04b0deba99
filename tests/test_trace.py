"""Tracing hooks, exit telemetry and the profiler-CSV summariser."""
import json
import types

import pytest
import torch

from orinfer_b200.utils import ncu_summary, trace

HEADER = ['ID', 'Process ID', 'Kernel Name', 'Block Size',
          'FBSP.TriageCompute.dram__bytes_read.sum', 'dram__bytes_write.sum',
          'gpu__time_duration.sum', 'gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed',
          'sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active',
          'sm__warps_active.avg.pct_of_peak_sustained_active', 'launch__registers_per_thread',
          'launch__grid_size', 'launch__block_size',
          'smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio',
          'smsp__average_warps_issue_stalled_barrier_per_issue_active.ratio',
          'smsp__average_warps_issue_stalled_wait_per_issue_active.ratio',
          'smsp__average_warps_issue_stalled_barrier_not_issued_per_issue_active.ratio']
UNITS = ['', '', '', '', 'Mbyte', 'Kbyte', 'ms', '%', '%', '%', 'register/thread', '', '',
         '', '', '', '']


def _csv(rows):
    q = lambda cells: ",".join('"%s"' % c for c in cells)
    return "\n".join(["==PROF== banner line", q(HEADER), q(UNITS)] + [q(r) for r in rows]) + "\n"


def test_ncu_summary_reads_counters_units_and_stalls():
    text = _csv([['0', '7', 'void qgemm_tc_kernel<1, 0, 4, 128>(Params)', '(576, 1, 1)',
                  '40.5', '2,000', '0.25', '61.5', '30.5', '28', '66', '608', '576',
                  '3.5', '0.25', '1.25', '9.0']])
    (l,) = ncu_summary.parse(text)
    assert l.kernel.startswith("void qgemm_tc_kernel")
    assert l.values["dram_read_mb"] == pytest.approx(40.5)
    assert l.values["dram_write_mb"] == pytest.approx(2.0)          # 2,000 Kbyte
    assert l.values["duration_us"] == pytest.approx(250.0)          # 0.25 ms
    assert l.values["registers"] == 66 and l.values["tensor_pct"] == 30.5
    assert l.top_stalls(2) == ["long_scoreboard 3.50", "wait 1.25"]  # *_not_issued is ignored
    md = ncu_summary.render([l], flops=2.0 * 2048 * 19456 * 2560, nbytes=0.0,
                            peaks=(6.5e12, 1.6e15, "test"))
    row = md.splitlines()[2]
    assert "qgemm_tc_kernel<1, 0, 4, 128>" in row and "| 608 x 576 |" in row
    assert "| 250.0 |" in row and "| 42.5 |" in row
    tflops = 2.0 * 2048 * 19456 * 2560 / 250e-6 / 1e12
    assert f"| {tflops:.1f} |" in row and f"| {tflops / 1600:.2f} |" in row


def test_ncu_summary_refuses_other_pages():
    with pytest.raises(ValueError):
        ncu_summary.parse('"a","b"\n"1","2"\n"3","4"\n')
    with pytest.raises(ValueError):
        ncu_summary.parse("")


def test_trace_lines_follow_the_topic_list(monkeypatch, capsys):
    monkeypatch.delenv("ORINFER_TRACE", raising=False)
    trace.line("admit", rid=1)
    assert capsys.readouterr().err == ""
    monkeypatch.setenv("ORINFER_TRACE", "admit, layered")
    trace.line("admit", rid=1, prompt=5)
    trace.line("prefill_choose", x=1)
    err = capsys.readouterr().err.strip().splitlines()
    assert err == ['ADMIT {"prompt": 5, "rid": 1}']
    monkeypatch.setenv("ORINFER_TRACE", "all")
    assert trace.enabled("prefill_choose")


def test_spans_are_free_when_off_and_totals_rank_by_time(monkeypatch):
    monkeypatch.delenv("ORINFER_NVTX", raising=False)
    monkeypatch.delenv("ORINFER_SPAN_PROFILE", raising=False)
    assert trace.span("x") is trace.span("y")            # shared null context
    trace.report(reset=True)
    trace.add("ffn", 3.0, count=2)
    trace.add("attn", 1.0)
    rep = trace.report(reset=True)
    assert list(rep) == ["ffn", "attn"]
    assert rep["ffn"] == {"count": 2, "total_ms": 3.0, "mean_us": 1500.0, "share": 0.75}
    assert trace.report() == {}


def test_engine_traces_and_exit_report(monkeypatch, capsys):
    from orinfer_b200.api.worker import EngineWorker
    from orinfer_b200.config import PRESETS, SchedulerOptions
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.models.weights import random_model
    monkeypatch.setenv("ORINFER_TRACE", "admit,prefill_choose")
    eng = Engine(random_model(PRESETS["tiny"], seed=0), kv_pages=8, max_context=256,
                 sched=SchedulerOptions(max_active=2, prefill_chunk=16))
    eng.generate([[1, 2, 3, 4, 5] * 5], max_new=2)
    err = capsys.readouterr().err.splitlines()
    admits = [json.loads(l.split(" ", 1)[1]) for l in err if l.startswith("ADMIT ")]
    chooses = [json.loads(l.split(" ", 1)[1]) for l in err if l.startswith("PREFILL_CHOOSE ")]
    assert admits[0]["prompt"] == 25 and admits[0]["cached"] == 0
    assert [c["chunks"][0][1:] for c in chooses] == [[0, 16], [16, 9]]
    EngineWorker._exit_report(types.SimpleNamespace(engine=eng))
    (sched,) = [l for l in capsys.readouterr().err.splitlines() if l.startswith("SCHEDULER ")]
    body = json.loads(sched.split(" ", 1)[1])
    assert body["engine"]["finished"] == 1 and "speculation" in body


@pytest.mark.gpu
def test_span_profile_times_layer_blocks_on_the_device(cuda, monkeypatch):
    from orinfer_b200.config import PRESETS
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.config import GraphMode, LoadOptions
    from orinfer_b200.models.weights import random_model
    monkeypatch.setenv("ORINFER_SPAN_PROFILE", "1")
    monkeypatch.setenv("ORINFER_NVTX", "1")
    trace.report(reset=True)
    eng = Engine(random_model(PRESETS["tiny"], seed=0).to(cuda), kv_pages=8, max_context=256,
                 load=LoadOptions(cuda_graph=GraphMode.OFF))
    eng.generate([[1, 2, 3, 4, 5] * 5], max_new=3)
    rep = trace.report(reset=True)
    layers = PRESETS["tiny"].layers
    assert rep["attn"]["count"] == rep["ffn"]["count"] == 3 * layers
    assert rep["attn"]["total_ms"] > 0 and abs(sum(v["share"] for v in rep.values()) - 1) < 1e-3
