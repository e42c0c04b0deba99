"""CLI verbs on CPU: make-model -> validate-model -> plan-model -> run-model -> batch."""
import json

from orinfer_b200.cli import build_parser, main


def test_parser_defaults_match_reference_table():
    a = build_parser().parse_args(["serve", "--preset", "tiny"])
    assert a.listen == "[::]:8088" and a.scheduler_policy == "latency"
    assert a.cuda_graph == "decode_only" and a.mtp_drafts == "auto"
    assert (a.prefix_cache_mib, a.kv_offload_mib, a.max_active_requests) == (4096, 0, 32)
    assert (a.prefill_budget_ms, a.target_tpot_ms, a.memory_reserve_mib) == (200.0, 400.0, 1024)
    assert (a.queue_timeout_ms, a.output_timeout_ms, a.drain_timeout_ms) == (0, 60000, 30000)
    assert build_parser().parse_args(["batch", "--preset", "tiny", "--input", "i", "--output",
                                      "o"]).scheduler_policy == "throughput"


def test_model_verbs(tmp_path, capsys):
    d = tmp_path / "m"
    assert main(["make-model", "--preset", "tiny", "--output", str(d)]) == 0
    assert main(["validate-model", str(d)]) == 0
    assert json.loads(capsys.readouterr().out.splitlines()[-1])["ok"]
    assert main(["plan-model", str(d)]) == 0
    plan = json.loads(capsys.readouterr().out)
    assert plan["target"] == "sm_100a" and len(plan["layers"]) == 2
    reqs = tmp_path / "r.json"
    reqs.write_text(json.dumps({"requests": [{"id": "a", "input_tokens": [1, 2, 3, 4],
                                              "max_new_tokens": 3}]}))
    common = ["--device", "cpu", "--max-active-requests", "4", "--prefill-chunk", "64",
              "--max-context", "256"]
    assert main(["run-model", str(d), "--requests", str(reqs)] + common) == 0
    rep = json.loads(capsys.readouterr().out)
    assert len(rep["requests"][0]["tokens"]) == 3 and rep["requests"][0]["prefill_tps"] > 0
    assert main(["score-model", str(d), "--tokens", "1,2,3,4,5"] + common) == 0
    score = json.loads(capsys.readouterr().out)
    assert len(score["probes"]) == 4 and score["nll"] > 0
    src, out = tmp_path / "in.jsonl", tmp_path / "out.jsonl"
    src.write_text(json.dumps({"messages": [{"role": "user", "content": "x"}], "max_tokens": 2,
                               "ignore_eos": True}) + "\n")
    assert main(["batch", str(d), "--input", str(src), "--output", str(out)] + common) == 0
    assert json.loads(out.read_text().splitlines()[0])["response"]["usage"]["completion_tokens"] == 2
    assert main(["validate-model", str(d)]) == 0


def test_validate_nccl_on_cpu_ranks():
    from orinfer_b200.parallel.selftest import main as selftest
    assert selftest(2, use_cuda=False) == 0


def test_models_registry_verbs(tmp_path, capsys):
    from orinfer_b200.cli import main
    model = tmp_path / "m"
    assert main(["make-model", "--preset", "tiny", "--output", str(model)]) == 0
    st = ["--state-dir", str(tmp_path / "state")]
    assert main(["models", *st, "import", "tiny", str(model)]) == 0
    assert main(["models", *st, "cp", "tiny", "tiny2"]) == 0
    capsys.readouterr()
    assert main(["models", *st, "list"]) == 0
    import json
    names = [e["name"] for e in json.loads(capsys.readouterr().out)]
    assert names == ["tiny", "tiny2"]
    assert main(["models", *st, "rm", "tiny"]) == 0
    assert main(["models", *st, "show", "tiny"]) == 2


def test_shipped_examples_run(tmp_path, capsys):
    """The files under examples/ are valid inputs of the verbs they document."""
    import json
    from pathlib import Path
    from orinfer_b200.api.chat_codec import ChatCodec  # noqa: F401  (the request schema lives there)
    from orinfer_b200.cli import main
    root = Path(__file__).resolve().parents[1] / "examples"
    common = ["--device", "cpu", "--cuda-graph", "off", "--prefix-cache-mib", "0"]
    assert main(["run-model", "--preset", "tiny", "--requests", str(root / "requests.json")]
                + common) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert [r["id"] for r in rep["requests"]] == ["short", "two-chunks"]
    assert [len(r["tokens"]) for r in rep["requests"]] == [8, 4]
    out = tmp_path / "out.jsonl"
    assert main(["batch", "--preset", "tiny", "--input", str(root / "batch.jsonl"), "--output",
                 str(out)] + common) == 0
    rows = [json.loads(x) for x in out.read_text().splitlines()]
    assert sorted(r.get("id", r.get("custom_id")) for r in rows) == ["a", "b"]
    body = json.loads((root / "chat-request.json").read_text())
    assert body["tools"][0]["function"]["strict"] and body["stream"]
    json.loads((root / "opencode.json").read_text())
    compile((root / "openai-python.py").read_text(), "openai-python.py", "exec")
