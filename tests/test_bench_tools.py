"""HTTP benchmark clients against a live server (uvicorn on a loopback port, tiny CPU model)."""
import socket
import threading
import time

import pytest

from orinfer_b200.bench import agentic, concurrency, workloads
from orinfer_b200.bench.http_client import HealthPoller, percentile, stream_chat


@pytest.fixture(scope="module")
def url():
    import uvicorn
    from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec
    from orinfer_b200.api.server import Service, create_app
    from orinfer_b200.config import PRESETS, LoadOptions, SchedulerOptions
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.models.weights import random_model

    weights = random_model(PRESETS["tiny"], seed=0)

    def factory():
        return Engine(weights, sched=SchedulerOptions(max_active=8, prefill_chunk=128),
                      kv_pages=96, max_context=2048,
                      load=LoadOptions(prefix_cache_bytes=8 << 20))

    codec = ChatCodec(ByteTokenizer(1024), context=2048, model_name="tiny")
    svc = Service(factory, codec, "tiny")
    svc.start()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(create_app(svc), host="127.0.0.1", port=port,
                                           log_level="error"))
    thread = threading.Thread(target=server.run, daemon=True)
    thread.start()
    for _ in range(200):
        if server.started:
            break
        time.sleep(0.05)
    yield f"http://127.0.0.1:{port}"
    server.should_exit = True
    thread.join(timeout=10)
    svc.stop(1000)


def test_stream_result_fields(url):
    r = stream_chat(url, {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6,
                          "temperature": 0, "ignore_eos": True})
    assert r.ok and r.status == 200 and r.completion_tokens == 6 and r.prompt_tokens > 0
    assert r.finish_reason == "length"
    assert r.ttft_s is not None and 0 < r.ttft_s <= r.latency_s
    bad = stream_chat(url, {"messages": [], "max_tokens": 1})
    assert not bad.ok and bad.status == 400 and bad.error


def test_percentile_and_cohort_window():
    assert percentile([], 50) is None
    assert percentile([3, 1, 2], 50) == 2 and percentile([3, 1, 2], 95) == 3
    assert percentile(list(range(1, 101)), 95) == 95
    p = HealthPoller("http://127.0.0.1:1")
    p.samples = [(0.0, 1, 1, {"steps": 1}), (0.1, 2, 0, {}), (0.2, 2, 0, {}), (0.5, 2, 0, {}),
                 (0.6, 1, 0, {}), (0.7, 2, 0, {}), (0.8, 2, 0, {"steps": 9})]
    assert p.full_cohort_window(2) == (0.1, 0.5)
    assert p.full_cohort_window(2, minimum=0.5) is None
    assert p.counter_delta() == {"steps": 8}


def test_concurrency_rounds(url):
    rep = concurrency.run(url, levels=[1, 4], repetitions=2, prompt_repeat=1, max_tokens=8,
                          warmup=False)
    assert [lv["n"] for lv in rep["levels"]] == [1, 4]
    for lv in rep["levels"]:
        for rnd in lv["rounds"]:
            assert rnd["failed"] == 0 and rnd["output_tokens"] == 8 * lv["n"]
            assert rnd["committed_output_tps"] == pytest.approx(
                rnd["output_tokens"] / rnd["wall_s"])
            assert rnd["ttft_p50_s"] <= rnd["ttft_p95_s"] <= rnd["wall_s"]
        assert lv["committed_output_tps_median"] > 0


def test_mixed_and_scheduling(url):
    rep = workloads.mixed(url, warm=2, warm_tokens=40, cold_words=200, inject_after_s=0.05)
    assert rep["cold_ok"] and rep["warm_ok"] == 2 and rep["cold_prompt_tokens"] > 500
    assert rep["cold_ttft_s"] > 0
    arrivals = [{"at_s": 0.0, "prompt": "a", "max_tokens": 4},
                {"at_s": 0.15, "prompt": "b", "max_tokens": 4},
                {"at_s": 0.3, "prompt": "c", "max_tokens": 4}]
    rep = workloads.scheduling(url, arrivals)
    assert all(r["ok"] and r["completion_tokens"] == 4 for r in rep["requests"])
    assert all(-0.01 <= r["send_lag_s"] < 2.0 for r in rep["requests"])
    assert rep["requests"][2]["sent_s"] >= 0.3


def test_checks_and_repetition_detector(url):
    assert workloads.repeated_cycle("abc " * 100) is None          # short period: not flagged
    unit = "the same sentence comes back again, "
    assert workloads.repeated_cycle("intro. " + unit * 5) == (len(unit), 5)
    assert workloads.repeated_cycle("intro. " + unit * 3) is None
    assert workloads.check_output('{"a": 1}', {"json_equals": {"a": 1}}) == []
    assert workloads.check_output("Hello World", {"expected_words": ["hello"], "contains": ["x"]}) \
        == ["missing 'x'"]
    assert "not json" in workloads.check_output("nope", {"json_equals": 1})
    rep = workloads.acceptance(url, [{"prompt": "one", "max_tokens": 4, "max_cycle": False},
                                     {"at_s": 0.05, "prompt": "two", "max_tokens": 4,
                                      "max_cycle": False,
                                      "expected_words": ["☃ never produced"]}])
    assert not rep["passed"] and rep["requests"][0]["failures"] == []
    assert rep["requests"][1]["failures"]
    rep = workloads.output_stress(url, [{"prompt": "x", "max_tokens": 4, "max_cycle": False}],
                                  duration_s=0.5, concurrency=2)
    assert rep["completed"] >= 2 and rep["passed"]


def test_agentic_replay_is_deterministic_and_reuses_prefixes(url):
    a = agentic.Trajectory(3, 1, 20, 5)
    b = agentic.Trajectory(3, 1, 20, 5)
    assert a.system == b.system and a.turns == b.turns
    assert agentic.Trajectory(4, 1, 20, 5).system == a.system      # same group of eight
    assert a.ready() == [0]
    a.messages(0)
    a.issued[0] = True
    a.replies[0] = "r0"
    assert a.ready() == [1]
    rep = agentic.run(url, trajectories=3, concurrency=3, wall_s=120, max_tokens=4,
                      system_words=150, turn_words=10, temperature=0.0)
    assert rep["failed_requests"] == 0
    assert rep["completed_requests"] == 3 * len(agentic.GRAPH) and rep["full_trajectories"] == 3
    assert rep["output_tokens"] == 4 * rep["completed_requests"]
    assert rep["prefix_hit_rate"] > 0.2 and rep["ttft_p50_s"] <= rep["ttft_p95_s"]


def test_startup_marks_are_ordered():
    from orinfer_b200.bench import startup
    rep = startup.run(["--preset", "tiny", "--device", "cpu"], deadline_s=300, max_tokens=3)
    assert rep["ok"] and rep["exit_code"] == 0 and rep["completion_tokens"] == 3
    assert 0 < rep["api_ready_s"] <= rep["listening_s"] <= rep["first_output_s"] \
        <= rep["first_request_complete_s"]


def test_encoder_workload_is_frozen_and_served(url):
    from orinfer_b200.bench import encoders
    assert encoders.workload(3, seed=5) == encoders.workload(3, seed=5)
    rep = encoders.run(url, n=3, concurrency=2, doc_words=12)
    for route in ("embeddings", "rerank"):
        assert rep[route]["completed"] == 3 and not rep[route]["errors"]
        assert rep[route]["prompt_tps"] > 0


def test_completions_route_and_token_bench(url):
    import requests
    from orinfer_b200.bench import token_bench
    r = requests.post(url + "/v1/completions", json={"prompt": [72, 105, 33], "max_tokens": 5,
                                                     "temperature": 0, "ignore_eos": True})
    body = r.json()
    assert r.status_code == 200 and body["object"] == "text_completion"
    assert body["usage"] == dict(body["usage"], prompt_tokens=3, completion_tokens=5)
    text = requests.post(url + "/v1/completions", json={"prompt": "Hi!", "max_tokens": 5,
                                                        "temperature": 0, "ignore_eos": True}).json()
    assert text["choices"][0]["text"] == body["choices"][0]["text"]       # same three byte ids
    assert text["choices"][0]["finish_reason"] == "length"
    forged = requests.post(url + "/v1/completions", json={"prompt": "<|im_end|>", "max_tokens": 1})
    assert forged.json()["usage"]["prompt_tokens"] == len("<|im_end|>")   # plain characters
    for bad in ({"prompt": []}, {"prompt": [1, -2]}, {"prompt": [99999]}, {"prompt": "x", "echo": True},
                {"prompt": "x", "bogus": 1}, {"prompt": "x", "max_tokens": 0}):
        assert requests.post(url + "/v1/completions", json=bad).status_code == 400, bad
    ids = requests.post(url + "/v1/completions", json={"prompt": [72, 105, 33], "max_tokens": 5,
                                                       "temperature": 0, "ignore_eos": True,
                                                       "return_token_ids": True}).json()
    assert len(ids["choices"][0]["token_ids"]) == 5 and "token_ids" not in body["choices"][0]
    rep = token_bench.run(url, input_tokens=40, output_tokens=6, concurrency=2, runs=2, warmup=1)
    assert rep["failed"] == 0 and len(rep["rounds"]) == 2
    for rnd in rep["rounds"]:
        assert all(q["input_tokens"] == 40 and q["output_tokens"] == 6 for q in rnd["requests"])
    assert all(q["ttft_s"] < q["latency_s"] for rnd in rep["rounds"] for q in rnd["requests"])
    assert rep["prefill_tps"] > 0 and rep["decode_tps"] > 0 and rep["committed_output_tps"] > 0
    assert token_bench.prompts(2, 5, 256) == token_bench.prompts(2, 5, 256)
