"""Managed runners as child processes behind the gateway (CPU runner, tiny checkpoint)."""
import json

import pytest
import torch
from fastapi.testclient import TestClient

from orinfer_b200.api import manager as M
from orinfer_b200.api.child_runner import ChildRunner, ProxyApp, RunnerStartError, weight_bytes


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    from orinfer_b200.config import PRESETS
    from orinfer_b200.engine.checkpoint import save_model
    from orinfer_b200.models.weights import random_model
    path = tmp_path_factory.mktemp("tiny-model")
    save_model(random_model(PRESETS["tiny"], seed=0), path)
    return path


def test_gateway_streams_through_a_child_process(model_dir, tmp_path):
    started, stopped = [], []

    def start(entry):
        child = ChildRunner(entry.path, entry.name, ["--device", "cpu", "--max-context", "512"],
                            start_timeout_s=300).start()
        started.append(child)
        return M.RunnerHandle(child, ProxyApp(child.base_url)), weight_bytes(entry.path)

    def stop(handle):
        handle.service.stop(30)
        stopped.append(handle.service.name)

    assert weight_bytes(model_dir) > 100_000
    m = M.ModelManager(tmp_path, start, stop)
    m.register("tiny", str(model_dir))
    with TestClient(M.create_gateway_app(m, sweep_s=3600)) as c:
        body = {"model": "tiny", "messages": [{"role": "user", "content": "hi"}],
                "max_tokens": 4, "temperature": 0, "ignore_eos": True}
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 200, r.text
        assert r.json()["usage"]["completion_tokens"] == 4 and r.json()["model"] == "tiny"
        with c.stream("POST", "/v1/chat/completions",
                      json=dict(body, stream=True, stream_options={"include_usage": True})) as s:
            assert s.headers["content-type"].startswith("text/event-stream")
            lines = [l for l in s.iter_lines() if l.startswith("data: ")]
        assert lines[-1] == "data: [DONE]"
        assert json.loads(lines[-2][6:])["usage"]["completion_tokens"] == 4
        bad = c.post("/v1/chat/completions", json=dict(body, bogus=1))
        assert bad.status_code == 400 and bad.json()["error"]["param"] == "bogus"   # relayed as is
        assert len(started) == 1 and started[0].alive() and m.running()[0]["leases"] == 0
        lines = c.get("/api/logs", params={"model": "tiny"}).json()["lines"]
        assert any(l.startswith("API READY") for l in lines)
        assert any(l.startswith("MODEL READY") for l in lines)
        assert c.get("/api/logs", params={"model": "ghost"}).status_code == 404
        # a runner that died is noticed by the next request and started again
        started[0].stop(30)
        back = c.post("/v1/chat/completions", json=body)
        assert back.status_code == 200 and back.json()["usage"]["completion_tokens"] == 4
        assert len(started) == 2 and m.restarts == 1 and started[1].alive()
        # one that dies between the liveness check and the relay answers 502 in the OpenAI
        # error shape, and the gateway stays up
        m._alive = lambda service: True
        started[1].stop(30)
        dead = c.post("/v1/chat/completions", json=body)
        assert dead.status_code == 502 and dead.json()["error"]["code"] == "runner_unavailable"
        assert c.get("/health").status_code == 200
    assert stopped.count("tiny") == 2 and not started[0].alive() and not started[1].alive()


def test_child_that_cannot_start_reports_its_stderr(tmp_path):
    with pytest.raises(RunnerStartError, match="exited with code"):
        ChildRunner(str(tmp_path / "missing"), "ghost", ["--device", "cpu"],
                    start_timeout_s=120).start()


def test_serve_listens_while_the_model_loads():
    """`serve` accepts connections before the weights are ready: /health says `starting`
    (503), requests are refused with 503, then the same listener turns ready."""
    import signal
    import socket
    import subprocess
    import sys
    import time

    import requests
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    proc = subprocess.Popen([sys.executable, "-m", "orinfer_b200", "serve", "--preset", "tiny",
                             "--device", "cpu", "--listen", f"127.0.0.1:{port}"],
                            stderr=subprocess.DEVNULL, start_new_session=True)
    url = f"http://127.0.0.1:{port}"
    seen, refused = [], None
    try:
        deadline = time.time() + 240
        while time.time() < deadline:
            try:
                r = requests.get(url + "/health", timeout=2)
            except requests.RequestException:
                time.sleep(0.05)
                continue
            seen.append((r.status_code, r.json()["status"]))
            if r.status_code == 200:
                break
            if refused is None:
                refused = requests.post(url + "/v1/chat/completions", timeout=5, json={
                    "messages": [{"role": "user", "content": "x"}]})
            time.sleep(0.1)
        assert seen[0] == (503, "starting") and seen[-1] == (200, "ready")
        assert refused is not None and refused.status_code == 503
        assert refused.json()["error"]["code"] == "not_ready"
    finally:
        proc.send_signal(signal.SIGTERM)
        assert proc.wait(timeout=60) == 0
