"""CLI verbs that talk to a running manager: ps, load, stop, run, transcribe, logs."""
import io
import json
import socket
import threading
import time
import wave

import pytest

from orinfer_b200 import cli
from orinfer_b200.api import manager as M


@pytest.fixture(scope="module")
def gateway(tmp_path_factory):
    import uvicorn
    from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec
    from orinfer_b200.api.server import Service, create_app
    from orinfer_b200.config import PRESETS, SchedulerOptions
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.models.weights import random_model
    weights = random_model(PRESETS["tiny"], seed=0)

    def start(entry):
        svc = Service(lambda: Engine(weights, sched=SchedulerOptions(max_active=4, prefill_chunk=64),
                                     kv_pages=24, max_context=512),
                      ChatCodec(ByteTokenizer(1024), context=512, model_name=entry.name), entry.name)
        svc.start()
        return M.RunnerHandle(svc, create_app(svc)), weights.nbytes()

    m = M.ModelManager(tmp_path_factory.mktemp("state"), start, lambda h: h.service.stop(1000))
    m.register("tiny", "/models/tiny")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(M.create_gateway_app(m, sweep_s=3600), host="127.0.0.1",
                                           port=port, log_level="error"))
    thread = threading.Thread(target=server.run, daemon=True)
    thread.start()
    for _ in range(200):
        if server.started:
            break
        time.sleep(0.05)
    yield f"http://127.0.0.1:{port}", m
    server.should_exit = True
    thread.join(timeout=10)


def test_load_ps_stop(gateway, capsys):
    url, m = gateway
    assert cli.main(["ps", "--url", url]) == 0
    assert json.loads(capsys.readouterr().out) == []
    assert cli.main(["load", "tiny", "--url", url, "--keep-alive", "30m"]) == 0
    loaded = json.loads(capsys.readouterr().out)
    assert loaded["names"] == ["tiny"] and loaded["keep_alive_s"] == 1800 and loaded["leases"] == 0
    assert cli.main(["ps", "--url", url]) == 0
    assert [x["name"] for x in json.loads(capsys.readouterr().out)] == ["tiny"]
    assert cli.main(["stop", "tiny", "--url", url]) == 0
    assert json.loads(capsys.readouterr().out) == {"model": "tiny", "stopped": True}
    assert cli.main(["stop", "tiny", "--url", url]) == 0
    assert json.loads(capsys.readouterr().out)["stopped"] is False
    assert cli.main(["load", "ghost", "--url", url]) == 2
    assert "ghost" in capsys.readouterr().err
    # a runner with a lease is refused unless forced
    r = m.acquire("tiny")
    with pytest.raises(M.ManagerError, match="in flight"):
        m.unload("tiny")
    assert m.unload("tiny", force=True) is True and m.running() == []
    m.release(r)


def test_run_and_transcribe(gateway, capsys, monkeypatch, tmp_path):
    url, _ = gateway
    params = json.dumps({"max_tokens": 4, "temperature": 0, "ignore_eos": True,
                         "logit_bias": {"104": 100}})
    assert cli.main(["run", "tiny", "say h", "--url", url, "--params", params]) == 0
    assert capsys.readouterr().out == "hhhh\n"
    monkeypatch.setattr("sys.stdin", io.StringIO("from a pipe"))
    assert cli.main(["run", "tiny", "--url", url, "--params", params]) == 0
    assert capsys.readouterr().out == "hhhh\n"
    assert cli.main(["run", "nope", "x", "--url", url]) == 2
    path = tmp_path / "a.wav"
    with wave.open(str(path), "wb") as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(16000)
        w.writeframes(b"\x00\x08" * 16000)
    assert cli.main(["transcribe", "tiny", str(path), "--url", url, "--language", "en",
                     "--max-tokens", "4"]) == 0
    assert capsys.readouterr().out.endswith("\n")
    assert cli.main(["ps", "--url", "http://127.0.0.1:9"]) == 3
