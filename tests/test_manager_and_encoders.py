"""Model manager semantics (registry, aliases, leases, budget eviction, keep-alive, negative
cache) with fake runners, and the embeddings / rerank endpoints on the tiny CPU model."""
import base64
import struct

import pytest
from fastapi import FastAPI
from fastapi.testclient import TestClient

from orinfer_b200.api import manager as M


class Clock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        return self.t


def _manager(tmp_path, budget=0, fail=()):
    started, stopped, clock = [], [], Clock()

    def start(entry):
        if entry.name in fail:
            raise RuntimeError("boom")
        started.append(entry.name)
        return f"svc:{entry.path}", 100

    m = M.ModelManager(tmp_path, start, stopped.append, budget, clock)
    return m, started, stopped, clock


def test_aliases_share_a_runner_and_registry_persists(tmp_path):
    m, started, stopped, _ = _manager(tmp_path)
    m.register("a", "/models/a", options={"tp": 2}, defaults={"temperature": 0.2})
    m.copy("a", "a-alias")
    m.register("a-fast", "/models/a", options={"tp": 4})          # different runner key
    r1, r2, r3 = m.acquire("a"), m.acquire("a-alias"), m.acquire("a-fast")
    assert r1 is r2 and r3 is not r1 and started == ["a", "a-fast"] and r1.leases == 2
    again = M.ModelManager(tmp_path, lambda e: ("x", 1), lambda s: None)
    assert [e.name for e in again.list()] == ["a", "a-alias", "a-fast"]
    assert again.show("a-alias").options == {"tp": 2}
    with pytest.raises(M.ManagerError):
        m.copy("missing", "x")
    m.release(r1); m.release(r2)
    m.remove("a")
    assert stopped == []                                          # alias still needs the runner
    m.remove("a-alias")
    assert stopped == ["svc:/models/a"]


def test_budget_evicts_idle_lru_and_refuses_when_all_in_use(tmp_path):
    m, started, stopped, clock = _manager(tmp_path, budget=250)
    for n in "abc":
        m.register(n, f"/models/{n}")
    ra = m.acquire("a"); clock.t = 1
    rb = m.acquire("b"); clock.t = 2
    with pytest.raises(M.ManagerError) as err:
        m.acquire("c")                                            # 300 > 250, nothing idle
    assert err.value.status == 503
    assert stopped == ["svc:/models/c"]                           # what did not fit was stopped again
    m.release(ra); clock.t = 3
    m.acquire("c")
    assert stopped[1:] == ["svc:/models/a"] and {r["names"][0] for r in m.running()} == {"b", "c"}
    m.release(rb)


def test_lifecycle_under_pressure_failures_and_dead_runners(tmp_path):
    """Room is made before a sized model starts; a request waits for capacity and a waiter
    that left is never loaded; concurrent requests share one start and one failure, and a
    later retry recovers; a runner that died is started again by the next request; memory
    pressure ignores a keep-alive of forever."""
    import threading
    import time
    starts, stopped, alive = [], [], {}
    fail = {"on": False}

    def start(entry):
        starts.append(entry.name)
        time.sleep(0.05)
        if fail["on"]:
            raise RuntimeError("boom")
        svc = f"svc:{entry.name}:{len(starts)}"
        alive[svc] = True
        return svc, 100

    m = M.ModelManager(tmp_path, start, stopped.append, 250, estimate=lambda e: 100,
                       alive=lambda s: alive.get(s, False), capacity_wait_s=2.0)
    for n in "abc":
        m.register(n, f"/models/{n}")
    ra, rb = m.acquire("a", keep_alive_s=-1), m.acquire("b", keep_alive_s=-1)
    # c waits for capacity; it is loaded once a lease comes back, evicting the idle model
    got = {}
    waiter = threading.Thread(target=lambda: got.setdefault("c", m.acquire("c")))
    waiter.start()
    time.sleep(0.2)
    assert starts == ["a", "b"] and waiter.is_alive()            # sized first: not started yet
    m.release(ra)
    waiter.join(5)
    assert got["c"].leases == 1 and stopped == ["svc:a:1"] and starts == ["a", "b", "c"]
    # a waiter whose client left is not loaded when space appears
    left = {"flag": False}
    err = {}

    def leaver():
        try:
            m.acquire("a", cancelled=lambda: left["flag"])
        except M.ManagerError as e:
            err["e"] = e
    t = threading.Thread(target=leaver)
    t.start()
    time.sleep(0.2)
    left["flag"] = True
    t.join(5)
    assert err["e"].status == 499 and starts == ["a", "b", "c"]
    m.release(rb); m.release(got["c"])
    # two requests for a model that cannot start share one attempt and one failure
    fail["on"] = True
    errors = []

    def want_a():
        try:
            m.acquire("a")
        except M.ManagerError as e:
            errors.append(e.status)
    pair = [threading.Thread(target=want_a) for _ in range(2)]
    [p.start() for p in pair]
    [p.join(5) for p in pair]
    assert errors == [503, 503] and starts.count("a") == 2        # the first load and this one
    fail["on"] = False
    m._failed.clear()                                             # the negative cache ran out
    ra = m.acquire("a")
    assert ra.leases == 1
    m.release(ra)
    # a runner that died is noticed by the next request and started again
    alive[ra.service] = False
    again = m.acquire("a")
    assert again.service != ra.service and m.restarts == 1 and alive[again.service]
    m.release(again)
    m.shutdown()


def test_keep_alive_sweep_and_negative_cache(tmp_path):
    m, started, stopped, clock = _manager(tmp_path, fail={"bad"})
    m.register("a", "/models/a"); m.register("bad", "/models/bad")
    r = m.acquire("a", keep_alive_s=5)
    assert m.sweep() == []                                        # leased
    m.release(r); clock.t = 4.9
    assert m.sweep() == []
    clock.t = 5.1
    assert len(m.sweep()) == 1 and stopped == ["svc:/models/a"]
    with pytest.raises(M.ManagerError):
        m.acquire("bad")
    started_before = list(started)
    with pytest.raises(M.ManagerError, match="failed to start"):
        m.acquire("bad")                                          # served from the negative cache
    assert started == started_before
    clock.t += M.NEGATIVE_CACHE_S + 1
    with pytest.raises(M.ManagerError):
        m.acquire("bad")                                          # retried after the window


def test_gateway_registry_routes(tmp_path):
    m, *_ = _manager(tmp_path)
    m.register("a", "/models/a")
    app = FastAPI()
    M.install(app, m)
    c = TestClient(app)
    assert c.post("/api/copy", json={"source": "a", "destination": "b"}).status_code == 200
    assert [x["name"] for x in c.get("/api/tags").json()["models"]] == ["a", "b"]
    assert c.post("/api/copy", json={"source": "zz", "destination": "b"}).status_code == 404
    assert c.request("DELETE", "/api/delete", json={"model": "a"}).status_code == 200
    assert [x["id"] for x in c.get("/v1/models").json()["data"]] == ["b"]


@pytest.fixture(scope="module")
def client():
    from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec
    from orinfer_b200.api.server import Service, create_app
    from orinfer_b200.config import PRESETS, SchedulerOptions
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.models.weights import random_model
    weights = random_model(PRESETS["tiny"], seed=0)
    svc = Service(lambda: Engine(weights, sched=SchedulerOptions(max_active=4, prefill_chunk=64),
                                 kv_pages=24, max_context=512),
                  ChatCodec(ByteTokenizer(1024), context=512, model_name="tiny"), "tiny")
    svc.start()
    with TestClient(create_app(svc)) as c:
        yield c
    svc.stop(1000)


def test_embeddings_endpoint(client):
    r = client.post("/v1/embeddings", json={"input": ["hello world", "hello world", "other"]}).json()
    assert r["object"] == "list" and len(r["data"]) == 3 and r["usage"]["prompt_tokens"] > 0
    a, b, c = (d["embedding"] for d in r["data"])
    assert a == b and a != c and len(a) == 256
    assert abs(sum(x * x for x in a) - 1.0) < 1e-4
    q = client.post("/v1/embeddings", json={"input": "hello world", "input_type": "query",
                                            "dimensions": 64, "encoding_format": "base64"}).json()
    vec = struct.unpack("<64f", base64.b64decode(q["data"][0]["embedding"]))
    assert abs(sum(x * x for x in vec) - 1.0) < 1e-4
    bad = client.post("/v1/embeddings", json={"input": [], "input_type": "document"})
    assert bad.status_code == 400 and bad.json()["error"]["param"] == "input"
    assert client.post("/v1/embeddings", json={"input": "x", "dimensions": 9999}).status_code == 400


def test_rerank_endpoint(client):
    body = {"query": "capital of France", "documents": ["Paris", {"text": "bananas"}, "Lyon"],
            "top_n": 2, "return_documents": True}
    r = client.post("/v1/rerank", json=body).json()
    assert len(r["results"]) == 2
    assert r["results"][0]["relevance_score"] >= r["results"][1]["relevance_score"]
    assert {x["index"] for x in r["results"]} <= {0, 1, 2} and "document" in r["results"][0]
    assert client.post("/rerank", json=body).json()["results"] == r["results"]
    assert client.post("/v1/rerank", json={"query": "", "documents": ["a"]}).status_code == 400


def test_gateway_forwards_by_model_and_releases_leases(tmp_path):
    """Two names, one runner: requests are forwarded to the runner serving the model and the
    lease ends with the response; an unknown model is a 404 in OpenAI error shape."""
    from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec
    from orinfer_b200.api.server import Service, create_app
    from orinfer_b200.config import PRESETS, SchedulerOptions
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.models.weights import random_model
    weights = random_model(PRESETS["tiny"], seed=0)
    started, stopped = [], []

    def start(entry):
        svc = Service(lambda: Engine(weights, sched=SchedulerOptions(max_active=4, prefill_chunk=64),
                                     kv_pages=24, max_context=512),
                      ChatCodec(ByteTokenizer(1024), context=512, model_name=entry.name), entry.name)
        svc.start()
        started.append(entry.name)
        return M.RunnerHandle(svc, create_app(svc)), weights.nbytes()

    def stop(handle):
        handle.service.stop(1000)
        stopped.append(handle.service.model_name)

    m = M.ModelManager(tmp_path, start, stop)
    m.register("tiny", "/models/tiny")
    m.copy("tiny", "tiny-alias")
    with TestClient(M.create_gateway_app(m, sweep_s=3600)) as c:
        body = {"model": "tiny-alias", "messages": [{"role": "user", "content": "hi"}],
                "max_tokens": 4, "temperature": 0, "ignore_eos": True}
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] == 4
        r2 = c.post("/v1/chat/completions", json=dict(body, model="tiny"))
        assert r2.json()["choices"][0]["message"] == r.json()["choices"][0]["message"]
        assert started == ["tiny-alias"] and m.running()[0]["leases"] == 0
        emb = c.post("/v1/embeddings", json={"model": "tiny", "input": "hello"})
        assert emb.status_code == 200 and len(emb.json()["data"][0]["embedding"]) == 256
        import io
        import wave
        wav = io.BytesIO()
        with wave.open(wav, "wb") as w:
            w.setnchannels(1)
            w.setsampwidth(2)
            w.setframerate(16000)
            w.writeframes(b"\x00\x10" * 8000)
        tr = c.post("/v1/audio/transcriptions", files={"file": ("a.wav", wav.getvalue())},
                    data={"model": "tiny", "max_tokens": "3"})
        assert tr.status_code == 200 and "text" in tr.json()
        assert c.post("/v1/audio/transcriptions", files={"file": ("a.wav", wav.getvalue())}
                      ).status_code == 400                          # no model named
        one = c.post("/api/embed", json={"model": "tiny", "input": ["alpha", "beta gamma"]})
        assert one.status_code == 200 and len(one.json()["embeddings"]) == 2
        assert len(one.json()["embeddings"][0]) == 256 and one.json()["prompt_eval_count"] > 5
        old = c.post("/api/embeddings", json={"model": "tiny", "prompt": "alpha"})
        assert old.status_code == 200
        assert old.json()["embedding"] == pytest.approx(one.json()["embeddings"][0], abs=1e-6)
        assert c.post("/api/embed", json={"model": "tiny", "input": []}).status_code == 400
        missing = c.post("/v1/chat/completions", json=dict(body, model="nope"))
        assert missing.status_code == 404 and missing.json()["error"]["code"] == "model_not_found"
        assert c.post("/api/generate", json={"model": "nope", "prompt": "x"}).status_code == 404
        assert [x["name"] for x in c.get("/api/ps").json()["models"]] == ["tiny", "tiny-alias"]
    assert stopped == ["tiny-alias"]                                # shutdown retired the runner


def test_discovery_reads_files_and_starts_nothing(tmp_path):
    """`/`, `/api/version`, `/api/tags`, `/api/ps` and `/api/show` of the gateway are answered
    from the registry and the model's files; no runner is started for them."""
    import json
    from fastapi.testclient import TestClient
    root = tmp_path / "model"
    root.mkdir()
    (root / "config.json").write_text(json.dumps(
        {"architectures": ["TestForCausalLM"],
         "text_config": {"hidden_size": 256, "num_hidden_layers": 4,
                         "max_position_embeddings": 8192}, "vision_config": {}}))
    (root / "tokenizer_config.json").write_text(json.dumps({"chat_template": "native jinja"}))
    starts = []
    m = M.ModelManager(tmp_path / "state", lambda e: starts.append(e.name), lambda s: None)
    m.register("fixture:2b", str(root), defaults={"temperature": 0.2})
    with TestClient(M.create_gateway_app(m, sweep_s=3600)) as c:
        for route in ("/", "/api/version", "/api/tags", "/api/ps"):
            assert c.get(route).status_code == 200, route
        assert c.get("/api/tags").json()["models"][0]["name"] == "fixture:2b"
        shown = c.post("/api/show", json={"model": "fixture:2b"}).json()
        assert shown["model_info"]["TestForCausalLM.context_length"] == 8192
        assert shown["model_info"]["TestForCausalLM.block_count"] == 4
        assert shown["template"] == "native jinja" and "vision" in shown["capabilities"]
        assert "temperature 0.2" in shown["parameters"]
        assert c.post("/api/show", json={"model": "absent"}).status_code == 404
        bad = c.post("/api/chat", content="{")
        assert bad.status_code == 400 and isinstance(bad.json()["error"], str)
    assert starts == []


def test_gateway_load_and_unload_requests_generate_nothing(tmp_path):
    """An Ollama request without a prompt loads the model (or, with keep_alive 0, unloads it)
    at the gateway: nothing is generated, an unload starts nothing, `/api/ps` shows when a
    model goes, malformed keep-alives are client errors."""
    from fastapi.testclient import TestClient
    starts, stops, seen = [], [], []

    class App:                                                   # a runner that must not be asked
        async def __call__(self, scope, receive, send):
            seen.append(scope["path"])
            raise AssertionError("no request may reach the runner")

    def start(entry):
        starts.append(entry.name)
        return M.RunnerHandle(object(), App()), 100

    m = M.ModelManager(tmp_path, start, lambda h: stops.append(1))
    m.register("fixture:2b", "/models/x")
    with TestClient(M.create_gateway_app(m, sweep_s=3600)) as c:
        gone = c.post("/api/generate", json={"model": "fixture:2b", "keep_alive": 0})
        assert gone.status_code == 200 and gone.json()["done_reason"] == "unload" and starts == []
        up = c.post("/api/generate", json={"model": "fixture:2b", "keep_alive": -1, "stream": False})
        assert up.json()["done_reason"] == "load" and up.json()["response"] == "" and starts == ["fixture:2b"]
        ps = c.get("/api/ps").json()["models"][0]
        assert ps["name"] == "fixture:2b" and ps["expires_at"] == "9999-12-31T23:59:59Z"
        chat = c.post("/api/chat", json={"model": "fixture:2b", "keep_alive": "5m"})
        assert chat.json()["done_reason"] == "load" and chat.json()["message"]["content"] == ""
        assert c.get("/api/ps").json()["models"][0]["expires_at"].startswith("20")
        down = c.post("/api/chat", json={"model": "fixture:2b", "messages": [], "keep_alive": 0})
        assert down.json()["done_reason"] == "unload" and stops == [1] and m.running() == []
        assert c.post("/api/generate", json={"model": "absent"}).status_code == 404
        bad = c.post("/api/generate", json={"model": "fixture:2b", "prompt": "hi", "keep_alive": {}})
        assert bad.status_code == 400 and isinstance(bad.json()["error"], str)
    assert seen == [] and starts == ["fixture:2b"]


def test_names_that_share_a_runner_keep_their_own_defaults(tmp_path):
    """An alias's sampling defaults are laid under each request at the gateway (the request's
    own fields win, alternative spellings of one limit are respected); Ollama bodies get them
    through `options` / `think`."""
    import json
    from fastapi.testclient import TestClient
    from starlette.responses import JSONResponse as Echo

    class App:
        async def __call__(self, scope, receive, send):
            body = (await receive())["body"]
            await Echo(json.loads(body))(scope, receive, send)

    starts = []

    def start(entry):
        starts.append(entry.name)
        return M.RunnerHandle(object(), App()), 1

    m = M.ModelManager(tmp_path, start, lambda h: None)
    m.register("base", "/models/x")
    m.register("warm", "/models/x", defaults={"temperature": 0.7, "max_tokens": 64,
                                              "enable_thinking": True})
    msgs = [{"role": "user", "content": "hi"}]
    with TestClient(M.create_gateway_app(m, sweep_s=3600)) as c:
        plain = c.post("/v1/chat/completions", json={"model": "base", "messages": msgs}).json()
        assert plain == {"model": "base", "messages": msgs}
        warm = c.post("/v1/chat/completions", json={"model": "warm", "messages": msgs}).json()
        assert warm["temperature"] == 0.7 and warm["max_tokens"] == 64 and warm["enable_thinking"]
        own = c.post("/v1/chat/completions", json={"model": "warm", "messages": msgs,
                                                   "temperature": 0, "max_completion_tokens": 8}).json()
        assert own["temperature"] == 0 and own["max_completion_tokens"] == 8
        assert "max_tokens" not in own                       # one limit, the request's spelling
        oll = c.post("/api/chat", json={"model": "warm", "messages": msgs,
                                        "options": {"top_p": 0.5}}).json()
        assert oll["options"] == {"top_p": 0.5, "temperature": 0.7, "num_predict": 64}
        assert oll["think"] is True
    assert starts == ["base"]                                # same files, same options: one runner


def test_max_loaded_models_caps_the_number_of_runners(tmp_path):
    starts, stopped = [], []
    m = M.ModelManager(tmp_path, lambda e: (starts.append(e.name) or f"svc:{e.name}", 1),
                       stopped.append, max_loaded=2)
    for n in "abc":
        m.register(n, f"/models/{n}")
    ra, rb = m.acquire("a"), m.acquire("b")
    with pytest.raises(M.ManagerError) as err:
        m.acquire("c")                                       # both in use, no waiting configured
    assert err.value.status == 503
    m.release(ra)
    m.acquire("c")
    assert "svc:a" in stopped and len(m.running()) == 2
    m.release(rb)


def test_serve_flags_of_the_reference_are_accepted():
    from orinfer_b200.cli import build_parser
    a = build_parser().parse_args([
        "serve", "--preset", "tiny", "--preprocess-workers", "3", "--preprocess-memory-mib",
        "512", "--request-body-mib", "8", "--max-loaded-models", "2", "--load-timeout-s", "120",
        "--gpu-lock", "/tmp/locks"])
    assert (a.preparation_workers, a.preparation_memory_mib, a.request_body_mib,
            a.max_loaded_models, a.load_timeout_s, a.gpu_lock) == (3, 512, 8, 2, 120.0, "/tmp/locks")
