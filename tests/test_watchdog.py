"""Step watchdog: a step past its deadline fails the service closed (host-side only)."""
import threading
import time

from orinfer_b200.engine.watchdog import StepWatchdog


def test_deadlines_trip_once_and_disarm_in_time_does_not():
    hits = []
    dog = StepWatchdog(lambda what, waited: hits.append((what, waited)), poll_s=0.01)
    with dog.guard("quick", 0.5):
        time.sleep(0.02)
    assert hits == [] and 0.02 <= dog.longest_s < 0.5
    dog.arm("ignored", 0)                                   # zero disables
    time.sleep(0.05)
    with dog.guard("slow", 0.05):
        time.sleep(0.2)
    assert len(hits) == 1 and hits[0][0] == "slow" and hits[0][1] >= 0.05
    with dog.guard("slow again", 0.02):                     # sticky: reported once
        time.sleep(0.1)
    assert len(hits) == 1 and dog.tripped == "slow"
    dog.close()


def test_stalled_step_fails_the_service_and_answers_clients():
    from fastapi.testclient import TestClient
    from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec
    from orinfer_b200.api.server import Service, create_app
    from orinfer_b200.config import PRESETS, SchedulerOptions
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.models.weights import random_model
    weights = random_model(PRESETS["tiny"], seed=0)
    release = threading.Event()

    def factory():
        eng = Engine(weights, sched=SchedulerOptions(max_active=2, prefill_chunk=64), kv_pages=16,
                     max_context=256)
        real, calls = eng.step, {"n": 0}

        def step():
            calls["n"] += 1
            if calls["n"] > 3:                               # after the warm-up: a host call that
                release.wait(12)                             # does not come back in time
            return real()
        eng.step = step
        return eng

    svc = Service(factory, ChatCodec(ByteTokenizer(1024), context=256, model_name="tiny"), "tiny",
                  step_timeout_ms=4000)
    svc.start()
    with TestClient(create_app(svc)) as c:
        assert c.get("/health").status_code == 200
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}],
                                                 "max_tokens": 4})
        assert r.status_code == 500 and r.json()["error"]["code"] == "engine_stalled"
        h = c.get("/health")
        assert h.status_code == 503 and "exceeded" in h.json()["reason"]
        assert "orinfer_watchdog_timeouts_total 1" in c.get("/metrics").text
        again = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]})
        assert again.status_code == 503                     # fails fast from now on
    release.set()
    svc.stop(1000)
