"""Leader / follower ranks of a multi-rank engine on CPU (gloo): the leader takes every
decision, followers replay the published device commands; a follower that stops replying
fails the leader closed within the deadline.  No GPU is involved."""
import time

import pytest

@pytest.fixture(autouse=True)
def _few_threads():
    """The leader rank lives in the test process: like the follower processes it should not
    claim every core for each small operator."""
    import torch
    before = torch.get_num_threads()
    torch.set_num_threads(2)
    yield
    torch.set_num_threads(before)


SPEC = dict(
    world=2, device="cpu", preset="tiny", group_timeout_s=120.0, kv_pages=32, max_context=512,
    max_rows=256,
    load=dict(cuda_graph="off", prefix_cache_bytes=0, tp=2),
    sched=dict(policy="latency", max_active=4, prefill_chunk=128),
)


def test_leader_and_follower_generate_like_spmd_ranks():
    from orinfer_b200.parallel.rank_worker import leader_engine
    engine, team = leader_engine(dict(SPEC), deadline_s=90.0)
    try:
        prompts = [[(7 * i + j) % 1000 + 1 for i in range(40)] for j in range(3)]
        out = engine.generate(prompts, max_new=6)
        team.channel.sync(90.0)
        assert all(len(o) == 6 for o in out)
        # the same prompts again: same tokens (the follower's KV / page rows stayed in step)
        again = engine.generate(prompts, max_new=6)
        assert again == out
        assert team.channel.failure is None
    finally:
        team.close(engine)
    assert all(p.returncode == 0 for p in team.procs)


def test_leader_keeps_the_prefix_cache_and_followers_follow_its_page_rows():
    from orinfer_b200.parallel.rank_worker import leader_engine
    spec = dict(SPEC, load=dict(SPEC["load"], prefix_cache_bytes=64 << 20))
    engine, team = leader_engine(spec, deadline_s=90.0)
    try:
        assert engine.prefix is not None
        shared = [(11 * i) % 997 + 1 for i in range(300)]           # two full pages and a bit
        first = engine.generate([shared + [5, 6, 7]], max_new=4)
        reqs = [engine.submit(shared + [8, 9], 4), engine.submit(shared + [5, 6, 7], 4)]
        while any(not r.finished for r in reqs):
            engine.step()
        team.channel.sync(90.0)
        assert all(r.cached_tokens >= 256 for r in reqs)            # both reuse the cached pages
        assert reqs[1].generated == first[0]                        # and the follower kept in step
        assert team.channel.failure is None
    finally:
        team.close(engine)
    assert all(p.returncode == 0 for p in team.procs)


def test_prompt_lookup_speculation_publishes_its_verification_packets(monkeypatch):
    """Drafts copied from earlier n-grams are verified in packets that the followers run too;
    the greedy text is what plain decoding gives."""
    from orinfer_b200.parallel.rank_worker import leader_engine
    monkeypatch.setenv("ORINFER_SINGLE_MTP_POLICY", "fixed3")
    prompt = [3, 1, 4, 1, 5, 9, 2, 6] * 6
    plain_engine, plain_team = leader_engine(dict(SPEC), deadline_s=90.0)
    try:
        plain = plain_engine.generate([prompt], max_new=16)[0]
    finally:
        plain_team.close(plain_engine)
    spec = dict(SPEC, load=dict(SPEC["load"], prompt_lookup=True, mtp_drafts=3))
    engine, team = leader_engine(spec, deadline_s=90.0)
    try:
        assert engine.spec.enabled and not engine.runner_has_mtp()
        # an oracle draft source makes every round propose (and accept) something
        engine.spec.drafts_for = lambda r, c: plain[len(r.generated):len(r.generated) + c]
        out = engine.generate([prompt], max_new=16)[0]
        team.channel.sync(90.0)
        st = engine.spec.statistics()
        assert out == plain
        assert st["rounds"] > 0 and st["accepted_draft_tokens"] > 0
        assert team.channel.failure is None
    finally:
        team.close(engine)
    assert all(p.returncode == 0 for p in team.procs)


def test_host_kv_tier_moves_pages_on_every_rank():
    """Page pressure sends cached prefixes to the host tier and a later hit brings them back:
    every rank saves and restores its own shard of the page on the leader's published commands,
    and the restored KV gives the same tokens."""
    from orinfer_b200.parallel.rank_worker import leader_engine
    spec = dict(SPEC, kv_pages=4, max_context=256,
                load=dict(SPEC["load"], prefix_cache_bytes=64 << 20, kv_offload_bytes=64 << 20),
                sched=dict(SPEC["sched"], max_active=1, prefill_chunk=256))
    engine, team = leader_engine(spec, deadline_s=90.0)
    try:
        base = [[(13 * i + 7 * j) % 997 + 1 for i in range(130)] for j in range(3)]
        first = [engine.generate([p], max_new=4)[0] for p in base]   # 3 usable pages: must evict
        assert engine.stats.offloaded_pages >= 1
        r = engine.submit(base[0], 4)
        while not r.finished:
            engine.step()
        team.channel.sync(90.0)
        assert engine.stats.restored_pages >= 1 and r.cached_tokens == 128
        assert r.generated == first[0]
        assert team.channel.failure is None
    finally:
        team.close(engine)
    assert all(p.returncode == 0 for p in team.procs)


def test_hybrid_model_keeps_prefix_cache_and_speculation_across_ranks(monkeypatch):
    """Recurrent state is per-rank device data: its copies are taken, restored and dropped by
    published commands under the leader's handles, and a verification round's accepted rows are
    committed on every rank.  Texts equal those of a plain multi-rank engine."""
    from orinfer_b200.parallel.rank_worker import leader_engine
    monkeypatch.setenv("ORINFER_SINGLE_MTP_POLICY", "fixed3")
    base = dict(SPEC, preset="tiny-hybrid")
    shared = [(11 * i) % 251 + 1 for i in range(128)]
    prompts = [shared + [5, 6, 7, 8, 5, 6, 7, 8, 5, 6], shared + [9, 8, 7]]
    plain_engine, plain_team = leader_engine(dict(base), deadline_s=90.0)
    try:
        assert plain_engine.recurrent
        plain = [plain_engine.generate([p], max_new=8)[0] for p in prompts]
    finally:
        plain_team.close(plain_engine)
    spec = dict(base, load=dict(SPEC["load"], prefix_cache_bytes=64 << 20, prompt_lookup=True,
                                mtp_drafts=3))
    engine, team = leader_engine(spec, deadline_s=90.0)
    try:
        assert engine.prefix is not None and engine.spec.enabled
        text = {}

        def drafts(r, c):                          # half-right drafts: accept one, reject the rest
            d = list(text[r.rid][len(r.generated):len(r.generated) + c])
            if len(d) > 1:
                d[1:] = [(t + 1) % 251 for t in d[1:]]
            return d

        engine.spec.drafts_for = drafts
        got = []
        for p, want in zip(prompts + prompts[:1], plain + plain[:1]):
            r = engine.submit(p, 8)
            text[r.rid] = want
            while not r.finished:
                engine.step()
            got.append(r)
        team.channel.sync(90.0)
        assert [r.generated for r in got] == plain + plain[:1]
        assert got[0].cached_tokens == 0 and got[1].cached_tokens == 128
        assert got[2].cached_tokens == 128
        st = engine.spec.statistics()
        assert 0 < st["accepted_draft_tokens"] < st["proposed_tokens"]
        assert engine.stats.stored_snapshots >= 1 and engine.stats.restored_snapshots == 2
        assert team.channel.failure is None
    finally:
        team.close(engine)
    assert all(p.returncode == 0 for p in team.procs)


def test_draft_head_speculation_runs_sharded_on_every_rank(monkeypatch):
    """With ``draft_head`` the shards carry the draft head (heads and FFN channels split like a
    decoder layer): the hidden rows it consumes are captured on every rank, its draft rounds
    are collective, and the text equals that of the same ranks without speculation."""
    from orinfer_b200.parallel.rank_worker import leader_engine
    monkeypatch.setenv("ORINFER_SINGLE_MTP_POLICY", "fixed2")
    base = dict(SPEC, mtp_layers=1, draft_head=True)
    prompts = [[(7 * i + 3 * j) % 500 + 1 for i in range(24)] for j in range(2)]
    plain_engine, plain_team = leader_engine(
        dict(base, load=dict(SPEC["load"], mtp_drafts=0)), deadline_s=90.0)
    try:
        assert not plain_engine.spec.enabled
        plain = plain_engine.generate(prompts, max_new=10)
    finally:
        plain_team.close(plain_engine)
    engine, team = leader_engine(dict(base, load=dict(SPEC["load"], mtp_drafts=2)),
                                 deadline_s=90.0)
    try:
        assert engine.runner_has_mtp() and engine.spec.enabled
        assert engine.w.mtp.layer.qkv.n < 2 * engine.w.global_config.q_heads * 64   # a shard
        out = engine.generate(prompts, max_new=10)
        team.channel.sync(90.0)
        assert out == plain
        st = engine.spec.statistics()
        assert st["rounds"] > 0 and st["proposed_tokens"] > 0
        assert not engine._mtp_backlog or all(r.finished for r in engine.running)
        assert team.channel.failure is None
    finally:
        team.close(engine)
    assert all(p.returncode == 0 for p in team.procs)


def test_ranks_cut_their_shards_out_of_a_model_directory(tmp_path):
    """A saved model served by two ranks: every rank reads the checkpoint on the host, keeps
    its shard and uploads that; the text is the unsharded model's up to the shard scales."""
    from orinfer_b200.config import PRESETS
    from orinfer_b200.engine.checkpoint import save_model
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.models.weights import random_model
    from orinfer_b200.parallel.rank_worker import leader_engine
    w = random_model(PRESETS["tiny"], seed=3)
    save_model(w, tmp_path / "m", "tiny")
    prompts = [[(5 * i + j) % 700 + 1 for i in range(30)] for j in range(2)]
    whole = Engine(w, kv_pages=16, max_context=512).generate(prompts, max_new=4)
    engine, team = leader_engine(dict(SPEC, preset=None, model_dir=str(tmp_path / "m")),
                                 deadline_s=90.0)
    try:
        assert engine.w.tp.world == 2 and engine.w.config.q_heads == PRESETS["tiny"].q_heads // 2
        out = engine.generate(prompts, max_new=4)
        team.channel.sync(90.0)
        same = sum(a == b for o, v in zip(out, whole) for a, b in zip(o, v))
        assert same >= 6, (out, whole)             # random weights: near-ties may flip a token
        assert team.channel.failure is None
    finally:
        team.close(engine)
    assert all(p.returncode == 0 for p in team.procs)


def test_follower_that_stops_replying_fails_the_leader_closed():
    from orinfer_b200.parallel.rank_channel import RankFailure
    from orinfer_b200.parallel.rank_worker import leader_engine
    spec = dict(SPEC, test_stall_after=2, group_timeout_s=6.0)
    engine, team = leader_engine(spec, deadline_s=3.0)
    t0 = time.monotonic()
    try:
        with pytest.raises((RankFailure, RuntimeError)):
            for _ in range(50):                       # the follower goes silent after 2 commands
                engine.generate([[1, 2, 3, 4, 5]], max_new=2)
                time.sleep(0.2)
        assert time.monotonic() - t0 < 40.0
        with pytest.raises((RankFailure, RuntimeError)):
            engine.generate([[1, 2, 3]], max_new=1)   # sticky
    finally:
        team.close(wait_s=2.0)


def _serve_tp2(device_args, timeout_s=300):
    """`orinfer serve --tp 2` as a subprocess; returns (proc, url) once /health is ready."""
    import socket
    import subprocess
    import sys

    import requests
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    proc = subprocess.Popen([sys.executable, "-m", "orinfer_b200", "serve", "--preset", "tiny",
                             "--tp", "2", "--listen", f"127.0.0.1:{port}", "--max-context", "512",
                             "--prefix-cache-mib", "0", *device_args],
                            stderr=subprocess.PIPE, text=True, start_new_session=True)
    url = f"http://127.0.0.1:{port}"
    deadline = time.time() + timeout_s
    while time.time() < deadline:
        if proc.poll() is not None:
            raise AssertionError("serve exited: " + proc.stderr.read()[-2000:])
        try:
            if requests.get(url + "/health", timeout=2).status_code == 200:
                return proc, url
        except requests.RequestException:
            pass
        time.sleep(0.2)
    proc.kill()
    raise AssertionError("serve --tp 2 never became ready")


def _chat_streams(url):
    import json

    import requests
    body = {"messages": [{"role": "user", "content": "hello there"}], "max_tokens": 5,
            "temperature": 0, "ignore_eos": True, "stream": True,
            "stream_options": {"include_usage": True}}
    with requests.post(url + "/v1/chat/completions", json=body, stream=True, timeout=120) as r:
        assert r.status_code == 200, r.text
        lines = [l.decode() for l in r.iter_lines() if l.startswith(b"data: ")]
    assert lines[-1] == "data: [DONE]"
    assert json.loads(lines[-2][6:])["usage"]["completion_tokens"] == 5
    plain = requests.post(url + "/v1/chat/completions", json=dict(body, stream=False), timeout=120)
    assert plain.status_code == 200 and plain.json()["usage"]["completion_tokens"] == 5


def test_serve_tp2_streams_a_chat_completion_on_cpu_ranks():
    import signal
    proc, url = _serve_tp2(["--device", "cpu", "--cuda-graph", "off"])
    try:
        _chat_streams(url)
    finally:
        proc.send_signal(signal.SIGTERM)
        assert proc.wait(timeout=90) == 0


@pytest.mark.gpu
def test_serve_tp2_streams_a_chat_completion_on_two_gpus(cuda):
    import signal

    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    proc, url = _serve_tp2([])
    try:
        _chat_streams(url)
        _chat_streams(url)                       # decode graphs captured by now: replay path
    finally:
        proc.send_signal(signal.SIGTERM)
        assert proc.wait(timeout=120) == 0
