"""Offline JSONL batch (journal, resume, ordering) and checkpoint round trip (CPU)."""
import json

import pytest
import torch

from orinfer_b200.api.batch_jsonl import BatchError, run_batch
from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec
from orinfer_b200.config import PRESETS, SchedulerOptions
from orinfer_b200.engine import checkpoint as C
from orinfer_b200.engine.engine import Engine
from orinfer_b200.models.weights import random_model


@pytest.fixture(scope="module")
def weights():
    return random_model(PRESETS["tiny"], seed=0)


def _engine(w):
    return Engine(w, sched=SchedulerOptions(max_active=4, prefill_chunk=64), kv_pages=24,
                  max_context=512)


def test_batch_journal_resume_and_order(weights, tmp_path):
    codec = ChatCodec(ByteTokenizer(1024), context=512)
    rows = [{"id": f"r{i}", "body": {"messages": [{"role": "user", "content": "shared " * 3 + str(i % 2)}],
                                     "max_tokens": 3, "temperature": 0, "ignore_eos": True}}
            for i in range(5)]
    rows.append({"id": "bad", "body": {"messages": [], "max_tokens": 3}})
    src, out = tmp_path / "in.jsonl", tmp_path / "out.jsonl"
    src.write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    counts = run_batch(_engine(weights), codec, src, out, order="auto", model_id="tiny")
    assert counts == {"total": 6, "skipped": 0, "completed": 5, "failed": 1}
    recs = {json.loads(l)["id"]: json.loads(l) for l in out.read_text().splitlines()}
    assert recs["bad"]["error"]["param"] == "messages"
    assert recs["r0"]["response"]["usage"]["completion_tokens"] == 3
    assert recs["r0"]["response"]["choices"][0]["message"] == recs["r2"]["response"]["choices"][0]["message"]
    with pytest.raises(BatchError):
        run_batch(_engine(weights), codec, src, out, model_id="tiny")
    again = run_batch(_engine(weights), codec, src, out, resume=True, model_id="tiny")
    assert again["skipped"] == 5 and again["failed"] == 1      # failed rows are retried
    with pytest.raises(BatchError, match="identity"):
        run_batch(_engine(weights), codec, src, out, resume=True, model_id="other")


def test_checkpoint_roundtrip_and_validation(weights, tmp_path):
    d = C.save_model(weights, tmp_path / "m")
    report = C.validate_model(d)
    assert report["ok"] and report["layers"] == 2
    loaded = C.load_model(d, verify=True)
    a = _engine(weights).generate([[1, 2, 3, 4]], max_new=4)
    b = _engine(loaded).generate([[1, 2, 3, 4]], max_new=4)
    assert a == b
    desc = json.loads((d / "cache" / "model.json").read_text())
    assert desc["target"] == "sm_100a" and desc["quantization_config"]["rotation"] == "signed-block128"
    desc["tensors"]["final_norm"] = "0" * 64
    (d / "cache" / "model.json").write_text(json.dumps(desc))
    with pytest.raises(C.CheckpointError, match="SHA-256"):
        C.validate_model(d)
