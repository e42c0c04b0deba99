"""Offline JSONL batch: every input line is a chat request (``{"id":..., "body":{...}}`` or
a bare request body); results are appended to an output journal as they finish.

Journal identity (input SHA-256, model, default request params) is kept in a sidecar
``<output>.meta.json``; ``resume`` skips ids already committed and retries failed ones;
``order="auto"`` sorts requests so that prompts sharing a prefix run next to each other
(prefix-tree ordering); a bounded writer thread appends and fsyncs about once a second.
Behaviour follows crates/orinfer-api/src/server/batch.rs:34-112,138-324 and
batch/files.rs:209-360 of the reference.
"""

from __future__ import annotations

import hashlib
import json
import os
import queue
import threading
import time
from pathlib import Path
from typing import Dict, List, Optional

from ..core.sampling import SamplingOptions
from .chat_codec import ChatCodec, RequestError
from .output_parser import OutputParser

SCHEMA = 1


class BatchError(RuntimeError):
    pass


def _scan_input(path: Path):
    sha = hashlib.sha256()
    rows = []
    with open(path, "rb") as f:
        for n, raw in enumerate(f):
            sha.update(raw)
            if not raw.strip():
                continue
            try:
                obj = json.loads(raw)
            except json.JSONDecodeError as e:
                raise BatchError(f"{path}:{n + 1}: invalid JSON ({e})")
            body = obj.get("body", obj) if isinstance(obj, dict) else None
            if not isinstance(body, dict):
                raise BatchError(f"{path}:{n + 1}: expected a JSON object")
            rid = str(obj.get("id", obj.get("custom_id", n))) if "body" in obj else str(n)
            rows.append((rid, body))
    ids = [r for r, _ in rows]
    if len(set(ids)) != len(ids):
        raise BatchError("duplicate request ids in the batch input")
    return rows, sha.hexdigest()


class _Writer(threading.Thread):
    def __init__(self, path: Path):
        super().__init__(daemon=True)
        self.q: "queue.Queue[Optional[dict]]" = queue.Queue(maxsize=1024)
        self.f = open(path, "a", encoding="utf-8")
        self.error: Optional[BaseException] = None

    def run(self):
        last_sync = time.monotonic()
        try:
            while True:
                try:
                    item = self.q.get(timeout=0.25)
                except queue.Empty:
                    item = False
                if item is None:
                    break
                if item:
                    self.f.write(json.dumps(item, ensure_ascii=False) + "\n")
                if time.monotonic() - last_sync >= 1.0:
                    self.f.flush()
                    os.fsync(self.f.fileno())
                    last_sync = time.monotonic()
        except BaseException as e:                  # surfaced by close()
            self.error = e
        finally:
            self.f.flush()
            os.fsync(self.f.fileno())
            self.f.close()

    def close(self):
        self.q.put(None)
        self.join()
        if self.error:
            raise BatchError(f"journal write failed: {self.error}")


def run_batch(engine, codec: ChatCodec, input_path, output_path, *, resume: bool = False,
              order: str = "input", default_request_params: Optional[dict] = None,
              model_id: str = "") -> Dict[str, int]:
    """Returns counts ``{"total", "skipped", "completed", "failed"}``."""
    input_path, output_path = Path(input_path), Path(output_path)
    rows, sha = _scan_input(input_path)
    meta_path = Path(str(output_path) + ".meta.json")
    identity = {"schema": SCHEMA, "input_sha256": sha, "model": model_id,
                "default_request_params": default_request_params or {}}
    done: Dict[str, bool] = {}
    if output_path.exists() and output_path.stat().st_size:
        if not resume:
            raise BatchError(f"{output_path} exists; pass resume to continue it")
        if not meta_path.exists() or json.loads(meta_path.read_text()) != identity:
            raise BatchError("journal identity differs from this run (input, model or "
                             "defaults changed)")
        with open(output_path, encoding="utf-8") as f:
            for line in f:
                try:
                    rec = json.loads(line)
                except json.JSONDecodeError:
                    continue                         # torn last line of a crashed run
                done[rec["id"]] = rec.get("error") is None
    meta_path.write_text(json.dumps(identity))
    todo = [(rid, body) for rid, body in rows if not done.get(rid, False)]
    prepared = []
    writer = _Writer(output_path)
    writer.start()
    counts = {"total": len(rows), "skipped": len(rows) - len(todo), "completed": 0, "failed": 0}
    for rid, body in todo:
        try:
            prepared.append((rid, codec.prepare(dict(body, stream=False),
                                                default_request_params)))
        except RequestError as e:
            writer.q.put({"id": rid, "error": e.body()["error"]})
            counts["failed"] += 1
    if order == "auto":
        prepared.sort(key=lambda it: it[1].prompt_ids)      # shared prefixes become adjacent
    pending = list(reversed(prepared))
    live = {}
    while pending or live:
        while pending and len(live) < engine.sched.max_active * 2:
            rid, p = pending.pop()
            req = engine.submit(p.prompt_ids, p.max_new, p.sampling, stop_ids=p.stop_ids,
                                ignore_eos=p.ignore_eos, cache_prompt=p.cache_prompt)
            live[req.rid] = (rid, p, req)
        engine.step()
        for key, (rid, p, req) in list(live.items()):
            if not req.finished:
                continue
            del live[key]
            toks = [t for t in req.generated if t not in req.stop_ids or req.ignore_eos]
            parser = OutputParser(thinking=p.thinking, stops=p.stop_strings)
            d = parser.feed(codec.tokenizer.decode(toks), final=True)
            msg = {"role": "assistant", "content": d.content}
            if d.reasoning:
                msg["reasoning_content"] = d.reasoning
            if d.tool_calls:
                from .output_parser import merge_tool_calls
                msg["tool_calls"] = merge_tool_calls(d.tool_calls)      # fragments -> calls
            writer.q.put({"id": rid, "response": {
                "choices": [{"index": 0, "message": msg,
                             "finish_reason": parser.finish_reason(req.finish_reason or "stop")}],
                "usage": {"prompt_tokens": len(req.prompt),
                          "completion_tokens": len(req.generated),
                          "prompt_tokens_details": {"cached_tokens": req.cached_tokens}}}})
            counts["completed"] += 1
    writer.close()
    return counts
