"""HTTP surface: OpenAI ``/v1/chat/completions`` (+ ``/render``), ``/v1/models``,
``/health``, ``/metrics`` and the Ollama routes, on FastAPI.

Route set, error body shape (``error.{message,type,param,code}``), 429 +
``Retry-After: 1`` on a full queue, 503 while not ready, the SSE chunk sequence (role
chunk, deltas, finish chunk, optional usage chunk, ``[DONE]``) and the request-id header
follow crates/orinfer-api/src/server/mod.rs:126-163,250-343,350-556 and
server/continuous.rs:424-449,774-776 of the reference.
"""

from __future__ import annotations

import asyncio
import json
import time
import uuid
from typing import Any, Callable, Dict, Optional

from fastapi import FastAPI, Request as HttpRequest
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from .chat_codec import ChatCodec, RequestError
from .metrics import Metrics
from .worker import EngineWorker, Job, Lifecycle

BODY_LIMIT = 32 << 20


def _error(status: int, message: str, code: Optional[str] = None, param: Optional[str] = None,
           err_type: str = "invalid_request_error", headers: Optional[dict] = None):
    return JSONResponse({"error": {"message": message, "type": err_type, "param": param,
                                   "code": code}}, status_code=status, headers=headers)


OPEN_PATHS = ("/health", "/", "/api/version")


def api_key() -> Optional[str]:
    """``ORINFER_API_KEY``: when set (and not empty) every route but the liveness ones wants
    ``Authorization: Bearer <key>`` (crates/orinfer-api/src/server/mod.rs:232-249)."""
    import os
    return os.environ.get("ORINFER_API_KEY") or None


def bearer_authorized(key: Optional[str], headers) -> bool:
    if key is None:
        return True
    import hmac
    value = headers.get("authorization") or ""
    return value.startswith("Bearer ") and hmac.compare_digest(value[7:].encode(), key.encode())


def refuse_unauthorized(key: Optional[str], request) -> Optional[JSONResponse]:
    if request.url.path in OPEN_PATHS or bearer_authorized(key, request.headers):
        return None
    return _error(401, "Invalid API key", code="invalid_api_key", err_type="authentication_error")


class Service:
    def __init__(self, engine_factory: Callable, codec: ChatCodec, model_name: str,
                 default_request_params: Optional[dict] = None, queue_timeout_ms: int = 0,
                 output_timeout_ms: int = 60000, preparation_workers: int = 4,
                 preparation_memory_mib: int = 1024, step_timeout_ms: int = 0,
                 exit_on_stall: bool = False):
        self.codec = codec
        self.model_name = model_name
        self.defaults = default_request_params or {}
        from .chat_codec import validate_defaults
        validate_defaults(codec, self.defaults)          # a bad default fails the start
        self.metrics = Metrics()
        self.lifecycle = Lifecycle()
        self.worker = EngineWorker(engine_factory, codec, self.metrics, self.lifecycle,
                                   queue_timeout_ms, step_timeout_ms, exit_on_stall)
        self.output_timeout_s = output_timeout_ms / 1e3
        self.started = time.time()
        from .preparation import PreparationPool
        self.preparation = PreparationPool(preparation_workers, preparation_memory_mib)

    def start(self, wait: bool = True) -> None:
        self.worker.start()
        if wait:
            self.worker.ready.wait()

    def stop(self, drain_ms: int = 30000) -> None:
        self.worker.stop(drain_ms / 1e3)

    # ------------------------------------------------------------------ chat
    async def submit_async(self, body: dict, loop) -> Job:
        """``submit`` with the preparation (template, tokeniser, grammar) on a pool thread,
        under the pool's worker and memory budgets."""
        from .preparation import estimate_bytes
        prepared = await self.preparation.run(
            lambda: self.codec.prepare(body, self.defaults), estimate_bytes(body))
        return self.submit(body, loop, prepared)

    def submit(self, body: dict, loop, prepared=None) -> Job:
        if prepared is None:
            prepared = self.codec.prepare(body, self.defaults)
        job = Job(prepared, "chatcmpl-" + uuid.uuid4().hex[:24], loop, asyncio.Queue())
        if self.lifecycle.state != Lifecycle.READY:
            raise RequestError("server is not ready", status=503, code="not_ready",
                               err_type="server_error")
        if not self.worker.try_submit(job):
            raise RequestError("request queue is full", status=429, code="queue_full",
                               err_type="rate_limit_error")
        return job

    async def events(self, job: Job):
        while True:
            try:
                ev = await asyncio.wait_for(job.events.get(), timeout=self.output_timeout_s)
            except asyncio.TimeoutError:
                job.cancelled = True
                yield {"type": "error", "status": 504, "message": "output stalled",
                       "code": "client_output_timeout"}
                return
            yield ev
            if ev["type"] in ("done", "error"):
                return

    def health(self) -> dict:
        eng = self.worker.engine
        out = {"status": self.lifecycle.state, "model": self.model_name,
               "uptime_s": round(time.time() - self.started, 3),
               "continuous_batching": True,
               "chat_capabilities": {
                   "chat_template_kwargs": True, "json_schema": True, "logprobs": True,
                   "streaming": True, "default_stream": bool(self.defaults.get("stream", False)),
                   "max_choices": 1, "response_formats": ["text", "json_object", "json_schema"],
                   "constraint_backend": "llguidance",
                   "tools": {"function": True, "strict": True, "required": True,
                             "incremental_arguments": True},
                   "max_top_logprobs": 20, "logit_bias": True, "stored_completions": False,
                   "images": False, "video": False,
                   "audio": getattr(self.codec, "audio", None) is not None,
                   "thinking_token_budget": True,
                   "prompt_cache": {"key": True, "retention": ["in-memory", "24h"],
                                    "persistent": False, "ttl_guaranteed": False}},
               "default_request_params": self.defaults}
        if self.lifecycle.reason:
            out["reason"] = self.lifecycle.reason
        if eng is not None:
            out["scheduler"] = eng.stats.as_dict()
            out["active"] = len(eng.running)
            out["queued"] = len(eng.waiting) + self.worker.jobs.qsize()
            if eng.prefix is not None:
                out["prefix_cache"] = eng.prefix.statistics().__dict__
            out["context"] = out["max_context"] = eng.max_context
            out["mtp"] = {"enabled": eng.runner_has_mtp() and eng.spec.enabled,
                          "max_drafts": eng.spec.max_drafts}
            out["prompt_lookup"] = {"enabled": bool(eng.spec.prompt_lookup and eng.spec.enabled)}
            out["active_requests"], out["queued_requests"] = out["active"], out["queued"]
            pager = getattr(eng.runner, "pager", None)
            if pager is not None:
                out["expert_pager"] = pager.stats.as_dict()
        out["preparation"] = self.preparation.snapshot()
        if getattr(self.codec, "boundary", None) is not None:
            out["tokenization_cache"] = self.codec.boundary.cache_statistics()
        images = getattr(self.codec, "images", None)
        if images is not None:
            out["image_cache"] = {"entries": len(images.cache._items), "bytes": images.cache.bytes,
                                  "budget_bytes": images.cache.budget}
            out["chat_capabilities"]["images"] = True
        out["output_pipeline"] = "thread" if self.worker.pipeline is not None else "inline"
        return out


def _chunk(job: Job, model: str, delta: dict, finish: Optional[str] = None,
           logprobs=None, usage=None) -> str:
    choice: Dict[str, Any] = {"index": 0, "delta": delta, "finish_reason": finish}
    if logprobs:
        choice["logprobs"] = {"content": logprobs}
    body = {"id": job.rid, "object": "chat.completion.chunk", "created": job.created_unix,
            "model": model, "choices": [choice] if delta is not None else []}
    if usage is not None:
        body["usage"] = usage
    return "data: " + json.dumps(body, ensure_ascii=False) + "\n\n"


def _delta_dict(d) -> dict:
    out: Dict[str, Any] = {}
    if d.content:
        out["content"] = d.content
    if d.reasoning:
        out["reasoning_content"] = d.reasoning
    if d.tool_calls:
        out["tool_calls"] = d.tool_calls
    return out


def create_app(service: Service, body_limit: int = BODY_LIMIT) -> FastAPI:
    app = FastAPI(title="orinfer-b200", docs_url=None, redoc_url=None)
    key = api_key()

    @app.middleware("http")
    async def request_id(request: HttpRequest, call_next):
        rid = request.headers.get("x-request-id") or uuid.uuid4().hex
        size = int(request.headers.get("content-length") or 0)
        resp = refuse_unauthorized(key, request)
        if resp is not None:
            pass
        elif size > body_limit:
            resp = _error(413, "request body too large", code="body_too_large")
        else:
            resp = await call_next(request)
        resp.headers["x-request-id"] = rid
        return resp

    @app.exception_handler(404)
    async def not_found(request: HttpRequest, exc):
        return _error(404, f"no route {request.method} {request.url.path}", code="not_found")

    @app.exception_handler(405)
    async def wrong_method(request: HttpRequest, exc):
        return _error(405, f"{request.method} is not allowed on {request.url.path}",
                      code="method_not_allowed")

    @app.get("/health")
    async def health():
        body = service.health()
        ok = service.lifecycle.state in (Lifecycle.READY, Lifecycle.DRAINING)
        return JSONResponse(body, status_code=200 if ok else 503)

    @app.get("/metrics")
    async def metrics():
        return PlainTextResponse(service.metrics.render(),
                                 media_type="text/plain; version=0.0.4")

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": service.model_name, "object": "model",
                                            "created": int(service.started),
                                            "owned_by": "orinfer"}]}

    @app.get("/v1/models/{model_id:path}")
    async def model(model_id: str):
        if model_id != service.model_name:
            return _error(404, f"model `{model_id}` is not served here", code="model_not_found",
                          param="model")
        return {"id": service.model_name, "object": "model", "created": int(service.started),
                "owned_by": "orinfer"}

    async def _json(request: HttpRequest):
        try:
            return json.loads(await request.body())
        except (json.JSONDecodeError, UnicodeDecodeError):
            raise RequestError("request body is not valid JSON")

    @app.post("/v1/chat/completions/render")
    async def render(request: HttpRequest):
        try:
            body = await _json(request)
            if isinstance(body, dict) and body.pop("return_mm_kwargs", False):
                raise RequestError("only false is supported: render returns token ids, no "
                                   "tensors", param="return_mm_kwargs")
            p = service.codec.prepare(body, service.defaults)
        except RequestError as e:
            return JSONResponse(e.body(), status_code=e.status)
        media = bool(p.images) or bool(p.audio)
        return {"model": p.model, "token_ids": p.prompt_ids, "token_count": len(p.prompt_ids),
                "multimodal": media,
                # the same under the names this server used first
                "prompt": p.prompt_text, "prompt_token_ids": p.prompt_ids,
                "prompt_tokens": len(p.prompt_ids), "max_tokens": p.max_new}

    @app.post("/v1/chat/completions")
    async def completions(request: HttpRequest):
        try:
            job = await service.submit_async(await _json(request), asyncio.get_running_loop())
        except RequestError as e:
            headers = {"Retry-After": "1"} if e.status == 429 else None
            return JSONResponse(e.body(), status_code=e.status, headers=headers)
        model = job.prepared.model
        if job.prepared.stream:
            async def sse():
                ended = False
                try:
                    async for ev in service.events(job):
                        ended = ended or ev["type"] in ("done", "error")
                        if ev["type"] == "start":
                            yield _chunk(job, model, {"role": "assistant", "content": ""})
                        elif ev["type"] == "delta":
                            yield _chunk(job, model, _delta_dict(ev["delta"]),
                                         logprobs=ev.get("logprobs"))
                        elif ev["type"] == "done":
                            yield _chunk(job, model, {}, finish=ev["finish_reason"])
                            if job.prepared.include_usage:
                                yield _chunk(job, model, None, usage=ev["usage"])
                            yield "data: [DONE]\n\n"
                        else:
                            yield "data: " + json.dumps({"error": {
                                "message": ev["message"], "type": "server_error", "param": None,
                                "code": ev.get("code")}}) + "\n\n"
                            yield "data: [DONE]\n\n"
                    if not ended:
                        # a stream that just stops is an error, not a short success
                        yield "data: " + json.dumps({"error": {
                            "message": "the response ended without a result",
                            "type": "server_error", "param": None,
                            "code": "incomplete_response"}}) + "\n\n"
                        yield "data: [DONE]\n\n"
                finally:
                    job.cancelled = True          # client went away or stream ended
            return StreamingResponse(sse(), media_type="text/event-stream")
        content, reasoning, calls, lps = "", "", [], []
        async for ev in service.events(job):
            if ev["type"] == "delta":
                content += ev["delta"].content
                reasoning += ev["delta"].reasoning
                calls += ev["delta"].tool_calls
                lps += ev.get("logprobs") or []
            elif ev["type"] == "error":
                return _error(ev.get("status", 500), ev["message"], ev.get("code"),
                              err_type="server_error" if ev.get("status", 500) >= 500
                              else "invalid_request_error")
            elif ev["type"] == "done":
                msg: Dict[str, Any] = {"role": "assistant", "content": content or None
                                       if calls else content}
                if reasoning:
                    msg["reasoning_content"] = reasoning
                if calls:
                    from .output_parser import merge_tool_calls
                    msg["tool_calls"] = merge_tool_calls(calls)
                choice: Dict[str, Any] = {"index": 0, "message": msg,
                                          "finish_reason": ev["finish_reason"]}
                if job.prepared.want_logprobs:
                    choice["logprobs"] = {"content": lps}
                return {"id": job.rid, "object": "chat.completion",
                        "created": int(time.time()), "model": model, "choices": [choice],
                        "usage": ev["usage"]}
        return _error(500, "request ended without a result", err_type="server_error")

    from .encoders import install as install_encoders
    from .ollama import install as install_ollama
    from .audio import install as install_audio
    from .completions import install as install_completions
    install_completions(app, service)
    install_encoders(app, service)
    install_ollama(app, service)
    install_audio(app, service)
    return app
