"""``POST /v1/completions``: raw-prompt completions, with the prompt given as text or as token
ids.

Not a route of the reference's own server — its benchmark harness drives competitors through
this OpenAI route (tools/bench/reference_bench.py:1-40: token-id prompts, ``ignore_eos``, fixed
seed), and exact-length token-id prompts are what makes HTTP-level prefill / decode rates
comparable with the engine harness.  No chat template, no thinking section, no tool parsing:
the output is the detokenised continuation.  ``return_token_ids`` adds the committed token ids
(one SSE chunk per token when streaming), which also makes the arrival of tokens visible when
their text is withheld or unprintable.
"""

from __future__ import annotations

import asyncio
import dataclasses
import json
import time
import uuid
from typing import Any, Dict

from fastapi import FastAPI
from fastapi import Request as HttpRequest
from fastapi.responses import JSONResponse, StreamingResponse

from .chat_codec import Prepared, RequestError

FIELDS = {"model", "prompt", "max_tokens", "temperature", "top_p", "top_k", "seed", "stop",
          "stream", "stream_options", "ignore_eos", "presence_penalty", "frequency_penalty",
          "repetition_penalty", "logit_bias", "n", "user", "echo", "cache_prompt",
          "return_token_ids"}


def prepare_completion(codec, body: Dict[str, Any], defaults=None) -> Prepared:
    if not isinstance(body, dict):
        raise RequestError("request body must be a JSON object")
    unknown = sorted(set(body) - FIELDS)
    if unknown:
        raise RequestError(f"unknown field `{unknown[0]}`", param=unknown[0])
    if body.get("echo"):
        raise RequestError("`echo` is not supported", param="echo")
    prompt = body.get("prompt")
    vocab = getattr(codec.tokenizer, "vocab", None)
    if isinstance(prompt, str) and prompt:
        ids = (codec.boundary.encode(codec.boundary.escape(prompt)) if codec.boundary
               else codec.tokenizer.encode(prompt))
        text = prompt
    elif isinstance(prompt, list) and prompt and all(
            isinstance(t, int) and not isinstance(t, bool) and 0 <= t and
            (vocab is None or t < vocab) for t in prompt):
        ids, text = list(prompt), ""
    else:
        raise RequestError("`prompt` must be a non-empty string or an array of token ids",
                           param="prompt")
    chat = {k: v for k, v in body.items() if k not in ("prompt", "echo", "return_token_ids")}
    chat.update(messages=[{"role": "user", "content": "."}], enable_thinking=False)
    base = codec.prepare(chat, defaults)
    if len(ids) >= codec.context:
        raise RequestError(f"the prompt of {len(ids)} tokens exceeds the context window of "
                           f"{codec.context} tokens", param="prompt",
                           code="context_length_exceeded")
    want = body.get("max_tokens", 16)
    if not isinstance(want, int) or want < 1:
        raise RequestError("`max_tokens` must be a positive integer", param="max_tokens")
    return dataclasses.replace(base, prompt_ids=ids, prompt_text=text, thinking=False, tools=[],
                               max_new=min(want, codec.context - len(ids)),
                               token_events=bool(body.get("return_token_ids")))


def install(app: FastAPI, service) -> None:
    def plain_chunk(rid, model, text, finish=None, usage=None, choices=True, token=None,
                    created=None):
        choice = {"index": 0, "text": text, "finish_reason": finish}
        if token is not None:
            choice["token_ids"] = [token]
        body = {"id": rid, "object": "text_completion",
                "created": int(time.time()) if created is None else created,
                "model": model, "choices": [choice] if choices else []}
        if usage is not None:
            body["usage"] = usage
        return "data: " + json.dumps(body, ensure_ascii=False) + "\n\n"

    @app.post("/v1/completions")
    async def completions(request: HttpRequest):
        try:
            try:
                body = json.loads(await request.body())
            except (json.JSONDecodeError, UnicodeDecodeError):
                raise RequestError("request body is not valid JSON")
            from .preparation import estimate_bytes
            prepared = await service.preparation.run(
                lambda: prepare_completion(service.codec, body, service.defaults),
                estimate_bytes(body))
            job = service.submit({}, asyncio.get_running_loop(), prepared)
        except RequestError as e:
            headers = {"Retry-After": "1"} if e.status == 429 else None
            return JSONResponse(e.body(), status_code=e.status, headers=headers)
        rid = "cmpl-" + uuid.uuid4().hex[:24]
        model = prepared.model
        if prepared.stream:
            import functools
            chunk = functools.partial(plain_chunk, created=job.created_unix)   # one per stream

            async def sse():
                try:
                    async for ev in service.events(job):
                        if ev["type"] == "token":
                            yield chunk(rid, model, "", token=ev["token"])
                        elif ev["type"] == "delta" and ev["delta"].content:
                            yield chunk(rid, model, ev["delta"].content)
                        elif ev["type"] == "done":
                            yield chunk(rid, model, "", finish=ev["finish_reason"])
                            if prepared.include_usage:
                                yield chunk(rid, model, "", usage=ev["usage"], choices=False)
                            yield "data: [DONE]\n\n"
                        elif ev["type"] == "error":
                            yield "data: " + json.dumps({"error": {
                                "message": ev["message"], "type": "server_error", "param": None,
                                "code": ev.get("code")}}) + "\n\n"
                            yield "data: [DONE]\n\n"
                finally:
                    job.cancelled = True
            return StreamingResponse(sse(), media_type="text/event-stream")
        text, token_ids = "", []
        async for ev in service.events(job):
            if ev["type"] == "token":
                token_ids.append(ev["token"])
            elif ev["type"] == "delta":
                text += ev["delta"].content
            elif ev["type"] == "error":
                status = ev.get("status", 500)
                return JSONResponse({"error": {"message": ev["message"], "param": None,
                                               "type": "server_error" if status >= 500
                                               else "invalid_request_error",
                                               "code": ev.get("code")}}, status_code=status)
            elif ev["type"] == "done":
                return {"id": rid, "object": "text_completion", "created": int(time.time()),
                        "model": model, "usage": ev["usage"],
                        "choices": [dict({"index": 0, "text": text,
                                          "finish_reason": ev["finish_reason"]},
                                         **({"token_ids": token_ids} if prepared.token_events
                                            else {}))]}
        return JSONResponse({"error": {"message": "request ended without a result",
                                       "type": "server_error", "param": None, "code": None}},
                            status_code=500)
