"""``POST /v1/audio/transcriptions``: multipart upload -> log-mel -> audio encoder features
overlaid on the placeholder rows of a transcription prompt -> ordinary generation.

Request fields and limits follow the reference (docs/audio.md:19-32,
crates/orinfer-api/src/server/audio.rs:18-370): ``file`` (at most 24 MiB and 1 200 s),
``language``, ``prompt``, ``temperature``, ``response_format`` ``json`` | ``text``; ``model`` is
accepted and echoed.  The front end runs on the preparation pool, like chat templating.
"""

from __future__ import annotations

import dataclasses
from typing import List, Optional, Tuple

from fastapi import FastAPI
from fastapi import Request as HttpRequest
from fastapi.responses import JSONResponse, PlainTextResponse

from ..models import audio as A
from .chat_codec import Prepared, RequestError

MAX_UPLOAD_BYTES = 24 << 20
AUDIO_TEXT = "<|audio_start|><|audio_pad|><|audio_end|>"


@dataclasses.dataclass
class BoundAudio:
    inputs: List[A.AudioInput]
    spans: List[Tuple[int, int]]


def prepare_transcription(codec, data: bytes, language: Optional[str], prompt: Optional[str],
                          temperature: float, max_tokens: Optional[int],
                          defaults: Optional[dict] = None) -> Prepared:
    tok = codec.tokenizer
    pad = tok.token_id("<|audio_pad|>")
    if pad is None:
        raise RequestError("this model takes no audio inputs", param="file")
    if len(data) > MAX_UPLOAD_BYTES:
        raise RequestError("audio file exceeds 24 MiB", param="file", status=413)
    try:
        audio = A.load_audio(data)
        n = audio.features
    except A.AudioError as e:
        raise RequestError(str(e), param="file")
    body = {"messages": [{"role": "user", "content": "."}], "temperature": temperature,
            "enable_thinking": False}
    if max_tokens is not None:
        body["max_tokens"] = max_tokens
    base = codec.prepare(body, defaults)
    b = codec.boundary
    ctl = b.controls if b is not None else (lambda t: t)
    esc = b.escape if b is not None else (lambda t: t)
    text = ""
    if prompt:
        if not isinstance(prompt, str):
            raise RequestError("`prompt` must be text", param="prompt")
        text += ctl("<|im_start|>system\n") + esc(prompt) + ctl("<|im_end|>\n")
    text += ctl(f"<|im_start|>user\n{AUDIO_TEXT}<|im_end|>\n<|im_start|>assistant\n")
    if language:
        if not isinstance(language, str) or len(language) > 32 or \
                not language.replace("-", "").isalnum():
            raise RequestError("`language` must be a language name or code", param="language")
        text += f"language {language}\n"
    ids = []
    for t in codec.encode_rendered(text):
        ids += [t] * n if t == pad else [t]
    text = codec.display(text)
    start = ids.index(pad)
    if len(ids) >= codec.context:
        raise RequestError(f"the audio needs {len(ids)} prompt tokens, beyond the context window "
                           f"of {codec.context}", param="file", code="context_length_exceeded")
    return dataclasses.replace(
        base, prompt_ids=ids, prompt_text=text, stream=False, thinking=False,
        max_new=min(base.max_new, codec.context - len(ids)),
        audio=BoundAudio([audio], [(start, start + n)]))


def install(app: FastAPI, service) -> None:
    import asyncio

    @app.post("/v1/audio/transcriptions")
    async def transcriptions(request: HttpRequest):
        try:
            form = await request.form()
            upload = form.get("file")
            if upload is None or not hasattr(upload, "read"):
                raise RequestError("multipart field `file` is required", param="file")
            data = await upload.read()
            fmt = form.get("response_format") or "json"
            if fmt not in ("json", "text"):
                raise RequestError("`response_format` must be json or text",
                                   param="response_format")
            try:
                temperature = float(form.get("temperature") or 0.0)
                max_tokens = int(form["max_tokens"]) if form.get("max_tokens") else None
            except ValueError:
                raise RequestError("`temperature` / `max_tokens` must be numbers",
                                   param="temperature")
            from .preparation import BASE_BYTES
            prepared = await service.preparation.run(
                lambda: prepare_transcription(service.codec, data, form.get("language"),
                                              form.get("prompt"), temperature, max_tokens,
                                              service.defaults),
                BASE_BYTES + 24 * len(data))
            job = service.submit({}, asyncio.get_running_loop(), prepared)
        except RequestError as e:
            headers = {"Retry-After": "1"} if e.status == 429 else None
            return JSONResponse(e.body(), status_code=e.status, headers=headers)
        text = ""
        async for ev in service.events(job):
            if ev["type"] == "delta":
                text += ev["delta"].content
            elif ev["type"] == "error":
                return JSONResponse({"error": {"message": ev["message"], "type": "server_error",
                                               "param": None, "code": ev.get("code")}},
                                    status_code=ev.get("status", 500))
            elif ev["type"] == "done":
                if fmt == "text":
                    return PlainTextResponse(text)
                return {"text": text, "usage": {"type": "tokens",
                                                "input_tokens": ev["usage"]["prompt_tokens"],
                                                "output_tokens": ev["usage"]["completion_tokens"],
                                                "total_tokens": ev["usage"]["total_tokens"]}}
        return JSONResponse({"error": {"message": "request ended without a result",
                                       "type": "server_error", "param": None, "code": None}},
                            status_code=500)
