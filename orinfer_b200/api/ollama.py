"""Ollama-compatible routes: requests are translated to the native chat request, responses
to Ollama's NDJSON stream (``stream`` defaults to true) with nanosecond durations.

Routes and semantics follow crates/orinfer-api/src/manager/ollama/mod.rs:47-59,
ollama/request.rs:9-75,76-280 (``think``, ``format``, ``tools``, ``options``,
``keep_alive`` forms) and ollama/response.rs:19-350; registry operations
(``pull``/``push``/``create``), raw prompts and template overrides answer explicit errors.
"""

from __future__ import annotations

import asyncio
import datetime as _dt
import json
import re
import time
from typing import Any, Dict, Optional

from fastapi import FastAPI, Request as HttpRequest
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from .chat_codec import RequestError

VERSION = "0.12.0"
OPTION_MAP = {"temperature": "temperature", "top_p": "top_p", "top_k": "top_k", "seed": "seed",
              "presence_penalty": "presence_penalty", "frequency_penalty": "frequency_penalty",
              "repeat_penalty": "repetition_penalty", "num_predict": "max_tokens",
              "stop": "stop"}


def parse_keep_alive(value) -> Optional[float]:
    """Seconds; None = default, negative = keep, 0 = unload now.  Accepts numbers and
    duration strings such as ``"1h30m"`` or ``"60s"``."""
    if value is None:
        return None
    if isinstance(value, (int, float)):
        return float(value)
    if isinstance(value, str):
        s = value.strip()
        if re.fullmatch(r"-?\d+(\.\d+)?", s):
            return float(s)
        total, pos = 0.0, 0
        sign = -1.0 if s.startswith("-") else 1.0
        s = s.lstrip("+-")
        units = {"ns": 1e-9, "us": 1e-6, "ms": 1e-3, "s": 1, "m": 60, "h": 3600}
        for m in re.finditer(r"(\d+(?:\.\d+)?)(ns|us|ms|s|m|h)", s):
            if m.start() != pos:
                raise RequestError("invalid keep_alive duration", param="keep_alive")
            total += float(m.group(1)) * units[m.group(2)]
            pos = m.end()
        if pos != len(s) or pos == 0:
            raise RequestError("invalid keep_alive duration", param="keep_alive")
        return sign * total
    raise RequestError("invalid keep_alive", param="keep_alive")


def _content(text, images):
    """Ollama ``images`` (bare base64 strings) -> ``image_url`` parts with a data URI whose
    media type is read from the file signature (PNG, JPEG or WebP only)."""
    if not images:
        return text
    import base64
    import binascii
    if not isinstance(images, list):
        raise RequestError("`images` must be an array of base64 strings", param="images")
    parts = [{"type": "text", "text": text or ""}]
    for item in images:
        try:
            head = base64.b64decode(item[:64] + "=" * (-len(item[:64]) % 4))[:16] \
                if isinstance(item, str) else None
        except (binascii.Error, ValueError):
            head = None
        if head is None:
            raise RequestError("invalid base64 image", param="images")
        if head.startswith(b"\x89PNG\r\n\x1a\n"):
            mime = "image/png"
        elif head.startswith(b"\xff\xd8\xff"):
            mime = "image/jpeg"
        elif head[:4] == b"RIFF" and head[8:12] == b"WEBP":
            mime = "image/webp"
        else:
            raise RequestError("images must be PNG, JPEG or WebP", param="images")
        parts.append({"type": "image_url", "image_url": {"url": f"data:{mime};base64,{item}"}})
    return parts


def _link_tool_messages(messages: list) -> list:
    """Ollama histories carry tool calls without ids and tool results named by ``tool_name``;
    the native history wants every call identified and every result bound to its call.  Calls
    without an id get ``call_N``; a result without ``tool_call_id`` answers the oldest open
    call of its ``tool_name`` (or the oldest open call when it names none)."""
    out, open_calls, made = [], [], 0
    for m in messages:
        if not isinstance(m, dict):
            out.append(m)
            continue
        m = dict(m)
        if m.get("role") == "assistant" and isinstance(m.get("tool_calls"), list):
            calls = []
            for c in m["tool_calls"]:
                if isinstance(c, dict):
                    c = dict(c)
                    if not c.get("id"):
                        made += 1
                        c["id"] = f"call_{made}"
                    c.setdefault("type", "function")
                    fn = c.get("function")
                    open_calls.append((c["id"], fn.get("name") if isinstance(fn, dict) else None))
                calls.append(c)
            m["tool_calls"] = calls
        elif m.get("role") == "tool":
            if m.get("tool_call_id"):
                open_calls = [c for c in open_calls if c[0] != m["tool_call_id"]]
            else:
                name = m.get("tool_name") or m.get("name")
                pick = next((c for c in open_calls if name and c[1] == name), None) \
                    or (open_calls[0] if open_calls else None)
                if pick is not None:
                    open_calls.remove(pick)
                    m["tool_call_id"] = pick[0]
        out.append(m)
    return out


class CallAssembler:
    """The native stream delivers a tool call as fragments (name first, then pieces of the
    argument text); this protocol shows a call once, whole, with its arguments as an object.
    ``feed`` returns the calls that became complete; ``flush`` what was cut off."""

    def __init__(self):
        self.open: Dict[int, Dict[str, str]] = {}

    def feed(self, fragments) -> list:
        for c in fragments:
            e = self.open.setdefault(c.get("index", 0), {"name": "", "arguments": ""})
            fn = c.get("function") or {}
            e["name"] += fn.get("name") or ""
            e["arguments"] += fn.get("arguments") or ""
        done = []
        for index in sorted(self.open):
            e = self.open[index]
            try:                                   # a proper prefix of an object never parses
                args = json.loads(e["arguments"]) if e["arguments"] else None
            except ValueError:
                continue
            if isinstance(args, dict):
                done.append({"function": {"name": e["name"], "arguments": args}})
                del self.open[index]
        return done

    def flush(self) -> list:
        from .messages import RAW_ARGUMENTS
        out = [{"function": {"name": e["name"],
                             "arguments": {RAW_ARGUMENTS: e["arguments"]} if e["arguments"] else {}}}
               for _i, e in sorted(self.open.items())]
        self.open = {}
        return out


def translate(body: Dict[str, Any], generate: bool) -> Dict[str, Any]:
    """Ollama request -> native chat request."""
    if not isinstance(body, dict):
        raise RequestError("request body must be a JSON object")
    if body.get("raw"):
        raise RequestError("raw prompts are not supported", param="raw")
    if body.get("template"):
        raise RequestError("template overrides are not supported", param="template")
    out: Dict[str, Any] = {"model": body.get("model")}
    if generate:
        msgs = []
        if body.get("system"):
            msgs.append({"role": "system", "content": body["system"]})
        msgs.append({"role": "user", "content": _content(body.get("prompt", ""),
                                                          body.get("images"))})
        if body.get("suffix"):
            raise RequestError("suffix is not supported", param="suffix")
        out["messages"] = msgs
    else:
        out["messages"] = _link_tool_messages(
            [dict({k: v for k, v in m.items() if k != "images"},
                  content=_content(m.get("content", ""), m["images"]))
             if isinstance(m, dict) and m.get("images") else m
             for m in body.get("messages") or []])
    out["output_limit"] = "clamp"
    opts = body.get("options") or {}
    for k, v in opts.items():
        if k in OPTION_MAP:
            out[OPTION_MAP[k]] = v
        elif k in ("num_ctx", "num_keep", "num_gpu", "num_thread", "num_batch", "min_p",
                   "typical_p", "mirostat", "mirostat_tau", "mirostat_eta", "repeat_last_n",
                   "tfs_z", "penalize_newline", "use_mmap", "numa", "main_gpu", "low_vram"):
            continue                                  # accepted, no native equivalent
        else:
            raise RequestError(f"unknown option `{k}`", param=f"options.{k}")
    if out.get("max_tokens") is not None and out["max_tokens"] < 0:
        out.pop("max_tokens")
    think = body.get("think")
    if think is not None:
        if isinstance(think, str):
            out["reasoning_effort"] = think
        else:
            out["enable_thinking"] = bool(think)
    fmt = body.get("format")
    if fmt == "json":
        out["response_format"] = {"type": "json_object"}
    elif isinstance(fmt, dict):
        out["response_format"] = {"type": "json_schema",
                                  "json_schema": {"name": "format", "schema": fmt}}
    elif fmt not in (None, ""):
        raise RequestError("format must be \"json\" or a JSON schema", param="format")
    if body.get("tools"):
        out["tools"] = body["tools"]
    if body.get("logprobs"):
        out["logprobs"] = True
        if body.get("top_logprobs") is not None:
            out["top_logprobs"] = body["top_logprobs"]
    parse_keep_alive(body.get("keep_alive"))
    out["stream"] = body.get("stream", True)
    return out


def _now() -> str:
    return _dt.datetime.now(_dt.timezone.utc).isoformat().replace("+00:00", "Z")


def install(app: FastAPI, service) -> None:
    def model_entry() -> dict:
        return {"name": service.model_name, "model": service.model_name,
                "modified_at": _now(), "size": 0, "digest": "",
                "details": {"format": "orinfer-e8p", "family": "orinfer",
                            "parameter_size": "", "quantization_level": "E8P-Q4A8"}}

    @app.get("/")
    async def root():
        return PlainTextResponse("Orinfer is running")

    @app.get("/api/version")
    async def version():
        return {"version": VERSION}

    @app.get("/api/tags")
    async def tags():
        return {"models": [model_entry()]}

    @app.get("/api/ps")
    async def ps():
        entry = model_entry()
        entry["expires_at"] = _now()
        entry["size_vram"] = 0
        return {"models": [entry]}

    @app.post("/api/show")
    async def show(request: HttpRequest):
        body = json.loads(await request.body() or b"{}")
        name = body.get("model") or body.get("name")
        if name not in (service.model_name, None):
            return JSONResponse({"error": f"model '{name}' not found"}, status_code=404)
        eng = service.worker.engine
        info = {} if eng is None else {"general.architecture": eng.cfg.arch,
                                       "context_length": eng.max_context}
        return {"details": model_entry()["details"], "model_info": info,
                "capabilities": ["completion", "tools", "thinking"], "template": "",
                "parameters": ""}

    async def run(request: HttpRequest, generate: bool):
        started = time.perf_counter_ns()
        try:
            body = json.loads(await request.body() or b"{}")
            if not generate and not body.get("messages") or generate and not body.get("prompt"):
                # an empty request only loads (or unloads) the model
                key = "response" if generate else "message"
                val = "" if generate else {"role": "assistant", "content": ""}
                return {"model": body.get("model"), "created_at": _now(), key: val,
                        "done": True, "done_reason": "load"}
            native = translate(body, generate)
            stream = native.pop("stream")
            native["stream"] = False
            job = service.submit(native, asyncio.get_running_loop())
        except RequestError as e:
            return JSONResponse({"error": e.message}, status_code=e.status)
        except json.JSONDecodeError:
            return JSONResponse({"error": "invalid JSON"}, status_code=400)
        model = body.get("model") or service.model_name
        first_token_ns: Optional[int] = None

        def frame(content="", thinking="", calls=None, done=False, final=None) -> dict:
            out: Dict[str, Any] = {"model": model, "created_at": _now()}
            if generate:
                out["response"] = content
                if thinking:
                    out["thinking"] = thinking
            else:
                msg: Dict[str, Any] = {"role": "assistant", "content": content}
                if thinking:
                    msg["thinking"] = thinking
                if calls:
                    msg["tool_calls"] = calls              # whole calls (CallAssembler)
                out["message"] = msg
            out["done"] = done
            if final:
                out.update(final)
            return out

        def finals(ev) -> dict:
            now = time.perf_counter_ns()
            u = ev["usage"]
            first = first_token_ns or now
            return {"done_reason": "length" if ev["finish_reason"] == "length" else "stop",
                    "total_duration": now - started, "load_duration": 0,
                    "prompt_eval_count": u["prompt_tokens"],
                    "prompt_eval_duration": first - started,
                    "eval_count": u["completion_tokens"], "eval_duration": now - first}

        assembler = CallAssembler()
        if stream:
            async def ndjson():
                nonlocal first_token_ns
                ended = False
                try:
                    async for ev in service.events(job):
                        ended = ended or ev["type"] in ("done", "error")
                        if ev["type"] == "delta":
                            first_token_ns = first_token_ns or time.perf_counter_ns()
                            d = ev["delta"]
                            whole = assembler.feed(d.tool_calls)
                            if d.content or d.reasoning or whole:
                                yield json.dumps(frame(d.content, d.reasoning, whole),
                                                 ensure_ascii=False) + "\n"
                        elif ev["type"] == "done":
                            yield json.dumps(frame(calls=assembler.flush(), done=True,
                                                   final=finals(ev))) + "\n"
                        elif ev["type"] == "error":
                            yield json.dumps({"error": ev["message"]}) + "\n"
                    if not ended:
                        # a stream that just stops is an error, not a short success
                        yield json.dumps({"error": "the response ended without a result"}) + "\n"
                finally:
                    job.cancelled = True
            return StreamingResponse(ndjson(), media_type="application/x-ndjson")
        content, thinking, calls = "", "", []
        async for ev in service.events(job):
            if ev["type"] == "delta":
                first_token_ns = first_token_ns or time.perf_counter_ns()
                content += ev["delta"].content
                thinking += ev["delta"].reasoning
                calls += assembler.feed(ev["delta"].tool_calls)
            elif ev["type"] == "error":
                return JSONResponse({"error": ev["message"]}, status_code=ev.get("status", 500))
            elif ev["type"] == "done":
                return frame(content, thinking, calls + assembler.flush(), True, finals(ev))
        return JSONResponse({"error": "request ended without a result"}, status_code=500)

    @app.post("/api/chat")
    async def chat(request: HttpRequest):
        return await run(request, False)

    @app.post("/api/generate")
    async def generate(request: HttpRequest):
        return await run(request, True)

    async def _embed(request: HttpRequest, legacy: bool):
        """Ollama embedding routes on top of the native encoder pass: ``/api/embed`` takes
        ``input`` (string or array) and answers ``embeddings`` (one vector per input);
        the older ``/api/embeddings`` takes ``prompt`` and answers one ``embedding``."""
        import asyncio
        from .encoders import embeddings as native_embeddings
        started = time.perf_counter_ns()
        try:
            body = await request.json()
            if not isinstance(body, dict):
                raise RequestError("request body must be a JSON object")
            value = body.get("prompt") if legacy else body.get("input")
            out = await asyncio.get_running_loop().run_in_executor(
                None, native_embeddings, service,
                {"input": value, "input_type": "document",
                 **({"dimensions": body["dimensions"]} if "dimensions" in body else {})})
        except RequestError as e:
            return JSONResponse({"error": e.message}, status_code=e.status)
        except (MemoryError, ValueError) as e:
            return JSONResponse({"error": str(e)}, status_code=400)
        vectors = [d["embedding"] for d in out["data"]]
        if legacy:
            return {"embedding": vectors[0]}
        return {"model": body.get("model") or service.model_name, "embeddings": vectors,
                "total_duration": time.perf_counter_ns() - started, "load_duration": 0,
                "prompt_eval_count": out["usage"]["prompt_tokens"]}

    @app.post("/api/embed")
    async def embed(request: HttpRequest):
        return await _embed(request, legacy=False)

    @app.post("/api/embeddings")
    async def embeddings_legacy(request: HttpRequest):
        return await _embed(request, legacy=True)

    @app.post("/api/copy")
    async def copy(request: HttpRequest):
        return JSONResponse({"error": "aliases need the model manager (orinfer serve "
                                      "without a model path)"}, status_code=501)

    @app.delete("/api/delete")
    async def delete(request: HttpRequest):
        return JSONResponse({"error": "unregistering needs the model manager"}, status_code=501)

    @app.api_route("/api/{path:path}", methods=["GET", "POST", "PUT", "DELETE", "HEAD"])
    async def unsupported(path: str):
        return JSONResponse({"error": f"/api/{path} is not supported by orinfer (registry "
                                      "operations such as pull, push and create are "
                                      "unavailable)"}, status_code=501)
