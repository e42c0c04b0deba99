"""Multi-model manager: a persistent registry of named models (with aliases), runners
started on demand and shared by every name that resolves to the same runner key, leases
that count requests in flight, a memory budget with idle eviction, a keep-alive sweep and a
short negative cache for failed starts.

The reference runs one child ``orinfer serve`` process per runner key behind a gateway
(crates/orinfer-api/src/manager/mod.rs:32-96,159-372,430-560,674-727; behaviour pinned by
manager/tests.rs:18-43).  Here a runner is an in-process ``Service`` (one engine thread each,
all sharing the GPU's one CUDA context), which keeps start-up at weight-load time and lets
runners share the process-wide kernel library; the registry, lease, budget and keep-alive
semantics are the same.  ``install`` adds the gateway routes that need the registry
(``/api/copy``, ``/api/delete``, ``/api/tags``, ``/api/ps``, model-dispatching chat).
"""

from __future__ import annotations

import json
import threading
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Dict, List, Optional

from fastapi import Request as HttpRequest
from fastapi.responses import JSONResponse, PlainTextResponse, Response

NEGATIVE_CACHE_S = 10.0
DEFAULT_KEEP_ALIVE_S = 300.0


class ManagerError(ValueError):
    def __init__(self, message: str, status: int = 400):
        super().__init__(message)
        self.status = status


@dataclass
class Entry:
    name: str
    path: str
    options: Dict[str, object] = field(default_factory=dict)     # execution-affecting options
    defaults: Dict[str, object] = field(default_factory=dict)    # sampling defaults (no fork)

    def runner_key(self) -> str:
        return json.dumps([str(Path(self.path).resolve()), self.options], sort_keys=True)


@dataclass
class Runner:
    key: str
    service: object
    bytes: int
    leases: int = 0
    last_used: float = field(default_factory=time.monotonic)
    keep_alive_s: float = DEFAULT_KEEP_ALIVE_S


class ModelManager:
    """``start(entry) -> (service, bytes)`` builds and starts a runner; ``stop(service)``
    retires it.  Both run under the transition lock, so starts and stops are serialised while
    models that are already up keep serving (their requests take only the table lock).

    ``estimate(entry) -> bytes`` (optional) sizes a model before it is started, so that room
    is made under the memory budget first; ``alive(service) -> bool`` (optional, default the
    service's own ``alive()``) lets a runner that died be noticed and started again by the
    next request.  When the budget is held by models in use, a request waits up to
    ``capacity_wait_s`` for one of them to go idle (a waiter whose client left is not loaded
    afterwards).  A start that failed is remembered for a short while and shared by everyone
    who was waiting for it."""

    def __init__(self, state_dir, start: Callable[[Entry], tuple], stop: Callable[[object], None],
                 memory_budget_bytes: int = 0, clock: Callable[[], float] = time.monotonic,
                 estimate: Optional[Callable[[Entry], int]] = None,
                 alive: Optional[Callable[[object], bool]] = None,
                 capacity_wait_s: float = 0.0, max_loaded: int = 0):
        self.state = Path(state_dir)
        self.state.mkdir(parents=True, exist_ok=True)
        self._start, self._stop = start, stop
        self._estimate, self._alive = estimate, alive
        self.capacity_wait_s = capacity_wait_s
        self.max_loaded = max_loaded               # 0: no limit on the number of runners
        self.budget = memory_budget_bytes
        self.clock = clock
        self._lock = threading.Lock()              # registry + runner table
        self._idle = threading.Condition(self._lock)   # a lease was returned / a runner left
        self._transition = threading.Lock()        # serialises starts / stops
        self.entries: Dict[str, Entry] = {}
        self.runners: Dict[str, Runner] = {}
        self._failed: Dict[str, tuple] = {}        # runner key -> (time, message)
        self.restarts = 0                          # runners found dead and started again
        self._load()

    # ------------------------------------------------------------------ registry
    def _file(self) -> Path:
        return self.state / "registry.json"

    def _load(self) -> None:
        if self._file().exists():
            for e in json.loads(self._file().read_text()):
                self.entries[e["name"]] = Entry(**e)

    def _save(self) -> None:
        tmp = self._file().with_suffix(".tmp")
        tmp.write_text(json.dumps([e.__dict__ for e in self.entries.values()], indent=1))
        tmp.replace(self._file())

    def register(self, name: str, path, options=None, defaults=None) -> Entry:
        if not name or "/" in name.strip("/") and name.startswith("/"):
            raise ManagerError("invalid model name")
        with self._lock:
            e = Entry(name, str(path), dict(options or {}), dict(defaults or {}))
            self.entries[name] = e
            self._save()
            return e

    def copy(self, source: str, destination: str) -> Entry:
        """An alias: same path and options (so the same runner), its own name."""
        with self._lock:
            if source not in self.entries:
                raise ManagerError(f"model '{source}' not found", 404)
            src = self.entries[source]
            e = Entry(destination, src.path, dict(src.options), dict(src.defaults))
            self.entries[destination] = e
            self._save()
            return e

    def remove(self, name: str) -> None:
        with self._lock:
            if name not in self.entries:
                raise ManagerError(f"model '{name}' not found", 404)
            key = self.entries.pop(name).runner_key()
            self._save()
            orphan = all(e.runner_key() != key for e in self.entries.values())
        if orphan:
            self._retire(key, force=False)

    def list(self) -> List[Entry]:
        with self._lock:
            return sorted(self.entries.values(), key=lambda e: e.name)

    def show(self, name: str) -> Entry:
        with self._lock:
            if name not in self.entries:
                raise ManagerError(f"model '{name}' not found", 404)
            return self.entries[name]

    # ------------------------------------------------------------------ runners
    def _is_alive(self, service) -> bool:
        if self._alive is not None:
            return bool(self._alive(service))
        probe = getattr(getattr(service, "service", service), "alive", None)
        return bool(probe()) if callable(probe) else True

    def _lease(self, key: str, keep_alive_s: Optional[float]) -> Optional[Runner]:
        """Under the table lock: a lease on the live runner of ``key``, or None (a runner
        that died is taken out of the table here; its successor is started by the caller)."""
        r = self.runners.get(key)
        if r is None:
            return None
        if not self._is_alive(r.service):
            del self.runners[key]
            self.restarts += 1
            self._idle.notify_all()
            threading.Thread(target=self._stop, args=(r.service,), daemon=True).start()
            return None
        r.leases += 1
        r.last_used = self.clock()
        if keep_alive_s is not None:
            r.keep_alive_s = keep_alive_s
        return r

    def _check_failed(self, name: str, key: str) -> None:
        failed = self._failed.get(key)
        if failed and self.clock() - failed[0] < NEGATIVE_CACHE_S:
            raise ManagerError(f"model '{name}' failed to start: {failed[1]}", 503)

    def acquire(self, name: str, keep_alive_s: Optional[float] = None,
                cancelled: Optional[Callable[[], bool]] = None) -> Runner:
        """Lease on the runner serving ``name`` (started if needed).  Pair with ``release``.
        ``cancelled``: polled while waiting; a caller that has left gets no runner started."""
        entry = self.show(name)
        key = entry.runner_key()
        gone = cancelled or (lambda: False)
        with self._lock:
            r = self._lease(key, keep_alive_s)
            if r is not None:
                return r
            self._check_failed(name, key)
        with self._transition:
            if gone():
                raise ManagerError("the request was cancelled while waiting to start", 499)
            with self._lock:                        # someone else may have started it meanwhile
                r = self._lease(key, keep_alive_s)
                if r is not None:
                    return r
                self._check_failed(name, key)       # ... or failed to: the failure is shared
            try:
                if self._estimate is not None:
                    self._make_room(int(self._estimate(entry)), gone)   # before it takes memory
                service, nbytes = self._start(entry)
            except ManagerError:
                raise
            except Exception as exc:                # noqa: BLE001 - reported to the client
                with self._lock:
                    self._failed[key] = (self.clock(), str(exc))
                raise ManagerError(f"model '{name}' failed to start: {exc}", 503) from exc
            try:
                self._make_room(nbytes, gone)
            except ManagerError:
                self._stop(service)                 # it does not fit after all
                raise
            r = Runner(key, service, nbytes, leases=1, last_used=self.clock(),
                       keep_alive_s=DEFAULT_KEEP_ALIVE_S if keep_alive_s is None else keep_alive_s)
            with self._lock:
                self.runners[key] = r
                self._failed.pop(key, None)
            return r

    def release(self, runner: Runner) -> None:
        with self._lock:
            runner.leases = max(runner.leases - 1, 0)
            runner.last_used = self.clock()
            self._idle.notify_all()

    def _make_room(self, nbytes: int, cancelled: Callable[[], bool] = lambda: False) -> None:
        """Idle eviction under the memory budget: least recently used idle runners go first
        (whatever their keep-alive).  With every runner in use the caller waits up to
        ``capacity_wait_s`` for a lease to come back."""
        if self.budget <= 0 and self.max_loaded <= 0:
            return
        deadline = time.monotonic() + self.capacity_wait_s
        while True:
            with self._lock:
                used = sum(r.bytes for r in self.runners.values())
                fits = self.budget <= 0 or used + nbytes <= self.budget
                if fits and (self.max_loaded <= 0 or len(self.runners) < self.max_loaded):
                    return
                idle = sorted((r for r in self.runners.values() if r.leases == 0),
                              key=lambda r: r.last_used)
                if not idle:
                    left = deadline - time.monotonic()
                    if left <= 0 or 0 < self.budget < nbytes:
                        raise ManagerError("memory budget exhausted by models in use", 503)
                    self._idle.wait(min(left, 0.05))
                    if cancelled():
                        raise ManagerError("the request was cancelled while waiting for "
                                           "memory", 499)
                    continue
                victim = idle[0].key
            self._retire(victim, force=True, locked=True)

    def _retire(self, key: str, force: bool, locked: bool = False) -> bool:
        def go():
            with self._lock:
                r = self.runners.get(key)
                if r is None or (r.leases > 0 and not force):
                    return False
                if r.leases > 0:
                    return False
                del self.runners[key]
                self._idle.notify_all()
            self._stop(r.service)
            return True
        if locked:
            return go()
        with self._transition:
            return go()

    def sweep(self) -> List[str]:
        """Retires idle runners whose keep-alive has run out (0 = retire as soon as idle;
        negative = keep forever).  Returns the retired runner keys."""
        now = self.clock()
        with self._lock:
            due = [r.key for r in self.runners.values()
                   if r.leases == 0 and r.keep_alive_s >= 0 and now - r.last_used >= r.keep_alive_s]
        return [k for k in due if self._retire(k, force=False)]

    def running(self) -> List[dict]:
        with self._lock:
            names = {}
            for e in self.entries.values():
                names.setdefault(e.runner_key(), []).append(e.name)
            return [{"names": sorted(names.get(r.key, [])), "bytes": r.bytes, "leases": r.leases,
                     "idle_s": round(self.clock() - r.last_used, 3),
                     "keep_alive_s": r.keep_alive_s} for r in self.runners.values()]

    def load(self, name: str, keep_alive_s: Optional[float] = None) -> dict:
        """Start the runner of ``name`` ahead of its first request (optionally setting its
        keep-alive) and return its entry of ``running()``."""
        self.release(self.acquire(name, keep_alive_s))
        return next(r for r in self.running() if name in r["names"])

    def unload(self, name: str, force: bool = False) -> bool:
        """Stop the runner of ``name`` and keep its registration.  A runner with requests in
        flight is refused (409) unless ``force``, which ends them.  False when not loaded."""
        key = self.show(name).runner_key()
        with self._transition:
            with self._lock:
                r = self.runners.get(key)
                if r is None:
                    return False
                if r.leases > 0 and not force:
                    raise ManagerError(f"model '{name}' has {r.leases} requests in flight", 409)
                del self.runners[key]
            self._stop(r.service)
            return True

    def unload_or_expire(self, name: str) -> bool:
        """Unload now when idle; a model with requests in flight gets a keep-alive of zero, so
        it goes as soon as they end.  False when it was not loaded."""
        try:
            return self.unload(name, force=False)
        except ManagerError:
            key = self.show(name).runner_key()
            with self._lock:
                r = self.runners.get(key)
                if r is not None:
                    r.keep_alive_s = 0.0
            return r is not None

    def logs(self, name: str) -> List[str]:
        """Recent stderr lines of the runner serving ``name`` (child-process runners keep a
        tail; in-process ones have none); 409 when the model is not loaded."""
        key = self.show(name).runner_key()
        with self._lock:
            r = self.runners.get(key)
        if r is None:
            raise ManagerError(f"model '{name}' is not running", 409)
        child = getattr(r.service, "service", r.service)
        return list(getattr(child, "tail", []))

    def shutdown(self) -> None:
        with self._transition:
            with self._lock:
                rs, self.runners = list(self.runners.values()), {}
            for r in rs:
                self._stop(r.service)


def apply_entry_defaults(payload: dict, defaults: Dict[str, object], ollama: bool) -> dict:
    """The request with the sampling defaults of the name it was sent to underneath it (the
    request's own fields win).  Names that share a runner keep their own defaults this way.
    Ollama bodies take them through ``options`` / ``think``; defaults without an Ollama
    spelling are left to the native routes."""
    if not defaults:
        return payload
    if not ollama:
        from .chat_codec import merge_defaults
        return merge_defaults(payload, defaults)
    from .ollama import OPTION_MAP
    spelling = {native: name for name, native in OPTION_MAP.items()}
    out = dict(payload)
    options = dict(out.get("options") or {})
    for key, value in defaults.items():
        if key in spelling:
            options.setdefault(spelling[key], value)
        elif key == "max_completion_tokens":
            options.setdefault("num_predict", value)
        elif key in ("enable_thinking", "reasoning_effort"):
            out.setdefault("think", value)
    if options:
        out["options"] = options
    return out


def describe(entry: Entry) -> dict:
    """What `/api/show` says about a registered model, read from its files alone: no runner is
    started and nothing touches a GPU.  Geometry from ``config.json``, the chat template from
    ``chat_template.jinja`` or ``tokenizer_config.json``, capabilities from the geometry (an
    encoder embeds, a decoder completes, calls tools and thinks; a vision section adds
    ``vision``)."""
    root = Path(entry.path)

    def read(name):
        try:
            return json.loads((root / name).read_text())
        except (OSError, ValueError):
            return {}
    cfg = read("config.json")
    text = cfg.get("text_config") if isinstance(cfg.get("text_config"), dict) else cfg
    arch = str(cfg.get("arch") or (cfg.get("architectures") or ["orinfer"])[0])
    template = ""
    if (root / "chat_template.jinja").exists():
        template = (root / "chat_template.jinja").read_text()
    else:
        template = str(read("tokenizer_config.json").get("chat_template") or "")
    encoder = bool(cfg.get("bidirectional"))
    caps = ["embedding"] if encoder else ["completion", "tools", "thinking"]
    if "vision_config" in cfg or entry.options.get("vision"):
        caps.append("vision")
    info = {"general.architecture": arch}
    for key, field_ in (("context_length", "max_context"), ("embedding_length", "hidden"),
                        ("block_count", "layers"), ("vocab_size", "vocab")):
        value = text.get(field_)
        if value is None:
            value = {"max_context": text.get("max_position_embeddings"),
                     "hidden": text.get("hidden_size"),
                     "layers": text.get("num_hidden_layers"),
                     "vocab": text.get("vocab_size")}[field_]
        if value is not None:
            info[f"{arch}.{key}"] = value
    limit = entry.options.get("max_context")
    if limit:
        info[f"{arch}.context_length"] = limit
    return {"details": {"family": arch, "format": "safetensors", "path": entry.path,
                        "quantization_level": "E8P-Q4A8"},
            "model_info": info, "capabilities": caps, "template": template,
            "parameters": "\n".join(f"{k} {v}" for k, v in sorted(entry.defaults.items()))}


def install(app, manager: ModelManager) -> None:
    """Registry routes of the Ollama surface on a gateway app."""
    def fail(e: ManagerError):
        return JSONResponse({"error": str(e)}, status_code=e.status)

    @app.get("/")
    async def root():
        return PlainTextResponse("Orinfer is running")

    @app.get("/api/version")
    async def version():
        from .. import __version__
        return {"version": __version__}

    @app.post("/api/show")
    async def show(request: HttpRequest):
        try:
            body = json.loads(await request.body() or b"{}")
        except ValueError:
            return JSONResponse({"error": "invalid JSON"}, status_code=400)
        try:
            return describe(manager.show(body.get("model") or body.get("name") or ""))
        except ManagerError as e:
            return fail(e)

    @app.get("/api/tags")
    async def tags():
        return {"models": [{"name": e.name, "model": e.name, "details": {"path": e.path}}
                           for e in manager.list()]}

    @app.get("/api/ps")
    async def ps():
        import datetime
        now = datetime.datetime.now(datetime.timezone.utc)

        def expires(r):
            if r["keep_alive_s"] < 0:
                return "9999-12-31T23:59:59Z"                # kept until told otherwise
            left = r["keep_alive_s"] - (r["idle_s"] if r["leases"] == 0 else 0.0)
            return (now + datetime.timedelta(seconds=max(left, 0.0))).strftime(
                "%Y-%m-%dT%H:%M:%SZ")
        return {"models": [{"name": n, "model": n, "size": r["bytes"], "size_vram": r["bytes"],
                            "leases": r["leases"], "expires_at": expires(r)}
                           for r in manager.running() for n in r["names"]]}

    @app.post("/api/copy")
    async def copy(request: HttpRequest):
        body = await request.json()
        try:
            manager.copy(body.get("source", ""), body.get("destination", ""))
        except ManagerError as e:
            return fail(e)
        return JSONResponse({}, status_code=200)

    @app.delete("/api/delete")
    async def delete(request: HttpRequest):
        body = await request.json()
        try:
            manager.remove(body.get("model") or body.get("name") or "")
        except ManagerError as e:
            return fail(e)
        return JSONResponse({}, status_code=200)

    @app.post("/api/load")
    async def load(request: HttpRequest):
        import asyncio
        body = await request.json()
        keep = body.get("keep_alive")
        if keep is not None:
            from .ollama import parse_keep_alive
            keep = parse_keep_alive(keep)
        try:
            return await asyncio.get_running_loop().run_in_executor(
                None, manager.load, body.get("model") or "", keep)
        except ManagerError as e:
            return fail(e)

    @app.post("/api/stop")
    async def stop(request: HttpRequest):
        import asyncio
        body = await request.json()
        try:
            stopped = await asyncio.get_running_loop().run_in_executor(
                None, manager.unload, body.get("model") or "", bool(body.get("force")))
        except ManagerError as e:
            return fail(e)
        return {"model": body.get("model"), "stopped": stopped}

    @app.get("/api/logs")
    async def logs(model: str = ""):
        try:
            return {"model": model, "lines": manager.logs(model)}
        except ManagerError as e:
            return fail(e)

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": e.name, "object": "model", "owned_by": "orinfer"}
                                           for e in manager.list()]}


# ---------------------------------------------------------------- gateway
class _Forward(Response):
    """ASGI response that replays the already-read body into a runner's own app and releases
    the runner's lease when the response (also a streamed one) has finished."""

    def __init__(self, app, body: bytes, done: Callable[[], None]):
        super().__init__()
        self.app, self.replay, self.done = app, body, done

    async def __call__(self, scope, receive, send):
        replayed = False

        async def rcv():
            nonlocal replayed
            if not replayed:
                replayed = True
                return {"type": "http.request", "body": self.replay, "more_body": False}
            return await receive()

        try:
            await self.app(scope, rcv, send)
        finally:
            self.done()


@dataclass
class RunnerHandle:
    service: object
    app: object


def create_gateway_app(manager: ModelManager, sweep_s: float = 5.0):
    """One listener for every registered model: OpenAI and Ollama inference routes are
    forwarded to the runner that serves the request's ``model`` (started on demand, leased for
    the life of the response); registry routes are served here.  ``start`` of the manager must
    return ``(RunnerHandle, bytes)``."""
    import asyncio
    import json as _json

    from fastapi import FastAPI

    app = FastAPI(title="orinfer-b200 gateway", docs_url=None, redoc_url=None)
    from .server import api_key, refuse_unauthorized
    key = api_key()

    @app.middleware("http")
    async def authorise(request: HttpRequest, call_next):
        refused = refuse_unauthorized(key, request)
        return refused if refused is not None else await call_next(request)

    install(app, manager)

    def openai_error(e: ManagerError):
        return JSONResponse({"error": {"message": str(e), "type": "invalid_request_error"
                                       if e.status < 500 else "server_error", "param": "model",
                                       "code": "model_not_found" if e.status == 404 else None}},
                            status_code=e.status)

    async def forward(request: HttpRequest, ollama: bool):
        body = await request.body()
        payload = {}
        try:
            if request.headers.get("content-type", "").startswith("multipart/form-data"):
                form = await request.form()          # parsed from the body that was just cached
                name = form["model"]
                if not isinstance(name, str):
                    raise TypeError("model")
            else:
                payload = _json.loads(body)
                name = payload["model"]
        except (ValueError, KeyError, TypeError):
            err = ManagerError("the request must name its `model` (JSON field or form field)", 400)
            return fail_ollama(err) if ollama else openai_error(err)
        keep = None
        if ollama and "keep_alive" in payload:
            from .chat_codec import RequestError
            from .ollama import parse_keep_alive
            try:
                keep = parse_keep_alive(payload["keep_alive"])
            except RequestError as e:
                return JSONResponse({"error": e.message}, status_code=400)
        run = asyncio.get_running_loop().run_in_executor
        generate = request.url.path == "/api/generate"
        if ollama and request.url.path in ("/api/generate", "/api/chat") \
                and not payload.get("prompt" if generate else "messages"):
            # no prompt: the request only loads the model or, with keep_alive 0, unloads it;
            # nothing is generated and an unload starts nothing
            import datetime
            try:
                if keep == 0:
                    manager.show(name)
                    await run(None, manager.unload_or_expire, name)
                    reason = "unload"
                else:
                    await run(None, manager.load, name, keep)
                    reason = "load"
            except ManagerError as e:
                return fail_ollama(e)
            stamp = datetime.datetime.now(datetime.timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ")
            empty = {"response": ""} if generate else {"message": {"role": "assistant",
                                                                   "content": ""}}
            return JSONResponse(dict(empty, model=name, created_at=stamp, done=True,
                                     done_reason=reason))
        if payload:
            try:                                     # the addressed name's own defaults
                merged = apply_entry_defaults(payload, manager.show(name).defaults, ollama)
            except ManagerError as e:
                return fail_ollama(e) if ollama else openai_error(e)
            if merged is not payload:
                body = _json.dumps(merged, ensure_ascii=False).encode()
        try:
            runner = await run(None, manager.acquire, name, keep)
        except ManagerError as e:
            return fail_ollama(e) if ollama else openai_error(e)
        return _Forward(runner.service.app, body, lambda: manager.release(runner))

    def fail_ollama(e: ManagerError):
        return JSONResponse({"error": str(e)}, status_code=e.status)

    def handler(ollama: bool):
        async def route(request: HttpRequest):
            return await forward(request, ollama)
        return route

    for path in ("/v1/chat/completions", "/v1/chat/completions/render", "/v1/completions",
                 "/v1/embeddings",
                 "/v1/rerank", "/rerank", "/v1/audio/transcriptions"):
        app.add_api_route(path, handler(False), methods=["POST"])
    for path in ("/api/chat", "/api/generate", "/api/embed", "/api/embeddings"):
        app.add_api_route(path, handler(True), methods=["POST"])

    @app.get("/health")
    async def health():
        return {"status": "ready", "models": [e.name for e in manager.list()],
                "running": manager.running()}

    @app.on_event("startup")
    async def start_sweeper():
        async def loop():
            while True:
                await asyncio.sleep(sweep_s)
                await asyncio.get_running_loop().run_in_executor(None, manager.sweep)
        app.state.sweeper = asyncio.create_task(loop())

    @app.on_event("shutdown")
    async def stop_all():
        app.state.sweeper.cancel()
        manager.shutdown()

    return app
