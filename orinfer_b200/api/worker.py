"""The serving loop: one OS thread owns the engine (and its CUDA context); HTTP handlers
hand it jobs through a bounded queue and receive events on per-request mailboxes.

Per iteration, like the reference's continuous worker
(crates/orinfer-api/src/server/continuous.rs:470-1009): receive waiting jobs (queue
deadline), mark cancelled ones, admit, advance the engine one packet, deliver tokens
through the output parser, publish statistics.  A fatal engine error flips the
lifecycle to ``failed`` (``/health`` answers 503) and fails every open request;
request-level errors fail only that request.
"""

from __future__ import annotations

import asyncio
import queue
import threading
import time
import traceback
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

from ..engine.engine import Engine
from ..engine.request import Request
from .chat_codec import ChatCodec, Prepared, RequestError
from .grammar import GrammarConstraint, GrammarError, ThinkingBudget
from .metrics import Metrics
from .output_parser import Delta, OutputParser

QUEUE_CAPACITY = 128


class Lifecycle:
    STARTING, READY, DRAINING, FAILED = "starting", "ready", "draining", "failed"

    def __init__(self):
        self.state = self.STARTING
        self.reason: Optional[str] = None
        self._lock = threading.Lock()

    def set(self, state: str, reason: Optional[str] = None) -> None:
        with self._lock:
            if self.state != self.FAILED:
                self.state, self.reason = state, reason


@dataclass
class Job:
    prepared: Prepared
    rid: str
    loop: Optional[asyncio.AbstractEventLoop] = None
    events: Any = None                           # asyncio.Queue or queue.Queue
    created: float = field(default_factory=time.monotonic)
    created_unix: int = field(default_factory=lambda: int(time.time()))   # `created` of every chunk
    cancelled: bool = False
    stop_requested: bool = False                 # the output side saw a stop string
    started_at: Optional[float] = None           # handed to the engine (end of queueing)
    request: Optional[Request] = None
    parser: Optional[OutputParser] = None
    pending_bytes: bytes = b""
    text_tokens: List[int] = field(default_factory=list)
    first_token_at: Optional[float] = None
    logprob_entries: List[dict] = field(default_factory=list)

    def post(self, event: dict) -> None:
        if self.loop is not None:
            try:
                self.loop.call_soon_threadsafe(self.events.put_nowait, event)
            except RuntimeError:            # the server's loop is gone: nobody is listening
                self.cancelled = True
        else:
            self.events.put_nowait(event)


class CallJob:
    """A function to run on the engine thread between two engine steps (encoder passes,
    introspection); the result comes back through ``future``."""

    def __init__(self, fn: Callable[[Engine], Any]):
        import concurrent.futures
        self.fn = fn
        self.future: "concurrent.futures.Future" = concurrent.futures.Future()
        self.cancelled = False


class OutputPipeline(threading.Thread):
    """Detokenisation, parsing and event delivery on their own thread, so the engine thread goes
    straight back to the next forward pass (the reference overlaps its output pipeline with the
    next iteration the same way, crates/orinfer-api/src/server/continuous.rs:31-48,103-200).
    Items arrive in commit order and are handled in that order; everything produced by one
    drain of the queue reaches an event loop in a single ``call_soon_threadsafe``."""

    def __init__(self, worker: "EngineWorker"):
        super().__init__(name="orinfer-output", daemon=True)
        self.worker = worker
        self.items: "queue.SimpleQueue" = queue.SimpleQueue()
        self.start()

    def push(self, item) -> None:
        self.items.put(item)

    def close(self) -> None:
        self.items.put(None)
        self.join(timeout=10)

    @staticmethod
    def _deliver(pairs) -> None:                 # runs on the event loop
        for job, event in pairs:
            job.events.put_nowait(event)

    def run(self) -> None:
        closing = False
        while not closing:
            batch = [self.items.get()]
            while True:
                try:
                    batch.append(self.items.get_nowait())
                except queue.Empty:
                    break
            by_loop: Dict[int, list] = {}

            def sink(job: Job, event: dict) -> None:
                if job.loop is None:
                    job.events.put_nowait(event)
                else:
                    by_loop.setdefault(id(job.loop), [job.loop, []])[1].append((job, event))

            for item in batch:
                if item is None:
                    closing = True
                    continue
                try:
                    if item[0] == "token":
                        self.worker._emit_token(*item[1:], sink)
                    else:
                        self.worker._emit_finish(*item[1:], sink)
                except Exception:                # noqa: BLE001 - one request, not the server
                    traceback.print_exc()
                    sink(item[1], {"type": "error", "status": 500,
                                   "message": "output pipeline failure", "code": "output_failure"})
            for loop, pairs in by_loop.values():
                try:
                    loop.call_soon_threadsafe(self._deliver, pairs)
                except RuntimeError:             # the server's loop is gone
                    for job, _ in pairs:
                        job.cancelled = True


class EngineWorker(threading.Thread):
    def __init__(self, engine_factory: Callable[[], Engine], codec: ChatCodec, metrics: Metrics,
                 lifecycle: Lifecycle, queue_timeout_ms: int = 0, step_timeout_ms: int = 0,
                 exit_on_stall: bool = False):
        super().__init__(name="orinfer-gpu", daemon=True)
        # a step that runs past step_timeout_ms fails the service closed (engine/watchdog.py)
        self.step_timeout_s = step_timeout_ms / 1e3
        self.exit_on_stall = exit_on_stall
        self.watchdog = None
        import os
        # ORINFER_ASYNC_OUTPUT=0 keeps detokenisation and parsing on the engine thread
        self.async_output = os.environ.get("ORINFER_ASYNC_OUTPUT", "1") != "0"
        self.pipeline: Optional[OutputPipeline] = None
        self.engine_factory = engine_factory
        self.engine: Optional[Engine] = None
        self.codec = codec
        self.metrics = metrics
        self.lifecycle = lifecycle
        self.jobs: "queue.Queue[Job]" = queue.Queue(maxsize=QUEUE_CAPACITY)
        self.active: Dict[int, Job] = {}
        self.queue_timeout_s = queue_timeout_ms / 1e3 if queue_timeout_ms else None
        self._stop = threading.Event()
        self.ready = threading.Event()

    # ------------------------------------------------------------------ submission
    def try_submit(self, job: Job) -> bool:
        if self.lifecycle.state != Lifecycle.READY:
            return False
        try:
            self.jobs.put_nowait(job)
        except queue.Full:
            return False
        self.metrics.set("requests_waiting", self.jobs.qsize())
        return True

    def stop(self, drain_s: float = 30.0) -> None:
        self.lifecycle.set(Lifecycle.DRAINING)
        deadline = time.monotonic() + drain_s
        while (self.active or not self.jobs.empty()) and time.monotonic() < deadline:
            time.sleep(0.01)
        self._stop.set()

    # ------------------------------------------------------------------ the loop
    def run(self) -> None:
        try:
            if self.step_timeout_s > 0:
                from ..engine.watchdog import StepWatchdog
                self.watchdog = StepWatchdog(self._stalled)
            self.engine = self.engine_factory()
            self._warmup()
            self._instrument()
            self._gauges()
            if self.async_output:
                self.pipeline = OutputPipeline(self)
            self.lifecycle.set(Lifecycle.READY)
            self.ready.set()
            while not self._stop.is_set():
                self._receive()
                if not self.engine.has_work():
                    try:
                        job = self.jobs.get(timeout=0.05)
                        self._start(job)
                    except queue.Empty:
                        pass
                    continue
                t0 = time.monotonic()
                if self.watchdog is not None:
                    self.watchdog.arm("engine step", self.step_timeout_s)
                self.engine.step()
                if self.watchdog is not None:
                    self.watchdog.disarm()
                    if self.watchdog.tripped:
                        raise RuntimeError(f"{self.watchdog.tripped} ran past its deadline")
                self.metrics.add("compute_seconds_total", time.monotonic() - t0)
                self._reap()
                self.metrics.set("requests_running", len(self.active))
                self.metrics.set("requests_waiting", self.jobs.qsize())
                if self.engine.stats.iterations % 32 == 0:
                    self._gauges()
            if self.pipeline is not None:
                self.pipeline.close()
            self._exit_report()
        except Exception as exc:                     # fatal: fail closed
            self.lifecycle.set(Lifecycle.FAILED, f"{type(exc).__name__}: {exc}")
            self.metrics.set("backend_healthy", 0)
            traceback.print_exc()
            for job in list(self.active.values()):
                job.post({"type": "error", "status": 500, "message": "engine failure",
                          "code": "engine_failure"})
            self.ready.set()

    def _gauges(self) -> None:
        """Slow-moving engine state for dashboards: free KV pages, prefix-cache hit rate and
        pages, speculation acceptance, graph replays."""
        eng, m = self.engine, self.metrics
        m.set("kv_pages_free", eng.pool.available)
        m.set("graph_replays_total", eng.stats.graph_hits)
        spec = eng.spec.statistics()
        m.set("speculation_acceptance_rate", spec.get("acceptance_rate", 0.0))
        m.set("speculation_rounds_total", spec.get("rounds", 0))
        m.level("batch_plan_seconds_total", eng.stats.batch_inputs_s)
        m.level("sampling_request_failures_total", eng.stats.failed_requests)
        pool = getattr(eng, "_prefill_graphs", None)
        if pool is not None and hasattr(pool, "evictions"):
            m.level("program_reclaims_total", pool.evictions)
        if eng.on_gpu:
            import torch
            free = torch.cuda.mem_get_info(eng.device)[0]
            m.set("device_rank_free_bytes_min", free)      # one rank per process
            m.set("device_rank_free_bytes_max", free)
        if eng.prefix is not None:
            st = eng.prefix.statistics()
            page = eng.kv.bytes_per_page(eng.cfg, eng.cfg.mtp_layers)
            m.set("prefix_cache_hit_rate", st.hit_rate)
            m.set("prefix_cache_device_pages", st.device_pages)
            m.set("prefix_cache_host_pages", st.host_pages)
            m.set("prefix_cache_device_entries", st.device_pages)
            m.set("prefix_cache_device_bytes", st.device_pages * page)
            m.set("prefix_cache_host_entries", st.host_pages)
            m.set("prefix_cache_host_bytes", st.host_pages * page)
            m.level("prefix_cache_evictions_total", st.evicted)
            dropped = max(st.offloaded - st.restored - st.host_pages, 0)
            m.level("prefix_cache_host_evictions_total", dropped)

    def _instrument(self) -> None:
        """Time the engine's admission pass and its prefix-cache store / host restore calls for
        the ``admission_seconds_total`` counter and the ``prefix_store`` / ``prefix_restore``
        histograms (wrappers on the host side; the engine itself is unchanged)."""
        eng, metrics = self.engine, self.metrics

        def timed(fn, record):
            def call(*a, **k):
                t0 = time.monotonic()
                out = fn(*a, **k)
                record(time.monotonic() - t0, a, out)
                return out
            return call

        eng._admit = timed(eng._admit, lambda dt, a, out: metrics.add(
            "admission_seconds_total", dt) if dt > 1e-5 else None)
        eng._restore_host_pages = timed(
            eng._restore_host_pages,
            lambda dt, a, out: (metrics.observe("prefix_restore", dt),
                                metrics.add("prefix_restore_seconds_total", dt))
            if dt > 1e-5 else None)
        if eng.prefix is not None:
            eng.prefix.insert = timed(eng.prefix.insert,
                                      lambda dt, a, out: metrics.observe("prefix_store", dt))

    def _stalled(self, what: str, waited_s: float) -> None:
        """Watchdog thread: the engine thread is stuck inside a step.  Fail closed, answer the
        clients, and optionally leave the process without running exit hooks."""
        import os
        import sys
        self.lifecycle.set(Lifecycle.FAILED, f"{what} exceeded {self.step_timeout_s:.1f} s")
        self.metrics.set("backend_healthy", 0)
        self.metrics.add("watchdog_timeouts_total")
        print(f"WATCHDOG {what} still running after {waited_s:.1f} s; failing closed",
              file=sys.stderr, flush=True)
        for job in list(self.active.values()):
            job.post({"type": "error", "status": 500, "message": "engine stalled",
                      "code": "engine_stalled"})
        if self.exit_on_stall:
            os._exit(70)

    def _exit_report(self) -> None:
        """Telemetry lines at shutdown: ``SCHEDULER {json}`` (engine statistics, speculation,
        prefix cache) and the device-timed spans when span profiling is on."""
        import json
        import sys
        from ..utils import trace
        eng = self.engine
        body = {"engine": eng.stats.as_dict(), "speculation": eng.spec.statistics()}
        if eng.prefix is not None:
            body["prefix_cache"] = eng.prefix.statistics().__dict__
        print(f"SCHEDULER {json.dumps(body, default=str)}", file=sys.stderr, flush=True)
        trace.dump()

    def _warmup(self) -> None:
        if self.engine.cfg.bidirectional:
            self.engine.encode([0, 1])
        else:
            self.engine.generate([[0]], max_new=1)

    def _receive(self) -> None:
        for _ in range(QUEUE_CAPACITY):
            try:
                job = self.jobs.get_nowait()
            except queue.Empty:
                return
            self._start(job)

    def call(self, fn: Callable[[Engine], Any], timeout: Optional[float] = 60.0):
        """Runs ``fn(engine)`` on the engine thread and returns its result."""
        job = CallJob(fn)
        if not self.try_submit(job):
            raise RequestError("request queue is full", status=429, code="queue_full",
                               err_type="rate_limit_error")
        return job.future.result(timeout=timeout)

    def _start(self, job) -> None:
        if isinstance(job, CallJob):
            try:
                job.future.set_result(job.fn(self.engine))
            except Exception as exc:                 # noqa: BLE001 - belongs to the caller
                job.future.set_exception(exc)
            return
        now = time.monotonic()
        if job.cancelled:
            return
        if self.queue_timeout_s is not None and now - job.created > self.queue_timeout_s:
            job.post({"type": "error", "status": 408, "message": "request waited too long",
                      "code": "request_queue_timeout", "retryable": True})
            return
        p = job.prepared
        try:
            constraint = self._constraint(p)
            job.parser = OutputParser(thinking=p.thinking, stops=p.stop_strings,
                                      json_mode=p.json_schema is not None or p.json_object,
                                      tools=bool(p.tools),
                                      tool_format=getattr(self.codec, "tool_format", "xml"))
            req = self.engine.submit(p.prompt_ids, p.max_new, p.sampling, stop_ids=p.stop_ids,
                                     ignore_eos=p.ignore_eos, want_logprobs=p.want_logprobs,
                                     constraint=constraint, cache_prompt=p.cache_prompt,
                                     **self._media(p),
                                     on_token=lambda r, tok, j=job: self._on_token(j, r, tok))
        except (RequestError, GrammarError, ValueError) as exc:
            job.post({"type": "error", "status": 400, "message": str(exc),
                      "code": getattr(exc, "code", None)})
            self.metrics.add("request_errors_total")
            return
        job.request = req
        self.active[req.rid] = job
        self.metrics.observe("queue", now - job.created)
        job.started_at = now
        job.post({"type": "start"})

    def _media(self, p: Prepared) -> dict:
        """Engine arguments for the images of a prepared request: encoder features (cached by
        image content) bound to their placeholder spans, and the rotary positions."""
        from ..engine.request import MediaSpan
        audio = getattr(p, "audio", None)
        if audio is not None:
            from ..models.audio import AudioEncoder
            if getattr(self, "_audio", None) is None:
                enc = AudioEncoder(self.engine.cfg.hidden, seed=0)
                if self.engine.on_gpu:
                    enc = enc.to(self.engine.device).half()
                self._audio = enc
            spans = [MediaSpan(a, b, self._audio.encode(x), x.digest())
                     for x, (a, b) in zip(audio.inputs, audio.spans)]
            self.metrics.add("audio_inputs_total", len(spans))
            return {"media": spans}
        bound = getattr(p, "images", None)
        if bound is None:
            return {}
        from ..models.vision import FeatureCache, VisionEncoder
        if getattr(self, "_vision", None) is None:
            enc = VisionEncoder(self.codec.images.spec, seed=0)
            if self.engine.on_gpu:
                enc = enc.to(self.engine.device).half()
            self._vision = (enc, FeatureCache())
        enc, cache = self._vision
        spans = [MediaSpan(a, b, cache.get(im, enc), im.digest())
                 for im, (a, b) in zip(bound.images, bound.spans)]
        self.metrics.add("image_inputs_total", len(spans))
        return {"media": spans, "rope_positions": bound.rope_positions,
                "rope_delta": bound.rope_delta}

    def _constraint(self, p: Prepared):
        tok = self.codec.tokenizer
        inner = None
        if p.json_schema is not None or p.json_object:
            inner = GrammarConstraint(tok, self.engine.cfg.vocab, p.json_schema, p.stop_ids)
        elif getattr(self.codec, "tool_format", "xml") == "xml" and p.tools:
            from . import tool_grammar
            if tool_grammar.applies(p.tools, p.tool_choice, p.parallel_tool_calls):
                try:
                    text = tool_grammar.recipe(tok, p.tools, p.tool_choice, p.parallel_tool_calls)
                except ValueError as e:
                    raise RequestError(str(e), param="tool_choice")
                inner = GrammarConstraint.from_lark(tok, self.engine.cfg.vocab, text, p.stop_ids)
        elif (getattr(self.codec, "tool_format", "xml") == "dsml" and p.tools
              and p.tool_choice == "required"):
            from .dsml import grammar as dsml_grammar
            inner = GrammarConstraint.from_lark(
                tok, self.engine.cfg.vocab,
                dsml_grammar(p.tools, required=True, parallel=p.parallel_tool_calls), p.stop_ids)
        if p.thinking and p.thinking_budget is not None:
            return ThinkingBudget(tok.encode("</think>"), p.thinking_budget, p.max_new, inner)
        if p.thinking and inner is not None:
            return ThinkingBudget(tok.encode("</think>"), p.max_new, p.max_new, inner)
        return inner

    # ------------------------------------------------------------------ token delivery
    def _on_token(self, job: Job, req: Request, tok: int) -> None:
        """Engine thread, once per committed token: the cheap part (cancellation, first-token
        mark, stop-token test); text work goes to the output pipeline."""
        if job.cancelled or job.stop_requested:
            self.engine.cancel(req)
            if job.stop_requested:
                req.finish_reason = "stop"
            return
        if job.first_token_at is None:
            job.first_token_at = time.monotonic()
            self.metrics.observe("time_to_first_token", job.first_token_at - job.created)
            self.metrics.observe("prefill", job.first_token_at - (job.started_at or job.created))
        is_stop = tok in req.stop_ids and not req.ignore_eos
        lp = req.logprobs[-1] if (req.logprobs and job.prepared.want_logprobs
                                  and not is_stop) else None
        if self.pipeline is not None:
            self.pipeline.push(("token", job, tok, is_stop, lp))
            return
        self._emit_token(job, tok, is_stop, lp, Job.post)
        if job.stop_requested:
            self.engine.cancel(req)
            req.finish_reason = "stop"

    def _emit_token(self, job: Job, tok: int, is_stop: bool, lp, sink) -> None:
        """Bytes -> complete UTF-8 -> parser -> deltas.  ``sink(job, event)`` delivers."""
        piece = b"" if is_stop else self.codec.tokenizer.token_bytes(tok)
        job.pending_bytes += piece
        text, job.pending_bytes = _utf8_prefix(job.pending_bytes)
        if lp is not None:
            _t, logprob, top = lp
            job.logprob_entries.append({
                "token": piece.decode("utf-8", errors="replace"), "logprob": logprob,
                "bytes": list(piece),
                "top_logprobs": [{"token": self.codec.tokenizer.token_bytes(i).decode(
                    "utf-8", errors="replace"), "logprob": l,
                    "bytes": list(self.codec.tokenizer.token_bytes(i))} for i, l in top]})
        if getattr(job.prepared, "token_events", False) and not is_stop:
            sink(job, {"type": "token", "token": int(tok)})    # one event per committed token
        delta = job.parser.feed(text)
        if not delta.empty():
            sink(job, {"type": "delta", "delta": delta, "logprobs": self._take_logprobs(job)})
        if job.parser.stopped:
            job.stop_requested = True                          # the engine thread cancels it

    @staticmethod
    def _take_logprobs(job: Job):
        out, job.logprob_entries = job.logprob_entries, []
        return out

    def _reap(self) -> None:
        for rid, job in list(self.active.items()):
            req = job.request
            if job.cancelled and not req.finished:
                self.engine.cancel(req)
            if not req.finished:
                continue
            del self.active[rid]
            if self.pipeline is not None:
                self.pipeline.push(("finish", job, req))
            else:
                self._emit_finish(job, req, Job.post)

    def _emit_finish(self, job: Job, req: Request, sink) -> None:
        tail = job.parser.feed(job.pending_bytes.decode("utf-8", errors="replace"), final=True)
        if not tail.empty() or job.logprob_entries:
            sink(job, {"type": "delta", "delta": tail, "logprobs": self._take_logprobs(job)})
        if req.error:
            # the request failed on its own (a constraint that cannot go on, logits that are
            # not finite): its client gets the reason, nobody else notices
            self.metrics.add("requests_failed_total")
            sink(job, {"type": "error", "status": 500, "message": req.error,
                       "code": "generation_failed"})
            return
        reason = req.finish_reason or "stop"
        if reason == "cancelled" or job.parser.stopped:
            reason = "stop"
        now = time.monotonic()
        self.metrics.observe("latency", now - job.created)
        if req.finished_at is not None:
            self.metrics.observe("finalize", max(now - req.finished_at, 0.0))
        if job.first_token_at:
            self.metrics.observe("decode", now - job.first_token_at)
        self.metrics.add("requests_total")
        self.metrics.add("prompt_tokens_total", len(req.prompt))
        self.metrics.add("completion_tokens_total", len(req.generated))
        self.metrics.add("generated_tokens_total", len(req.generated))
        self.metrics.add("cached_tokens_total", req.cached_tokens)
        self.metrics.add("cached_prompt_tokens_total", req.cached_tokens)
        reasoning = 0
        if job.prepared.thinking:
            close = self.codec.tokenizer.encode("</think>")
            gen = req.generated
            reasoning = next((i for i in range(len(gen)) if gen[i:i + len(close)] == close),
                             len(gen))
        sink(job, {"type": "done", "finish_reason": job.parser.finish_reason(reason),
                   "usage": {"prompt_tokens": len(req.prompt),
                             "completion_tokens": len(req.generated),
                             "total_tokens": len(req.prompt) + len(req.generated),
                             "completion_tokens_details": {"reasoning_tokens": reasoning},
                             "prompt_tokens_details": {"cached_tokens": req.cached_tokens}}})


def _utf8_prefix(data: bytes):
    """Longest prefix that is complete UTF-8, and the withheld remainder."""
    for cut in range(len(data), max(len(data) - 4, -1), -1):
        try:
            return data[:cut].decode("utf-8"), data[cut:]
        except UnicodeDecodeError:
            continue
    return data.decode("utf-8", errors="replace"), b""
