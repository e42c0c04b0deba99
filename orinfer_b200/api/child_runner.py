"""Managed runners as child processes: one ``orinfer serve MODEL`` per loaded model behind the
gateway, so retiring a model returns all of its device memory and a crashing runner cannot
take the gateway down.

The reference's manager does the same (crates/orinfer-api/src/manager/mod.rs:137-148,159-727:
a runner process per (model path, execution options), started on demand, kept alive while
leased, stopped by keep-alive expiry or memory pressure).  ``ChildRunner`` owns the process;
``ProxyApp`` is the ASGI application the gateway forwards to — it relays the request to the
child's loopback listener and streams the reply back chunk by chunk, so SSE and NDJSON
responses arrive as they are produced.
"""

from __future__ import annotations

import os
import signal
import socket
import subprocess
import sys
import threading
import time
from pathlib import Path
from typing import List, Optional

HOP_HEADERS = {b"connection", b"keep-alive", b"transfer-encoding", b"te", b"trailer", b"upgrade",
               b"proxy-authorization", b"proxy-authenticate", b"host", b"content-length"}


class RunnerStartError(RuntimeError):
    pass


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def weight_bytes(model_dir) -> int:
    """Bytes of the weight files of a model directory (what the runner will hold on the GPU)."""
    return sum(p.stat().st_size for p in Path(model_dir).rglob("*.safetensors"))


class ChildRunner:
    def __init__(self, model_dir: str, name: str, serve_args: Optional[List[str]] = None,
                 start_timeout_s: float = 600.0, env: Optional[dict] = None):
        self.model_dir, self.name = str(model_dir), name
        self.serve_args = list(serve_args or [])
        self.start_timeout_s = start_timeout_s
        self.env = env
        self.port = 0
        self.proc: Optional[subprocess.Popen] = None
        self.tail: List[str] = []
        self._ready = threading.Event()

    @property
    def base_url(self) -> str:
        return f"http://127.0.0.1:{self.port}"

    def start(self) -> "ChildRunner":
        self.port = _free_port()
        cmd = [sys.executable, "-m", "orinfer_b200", "serve", self.model_dir, "--model", self.name,
               "--listen", f"127.0.0.1:{self.port}", *self.serve_args]
        self.proc = subprocess.Popen(cmd, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE,
                                     text=True, env=self.env, start_new_session=True)
        threading.Thread(target=self._watch, daemon=True).start()
        deadline = time.monotonic() + self.start_timeout_s
        while time.monotonic() < deadline:
            if self._ready.wait(0.05) and self._accepts():
                return self
            if self.proc.poll() is not None:
                raise RunnerStartError(f"runner for {self.name} exited with code "
                                       f"{self.proc.returncode}: " + " | ".join(self.tail[-5:]))
        self.stop(5)
        raise RunnerStartError(f"runner for {self.name} did not become ready in "
                               f"{self.start_timeout_s:.0f} s")

    def _watch(self) -> None:
        for line in self.proc.stderr:
            self.tail.append(line.rstrip())
            del self.tail[:-40]
            if line.startswith("API READY"):
                self._ready.set()

    def _accepts(self) -> bool:
        try:
            with socket.create_connection(("127.0.0.1", self.port), timeout=0.2):
                return True
        except OSError:
            return False

    def alive(self) -> bool:
        return self.proc is not None and self.proc.poll() is None

    def stop(self, timeout_s: float = 30.0) -> None:
        """SIGTERM (the runner drains), then SIGKILL of this runner's own process group."""
        if self.proc is None or self.proc.poll() is not None:
            return
        self.proc.send_signal(signal.SIGTERM)
        try:
            self.proc.wait(timeout=timeout_s)
        except subprocess.TimeoutExpired:
            os.killpg(self.proc.pid, signal.SIGKILL)
            self.proc.wait()


class ProxyApp:
    """ASGI application relaying every request to ``base_url`` with streaming replies."""

    def __init__(self, base_url: str, timeout_s: float = 3600.0):
        self.base_url = base_url.rstrip("/")
        self.timeout_s = timeout_s

    async def __call__(self, scope, receive, send):
        import httpx
        body = b""
        while True:
            msg = await receive()
            if msg["type"] == "http.disconnect":
                return
            body += msg.get("body", b"")
            if not msg.get("more_body"):
                break
        headers = [(k.decode("latin-1"), v.decode("latin-1")) for k, v in scope["headers"]
                   if k.lower() not in HOP_HEADERS]
        url = self.base_url + scope["path"]
        if scope.get("query_string"):
            url += "?" + scope["query_string"].decode("latin-1")
        started = False
        try:
            async with httpx.AsyncClient(timeout=httpx.Timeout(self.timeout_s, connect=5.0)) as c:
                async with c.stream(scope["method"], url, content=body, headers=headers) as r:
                    await send({"type": "http.response.start", "status": r.status_code,
                                "headers": [(k.lower().encode("latin-1"), v.encode("latin-1"))
                                            for k, v in r.headers.items()
                                            if k.lower().encode() not in HOP_HEADERS]})
                    started = True
                    async for chunk in r.aiter_raw():
                        await send({"type": "http.response.body", "body": chunk,
                                    "more_body": True})
                    await send({"type": "http.response.body", "body": b"", "more_body": False})
        except httpx.HTTPError as e:
            if started:                 # the reply is already under way: just end it
                await send({"type": "http.response.body", "body": b"", "more_body": False})
                return
            payload = ('{"error": {"message": "runner unreachable: %s", "type": "server_error", '
                       '"param": null, "code": "runner_unavailable"}}'
                       % type(e).__name__).encode()
            await send({"type": "http.response.start", "status": 502,
                        "headers": [(b"content-type", b"application/json")]})
            await send({"type": "http.response.body", "body": payload, "more_body": False})
