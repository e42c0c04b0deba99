"""Start-up time: from launching ``orinfer serve`` to ``API READY`` and to the first complete
streaming chat request.

The two columns "Serve->API s" and "Serve->first output s" of the reference's performance
table come from tools/bench/startup.py: the clock starts when the CLI process is spawned; the
first mark is the ``API READY`` line on stderr, the second is the first non-empty text,
reasoning or tool delta of a streaming request sent as soon as the listener accepts.

    python -m orinfer_b200.bench.startup -- MODEL_DIR --cuda-graph decode_only
"""

from __future__ import annotations

import argparse
import json
import signal
import socket
import subprocess
import sys
import threading
import time

from .http_client import stream_chat


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run(serve_args, port: int | None = None, deadline_s: float = 600.0, max_tokens: int = 8,
        env=None) -> dict:
    port = port or free_port()
    cmd = [sys.executable, "-m", "orinfer_b200", "serve", *serve_args,
           "--listen", f"127.0.0.1:{port}"]
    t0 = time.perf_counter()
    proc = subprocess.Popen(cmd, stderr=subprocess.PIPE, stdout=subprocess.DEVNULL, text=True,
                            env=env)
    marks = {}
    tail = []

    def watch():
        for line in proc.stderr:
            tail.append(line.rstrip())
            del tail[:-40]
            if line.startswith("WARMUP READY"):
                marks.setdefault("warmup_ready_s", time.perf_counter() - t0)
            if line.startswith("API READY"):
                marks.setdefault("api_ready_s", time.perf_counter() - t0)

    watcher = threading.Thread(target=watch, daemon=True)
    watcher.start()
    url = f"http://127.0.0.1:{port}"
    result = None
    try:
        while time.perf_counter() - t0 < deadline_s and proc.poll() is None:
            if "api_ready_s" not in marks:
                time.sleep(0.01)
                continue
            try:
                with socket.create_connection(("127.0.0.1", port), timeout=0.2):
                    pass
            except OSError:
                time.sleep(0.01)
                continue
            marks["listening_s"] = time.perf_counter() - t0
            result = stream_chat(url, {"messages": [{"role": "user", "content": "Say hello."}],
                                       "max_tokens": max_tokens, "temperature": 0,
                                       "enable_thinking": False}, timeout=deadline_s)
            break
    finally:
        if proc.poll() is None:
            proc.send_signal(signal.SIGTERM)
            try:
                proc.wait(timeout=60)
            except subprocess.TimeoutExpired:
                proc.kill()
                proc.wait()
        watcher.join(timeout=5)
    out = {"command": cmd, "exit_code": proc.returncode, **marks,
           "ok": bool(result and result.ok)}
    if result is not None:
        mark = result.first_output or result.first_event
        out["first_output_s"] = (mark - t0) if mark else None
        out["first_request_complete_s"] = result.end - t0
        out["completion_tokens"] = result.completion_tokens
        out["error"] = result.error
    else:
        out["stderr_tail"] = tail[-10:]
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--deadline", type=float, default=600.0)
    ap.add_argument("serve_args", nargs=argparse.REMAINDER,
                    help="arguments of `orinfer serve` after `--`")
    a = ap.parse_args(argv)
    args = [x for x in a.serve_args if x != "--"]
    rep = run(args, deadline_s=a.deadline)
    print(json.dumps(rep, indent=1))
    return 0 if rep["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
