"""Model pull against a local hub: listing, resume after a cut connection, verification."""
import hashlib
import json
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from urllib.parse import parse_qs, urlparse

import pytest

from orinfer_b200.api import pull as P

FILES = {"cache/model.json": b'{"schema": 1}', "weights/a.safetensors": bytes(range(256)) * 400,
         "tokenizer.json": b"{}"}
SHA = "ab" * 20


class Hub(BaseHTTPRequestHandler):
    cut_after = {}           # path -> bytes to send before dropping the connection (once)
    ranges = []
    ignore_range = False

    def log_message(self, *a):
        pass

    def _json(self, obj):
        body = json.dumps(obj).encode()
        self.send_response(200)
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)

    def do_GET(self):
        url = urlparse(self.path)
        if url.path == "/api/models/org/m/revision/main":
            return self._json({"sha": SHA, "siblings": [
                {"rfilename": n, "size": len(b),
                 "lfs": {"sha256": hashlib.sha256(b).hexdigest()} if n.endswith("tensors") else None}
                for n, b in FILES.items()]})
        if url.path == "/api/models/org/bad/revision/main":
            return self._json({"sha": SHA, "siblings": [{"rfilename": "../evil", "size": 1}]})
        if url.path == "/api/models/org/empty/revision/main":
            return self._json({"sha": SHA, "siblings": [{"rfilename": "x.bin", "size": 1}]})
        if url.path == "/api/v1/models/org/m/repo/files":
            return self._json({"Data": {"Files": [{"Type": "tree", "Path": "cache"}] + [
                {"Type": "blob", "Path": n, "Size": len(b),
                 "Sha256": hashlib.sha256(b).hexdigest()} for n, b in FILES.items()]}})
        name = None
        if url.path.startswith(f"/org/m/resolve/{SHA}/"):
            name = url.path[len(f"/org/m/resolve/{SHA}/"):]
        elif url.path == "/api/v1/models/org/m/repo":
            name = parse_qs(url.query)["FilePath"][0]
        if name not in FILES:
            self.send_response(404)
            self.end_headers()
            return
        data = FILES[name]
        start = 0
        rng = self.headers.get("Range")
        if rng and not Hub.ignore_range:
            Hub.ranges.append((name, rng))
            start = int(rng[len("bytes="):-1])
            self.send_response(206)
            self.send_header("Content-Range", f"bytes {start}-{len(data) - 1}/{len(data)}")
        else:
            self.send_response(200)
        self.send_header("Content-Length", str(len(data) - start))
        self.end_headers()
        cut = Hub.cut_after.pop(name, None)
        if cut is not None:
            self.wfile.write(data[start:start + cut])
            self.wfile.flush()
            self.connection.close()
            return
        self.wfile.write(data[start:])


@pytest.fixture()
def hub(monkeypatch):
    server = ThreadingHTTPServer(("127.0.0.1", 0), Hub)
    threading.Thread(target=server.serve_forever, daemon=True).start()
    base = f"http://127.0.0.1:{server.server_port}"
    monkeypatch.setenv("ORINFER_HF_ENDPOINT", base)
    monkeypatch.setenv("ORINFER_MODELSCOPE_ENDPOINT", base)
    Hub.cut_after, Hub.ranges, Hub.ignore_range = {}, [], False
    yield base
    server.shutdown()


def test_source_and_path_rules():
    assert P.parse_source("hf:org/m") == ("hf", "org", "main")[:1] + ("org/m", "main")
    assert P.parse_source("modelscope:org/m@v2") == ("modelscope", "org/m", "v2")
    for bad in ("org/m", "s3:org/m", "hf:m", "hf:org/.m", "hf:a/b/c"):
        with pytest.raises(P.PullError):
            P.parse_source(bad)
    for bad in ("../x", "/abs", "a//b", "a/./b", "a\\b", ""):
        with pytest.raises(P.PullError):
            P.safe_path(bad)
    assert P.safe_path("cache/model.json") == "cache/model.json"


def test_pull_resumes_after_a_cut_connection(hub, tmp_path):
    Hub.cut_after = {"weights/a.safetensors": 50000}
    naps = []
    snap = P.pull("hf:org/m", tmp_path, sleep=naps.append)
    for name, body in FILES.items():
        assert (snap / name).read_bytes() == body
    assert Hub.ranges == [("weights/a.safetensors", "bytes=49152-")] and naps == [1.0]
    assert not list(snap.rglob("*.part"))
    assert json.loads((snap / ".orinfer-source.json").read_text())["version"] == SHA
    Hub.ranges.clear()
    again = P.pull("hf:org/m", tmp_path, sleep=naps.append)           # nothing fetched again
    assert again == snap and Hub.ranges == [] and naps == [1.0]
    ms = P.pull("modelscope:org/m", tmp_path, sleep=naps.append)
    assert ms != snap and (ms / "weights/a.safetensors").read_bytes() == FILES["weights/a.safetensors"]


def test_partial_files_hash_mismatch_and_bad_listings(hub, tmp_path):
    body = FILES["weights/a.safetensors"]
    sha = hashlib.sha256(body).hexdigest()
    url = f"{hub}/org/m/resolve/{SHA}/weights/a.safetensors"
    target = tmp_path / "a.bin"
    (tmp_path / "a.bin.part").write_bytes(body[:5000])
    P.download(url, target, len(body), sha, sleep=lambda s: None)
    assert target.read_bytes() == body and Hub.ranges[-1][1] == "bytes=5000-"
    (tmp_path / "b.bin.part").write_bytes(body)                       # complete part: just renamed
    n = len(Hub.ranges)
    P.download(url, tmp_path / "b.bin", len(body), sha, sleep=lambda s: None)
    assert (tmp_path / "b.bin").read_bytes() == body and len(Hub.ranges) == n
    (tmp_path / "c.bin.part").write_bytes(b"\xff" * 5000)             # corrupt prefix
    naps = []                                                          # dropped, fetched afresh
    P.download(url, tmp_path / "c.bin", len(body), sha, sleep=naps.append)
    assert (tmp_path / "c.bin").read_bytes() == body and naps == [1.0]
    with pytest.raises(P.PullError, match="hash mismatch"):
        P.download(url, tmp_path / "c2.bin", len(body), "0" * 64, sleep=naps.append)
    assert not (tmp_path / "c2.bin").exists() and len(naps) == 4
    Hub.ignore_range = True                                            # server restarts at zero
    (tmp_path / "d.bin.part").write_bytes(b"\xff" * 100)
    P.download(url, tmp_path / "d.bin", len(body), sha, sleep=lambda s: None)
    assert (tmp_path / "d.bin").read_bytes() == body
    with pytest.raises(P.PullError, match="incomplete"):
        P.download(url, tmp_path / "e.bin", len(body) + 1, None, sleep=lambda s: None)
    with pytest.raises(P.PullError, match="invalid sha256"):
        P.download(url, tmp_path / "f.bin", None, "zz", sleep=lambda s: None)
    with pytest.raises(P.PullError, match="unsafe"):
        P.list_files("hf:org/bad")
    with pytest.raises(P.PullError, match="cache/model.json"):
        P.list_files("hf:org/empty")
    with pytest.raises(P.PullError, match="cannot list"):
        P.list_files("hf:org/missing")
