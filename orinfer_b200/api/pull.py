"""``orinfer models pull``: fetch a native model snapshot from Hugging Face or ModelScope with
resumable downloads, verify it, and register it with the manager.

Only already-converted models are pulled (the repository must hold ``cache/model.json``);
nothing is quantised or compiled online.  Behaviour follows the reference's
crates/orinfer-api/src/manager/pull.rs: the file list and an immutable version come from the
hub's metadata (HF: commit sha + ``siblings`` with size and LFS sha256; ModelScope:
``Data.Files``, version = sha256 of that list), file names must be safe relative paths, each
file goes to ``<name>.part`` and resumes with ``Range: bytes=<offset>-`` (the reply's
``Content-Range`` must start at that offset), four attempts with 1/2/4 s back-off, size and
sha256 are checked before the rename, a complete file that verifies is not fetched again, and
the snapshot directory is keyed by sha256(``source@version``).
"""

from __future__ import annotations

import hashlib
import json
import os
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, List, Optional, Tuple
from urllib.parse import quote, urlencode

import requests

HF_ENDPOINT = "https://huggingface.co"
MODELSCOPE_ENDPOINT = "https://modelscope.cn"
ATTEMPTS = 4


class PullError(RuntimeError):
    pass


@dataclass
class RemoteFile:
    name: str
    url: str
    size: Optional[int]
    sha256: Optional[str]


def safe_path(name: str) -> str:
    parts = name.split("/")
    if not name or name.startswith("/") or "\\" in name or "\0" in name or \
            any(p in ("", ".", "..") for p in parts):
        raise PullError(f"unsafe file name in repository: {name!r}")
    return name


def parse_source(source: str) -> Tuple[str, str, str]:
    """``hf:org/repo[@revision]`` or ``modelscope:org/repo[@revision]`` -> (hub, repo, revision)."""
    hub, sep, rest = source.partition(":")
    if not sep or hub not in ("hf", "modelscope"):
        raise PullError("source must look like hf:org/repo[@revision] or modelscope:org/repo")
    repo, _, revision = rest.partition("@")
    if repo.count("/") != 1 or any(not p or p.startswith(".") for p in repo.split("/")):
        raise PullError("repository must be org/name")
    return hub, repo, revision or ("main" if hub == "hf" else "master")


def _headers(token: Optional[str]) -> dict:
    return {"Authorization": f"Bearer {token}"} if token else {}


def list_files(source: str, token: Optional[str] = None, session=None
               ) -> Tuple[str, List[RemoteFile]]:
    """(immutable version, files) of a repository."""
    http = session or requests
    hub, repo, revision = parse_source(source)
    files: List[RemoteFile] = []
    try:
        if hub == "hf":
            base = os.environ.get("ORINFER_HF_ENDPOINT", HF_ENDPOINT).rstrip("/")
            r = http.get(f"{base}/api/models/{repo}/revision/{quote(revision, safe='')}",
                         params={"blobs": "true"}, headers=_headers(token), timeout=60)
            r.raise_for_status()
            meta = r.json()
            version = meta.get("sha") or ""
            if len(version) != 40 or any(c not in "0123456789abcdefABCDEF" for c in version):
                raise PullError("invalid HF commit identity")
            for f in meta.get("siblings") or []:
                name = safe_path(f["rfilename"])
                files.append(RemoteFile(name, f"{base}/{repo}/resolve/{version}/{quote(name)}",
                                        f.get("size"), (f.get("lfs") or {}).get("sha256")))
        else:
            base = os.environ.get("ORINFER_MODELSCOPE_ENDPOINT", MODELSCOPE_ENDPOINT).rstrip("/")
            r = http.get(f"{base}/api/v1/models/{repo}/repo/files",
                         params={"Revision": revision, "Recursive": "true"},
                         headers=_headers(token), timeout=60)
            r.raise_for_status()
            listing = r.json()["Data"]["Files"]
            version = hashlib.sha256(json.dumps(listing, sort_keys=True).encode()).hexdigest()
            for f in listing:
                if f.get("Type") == "tree":
                    continue
                name = safe_path(f["Path"])
                url = f"{base}/api/v1/models/{repo}/repo?" + urlencode(
                    {"Revision": revision, "FilePath": name})
                files.append(RemoteFile(name, url, f.get("Size"), f.get("Sha256")))
    except (requests.RequestException, KeyError, TypeError, ValueError) as e:
        raise PullError(f"cannot list {source}: {e}") from None
    if not any(f.name == "cache/model.json" for f in files):
        raise PullError("repository must contain a native model (cache/model.json)")
    return version, files


def file_sha256(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def _verifies(path: Path, size: Optional[int], sha: Optional[str]) -> bool:
    return path.is_file() and (size is None or path.stat().st_size == size) and \
        (sha is None or file_sha256(path) == sha)


def download(url: str, target: Path, size: Optional[int] = None, sha256: Optional[str] = None,
             token: Optional[str] = None, session=None,
             sleep: Callable[[float], None] = time.sleep) -> None:
    if sha256 is not None and (len(sha256) != 64 or
                               any(c not in "0123456789abcdef" for c in sha256.lower())):
        raise PullError("hub metadata holds an invalid sha256")
    if _verifies(target, size, sha256):
        return
    http = session or requests
    target.parent.mkdir(parents=True, exist_ok=True)
    part = target.with_name(target.name + ".part")
    if size is not None and part.is_file() and part.stat().st_size >= size:
        if _verifies(part, size, sha256):
            os.replace(part, target)
            return
        part.unlink()
    last = "no attempt made"
    for attempt in range(ATTEMPTS):
        try:
            offset = part.stat().st_size if part.is_file() else 0
            headers = _headers(token)
            if offset:
                headers["Range"] = f"bytes={offset}-"
            with http.get(url, headers=headers, stream=True, timeout=60) as r:
                r.raise_for_status()
                resume = r.status_code == 206
                if resume and not (r.headers.get("Content-Range") or "").startswith(
                        f"bytes {offset}-"):
                    raise PullError("download returned an unexpected byte range")
                with open(part, "ab" if resume else "wb") as f:
                    for block in r.iter_content(16 << 10):   # what arrived before a cut is kept
                        f.write(block)
                    f.flush()
                    os.fsync(f.fileno())
            if size is not None and part.stat().st_size != size:
                raise PullError("incomplete model download")
            if sha256 is not None and file_sha256(part) != sha256.lower():
                part.unlink()
                raise PullError("model file hash mismatch")
            os.replace(part, target)
            return
        except (requests.RequestException, PullError, OSError) as e:
            last = str(e)
        if attempt < ATTEMPTS - 1:
            sleep(float(1 << attempt))
    raise PullError(f"{url}: {last}")


def pull(source: str, root: Path, token: Optional[str] = None, session=None,
         sleep: Callable[[float], None] = time.sleep,
         progress: Optional[Callable[[str, int, int], None]] = None) -> Path:
    """Download (or complete) the snapshot of ``source`` under ``root``; returns its
    directory.  Safe to re-run: finished files are kept, partial ones resume."""
    version, files = list_files(source, token, session)
    key = hashlib.sha256(f"{source}@{version}".encode()).hexdigest()
    snapshot = Path(root) / "snapshots" / key
    for i, f in enumerate(files):
        if progress:
            progress(f.name, i, len(files))
        download(f.url, snapshot / f.name, f.size, f.sha256, token, session, sleep)
    (snapshot / ".orinfer-source.json").write_text(json.dumps(
        {"source": source, "version": version, "files": len(files)}))
    return snapshot
