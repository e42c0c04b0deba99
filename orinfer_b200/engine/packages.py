"""Model packages: one ``.tar.xz`` / ``.tar.gz`` archive holding a single model directory
named by the SHA-256 of its descriptor, installed into a cache directory.

Installation validates in a private staging directory on the cache's filesystem and publishes
with one rename: unsafe member paths (absolute, ``..``), links, devices and a second top-level
directory are rejected before anything is written outside staging; an already installed
package is never replaced, also under concurrent installers (the rename fails instead).
Cache lookup order: ``$ORINFER_MODEL_CACHE``, ``$XDG_CACHE_HOME/orinfer/models``,
``~/.cache/orinfer/models``.  The reference installs its execution packages the same way
(crates/orinfer-engine/src/operators/install.rs:19-140, operators.rs:64-131); here the archive
carries the quantised checkpoint itself, since kernels are linked into the library instead of
being shipped as per-model cubins.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import tarfile
import tempfile
from pathlib import Path
from typing import Optional

from .checkpoint import CheckpointError, validate_model


class PackageError(ValueError):
    pass


def cache_dir(explicit: Optional[str] = None) -> Path:
    if explicit:
        return Path(explicit)
    if os.environ.get("ORINFER_MODEL_CACHE"):
        return Path(os.environ["ORINFER_MODEL_CACHE"])
    base = os.environ.get("XDG_CACHE_HOME") or os.path.join(os.path.expanduser("~"), ".cache")
    return Path(base) / "orinfer" / "models"


def digest_of(model_dir) -> str:
    return hashlib.sha256((Path(model_dir) / "cache" / "model.json").read_bytes()).hexdigest()


def create(model_dir, out_path) -> str:
    """Packs ``model_dir`` as ``<digest>/...`` into ``out_path`` (.tar.xz or .tar.gz)."""
    validate_model(model_dir)
    digest = digest_of(model_dir)
    mode = "w:xz" if str(out_path).endswith(".xz") else "w:gz"
    with tarfile.open(out_path, mode) as tar:
        for p in sorted(Path(model_dir).rglob("*")):
            if p.is_file() and not p.is_symlink():
                tar.add(p, arcname=f"{digest}/{p.relative_to(model_dir)}", recursive=False)
    return digest


def _is_hex_digest(name: str) -> bool:
    return len(name) == 64 and all(c in "0123456789abcdef" for c in name)


def install(archive, cache: Optional[str] = None) -> Path:
    cache_path = cache_dir(cache)
    with open(archive, "rb") as f:
        magic = f.read(6)
    if not (magic.startswith(b"\xfd7zXZ\x00") or magic.startswith(b"\x1f\x8b")):
        raise PackageError("expected a .tar.xz or .tar.gz model package")
    cache_path.mkdir(parents=True, exist_ok=True)
    staging = Path(tempfile.mkdtemp(prefix=".install-", dir=cache_path))
    try:
        root = None
        with tarfile.open(archive, "r:*") as tar:
            for m in tar:
                parts = Path(m.name).parts
                if not parts or m.name.startswith("/") or any(p in ("..", ".") for p in parts):
                    raise PackageError(f"unsafe archive path {m.name!r}")
                if not _is_hex_digest(parts[0]):
                    raise PackageError("malformed package digest")
                if root is not None and parts[0] != root:
                    raise PackageError("expected one package directory")
                root = parts[0]
                if m.isdir():
                    (staging / m.name).mkdir(parents=True, exist_ok=True)
                    continue
                if not m.isfile():
                    raise PackageError(f"archive member {m.name!r} is not a regular file")
                dest = staging / m.name
                dest.parent.mkdir(parents=True, exist_ok=True)
                src = tar.extractfile(m)
                with open(dest, "wb") as out:
                    shutil.copyfileobj(src, out)
        if root is None:
            raise PackageError("empty package")
        try:
            validate_model(staging / root)
        except (CheckpointError, OSError, KeyError) as e:
            raise PackageError(f"package does not hold a valid model: {e}") from e
        if digest_of(staging / root) != root:
            raise PackageError("package digest does not match its descriptor")
        final = cache_path / root
        try:
            os.rename(staging / root, final)       # fails if another installer won the race
        except OSError as e:
            raise PackageError("package already installed; existing files were not changed") \
                from e
        return final
    finally:
        shutil.rmtree(staging, ignore_errors=True)


def resolve(name_or_path: str, cache: Optional[str] = None) -> Path:
    """A directory path, or the digest (or unique digest prefix) of an installed package."""
    p = Path(name_or_path)
    if p.is_dir():
        return p
    hits = [d for d in cache_dir(cache).glob(f"{name_or_path}*") if d.is_dir()]
    if len(hits) != 1:
        raise PackageError(f"{name_or_path!r} is neither a directory nor one installed package")
    return hits[0]
