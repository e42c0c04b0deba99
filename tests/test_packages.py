"""Model package archives: create, install once, reject unsafe or inconsistent archives."""
import io
import tarfile

import pytest

from orinfer_b200.config import PRESETS
from orinfer_b200.engine import packages as P
from orinfer_b200.engine.checkpoint import save_model
from orinfer_b200.models.weights import random_model


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    d = tmp_path_factory.mktemp("model")
    save_model(random_model(PRESETS["tiny"], seed=0), d)
    return d


def test_create_install_resolve_and_no_replace(model_dir, tmp_path):
    arc = tmp_path / "m.tar.xz"
    digest = P.create(model_dir, arc)
    cache = tmp_path / "cache"
    path = P.install(arc, str(cache))
    assert path == cache / digest and (path / "model.safetensors").exists()
    assert not list(cache.glob(".install-*"))                     # staging is gone
    assert P.resolve(digest[:10], str(cache)) == path
    with pytest.raises(P.PackageError, match="already installed"):
        P.install(arc, str(cache))


def _tar(path, members, mode="w:gz"):
    with tarfile.open(path, mode) as tar:
        for name, data, kind in members:
            info = tarfile.TarInfo(name)
            if kind == "file":
                info.size = len(data)
                tar.addfile(info, io.BytesIO(data))
            elif kind == "link":
                info.type = tarfile.SYMTYPE
                info.linkname = data.decode()
                tar.addfile(info)


def test_unsafe_and_malformed_archives_are_rejected(tmp_path):
    d = "a" * 64
    cases = {
        "traversal": [(f"{d}/../evil", b"x", "file")],
        "absolute": [("/etc/evil", b"x", "file")],
        "symlink": [(f"{d}/link", b"/etc/passwd", "link")],
        "two roots": [(f"{d}/a", b"x", "file"), ("b" * 64 + "/a", b"x", "file")],
        "bad digest": [("model/a", b"x", "file")],
        "not a model": [(f"{d}/a", b"x", "file")],
    }
    for name, members in cases.items():
        arc = tmp_path / f"{name.replace(' ', '_')}.tar.gz"
        _tar(arc, members)
        with pytest.raises(P.PackageError):
            P.install(arc, str(tmp_path / "cache"))
        assert not (tmp_path / "evil").exists()
    (tmp_path / "plain.bin").write_bytes(b"not an archive")
    with pytest.raises(P.PackageError, match="tar"):
        P.install(tmp_path / "plain.bin", str(tmp_path / "cache"))


def test_cli_package_roundtrip(model_dir, tmp_path):
    from orinfer_b200.cli import main
    arc = tmp_path / "m.tar.gz"
    assert main(["package", "create", str(model_dir), "--output", str(arc)]) == 0
    assert main(["package", "install", str(arc), "--cache", str(tmp_path / "c")]) == 0
    assert main(["package", "install", str(arc), "--cache", str(tmp_path / "c")]) == 2
