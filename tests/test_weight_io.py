"""C++ safetensors reader: index, parallel copy, SHA-256 verification."""
import hashlib

import pytest
import torch
from safetensors.torch import save_file

from orinfer_b200.engine import weight_io as W


def test_reader_matches_safetensors_and_verifies(tmp_path):
    g = torch.Generator().manual_seed(0)
    t = {"a.int8": torch.randint(-128, 127, (37, 256), generator=g, dtype=torch.int8),
         "b.packed": torch.randint(-2 ** 31, 2 ** 31 - 1, (3, 40, 16), generator=g, dtype=torch.int32),
         "c.scale": torch.randn(40, generator=g).half(), "d": torch.randn(5, 7, generator=g),
         "empty": torch.zeros(0, dtype=torch.float16)}
    path = tmp_path / "m.safetensors"
    save_file(t, str(path), metadata={"codec": "x-v1", "layout": 'quoted "name"'})
    got, meta = W.read_tensors(path, workers=3)
    assert set(got) == set(t) and meta == {"codec": "x-v1", "layout": 'quoted "name"'}
    for k in t:
        assert got[k].dtype == t[k].dtype and torch.equal(got[k], t[k])
    digests = {k: hashlib.sha256(v.numpy().tobytes()).hexdigest() for k, v in t.items()}
    assert W.sha256_hex(t["b.packed"]) == digests["b.packed"]
    W.read_tensors(path, workers=2, digests=digests)
    digests["c.scale"] = "0" * 64
    with pytest.raises(W.WeightReadError, match="c.scale"):
        W.read_tensors(path, digests=digests)


def test_reader_rejects_truncated_and_malformed_files(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00{\"a\":")
    with pytest.raises(W.WeightReadError):
        W.read_tensors(p)
    save_file({"x": torch.zeros(1024)}, str(tmp_path / "ok.safetensors"))
    raw = (tmp_path / "ok.safetensors").read_bytes()
    (tmp_path / "cut.safetensors").write_bytes(raw[:-100])
    with pytest.raises(W.WeightReadError, match="outside the file"):
        W.read_tensors(tmp_path / "cut.safetensors")
