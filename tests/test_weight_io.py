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


def test_tensors_are_created_in_an_arena_and_streamed_through_bounded_staging(tmp_path):
    """With a target device small tensors are views of one arena allocation and large ones
    stand alone; the staged walk (what a GPU load does) moves the file through two small
    staging buffers, in several batches, and gives the same bytes and digests."""
    g = torch.Generator().manual_seed(1)
    t = {f"t{i:02d}": torch.randint(-128, 127, (17 + 13 * i, 64), generator=g, dtype=torch.int8)
         for i in range(12)}
    t["big"] = torch.randn(300, 128, generator=g)                      # 150 KiB: stands alone
    t["half"] = torch.randn(33, generator=g).half()
    t["empty"] = torch.zeros(0, dtype=torch.int32)
    path = tmp_path / "m.safetensors"
    save_file(t, str(path))
    digests = {k: hashlib.sha256(v.numpy().tobytes()).hexdigest() for k, v in t.items()}
    for staged in (False, True):
        got, _ = W.read_tensors(path, workers=3, device="cpu", digests=digests, staged=staged,
                                staging_bytes=16 << 10, arena_limit=64 << 10)
        for k in t:
            assert got[k].dtype == t[k].dtype and torch.equal(got[k], t[k]), (k, staged)
        small = [k for k in t if t[k].numel() * t[k].element_size() <= 64 << 10 and t[k].numel()]
        bases = {got[k].untyped_storage().data_ptr() for k in small}
        assert len(bases) == 1                                          # one arena
        assert got["big"].untyped_storage().data_ptr() not in bases
        assert all(got[k].data_ptr() % 256 == 0 for k in small)
    bad = dict(digests, t05="0" * 64)
    with pytest.raises(W.WeightReadError, match="t05"):
        W.read_tensors(path, device="cpu", digests=bad, staged=True, staging_bytes=16 << 10)
    sizes = [100, 5000, 300, 9000, 20000, 1]
    assert W.plan_batches(sizes, 8192) == [[0, 1, 2], [3], [4], [5]]
    offs, total = W.plan_arena(sizes, 6000)
    assert offs == [0, 256, 5376, None, None, 5888] and total == 6144
