"""The allocation-free argmax entry point, called through its exported C symbol.

Some hosts of the kernel library cannot call cudaMalloc once they are running (a
real-time loop that must stay off the allocator lock, or a process whose device memory
was carved up in advance by another runtime), so they cannot supply the scratch
buffers that ``orinfer_argmax`` wants.  ``orinfer_argmax_noalloc`` keeps its scratch in
a fixed array inside the library.  This test checks it against the ordinary entry
point on two calls in a row (the array is reused and never cleared), and that sizes
beyond the built-in scratch are refused.  The file sorts last so a run that stops at
the first failure has already covered everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from orinfer_b200.ops import native
    lib = native.lib()
    fn = lib.orinfer_argmax_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


def test_noalloc_argmax_matches_regular_entry_point_twice(cuda):
    from orinfer_b200.ops import functional as F
    from orinfer_b200.ops import native
    fn = _entry()
    g = torch.Generator().manual_seed(12)
    stream = torch.cuda.current_stream().cuda_stream
    for rows, vocab in ((7, 151936), (3, 5000)):        # second call reuses the dirty scratch
        logits = torch.randn(rows, vocab, generator=g).to(cuda)
        logits[0, 11] = logits[0, vocab - 2] = 77.0     # tie -> lowest index
        if rows > 2:
            logits[2, 3] = float("inf")                 # non-finite row -> -1
        want = F.argmax(logits)
        got = torch.full((rows,), -7, dtype=torch.int32, device=cuda)
        before = torch.cuda.memory_allocated()
        rc = fn(logits.data_ptr(), rows, vocab, got.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(got, want)
        assert int(got[0]) == 11 and int(got[2]) == -1
    assert native.read_status() == 0


def test_noalloc_argmax_rejects_sizes_beyond_its_scratch(cuda):
    fn = _entry()
    logits = torch.zeros(4, 64, device=cuda)
    out = torch.zeros(4, dtype=torch.int32, device=cuda)
    stream = torch.cuda.current_stream().cuda_stream
    assert fn(logits.data_ptr(), 257, 64, out.data_ptr(), stream) == -1
    assert fn(logits.data_ptr(), 4, (1 << 20) + 1, out.data_ptr(), stream) == -1
    assert fn(logits.data_ptr(), -1, 64, out.data_ptr(), stream) == -1
    assert fn(logits.data_ptr(), 0, 64, out.data_ptr(), stream) == 0
    assert fn(logits.data_ptr(), 4, 64, out.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert out.tolist() == [0, 0, 0, 0]
