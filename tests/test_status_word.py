"""The device status word: a bounded wait that runs out is reported, and the engine turns a
non-zero word into a fatal error that fails the service closed."""
import ctypes

import pytest
import torch


@pytest.mark.gpu
def test_wait_that_runs_out_sets_the_status_word(cuda):
    """`orinfer_ag_wait` with the sequence counter ahead of flags that nothing sets: the
    single waiting thread gives up after the (shortened) limit, the kernel returns and the
    status word names the peer wait and the source rank.  Nothing faults or spins on."""
    from orinfer_b200.ops import native
    from orinfer_b200.parallel.fused import _AgIn
    lib = native.lib()
    lib.orinfer_ag_wait.argtypes = [ctypes.POINTER(_AgIn), ctypes.c_int, ctypes.c_void_p]
    lib.orinfer_ag_wait.restype = ctypes.c_int
    flags = torch.zeros(8, dtype=torch.int32, device=cuda)          # never bumped
    sent = torch.ones(1, dtype=torch.int32, device=cuda)            # "wait for sequence 1"
    native.set_wait_limit_us(1000)
    try:
        ag = _AgIn(flags.data_ptr(), sent.data_ptr(), 2, 4)
        native.check(lib.orinfer_ag_wait(ctypes.byref(ag), 8, native.stream()), "ag_wait")
        reader = native.StatusReader()
        reader.enqueue()
        torch.cuda.synchronize()
        assert reader.value() == (5 << 16) | 0x100, hex(reader.value())
        assert native.read_status() == (5 << 16) | 0x100
    finally:
        native.clear_status()
        native.set_wait_limit_us(1_000_000)
    assert native.read_status() == 0
    # the context is still usable
    assert int(torch.arange(10, device=cuda).sum()) == 45


def test_engine_fails_closed_on_a_nonzero_status_word():
    from orinfer_b200.config import PRESETS
    from orinfer_b200.core.policy import EngineError, ErrorKind
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.models.weights import random_model

    class StubStatus:
        def __init__(self):
            self.word = 0
            self.enqueued = 0

        def enqueue(self):
            self.enqueued += 1

        def value(self):
            return self.word

    eng = Engine(random_model(PRESETS["tiny"], seed=0), kv_pages=16, max_context=256)
    eng._status = stub = StubStatus()
    req = eng.submit([1, 2, 3, 4], 8)
    eng.step()
    assert stub.enqueued >= 1 and len(req.generated) == 1
    stub.word = (5 << 16) | 3                       # a peer wait of source rank 3 ran out
    with pytest.raises(EngineError) as err:
        eng.step()
    assert err.value.kind is ErrorKind.NCCL and err.value.fatal
    assert "peer wait" in str(err.value)
    stub.word = 0                                    # sticky: the engine stays failed
    with pytest.raises(EngineError):
        eng.step()


def test_expect_device_refuses_a_foreign_device(monkeypatch):
    from orinfer_b200.ops import native

    class FakeLib:
        @staticmethod
        def orinfer_current_device():
            return 0

    monkeypatch.setattr(native, "_load", lambda: FakeLib)
    native.expect_device("cuda:0")
    with pytest.raises(native.KernelError):
        native.expect_device("cuda:1")
