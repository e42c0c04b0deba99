"""Rank control plane on CPU threads: lock-step broadcast, two-phase decisions, deadlines,
sticky fail-closed failure, with failures injected on the host (no GPU involved)."""
import time

import pytest

from orinfer_b200.parallel import team as T

OP_ECHO, OP_FREE, OP_PLAN, OP_COMMIT, OP_ROLLBACK, OP_REDUCE, OP_KEY = range(7)


def _team(n=4, fast_ms=400, state=None, comm=None):
    state = state if state is not None else {}

    def handler(rank, op, args):
        if op == OP_ECHO:
            return rank * 100 + args[0]
        if op == OP_FREE:
            return state.get("free", [10, 7, 9, 8])[rank]
        if op == OP_PLAN:
            return 0 if rank in state.get("refuse", ()) else 1
        if op == OP_COMMIT:
            state.setdefault("committed", []).append(rank)
            return 1
        if op == OP_ROLLBACK:
            state.setdefault("rolled_back", []).append(rank)
            return 1
        if op == OP_REDUCE:
            return int(comm.all_reduce(rank, [float(rank + 1)], timeout_ms=300)[0])
        if op == OP_KEY:
            return state.get("keys", [5, 5, 5, 5])[rank]
        raise ValueError(op)

    return T.Team(n, handler, fast_ms=fast_ms, heavy_ms=2000), state


def test_broadcast_is_lock_step_and_ordered():
    team, _ = _team()
    try:
        for i in range(50):
            assert team.broadcast(OP_ECHO, [i]) == [r * 100 + i for r in range(4)]
        assert team.failure() is None
    finally:
        team.close()


def test_two_phase_budget_agreement_and_rollback():
    team, state = _team()
    try:
        assert team.budget(OP_FREE) == 7                      # admission uses the min over ranks
        assert team.agree(OP_KEY) == 5
        state["keys"] = [5, 5, 6, 5]
        with pytest.raises(ValueError):
            team.agree(OP_KEY)
        assert team.save(OP_PLAN, OP_COMMIT, OP_ROLLBACK) and sorted(state["committed"]) == [0, 1, 2, 3]
        state["refuse"] = {2}
        assert not team.save(OP_PLAN, OP_COMMIT, OP_ROLLBACK)
        assert sorted(state["rolled_back"]) == [0, 1, 2, 3] and len(state["committed"]) == 4
    finally:
        team.close()


@pytest.mark.parametrize("kind,expect", [(T.DROP_REPLY, T.TIMEOUT), (T.DELAY_MS, T.TIMEOUT),
                                         (T.ERROR_CODE, T.RANK_ERROR),
                                         (T.EXIT_THREAD, T.DISCONNECTED)])
def test_first_failure_is_sticky_and_later_commands_fail_fast(kind, expect):
    team, _ = _team()
    try:
        assert team.broadcast(OP_ECHO, [1])[3] == 301
        team.inject(2, kind, value=900 if kind == T.DELAY_MS else 77)
        with pytest.raises(T.TeamFailure) as err:
            team.broadcast(OP_ECHO, [2])
        assert err.value.result == expect and err.value.rank == 2
        if kind == T.ERROR_CODE:
            assert err.value.code == 77
        t0 = time.monotonic()
        with pytest.raises(T.TeamFailure) as again:
            team.broadcast(OP_ECHO, [3])
        assert again.value.result == T.STICKY and time.monotonic() - t0 < 0.1
        assert team.failure()[0] == 2
    finally:
        team.close()


def test_handler_exception_marks_rank_failed():
    team, _ = _team()
    try:
        with pytest.raises(T.TeamFailure) as err:
            team.broadcast(99)
        assert err.value.result == T.RANK_ERROR
    finally:
        team.close()


def test_fake_collective_and_rank_that_never_joins():
    comm = T.FakeComm(4)
    team, _ = _team(comm=comm, fast_ms=1500)
    try:
        assert team.broadcast(OP_REDUCE) == [10, 10, 10, 10]
        assert comm.calls == 1
        comm.fail_next(1, 13)                                  # rank 1 errors out of the collective
        with pytest.raises(T.TeamFailure) as err:              # peers time out inside it, bounded
            team.broadcast(OP_REDUCE)
        assert err.value.result == T.RANK_ERROR
        assert team.failure() is not None
    finally:
        team.close()
        comm.close()


def test_preflight_gate():
    assert T.preflight([lambda: True] * 3, timeout_s=1.0)
    assert not T.preflight([lambda: True, lambda: False], timeout_s=1.0)
    assert not T.preflight([lambda: True, lambda: time.sleep(0.5) or True], timeout_s=0.1)


def test_worker_cpu_sets_are_parsed_checked_and_applied(monkeypatch):
    """``ORINFER_WORKER_CPUS``: one CPU set per rank; malformed, overlapping or unavailable
    sets are refused; a rank pins itself to its set."""
    import os
    from orinfer_b200.parallel import affinity as A
    assert A.parse("0-2,5;3,4", 2) == [[0, 1, 2, 5], [3, 4]]
    assert A.parse(" 7 ", 1) == [[7]]
    for bad, ranks in (("0-1", 2), ("0;0", 2), ("0-1,1;2", 2), ("3-1;4", 2), ("a;1", 2),
                       ("0,;1", 2), (";1", 2), ("0;99999", 2), ("-1;2", 2)):
        with pytest.raises(A.AffinityError):
            A.parse(bad, ranks)
    assert A.configured(2, "") is None
    monkeypatch.delenv(A.VARIABLE, raising=False)
    assert A.bind_rank(0, 2) is None
    allowed = sorted(os.sched_getaffinity(0))
    outside = max(allowed) + 1
    with pytest.raises(A.AffinityError, match="not available"):
        A.configured(2, f"{allowed[0]};{outside}")
    if len(allowed) >= 2:
        monkeypatch.setenv(A.VARIABLE, f"{allowed[0]};{allowed[1]}")
        try:
            assert A.bind_rank(1, 2) == [allowed[1]]
            assert os.sched_getaffinity(0) == {allowed[1]}
        finally:
            os.sched_setaffinity(0, allowed)
