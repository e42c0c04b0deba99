"""CPU placement of rank processes.

``ORINFER_WORKER_CPUS`` names one CPU set per rank, sets separated by ``;``, CPUs and closed
ranges separated by ``,`` (``"0-7;8-15"``: rank 0 on CPUs 0..7, rank 1 on 8..15).  The list
must name exactly as many sets as there are ranks, a set may not be empty or repeat a CPU, two
ranks may not share one, and every CPU must be one this process may run on.  When the variable
is set, every rank pins itself before it creates its CUDA context and its reader threads, so a
rank's host work stays near its GPU and ranks do not migrate onto each other's cores.  Same
contract as the reference's worker placement
(crates/orinfer-engine/src/models/deepseek_v41/affinity.rs:18-143).
"""

from __future__ import annotations

import os
from typing import List, Optional, Sequence

VARIABLE = "ORINFER_WORKER_CPUS"
CPU_LIMIT = 4096


class AffinityError(ValueError):
    pass


def parse(value: str, ranks: int) -> List[List[int]]:
    """CPU ids per rank, each sorted ascending."""
    groups = value.split(";")
    if len(groups) != ranks:
        raise AffinityError(f"expected {ranks} worker CPU sets, found {len(groups)}")
    out = [_parse_set(g) for g in groups]
    seen = set()
    for cpus in out:
        for cpu in cpus:
            if cpu in seen:
                raise AffinityError("worker CPU sets overlap")
            seen.add(cpu)
    return out


def _parse_set(text: str) -> List[int]:
    cpus = set()
    for part in text.split(","):
        part = part.strip()
        if not part:
            raise AffinityError("empty worker CPU entry")
        first, dash, last = part.partition("-")
        try:
            lo = int(first)
            hi = int(last) if dash else lo
        except ValueError as e:
            raise AffinityError(f"invalid worker CPU `{part}`") from e
        if lo < 0 or hi < lo or hi >= CPU_LIMIT:
            raise AffinityError(f"invalid worker CPU range `{part}`")
        for cpu in range(lo, hi + 1):
            if cpu in cpus:
                raise AffinityError("a worker CPU set repeats a CPU")
            cpus.add(cpu)
    if not cpus:
        raise AffinityError("empty worker CPU set")
    return sorted(cpus)


def configured(ranks: int, value: Optional[str] = None) -> Optional[List[List[int]]]:
    """The placement the environment asks for, checked against the CPUs this process may
    use; None when the variable is not set."""
    value = os.environ.get(VARIABLE) if value is None else value
    if not value:
        return None
    sets = parse(value, ranks)
    allowed = os.sched_getaffinity(0)
    for cpus in sets:
        missing = [c for c in cpus if c not in allowed]
        if missing:
            raise AffinityError(f"worker CPUs {missing} are not available to this process")
    return sets


def bind(cpus: Sequence[int]) -> None:
    """Pins the calling process (all threads it creates afterwards) to ``cpus``."""
    try:
        os.sched_setaffinity(0, set(cpus))
    except OSError as e:
        raise AffinityError(f"failed to bind worker CPUs: {e}") from e


def bind_rank(rank: int, ranks: int) -> Optional[List[int]]:
    """Applies this rank's set when ``ORINFER_WORKER_CPUS`` is set; returns it."""
    sets = configured(ranks)
    if sets is None:
        return None
    bind(sets[rank])
    return sets[rank]
