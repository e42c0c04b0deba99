"""Launch-variant tables: which GEMM tile configuration serves which row range.

A table is JSON::

    {"device": "NVIDIA B200", "schema": 1,
     "gemm": [{"fmt": "q4", "n": 19456, "k": 2560, "m_lo": 257, "m_hi": 512,
               "mt": 2, "nb": 128, "splits": 1, "us": 61.2, "us_default": 64.0}, ...],
     "attention": [{"rows_lo": 1, "rows_hi": 1, "ctx_lo": 257, "ctx_hi": 1024, "kvh": 8,
                    "splits": 8, "us": 11.9, "us_default": 12.4}, ...]}

Every entry replaces the launch heuristics of the tensor-core GEMM for rows ``m_lo..m_hi`` of
one projection shape; shapes and row counts that no entry covers keep the heuristics.  The
optional ``attention`` list does the same for the key-axis split count of decode attention.  The
reference selects kernels per row range the same way (``KernelVariant{min_rows, max_rows}``,
crates/orinfer-model-sdk/src/operators/rows.rs:10-60) from tables written by its offline
tuners (python/orinfer_build/tuning/); here the tuner is ``orinfer_b200.tuning.gemm_tuner``.

``load_default`` is called when the kernel library is initialised: it applies the table named
by ``ORINFER_TUNING_TABLE`` (``off`` disables tuning), else ``data/b200.json`` beside this
file when present.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, List, Optional

FORMATS = {"w8": 0, "q4": 1, "q2": 2}
SCHEMA = 1
DEFAULT_PATH = Path(__file__).parent / "data" / "b200.json"
SPLITK_WORKSPACE_BYTES = 96 << 20


@dataclass(frozen=True)
class GemmVariant:
    fmt: str
    n: int
    k: int
    m_lo: int
    m_hi: int
    mt: int
    nb: int
    splits: int
    us: float = 0.0
    us_default: float = 0.0

    def problems(self) -> List[str]:
        """Why the kernel library would refuse this entry (empty = valid)."""
        bad = []
        if self.fmt not in FORMATS:
            bad.append(f"unknown format {self.fmt!r}")
        if self.m_lo < 1 or self.m_hi < self.m_lo:
            bad.append("row range must satisfy 1 <= m_lo <= m_hi")
        if self.n < 8 or self.k < 128 or self.k % 128:
            bad.append("n >= 8 and k a positive multiple of 128")
        if self.mt not in (1, 2, 4):
            bad.append("mt must be 1, 2 or 4")
        if self.nb not in (128, 64, 32):
            bad.append("nb must be 128, 64 or 32")
        if not 1 <= self.splits <= min(16, max(self.k // 128, 1)):
            bad.append("splits must be within 1..min(16, k/128)")
        elif self.splits > 1:
            if self.nb != 128 or self.n % 8:
                bad.append("split-K needs nb = 128 and n % 8 == 0")
            if self.splits * self.m_hi * self.n * 4 > SPLITK_WORKSPACE_BYTES:
                bad.append("split-K partials exceed the workspace")
        return bad


def parse(text: str) -> List[GemmVariant]:
    """Entries of a table; raises ValueError on a malformed table, an invalid entry or two
    entries of one shape whose row ranges overlap."""
    doc = json.loads(text)
    if not isinstance(doc, dict) or doc.get("schema") != SCHEMA:
        raise ValueError(f"tuning table: schema {SCHEMA} expected")
    out: List[GemmVariant] = []
    for i, e in enumerate(doc.get("gemm", [])):
        try:
            v = GemmVariant(**{k: e[k] for k in ("fmt", "n", "k", "m_lo", "m_hi", "mt", "nb",
                                                  "splits")},
                            us=float(e.get("us", 0.0)), us_default=float(e.get("us_default", 0.0)))
        except (KeyError, TypeError) as err:
            raise ValueError(f"tuning table: entry {i}: {err}") from None
        bad = v.problems()
        if bad:
            raise ValueError(f"tuning table: entry {i}: {'; '.join(bad)}")
        out.append(v)
    seen = {}
    for v in sorted(out, key=lambda v: (v.fmt, v.n, v.k, v.m_lo)):
        key = (v.fmt, v.n, v.k)
        if key in seen and v.m_lo <= seen[key]:
            raise ValueError(f"tuning table: overlapping row ranges for {key}")
        seen[key] = v.m_hi
    return out


def dump(variants: Iterable[GemmVariant], device: str) -> str:
    rows = [dict(fmt=v.fmt, n=v.n, k=v.k, m_lo=v.m_lo, m_hi=v.m_hi, mt=v.mt, nb=v.nb,
                 splits=v.splits, us=round(v.us, 2), us_default=round(v.us_default, 2))
            for v in sorted(variants, key=lambda v: (v.fmt, v.n, v.k, v.m_lo))]
    return json.dumps({"schema": SCHEMA, "device": device, "gemm": rows}, indent=1) + "\n"


def lookup(variants: Iterable[GemmVariant], fmt: str, m: int, n: int, k: int
           ) -> Optional[GemmVariant]:
    for v in variants:
        if v.fmt == fmt and v.n == n and v.k == k and v.m_lo <= m <= v.m_hi:
            return v
    return None


def merge_ranges(variants: Iterable[GemmVariant]) -> List[GemmVariant]:
    """Joins neighbouring row ranges of one shape that chose the same configuration."""
    out: List[GemmVariant] = []
    for v in sorted(variants, key=lambda v: (v.fmt, v.n, v.k, v.m_lo)):
        last = out[-1] if out else None
        if (last is not None and (last.fmt, last.n, last.k, last.mt, last.nb, last.splits)
                == (v.fmt, v.n, v.k, v.mt, v.nb, v.splits) and last.m_hi + 1 == v.m_lo):
            out[-1] = GemmVariant(v.fmt, v.n, v.k, last.m_lo, v.m_hi, v.mt, v.nb, v.splits,
                                  max(last.us, v.us), max(last.us_default, v.us_default))
        else:
            out.append(v)
    return out


# ---------------------------------------------------------------- decode attention splits
@dataclass(frozen=True)
class AttentionSplit:
    """Key-axis split count of the decode / verify attention kernel for packets of
    ``rows_lo..rows_hi`` rows whose longest context is within ``ctx_lo..ctx_hi`` tokens, on a
    model with ``kvh`` KV heads.  Replaces the heuristic of ``ops.functional.attention_splits``
    for that range (written by ``orinfer_b200.tuning.attention_tuner``)."""
    rows_lo: int
    rows_hi: int
    ctx_lo: int
    ctx_hi: int
    kvh: int
    splits: int
    us: float = 0.0
    us_default: float = 0.0

    def problems(self) -> List[str]:
        bad = []
        if self.rows_lo < 1 or self.rows_hi < self.rows_lo:
            bad.append("row range must satisfy 1 <= rows_lo <= rows_hi")
        if self.ctx_lo < 1 or self.ctx_hi < self.ctx_lo:
            bad.append("context range must satisfy 1 <= ctx_lo <= ctx_hi")
        if self.kvh < 1:
            bad.append("kvh must be positive")
        if not 1 <= self.splits <= 32:
            bad.append("splits must be within 1..32")
        return bad


ATTENTION: List[AttentionSplit] = []


def parse_attention(text: str) -> List[AttentionSplit]:
    doc = json.loads(text)
    if not isinstance(doc, dict) or doc.get("schema") != SCHEMA:
        raise ValueError(f"tuning table: schema {SCHEMA} expected")
    out: List[AttentionSplit] = []
    for i, e in enumerate(doc.get("attention", [])):
        try:
            v = AttentionSplit(**{k: int(e[k]) for k in ("rows_lo", "rows_hi", "ctx_lo", "ctx_hi",
                                                         "kvh", "splits")},
                               us=float(e.get("us", 0.0)),
                               us_default=float(e.get("us_default", 0.0)))
        except (KeyError, TypeError, ValueError) as err:
            raise ValueError(f"tuning table: attention entry {i}: {err}") from None
        bad = v.problems()
        if bad:
            raise ValueError(f"tuning table: attention entry {i}: {'; '.join(bad)}")
        out.append(v)
    for a in range(len(out)):
        for b in range(a + 1, len(out)):
            x, y = out[a], out[b]
            if (x.kvh == y.kvh and x.rows_lo <= y.rows_hi and y.rows_lo <= x.rows_hi
                    and x.ctx_lo <= y.ctx_hi and y.ctx_lo <= x.ctx_hi):
                raise ValueError(f"tuning table: attention entries {a} and {b} overlap")
    return out


def attention_lookup(max_kv_len: int, rows: int, kvh: int) -> Optional[int]:
    for v in ATTENTION:
        if v.kvh == kvh and v.rows_lo <= rows <= v.rows_hi and v.ctx_lo <= max_kv_len <= v.ctx_hi:
            return v.splits
    return None


def set_attention(entries: Iterable[AttentionSplit]) -> int:
    ATTENTION[:] = list(entries)
    return len(ATTENTION)


def dump_attention(entries: Iterable[AttentionSplit]) -> List[dict]:
    return [dict(rows_lo=v.rows_lo, rows_hi=v.rows_hi, ctx_lo=v.ctx_lo, ctx_hi=v.ctx_hi,
                 kvh=v.kvh, splits=v.splits, us=round(v.us, 2), us_default=round(v.us_default, 2))
            for v in sorted(entries, key=lambda v: (v.kvh, v.rows_lo, v.ctx_lo))]


def apply(variants: Iterable[GemmVariant], lib=None) -> int:
    """Replaces the kernel library's variant table; returns the number of entries set."""
    if lib is None:
        from ..ops import native
        lib = native.lib()
    lib.orinfer_qgemm_clear_variants()
    count = 0
    for v in variants:
        code = lib.orinfer_qgemm_set_variant(FORMATS[v.fmt], v.m_lo, v.m_hi, v.n, v.k, v.mt, v.nb,
                                             v.splits)
        if code != 0:
            raise ValueError(f"kernel library refused tuning entry {v} (code {code})")
        count += 1
    return count


def load_default(lib=None) -> int:
    name = os.environ.get("ORINFER_TUNING_TABLE", "")
    if name == "off":
        set_attention([])
        return apply([], lib)
    path = Path(name) if name else DEFAULT_PATH
    if not path.exists():
        if name:
            raise FileNotFoundError(f"ORINFER_TUNING_TABLE={name} does not exist")
        return 0
    text = path.read_text()
    set_attention(parse_attention(text))
    return apply(parse(text), lib)
