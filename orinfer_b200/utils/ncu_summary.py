"""Turns an Nsight Compute raw-page CSV into the short roofline summary kept under ``profiles/``.

    ncu -i capture.ncu-rep --page raw --csv > capture.csv
    python -m orinfer_b200.utils.ncu_summary capture.csv --flops 2.1e11 --bytes 5.2e7

Reads only counters (durations, DRAM bytes and throughput, tensor-pipe activity, occupancy,
registers, stall reasons); no source or instruction pages are read or produced.  One table row
per captured launch.  ``--flops`` / ``--bytes`` are the algorithmic work of one launch; with
them the achieved rates and the fractions of the measured peaks (``MEASURED_PEAKS.json`` at
the repository root, else the stated fallback) are added.  Same role as the reference's
``python/orinfer_build/validation/profile_summary.py`` (which attributes Nsight Systems graph
nodes to plan operations); here the unit of attribution is the kernel launch.
"""

from __future__ import annotations

import argparse
import csv
import io
import sys
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional

# counter -> (column label, unit conversion to the label's unit)
WANTED = {
    "gpu__time_duration.sum": "duration_us",
    "dram__bytes_read.sum": "dram_read_mb",
    "dram__bytes_write.sum": "dram_write_mb",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed": "dram_pct",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active": "tensor_pct",
    "sm__inst_executed_pipe_tensor.sum": "tensor_insts",
    "sm__warps_active.avg.pct_of_peak_sustained_active": "warps_active_pct",
    "sm__throughput.avg.pct_of_peak_sustained_elapsed": "sm_pct",
    "launch__registers_per_thread": "registers",
    "launch__shared_mem_per_block_dynamic": "smem_dynamic_kb",
    "launch__grid_size": "grid",
    "launch__block_size": "block",
}
STALL_PREFIX = "smsp__average_warps_issue_stalled_"
STALL_SUFFIX = "_per_issue_active.ratio"
_SCALE = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12,
          "ns": 1e-3, "us": 1.0, "ms": 1e3, "s": 1e6, "nsecond": 1e-3, "usecond": 1.0,
          "msecond": 1e3, "second": 1e6}


@dataclass
class Launch:
    kernel: str
    values: Dict[str, float] = field(default_factory=dict)
    stalls: Dict[str, float] = field(default_factory=dict)

    def top_stalls(self, n: int = 3) -> List[str]:
        ranked = sorted(self.stalls.items(), key=lambda kv: -kv[1])[:n]
        return [f"{k} {v:.2f}" for k, v in ranked if v > 0]


def _number(text: str) -> Optional[float]:
    try:
        return float(text.replace(",", ""))
    except ValueError:
        return None


def _short(name: str) -> str:
    """Column headers carry a unit/section prefix ("FBSP.TriageCompute.dram__..."): the
    counter starts at the first component that contains a double underscore."""
    parts = name.split(".")
    for i, part in enumerate(parts):
        if "__" in part:
            return ".".join(parts[i:])
    return name


def parse(text: str) -> List[Launch]:
    """Launches of a ``--page raw --csv`` dump (header row, unit row, one row per launch)."""
    rows = list(csv.reader(io.StringIO(text)))
    rows = [r for r in rows if r and not r[0].startswith("==")]
    if len(rows) < 3:
        raise ValueError("ncu summary: expected a header row, a unit row and launches")
    header, units = rows[0], rows[1]
    if "Kernel Name" not in header:
        raise ValueError("ncu summary: not a raw-page CSV (no 'Kernel Name' column)")
    name_col = header.index("Kernel Name")
    short = [_short(h) for h in header]
    out = []
    for row in rows[2:]:
        if len(row) != len(header):
            continue
        launch = Launch(row[name_col])
        for col, (counter, unit) in enumerate(zip(short, units)):
            value = _number(row[col])
            if value is None:
                continue
            label = WANTED.get(counter)
            if label is not None and label not in launch.values:
                if label.endswith("_mb"):
                    value = value * _SCALE.get(unit, 1.0) / 1e6
                elif label.endswith("_us"):
                    value = value * _SCALE.get(unit, 1.0)
                elif label.endswith("_kb"):
                    value = value * _SCALE.get(unit, 1.0) / 1e3
                launch.values[label] = value
            elif counter.startswith(STALL_PREFIX) and counter.endswith(STALL_SUFFIX):
                reason = counter[len(STALL_PREFIX):-len(STALL_SUFFIX)]
                if not reason.endswith("_not_issued"):
                    launch.stalls[reason] = value
        out.append(launch)
    return out


def kernel_label(name: str, width: int = 48) -> str:
    base = name.split("(")[0].replace("void ", "").strip()
    return base if len(base) <= width else base[:width - 1] + "…"


def render(launches: Iterable[Launch], flops: float = 0.0, nbytes: float = 0.0,
           peaks=None) -> str:
    """Markdown table; ``peaks`` = (bytes/s, flop/s, tag)."""
    cols = ["kernel", "grid x block", "regs", "duration us", "DRAM MB (r+w)", "DRAM %",
            "tensor %", "warps active %", "top stalls"]
    if nbytes:
        cols += ["GB/s", "of HBM peak"]
    if flops:
        cols += ["TFLOP/s", "of tensor peak"]
    lines = ["| " + " | ".join(cols) + " |", "| " + " | ".join("---" for _ in cols) + " |"]
    fmt = lambda v, spec="{:.1f}": "-" if v is None else spec.format(v)
    for l in launches:
        v = l.values.get
        dur = v("duration_us")
        traffic = None
        if v("dram_read_mb") is not None or v("dram_write_mb") is not None:
            traffic = (v("dram_read_mb") or 0.0) + (v("dram_write_mb") or 0.0)
        row = [kernel_label(l.kernel),
               f"{fmt(v('grid'), '{:.0f}')} x {fmt(v('block'), '{:.0f}')}",
               fmt(v("registers"), "{:.0f}"), fmt(dur), fmt(traffic), fmt(v("dram_pct")),
               fmt(v("tensor_pct")), fmt(v("warps_active_pct")), ", ".join(l.top_stalls()) or "-"]
        if nbytes:
            rate = nbytes / (dur * 1e-6) if dur else None
            row += [fmt(rate / 1e9 if rate else None),
                    fmt(rate / peaks[0] if rate and peaks else None, "{:.2f}")]
        if flops:
            rate = flops / (dur * 1e-6) if dur else None
            row += [fmt(rate / 1e12 if rate else None),
                    fmt(rate / peaks[1] if rate and peaks else None, "{:.2f}")]
        lines.append("| " + " | ".join(row) + " |")
    if peaks and (flops or nbytes):
        lines.append("")
        lines.append(f"Peaks: {peaks[0] / 1e9:.0f} GB/s copy, {peaks[1] / 1e12:.0f} TFLOP/s bf16 "
                     f"({peaks[2]}); durations are under the profiler (serialised, cold cache): "
                     "compare shares, take absolute times from CUDA events.")
    return "\n".join(lines) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("csv", help="output of `ncu -i X.ncu-rep --page raw --csv` ('-' = stdin)")
    ap.add_argument("--flops", type=float, default=0.0, help="algorithmic FLOPs of one launch")
    ap.add_argument("--bytes", type=float, default=0.0, help="algorithmic bytes of one launch")
    ap.add_argument("--kernel", default="", help="keep launches whose name contains this")
    a = ap.parse_args(argv)
    text = sys.stdin.read() if a.csv == "-" else open(a.csv).read()
    launches = [l for l in parse(text) if a.kernel in l.kernel]
    from ..bench.kernel_probe import peaks
    sys.stdout.write(render(launches, a.flops, a.bytes, peaks()))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
