"""Short text summary of an Nsight Compute report: the counters this backend's roofline claims rest on.

    ncu -i report.ncu-rep --page raw --csv | python -m tilebench_b200.profiling.ncu_summary
    python -m tilebench_b200.profiling.ncu_summary report.ncu-rep          # runs `ncu -i` itself

The reference extracts Duration, memory / compute throughput, block size, registers and shared memory
(scripts/profiling/ncu_writeup.py:37-44); this adds the two families the north star names: DRAM bytes and
throughput for the streaming kernels, tensor-pipe activity for the GEMMs, plus the warp stall reasons that
explain a low figure.  It reads counters only — never a source or instruction listing.
"""
from __future__ import annotations

import csv
import subprocess
import sys

KEYS = [
    "gpu__time_duration.sum",
    "launch__grid_size", "launch__block_size", "launch__registers_per_thread",
    "launch__shared_mem_per_block_dynamic", "launch__shared_mem_per_block_static",
    "sm__cycles_elapsed.avg.per_second",
    "dram__bytes_read.sum", "dram__bytes_write.sum",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",
    "lts__t_sector_hit_rate.pct",
    "sm__throughput.avg.pct_of_peak_sustained_elapsed",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
    "sm__warps_active.avg.pct_of_peak_sustained_active",
    "smsp__issue_active.avg.pct_of_peak_sustained_active",
    "l1tex__data_bank_conflicts_pipe_lsu_mem_shared.sum",
]
STALL_PREFIX = "smsp__average_warps_issue_stalled_"
STALL_SUFFIX = "_per_issue_active.ratio"


def summarise(rows: list[list[str]]) -> list[dict]:
    header, units, body = rows[0], rows[1], rows[2:]
    col = {name: i for i, name in enumerate(header)}
    out = []
    for r in body:
        d = {"kernel": r[col["Kernel Name"]]} if "Kernel Name" in col else {}
        for k in KEYS:
            if k in col and r[col[k]] != "":
                d[k] = f"{r[col[k]]} {units[col[k]]}".strip()
        stalls = []
        for name, i in col.items():
            if name.startswith(STALL_PREFIX) and name.endswith(STALL_SUFFIX):
                try:
                    v = float(r[i].replace(",", ""))
                except ValueError:
                    continue
                if v >= 0.05:
                    stalls.append((v, name[len(STALL_PREFIX):-len(STALL_SUFFIX)]))
        d["stalls"] = ", ".join(f"{n} {v:.2f}" for v, n in sorted(stalls, reverse=True)[:6])
        if "dram__bytes_read.sum" in col and "dram__bytes_write.sum" in col:
            d["dram traffic (read + write)"] = f"{r[col['dram__bytes_read.sum']]} + {r[col['dram__bytes_write.sum']]} {units[col['dram__bytes_read.sum']]}"
        out.append(d)
    return out


def to_markdown(entries: list[dict]) -> str:
    lines = []
    for e in entries:
        lines.append(f"### {e.get('kernel', '?')}\n")
        lines.append("| metric | value |\n|---|---|")
        for k, v in e.items():
            if k != "kernel":
                lines.append(f"| {k} | {v} |")
        lines.append("")
    return "\n".join(lines)


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if argv:
        text = subprocess.run(["ncu", "-i", argv[0], "--page", "raw", "--csv"], capture_output=True, text=True).stdout
    else:
        text = sys.stdin.read()
    rows = [r for r in csv.reader(text.splitlines()) if r]
    start = next((i for i, r in enumerate(rows) if "Kernel Name" in r), None)
    if start is None:
        print("no kernel rows found in the ncu CSV", file=sys.stderr)
        return 1
    print(to_markdown(summarise(rows[start:])))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
