"""Side-by-side table of this backend's summary CSVs and the reference's published B200 CSVs.

    python -m tilebench_b200.run_bench --operator weight_dequant --output-root out/l2x2          # reference protocol (2x L2 flush)
    python -m tilebench_b200.run_bench --operator weight_dequant --flush-mb 64 --output-root out/flush64
    python -m tilebench_b200.profiling.head_to_head --ours out/l2x2/B200/csv --ours-flush64 out/flush64/B200/csv \\
        --published /path/to/TileBench/results/B200/csv --out head_to_head.md

For every case of the four reference operators on the path it lists this backend's time under both
protocols beside the fastest published DSL backend (Triton / cuTile / TileLang, default and autotuned
CSVs), then sums up per operator: cases at or ahead of the best published time, and the geometric mean of
the ratio.  The published rows were taken on another B200 with a 64 MB eviction buffer (half of L2), so the
`flush64` column is the like-for-like one; the `2xL2` column is what the current reference timer would show.
"""
from __future__ import annotations

import argparse
import csv
import math
from pathlib import Path

OPERATORS = ("weight_dequant", "dequantize_rowwise", "matmul_int8", "matmul_fp32_fp16_fp8")
DSL = ("triton", "cutile", "tilelang")


def _params(text: str) -> dict:
    out = {}
    for part in text.split(","):
        if "=" in part:
            k, v = part.split("=", 1)
            out[k.strip()] = v.strip()
    return out


def _num(x):
    try:
        v = float(x)
        return v if v > 0 and not math.isnan(v) else None
    except (TypeError, ValueError):
        return None


def read_ours(path: Path) -> dict:
    rows = {}
    if not path.is_file():
        return rows
    for r in csv.DictReader(open(path)):
        rows[(frozenset(_params(r["params"]).items()), r["dtype"])] = (_num(r.get("cuda_ms")), _num(r.get("torch_ms")), r["params"])
    return rows


def read_published(path: Path) -> list:
    if not path.is_file():
        return []
    out = []
    for r in csv.DictReader(open(path)):
        best = min(((v, b) for b in DSL if (v := _num(r.get(f"{b}_ms"))) is not None), default=(None, None))
        out.append((_params(r["params"]), r["dtype"], best[0], best[1], _num(r.get("torch_ms"))))
    return out


def match(ours: dict, params: dict, dtype: str):
    """Our row whose parameters contain the published row's (ours also lists the case defaults)."""
    want = set(params.items())
    for (p, dt), val in ours.items():
        if dt == dtype and want <= set(p):
            return val
    return None


def operator_section(op: str, ours_dir: Path, flush_dir: Path | None, pub_dir: Path, max_rows: int) -> str:
    ours = read_ours(ours_dir / f"{op}_default.csv")
    ours64 = read_ours(flush_dir / f"{op}_default.csv") if flush_dir else {}
    lines = [f"### {op}", "",
             "| case | dtype | cuda 2xL2 ms | cuda flush64 ms | best published default | best published autotuned | flush64 / autotuned |",
             "|---|---|---|---|---|---|---|"]
    pub_default = read_published(pub_dir / f"{op}_default.csv")
    pub_auto = {(frozenset(p.items()), dt): (ms, who) for p, dt, ms, who, _ in read_published(pub_dir / f"{op}_autotune.csv")}
    ratios, ahead, total, table = [], 0, 0, []
    for params, dtype, dms, dwho, _ in pub_default:
        a = match(ours, params, dtype)
        b = match(ours64, params, dtype)
        ams, awho = pub_auto.get((frozenset(params.items()), dtype), (None, None))
        mine = (b or a or (None,))[0]
        best = min((x for x in (dms, ams) if x), default=None)
        if mine and best:
            total += 1
            ratios.append(mine / best)
            ahead += mine <= best
        cell = lambda v, w=None: "" if v is None else (f"{v:.4f}" + (f" ({w})" if w else ""))
        table.append((", ".join(f"{k}={v}" for k, v in params.items()), dtype, cell(a[0] if a else None), cell(b[0] if b else None),
                      cell(dms, dwho), cell(ams, awho), "" if not (mine and ams) else f"{mine / ams:.2f}"))
    step = max(1, len(table) // max_rows)
    shown = table[::step][-max_rows:] if len(table) > max_rows else table
    if table and table[-1] not in shown:
        shown.append(table[-1])
    lines += ["| " + " | ".join(r) + " |" for r in shown]
    if total:
        gm = math.exp(sum(math.log(x) for x in ratios) / len(ratios))
        lines += ["", f"{op}: {ahead} of {total} cases at or ahead of the fastest published DSL time; geometric mean of ours / best published = {gm:.2f} "
                      f"(min {min(ratios):.2f}, max {max(ratios):.2f}); {len(table)} published cases, every {step}th shown."]
    else:
        lines += ["", f"{op}: no matching rows (ours: {len(ours)}, published: {len(table)})."]
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--ours", required=True, help="csv folder written by run_bench under the reference protocol (2x L2 flush)")
    ap.add_argument("--ours-flush64", default=None, help="csv folder written by run_bench --flush-mb 64")
    ap.add_argument("--published", required=True, help="results/B200/csv of a TileBench checkout")
    ap.add_argument("--out", default=None)
    ap.add_argument("--max-rows", type=int, default=8)
    ap.add_argument("--operators", default=",".join(OPERATORS))
    args = ap.parse_args(argv)
    parts = [operator_section(op, Path(args.ours), Path(args.ours_flush64) if args.ours_flush64 else None, Path(args.published), args.max_rows)
             for op in args.operators.split(",") if op]
    text = "\n\n".join(parts) + "\n"
    if args.out:
        Path(args.out).write_text(text)
    else:
        print(text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
