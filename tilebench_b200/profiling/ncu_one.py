"""One Nsight Compute capture of one operator case, start to finish.

Shape of the reference's capture driver (scripts/profiling/ncu_one.py:60-100): build the `ncu` command
around the profiling harness, run it, check that what was captured is the operator's own kernel, and write
a short summary.  Differences that matter on shared GPUs:

  * the harness command is first run WITHOUT ncu and must exit 0 — a program that faults is never profiled;
  * `--clock-control none` always (ncu must not lock the clocks of a GPU other jobs will inherit);
  * kernels are selected by name (`-k regex:`), a handful of launches (`-c`), inside the harness's
    cudaProfilerStart/Stop range (`--profile-from-start off`), so the capture ends by itself.

    python -m tilebench_b200.profiling.ncu_one --operator gemm_fp8_blockscaled --case '{"S": 4096}' \\
        --out-dir profiles_out [--set full | --metrics a,b,c] [--dry-run]
"""
from __future__ import annotations

import argparse
import csv
import json
import re
import shlex
import subprocess
import sys
from pathlib import Path

from tilebench_b200.profiling import ncu_summary

#: Every kernel of the library starts with this prefix; an operator's capture may narrow it further.
KERNEL_PREFIX = "tb200_k_"
KERNEL_REGEX = {
    "dequant_int4_group": "tb200_k_dequant_int4",
    "dequant_int8_channel": "tb200_k_dequant_int8",
    "dequantize_rowwise": "tb200_k_dequant_int8",
    "weight_dequant": "tb200_k_weight_dequant",
    "quantize_fp8_block": "tb200_k_quant_fp8",
    "quantize_int4_group": "tb200_k_quant_int4",
    "gemm_w4a16": "tb200_k_(gemm|gemv)_w4a16",
    "gemm_fp8_blockscaled": "tb200_k_gemm_fp8",
    "matmul_int8": "tb200_k_gemm_i8",
    "matmul_fp32_fp16_fp8": "tb200_k_gemm_(f16|bf16|tf32|f8)_",
}


def kernel_regex(operator: str) -> str:
    return KERNEL_REGEX.get(operator, KERNEL_PREFIX)


def harness_command(operator: str, case: dict, python: str = sys.executable) -> list[str]:
    return [python, "-m", "tilebench_b200.profiling.harness", "--operator", operator, "--case", json.dumps(case, separators=(",", ":"))]


def ncu_command(operator: str, case: dict, report: Path, *, ncu: str = "ncu", launches: int = 2, section_set: str | None = "full",
                metrics: list[str] | None = None, python: str = sys.executable) -> list[str]:
    """The capture command; `metrics` (a short list, one pass or few) replaces `--set`."""
    cmd = [ncu]
    if metrics:
        cmd += ["--metrics", ",".join(metrics)]
    else:
        cmd += ["--set", section_set or "full"]
    cmd += ["--clock-control", "none", "--profile-from-start", "off", "-k", f"regex:{kernel_regex(operator)}",
            "-c", str(int(launches)), "-f", "-o", str(report.with_suffix(""))]
    return cmd + harness_command(operator, case, python)


def validate_capture(rows: list[list[str]], operator: str) -> list[str]:
    """Kernel names captured; raises if none, or if one is not the operator's own."""
    start = next((i for i, r in enumerate(rows) if "Kernel Name" in r), None)
    if start is None:
        raise RuntimeError("the report holds no kernel rows: nothing was captured")
    col = rows[start].index("Kernel Name")
    names = [r[col] for r in rows[start + 2:] if len(r) > col and r[col]]
    if not names:
        raise RuntimeError("the report holds no kernel rows: nothing was captured")
    rgx = re.compile(kernel_regex(operator))
    foreign = [n for n in names if not rgx.search(n)]
    if foreign:
        raise RuntimeError(f"captured kernels that are not {operator}'s: {foreign}")
    return names


def read_report(report: Path, ncu: str = "ncu") -> list[list[str]]:
    text = subprocess.run([ncu, "-i", str(report), "--page", "raw", "--csv"], capture_output=True, text=True).stdout
    return [r for r in csv.reader(text.splitlines()) if r]


def write_summary(path: Path, operator: str, case: dict, commands: list[list[str]], rows: list[list[str]]) -> None:
    start = next(i for i, r in enumerate(rows) if "Kernel Name" in r)
    body = ncu_summary.to_markdown(ncu_summary.summarise(rows[start:]))
    cmds = " &&\n    ".join(shlex.join(c) for c in commands)
    path.write_text(f"# {operator} {json.dumps(case)}\n\nCommand (plain run first, then under ncu; 1 GPU):\n\n    {cmds}\n\n{body}\n")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--operator", required=True)
    ap.add_argument("--case", default="{}")
    ap.add_argument("--out-dir", default="ncu_out")
    ap.add_argument("--set", dest="section_set", default="full")
    ap.add_argument("--metrics", default="", help="comma-separated metric names instead of --set")
    ap.add_argument("--launches", type=int, default=2)
    ap.add_argument("--ncu", default="ncu")
    ap.add_argument("--dry-run", action="store_true", help="print the two commands and stop")
    args = ap.parse_args(argv)
    case = json.loads(args.case)
    out_dir = Path(args.out_dir)
    tag = args.operator + "".join(f"_{k}{v}" for k, v in sorted(case.items()))
    report = out_dir / f"{tag}.ncu-rep"
    plain = harness_command(args.operator, case)
    capture = ncu_command(args.operator, case, report, ncu=args.ncu, launches=args.launches, section_set=args.section_set,
                          metrics=[m for m in args.metrics.split(",") if m])
    if args.dry_run:
        print(shlex.join(plain) + " &&\n" + shlex.join(capture))
        return 0
    out_dir.mkdir(parents=True, exist_ok=True)
    first = subprocess.run(plain)
    if first.returncode != 0:
        print(f"not profiled: the plain run exited {first.returncode}", file=sys.stderr)
        return 86
    if subprocess.run(capture).returncode != 0:
        print("ncu failed", file=sys.stderr)
        return 1
    rows = read_report(report, args.ncu)
    names = validate_capture(rows, args.operator)
    write_summary(out_dir / f"{tag}.md", args.operator, case, [plain, capture], rows)
    print(f"captured {len(names)} launch(es): {sorted(set(names))} -> {out_dir / (tag + '.md')}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
