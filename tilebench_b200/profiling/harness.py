"""One operator call inside a profiler range, for `ncu --profile-from-start off`.

Shape of the reference's NCU harness (scripts/profiling/ncu_generic_harness.py:73-84): seeded inputs,
three warm-up calls, one 2x-L2 flush, then exactly one `impl_cuda.run` between
torch.cuda.profiler.start() and stop().

    python -m tilebench_b200.profiling.harness --operator gemm_fp8_blockscaled --case '{"S": 4096}'
    ncu --set full --clock-control none --profile-from-start off -k regex:tb200_k_ -c 3 -o out \
        python -m tilebench_b200.profiling.harness --operator ... --case ...
"""
from __future__ import annotations

import argparse
import importlib
import json

import torch
import yaml

from tilebench_b200.core.dtypes import resolve_dtype
from tilebench_b200.core.timer import flush_l2_cache
from tilebench_b200.data.tensors import get_generator
from tilebench_b200.paths import operator_config


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--operator", required=True)
    ap.add_argument("--case", default="{}", help="JSON overrides of the operator's case_defaults")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seed", type=int, default=1)
    args = ap.parse_args()

    cfg = yaml.safe_load(open(operator_config(args.operator)))
    case = dict(cfg.get("case_defaults", {}))
    for k, v in cfg.get("case_grid", {}).items():
        case.setdefault(k, v[0] if isinstance(v, list) else None)
    case.update(json.loads(args.case))
    dtype = resolve_dtype(case.pop("dtype", "fp32"))
    impl = importlib.import_module(f"tilebench_b200.benchmarks.operators.{args.operator}.impl_cuda")
    inputs = get_generator(args.operator)(**case, dtype=dtype, device="cpu", seed=args.seed)
    inputs = tuple(x.cuda() if isinstance(x, torch.Tensor) else x for x in inputs)
    for _ in range(args.warmup):
        impl.run(*inputs)
    flush_l2_cache()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    out = impl.run(*inputs)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    outs = out if isinstance(out, (tuple, list)) else (out,)
    print(json.dumps({"operator": args.operator, "case": case, "out_shapes": [list(o.shape) for o in outs]}))


if __name__ == "__main__":
    main()
