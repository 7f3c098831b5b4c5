"""ncu CSV summariser on a canned export (no GPU, no ncu needed)."""
from tilebench_b200.profiling import ncu_summary

CSV = [
    ["ID", "Kernel Name", "gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum",
     "smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio",
     "smsp__average_warps_issue_stalled_wait_per_issue_active.ratio", "launch__grid_size"],
    ["", "", "us", "Mbyte", "Mbyte", "inst", "inst", ""],
    ["0", "tb200_k_dequant_int8_rowwise_bf16", "145.18", "268.73", "484.07", "3.30", "0.01", "1184"],
]


def test_summary_picks_counters_and_stalls():
    (e,) = ncu_summary.summarise(CSV)
    assert e["kernel"] == "tb200_k_dequant_int8_rowwise_bf16"
    assert e["gpu__time_duration.sum"] == "145.18 us" and e["launch__grid_size"] == "1184"
    assert e["dram traffic (read + write)"] == "268.73 + 484.07 Mbyte"
    assert e["stalls"] == "long_scoreboard 3.30"            # 0.01 is below the reporting threshold
    md = ncu_summary.to_markdown([e])
    assert md.startswith("### tb200_k_dequant_int8_rowwise_bf16") and "| dram__bytes_read.sum | 268.73 Mbyte |" in md


def test_capture_command_follows_the_shared_gpu_rules(capsys):
    from pathlib import Path
    from tilebench_b200.profiling import ncu_one
    cmd = ncu_one.ncu_command("gemm_fp8_blockscaled", {"S": 4096}, Path("out/x.ncu-rep"))
    i = cmd.index("--clock-control")
    assert cmd[i + 1] == "none"                                   # ncu must never lock the clocks
    assert cmd[cmd.index("--profile-from-start") + 1] == "off"
    assert cmd[cmd.index("-k") + 1] == "regex:tb200_k_gemm_fp8" and cmd[cmd.index("-c") + 1] == "2"
    assert cmd[cmd.index("--set") + 1] == "full" and cmd[-6:-4] == ["-m", "tilebench_b200.profiling.harness"]
    few = ncu_one.ncu_command("dequant_int8_channel", {}, Path("o.ncu-rep"), metrics=["gpu__time_duration.sum"])
    assert "--set" not in few and few[few.index("--metrics") + 1] == "gpu__time_duration.sum"
    assert ncu_one.main(["--operator", "matmul_int8", "--case", '{"K": 4096}', "--dry-run"]) == 0
    plain, capture = capsys.readouterr().out.strip().split(" &&\n")
    assert "ncu" not in plain.split()[0] and capture.startswith("ncu ") and capture.endswith(plain)   # plain run first, same command


def test_capture_validation_names_foreign_kernels():
    import pytest
    from tilebench_b200.profiling import ncu_one
    assert ncu_one.validate_capture(CSV, "dequant_int8_channel") == ["tb200_k_dequant_int8_rowwise_bf16"]
    with pytest.raises(RuntimeError, match="not gemm_w4a16's"):
        ncu_one.validate_capture(CSV, "gemm_w4a16")
    with pytest.raises(RuntimeError, match="nothing was captured"):
        ncu_one.validate_capture([["ID", "Kernel Name"], ["", ""]], "gemm_w4a16")


def test_role_cycle_variant_adds_its_reader_and_leaves_the_product_library_alone():
    """The diagnostic build (-DTB200_ROLE_CYCLES) is a separate library with one extra entry point; the product library
    does not export it (its exports are pinned against include/tb200.h in test_abi.py)."""
    import ctypes
    from tilebench_b200.csrc import build
    from tilebench_b200.profiling import role_cycles
    variant = ctypes.CDLL(str(build.build_variant("role_cycles", ["TB200_ROLE_CYCLES=1"], role_cycles.VARIANT_SOURCES)))
    assert hasattr(variant, "tb200_w4a16_role_cycles") and hasattr(variant, "tb200_fp8_role_cycles")
    assert hasattr(variant, "tb200_gemm_w4a16")
    product = ctypes.CDLL(str(build.build_library()))
    assert not hasattr(product, "tb200_w4a16_role_cycles") and not hasattr(product, "tb200_fp8_role_cycles")
