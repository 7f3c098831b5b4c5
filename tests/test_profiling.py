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
