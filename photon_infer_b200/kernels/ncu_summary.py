"""Short text summaries of Nsight Compute output, as kept under ``profiles/``.

    python -m photon_infer_b200.kernels.ncu_summary launches launches.csv [--per N]
        ``launches.csv``: what ``ncu --metrics gpu__time_duration.sum --csv --log-file launches.csv <command>`` wrote.
        Prints the summed device time and, per kernel name, total, count and mean (divided by ``--per`` units,
        e.g. the number of steps that were captured).

    python -m photon_infer_b200.kernels.ncu_summary report prof.ncu-rep
        ``prof.ncu-rep``: what ``ncu --set full -o prof <command>`` wrote.  Calls ``ncu -i prof.ncu-rep --page raw
        --csv`` and prints, per captured launch, the figures the summaries quote (duration, registers, occupancy
        limits, DRAM and L2 traffic, tensor pipe, issue slots, stall reasons).
"""
from __future__ import annotations

import argparse
import collections
import csv
import subprocess
import sys

REPORT_METRICS = [
    ("gpu__time_duration.sum", "duration"),
    ("sm__cycles_elapsed.avg.per_second", "SM clock during the capture"),
    ("launch__grid_size", "grid size (blocks)"),
    ("launch__block_size", "block size (threads)"),
    ("launch__registers_per_thread", "registers per thread"),
    ("launch__occupancy_limit_registers", "blocks per SM allowed by registers"),
    ("launch__occupancy_limit_shared_mem", "blocks per SM allowed by shared memory"),
    ("launch__waves_per_multiprocessor", "waves per SM"),
    ("dram__bytes_read.sum", "DRAM bytes read"),
    ("dram__bytes_write.sum", "DRAM bytes written"),
    ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "DRAM throughput, % of peak"),
    ("lts__t_bytes.sum", "L2 bytes"),
    ("lts__throughput.avg.pct_of_peak_sustained_elapsed", "L2 throughput, % of peak"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "tensor pipe active, % of active cycles"),
    ("sm__inst_executed_pipe_xu.avg.pct_of_peak_sustained_active", "XU pipe (exp2, rcp), % of active cycles"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "warps active, % of peak"),
    ("smsp__issue_active.avg.pct_of_peak_sustained_active", "issue slots used, %"),
    ("smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio", "stall: long scoreboard per issue"),
    ("smsp__average_warps_issue_stalled_short_scoreboard_per_issue_active.ratio", "stall: short scoreboard per issue"),
    ("smsp__average_warps_issue_stalled_wait_per_issue_active.ratio", "stall: fixed-latency wait per issue"),
    ("smsp__average_warps_issue_stalled_barrier_per_issue_active.ratio", "stall: barrier per issue"),
    ("smsp__average_warps_issue_stalled_math_pipe_throttle_per_issue_active.ratio", "stall: math pipe throttle per issue"),
    ("smsp__average_warps_issue_stalled_lg_throttle_per_issue_active.ratio", "stall: load/store queue per issue"),
]


def launches(path: str, per: float) -> None:
    with open(path) as f:
        lines = [line for line in f if not line.startswith("==")]
    total = 0.0
    by_name = collections.OrderedDict()
    for row in csv.DictReader(lines):
        value = float(row["Metric Value"].replace(",", ""))
        if row["Metric Unit"] == "ns":
            value /= 1000.0
        name = row["Kernel Name"][:72]
        entry = by_name.setdefault(name, [0.0, 0])
        entry[0] += value
        entry[1] += 1
        total += value
    print(f"total {total / per:.1f} us per unit ({sum(c for _, c in by_name.values()) / per:.1f} launches)")
    for name, (value, count) in sorted(by_name.items(), key=lambda item: -item[1][0]):
        print(f"{value / per:9.1f} us {count / per:6.1f} x {value / count:8.2f} us  {name}")


def report(path: str) -> None:
    out = subprocess.run(["ncu", "-i", path, "--page", "raw", "--csv"], capture_output=True, text=True, check=True).stdout
    rows = list(csv.reader(out.splitlines()))
    header, units = rows[0], rows[1]
    index = {h: i for i, h in enumerate(header)}
    for row in rows[2:]:
        grid = row[index["launch__grid_size"]] if "launch__grid_size" in index else "?"
        block = row[index["launch__block_size"]] if "launch__block_size" in index else "?"
        print(f"{row[index['Kernel Name']][:60]}  (grid {grid} x {block} threads)")
        for metric, label in REPORT_METRICS:
            if metric in index and metric not in ("launch__grid_size", "launch__block_size"):
                print(f"    {label:55s} {row[index[metric]][:24]:>14s} {units[index[metric]]}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    a = sub.add_parser("launches")
    a.add_argument("csv")
    a.add_argument("--per", type=float, default=1.0)
    b = sub.add_parser("report")
    b.add_argument("rep")
    args = ap.parse_args(argv)
    if args.what == "launches":
        launches(args.csv, args.per)
    else:
        report(args.rep)
    return 0


if __name__ == "__main__":
    sys.exit(main())
