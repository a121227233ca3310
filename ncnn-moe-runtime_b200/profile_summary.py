"""Turns an ncu report into the short text summary kept under profiles/ and records the DRAM traffic per
launch that bench.py reports next to the algorithmic bytes.

    ncu -i <file>.ncu-rep --page raw --csv > raw.csv        # works without a GPU
    python ncnn-moe-runtime_b200/profile_summary.py raw.csv --workload headline --algorithmic-bytes 205914112 \\
        --command "<the full profiling command>" --out profiles/sample_rows_kernel_f32_headline.md

Nothing here runs on a GPU; profiles/ holds only the text this writes.
"""
from __future__ import annotations

import argparse
import csv
import json
from pathlib import Path

METRICS = [
    ("gpu__time_duration.sum", "duration"),
    ("dram__bytes_read.sum", "DRAM bytes read"),
    ("dram__bytes_write.sum", "DRAM bytes written"),
    ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "DRAM throughput, % of peak"),
    ("launch__grid_size", "grid size"),
    ("launch__block_size", "block size"),
    ("launch__registers_per_thread", "registers per thread"),
    ("launch__shared_mem_per_block_dynamic", "dynamic shared memory per block"),
    ("launch__waves_per_multiprocessor", "waves per SM"),
    ("launch__occupancy_limit_shared_mem", "occupancy limit, shared memory (blocks)"),
    ("launch__occupancy_limit_registers", "occupancy limit, registers (blocks)"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "warps active, % of peak"),
    ("smsp__inst_executed.sum", "warp instructions executed"),
    ("smsp__issue_active.avg.pct_of_peak_sustained_active", "issue slots used, %"),
    ("l1tex__data_bank_conflicts_pipe_lsu_mem_shared.sum", "shared-memory bank conflicts"),
    ("smsp__inst_executed_op_shared_ld.sum", "shared loads (warp instructions)"),
    ("sass__inst_executed_local_loads", "local-memory loads (warp instructions)"),
    ("sass__inst_executed_local_stores", "local-memory stores (warp instructions)"),
    ("lts__t_sector_hit_rate.pct", "L2 hit rate, %"),
]
STALL_PREFIX = "smsp__average_warps_issue_stalled_"
STALL_SUFFIX = "_per_issue_active.ratio"


def to_bytes(value: str, unit: str) -> float:
    scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}.get(unit, 1.0)
    return float(value.replace(",", "")) * scale


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("raw_csv")
    parser.add_argument("--workload", required=True, help="key of this capture in profiles/traffic.json")
    parser.add_argument("--algorithmic-bytes", type=float, required=True)
    parser.add_argument("--command", required=True)
    parser.add_argument("--title", default=None)
    parser.add_argument("--scale", type=float, default=1.0, help="units of a full launch per unit of the captured launch (small captures)")
    parser.add_argument("--out", required=True)
    args = parser.parse_args()

    rows = list(csv.reader(open(args.raw_csv)))
    header, units, launches = rows[0], rows[1], rows[2:]
    column = {name: index for index, name in enumerate(header)}
    kernel = launches[0][column["Kernel Name"]] if "Kernel Name" in column else "kernel"
    lines = [f"# {args.title or kernel} — {args.workload}", "", "Command (ncu only after the same command line had exited 0 without it):", "", f"    {args.command}", "",
             f"Captured launches: {len(launches)}.  Read here with `ncu -i <report> --page raw --csv`.", "", "| metric | " + " | ".join(f"launch {i + 1}" for i in range(len(launches))) + " |",
             "|---|" + "---:|" * len(launches)]
    for name, label in METRICS:
        if name in column:
            unit = units[column[name]]
            lines.append(f"| {label}{' (' + unit + ')' if unit else ''} | " + " | ".join(launch[column[name]] for launch in launches) + " |")
    stalls = []
    for name, index in column.items():
        if name.startswith(STALL_PREFIX) and name.endswith(STALL_SUFFIX):
            value = sum(float(launch[index]) for launch in launches) / len(launches)
            stalls.append((value, name[len(STALL_PREFIX):-len(STALL_SUFFIX)]))
    stalls.sort(reverse=True)
    lines += ["", "Warp stall reasons (cycles stalled per issued instruction, mean over the launches): " +
              ", ".join(f"{name} {value:.2f}" for value, name in stalls if value >= 0.005) + "."]
    traffic = None
    if "dram__bytes_read.sum" in column and "dram__bytes_write.sum" in column:
        per_launch = [to_bytes(launch[column["dram__bytes_read.sum"]], units[column["dram__bytes_read.sum"]]) +
                      to_bytes(launch[column["dram__bytes_write.sum"]], units[column["dram__bytes_write.sum"]]) for launch in launches]
        traffic = sum(per_launch) / len(per_launch) * args.scale
        lines += ["", f"DRAM traffic per launch: {traffic / 1e6:.2f} MB" + (f" (captured launch scaled by {args.scale:g})" if args.scale != 1.0 else "") +
                  f" against {args.algorithmic_bytes / 1e6:.2f} MB of algorithmic bytes (one logits read per row): {traffic / args.algorithmic_bytes:.3f}x."]
    out = Path(args.out)
    out.write_text("\n".join(lines) + "\n")
    if traffic is not None:
        table_path = out.parent / "traffic.json"
        table = json.loads(table_path.read_text()) if table_path.exists() else {}
        table[args.workload] = {"dram_bytes_per_launch": int(round(traffic)), "algorithmic_bytes_per_launch": int(args.algorithmic_bytes),
                                "source": out.name}
        table_path.write_text(json.dumps(table, indent=1, sort_keys=True) + "\n")
    print(out)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
