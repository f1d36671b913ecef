"""Condenses an Nsight Compute report into the handful of figures used for roofline notes.

    python benchmarks/ncu_summary.py report.ncu-rep [more.ncu-rep ...]

Reads the report with ``ncu -i <file> --page raw --csv`` (works on a machine without a GPU) and
prints, per captured launch: kernel name, grid / block, registers, duration, DRAM bytes and
throughput, tensor-pipe activity, achieved warps and the dominant stall reasons.
"""
from __future__ import annotations

import csv
import io
import subprocess
import sys

KEYS = [
    ("gpu__time_duration.sum", "duration"),
    ("dram__bytes_read.sum", "dram read"),
    ("dram__bytes_write.sum", "dram write"),
    ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "dram throughput % of peak"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "tensor pipe active % (legacy mma)"),
    ("sm__pipe_tensor_subpipe_umma_cycles_active.avg.pct_of_peak_sustained_active", "tensor pipe active % (tcgen05)"),
    ("sm__inst_executed_pipe_uniform_op_utcmma.sum", "tcgen05.mma instructions"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "achieved occupancy %"),
    ("launch__registers_per_thread", "registers / thread"),
    ("launch__grid_size", "grid"),
    ("launch__block_size", "block"),
    ("launch__shared_mem_per_block_dynamic", "dynamic smem / block"),
    ("sm__throughput.avg.pct_of_peak_sustained_elapsed", "sm throughput %"),
    ("lts__t_sector_hit_rate.pct", "L2 hit rate %"),
]


def summarize(path: str) -> str:
    res = subprocess.run(["ncu", "-i", path, "--page", "raw", "--csv"], capture_output=True, text=True)
    if res.returncode != 0:
        return f"{path}: ncu failed: {res.stderr.strip()[:200]}"
    rows = list(csv.reader(io.StringIO(res.stdout)))
    if len(rows) < 3:
        return f"{path}: empty report"
    hdr, units = rows[0], rows[1]
    out = [f"report: {path}"]
    for r in rows[2:]:
        rec = dict(zip(hdr, r))
        unit = dict(zip(hdr, units))
        out.append(f"kernel: {rec.get('Kernel Name', '?')}")
        for key, label in KEYS:
            if key in rec and rec[key] != "":
                out.append(f"  {label:42s} {rec[key]} {unit.get(key, '')}")
        stalls = []
        for h in hdr:
            if h.startswith("smsp__average_warps_issue_stalled_") and h.endswith("_per_issue_active.ratio"):
                try:
                    stalls.append((float(rec[h]), h[len("smsp__average_warps_issue_stalled_"):-len("_per_issue_active.ratio")]))
                except ValueError:
                    pass
        stalls.sort(reverse=True)
        if stalls:
            out.append("  top stalls (warps per issue):            " + ", ".join(f"{n} {v:.2f}" for v, n in stalls[:5]))
    return "\n".join(out)


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        print(__doc__)
        return 2
    for p in argv:
        print(summarize(p))
        print()
    return 0


if __name__ == "__main__":
    sys.exit(main())
