"""Short text summary of a Nsight Compute capture: the handful of counters a roofline reading needs.

    python -m elfa_b200.utils.ncu_summary prof.ncu-rep            # runs `ncu -i prof.ncu-rep --page raw --csv`
    ncu -i prof.ncu-rep --page raw --csv | python -m elfa_b200.utils.ncu_summary -

One markdown table per captured launch: duration, DRAM bytes and throughput, tensor-pipe and issue utilisation,
warps, registers, grid, and the largest stall reasons per issued instruction. Reading a report needs no GPU.

reference: ``scripts/profile.sh:27-42`` (``ncu --set=full`` / ``ncu --kernel-name``: capture only, nothing reads it).
"""
from __future__ import annotations

import csv
import io
import subprocess
import sys
from typing import Dict, List

WANTED = [
    ("gpu__time_duration.sum", "duration"),
    ("dram__bytes_read.sum", "DRAM read"),
    ("dram__bytes_write.sum", "DRAM written"),
    ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "DRAM throughput, % of peak"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "tensor pipe active, %"),
    ("sm__inst_executed_pipe_xu.avg.pct_of_peak_sustained_active", "MUFU pipe (exp, rsqrt), % of peak"),
    ("sm__throughput.avg.pct_of_peak_sustained_elapsed", "SM throughput, % of peak"),
    ("smsp__issue_active.avg.pct_of_peak_sustained_active", "issue slots used, %"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "warps active, % of slots"),
    ("smsp__inst_executed.sum", "warp instructions"),
    ("launch__registers_per_thread", "registers / thread"),
    ("launch__grid_size", "grid"),
    ("launch__block_size", "block"),
]
STALL_PREFIX = "smsp__average_warps_issue_stalled_"
STALL_SUFFIX = "_per_issue_active.ratio"


def parse(csv_text: str) -> List[Dict[str, str]]:
    """Rows of ``--page raw --csv`` output -> one ``{metric: "value unit"}`` dict per launch (plus ``"Kernel Name"``)."""
    lines = [ln for ln in csv_text.splitlines() if ln.startswith('"')]
    rows = list(csv.reader(io.StringIO("\n".join(lines))))
    if len(rows) < 3:
        return []
    header, units = rows[0], rows[1]
    out = []
    for r in rows[2:]:
        d = {}
        for name, unit, val in zip(header, units, r):
            d[name] = f"{val} {unit}".strip() if name != "Kernel Name" else val
        out.append(d)
    return out


def summarise(launch: Dict[str, str], top_stalls: int = 4) -> str:
    lines = [f"### `{launch.get('Kernel Name', '?')[:100]}`", "", "| metric | value |", "|---|---|"]
    for key, label in WANTED:
        if key in launch:
            lines.append(f"| {label} | {launch[key]} |")
    # load balance over the SMs: a tail shows as a busiest SM far above the average
    cyc = {}
    for key in ("sm__cycles_active.avg", "sm__cycles_active.max", "sm__cycles_active.min", "sm__cycles_elapsed.max"):
        try:
            cyc[key] = float(launch[key].split()[0].replace(",", ""))
        except (KeyError, ValueError, IndexError):
            pass
    if len(cyc) == 4:
        lines.append(f"| SM active cycles avg / max / min (elapsed max) | {cyc['sm__cycles_active.avg'] / 1e3:.0f} K / "
                     f"{cyc['sm__cycles_active.max'] / 1e3:.0f} K / {cyc['sm__cycles_active.min'] / 1e3:.0f} K "
                     f"({cyc['sm__cycles_elapsed.max'] / 1e3:.0f} K) |")
    stalls = []
    for k, v in launch.items():
        if k.startswith(STALL_PREFIX) and k.endswith(STALL_SUFFIX):
            try:
                stalls.append((float(v.split()[0].replace(",", "")), k[len(STALL_PREFIX):-len(STALL_SUFFIX)]))
            except ValueError:
                pass
    stalls = [s for s in sorted(stalls, reverse=True) if s[1] != "selected"][:top_stalls]
    if stalls:
        lines.append("| stall cycles per issued instruction | " + ", ".join(f"{n} {v:.2f}" for v, n in stalls) + " |")
    return "\n".join(lines)


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1:
        print(__doc__)
        return 2
    if argv[0] == "-":
        text = sys.stdin.read()
    else:
        text = subprocess.run(["ncu", "-i", argv[0], "--page", "raw", "--csv"], capture_output=True, text=True, check=True).stdout
    launches = parse(text)
    if not launches:
        print("no launches found in the report", file=sys.stderr)
        return 1
    print("\n\n".join(summarise(x) for x in launches))
    return 0


if __name__ == "__main__":
    sys.exit(main())
