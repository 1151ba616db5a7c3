"""Turn memory-probe snapshots (``# key=value`` headers written by the trainers) and sweep limit files into
CSV / Markdown tables: peak memory versus T per configuration and the max-T-before-OOM table.  Counterpart of
Tests/mem_scaling_table.py and Tests/bluscriptcp/mem_scaling_table.py."""
from __future__ import annotations

import argparse
import glob
import os
import re
from typing import Dict, List


def parse_header_file(path: str) -> Dict[str, str]:
    out: Dict[str, str] = {"file": os.path.basename(path)}
    for line in open(path, errors="replace"):
        if not line.startswith("#"):
            continue
        for k, v in re.findall(r"([A-Za-z_][A-Za-z0-9_]*)=([^\s]+)", line):
            out.setdefault(k, v)
    return out


def collect(snap_dir: str) -> List[Dict[str, str]]:
    rows = [parse_header_file(p) for p in sorted(glob.glob(os.path.join(snap_dir, "*.txt"))) if not os.path.basename(p).startswith(("log_", "limits_"))]
    return [r for r in rows if "impl" in r]


def table_md(rows: List[Dict[str, str]]) -> str:
    cols = ["impl", "label", "attn_mode", "rotator", "world_size", "T", "CUDA_MEMGETINFO_USED_MB", "reserved_mb", "active_mb", "internal_frag_pct"]
    rows = sorted(rows, key=lambda r: (r.get("label", ""), r.get("attn_mode", ""), int(r.get("world_size", 0)), int(r.get("T", 0))))
    lines = ["| " + " | ".join(cols) + " |", "|" + "---|" * len(cols)]
    for r in rows:
        lines.append("| " + " | ".join(r.get(c, "") for c in cols) + " |")
    return "\n".join(lines)


def limits_md(snap_dir: str) -> str:
    lines = ["| label | mode | rotator | ws | max T ok | first T fail |", "|---|---|---|---|---|---|"]
    for p in sorted(glob.glob(os.path.join(snap_dir, "limits_*.txt"))):
        h = parse_header_file(p)
        lines.append(f"| {h.get('label', '')} | {h.get('mode', '')} | {h.get('rotator', '')} | {h.get('ws', '')} | {h.get('max_T_ok', '')} | {h.get('first_T_fail', '')} |")
    return "\n".join(lines)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("snap_dir")
    ap.add_argument("--csv", default="")
    a = ap.parse_args(argv)
    rows = collect(a.snap_dir)
    print(table_md(rows))
    print()
    print(limits_md(a.snap_dir))
    if a.csv:
        keys = sorted({k for r in rows for k in r})
        with open(a.csv, "w") as f:
            f.write(",".join(keys) + "\n")
            for r in rows:
                f.write(",".join(r.get(k, "") for k in keys) + "\n")


if __name__ == "__main__":
    main()
