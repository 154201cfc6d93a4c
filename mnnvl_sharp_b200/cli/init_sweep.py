"""Peer-access initialisation latency versus rank count.

    python -m mnnvl_sharp_b200.cli.init_sweep rack.yaml [--rank-counts 1,2,4,8] [--repeats 3]
                                              [--sharp-backend legacy|tma_async] [--out-dir DIR]

For every (rank count, repeat) the launcher runs the benchmark with `--init-only --json`, the
log goes to `rank_<N>_repeat_<r>.log`, and the JSON summary (the last stdout line that starts
with `{` and ends with `}`) becomes one row of `init_latency.csv` with the reference project's
schema (scripts/run_init_sweep.py:143-152). Differences from that script: each row is appended
as soon as it exists and points already in the CSV are skipped, so a sweep that was interrupted
(or whose later points failed) resumes instead of starting over; the default rank counts are
1, 2, 4, 8 for a single 8-GPU box (counts above the inventory are dropped and the inventory
total is added, as in the reference :110-118).
"""
from __future__ import annotations

import argparse
import csv
import json
import statistics
import subprocess
import sys
from pathlib import Path

from ..utils import rack as racklib

DEFAULT_RANK_COUNTS = [1, 2, 4, 8, 16, 32, 64, 72]
FIELDS = racklib.CSV_HEADER.split(",")


def parse_rank_counts(text: str) -> list[int]:
    out = []
    for token in text.split(","):
        token = token.strip()
        if not token:
            continue
        value = int(token)
        if value <= 0:
            raise ValueError("rank counts must be positive")
        out.append(value)
    return out


def select_rank_counts(requested: list[int], total: int) -> list[int]:
    counts = [c for c in requested if c <= total]
    if total >= 4 and total not in counts:
        counts.append(total)
    return sorted(set(counts))


def extract_json_line(stdout: str) -> dict:
    for line in reversed(stdout.splitlines()):
        line = line.strip()
        if line.startswith("{") and line.endswith("}"):
            return json.loads(line)
    raise RuntimeError("no JSON summary line in the benchmark output")


def existing_rows(csv_path: Path) -> set[tuple[int, int, str]]:
    if not csv_path.exists():
        return set()
    with csv_path.open(newline="") as f:
        return {(int(r["rank_count"]), int(r["repeat"]), r["sharp_backend"]) for r in csv.DictReader(f)}


def run_one(rack_yaml: Path, rank_count: int, selection: str, backend: str, log_path: Path, launcher=None) -> dict:
    cmd = launcher or [sys.executable, "-m", "mnnvl_sharp_b200.cli.run"]
    cmd = list(cmd) + [str(rack_yaml), "--rank-count", str(rank_count), "--rank-selection", selection,
                       "--sharp-backend", backend, "--init-only", "--json", "--bytes", "1073741824"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log_path.write_text(f"$ {' '.join(cmd)}\n--- stdout ---\n{proc.stdout}\n--- stderr ---\n{proc.stderr}\n")
    if proc.returncode != 0:
        raise RuntimeError(f"rank_count={rank_count} failed with exit code {proc.returncode}; see {log_path}")
    return extract_json_line(proc.stdout)


def main(argv: list[str] | None = None, launcher=None) -> int:
    p = argparse.ArgumentParser(description="Sweep peer-access initialisation latency.")
    p.add_argument("rack_yaml", type=Path)
    p.add_argument("--rank-counts", default=",".join(str(x) for x in DEFAULT_RANK_COUNTS))
    p.add_argument("--rank-selection", choices=["balanced", "prefix"], default="balanced")
    p.add_argument("--sharp-backend", choices=["legacy", "tma_async"], default="legacy")
    p.add_argument("--repeats", type=int, default=3)
    p.add_argument("--out-dir", type=Path, default=Path("results/init_sweep"))
    args = p.parse_args(argv)
    if args.repeats <= 0:
        raise SystemExit("--repeats must be positive")
    total = racklib.available_rank_count(args.rack_yaml)
    counts = select_rank_counts(parse_rank_counts(args.rank_counts), total)
    if not counts:
        raise SystemExit(f"no requested rank counts fit rack.yaml total device count {total}")
    args.out_dir.mkdir(parents=True, exist_ok=True)
    csv_path = args.out_dir / "init_latency.csv"
    done = existing_rows(csv_path)
    new_file = not csv_path.exists()
    failures = 0
    with csv_path.open("a", newline="") as f:
        writer = csv.DictWriter(f, fieldnames=FIELDS)
        if new_file:
            writer.writeheader()
            f.flush()
        for count in counts:
            for repeat in range(args.repeats):
                if (count, repeat, args.sharp_backend) in done:
                    continue
                log_path = args.out_dir / f"rank_{count}_repeat_{repeat}.log"
                try:
                    summary = run_one(args.rack_yaml.resolve(), count, args.rank_selection, args.sharp_backend, log_path,
                                      launcher)
                except Exception as ex:  # noqa: BLE001
                    print(f"warning: {ex}", file=sys.stderr)
                    failures += 1
                    continue
                writer.writerow({"rank_count": count, "repeat": repeat, "sharp_backend": args.sharp_backend,
                                 **{k: summary[k] for k in FIELDS[3:]}})
                f.flush()
    from . import plot_init_latency

    plot_path = plot_init_latency.plot(csv_path, args.out_dir / "init_latency.png")
    grouped: dict[int, list[float]] = {}
    with csv_path.open(newline="") as f:
        for row in csv.DictReader(f):
            grouped.setdefault(int(row["rank_count"]), []).append(float(row["peer_init_ms"]))
    for count in sorted(grouped):
        print(f"rank_count={count} peer_init_ms_median={statistics.median(grouped[count]):.3f}")
    print(f"wrote {csv_path}")
    if plot_path is not None:
        print(f"wrote {plot_path}")
    return 1 if failures else 0


if __name__ == "__main__":
    raise SystemExit(main())
