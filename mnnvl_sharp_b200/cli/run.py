"""Launcher: one rank process per selected GPU.

    python -m mnnvl_sharp_b200.cli.run rack.yaml [--rank-count N] [--rank-selection balanced|prefix]
                                       [--emit-dir DIR] [benchmark flags ...]

The job of the reference project's scripts/run_mnnvl_sharp.sh: build the native parts if
needed, derive the rank plan from the inventory, write the launch artefacts (host list,
ssh config, selected-entries table, rankfile, rank count; reference :184-216) and start the
ranks. When every selected tray is this machine the ranks are started locally by the
benchmark binary itself (its own control plane replaces mpirun). A plan that spans several
hosts needs a process manager that can start remote processes; the artefacts are then written
to --emit-dir for use with one (exit code 3), because this package's control plane is
single-host. All flags after the inventory are passed to the binary unchanged, and
--rank-count is appended when the user did not give it (reference :246-250).

Environment: MNNVL_SSH_USER, MNNVL_SSH_IDENTITY, MNNVL_SSH_KNOWN_HOSTS (ssh config contents),
MNNVL_LOCAL_LABEL (this machine's tray label; default: short host name).
"""
from __future__ import annotations

import os
import socket
import subprocess
import sys
import tempfile
from pathlib import Path

from .. import _build
from ..utils import rack as racklib


def scan(args: list[str]) -> tuple[str | None, str]:
    """Find --rank-count / --rank-selection among the pass-through flags without consuming them."""
    count, selection = None, "balanced"
    i = 0
    while i < len(args):
        if args[i] in ("--rank-count", "--rank-selection"):
            if i + 1 >= len(args):
                raise SystemExit(f"error: {args[i]} requires a value")
            if args[i] == "--rank-count":
                count = args[i + 1]
            else:
                selection = args[i + 1]
            i += 2
        else:
            i += 1
    if selection not in ("balanced", "prefix"):
        raise SystemExit("error: --rank-selection must be balanced or prefix")
    return count, selection


def write_artefacts(directory: Path, texts: dict) -> None:
    directory.mkdir(parents=True, exist_ok=True)
    (directory / "hosts.txt").write_text(texts["hosts"])
    (directory / "ssh_config").write_text(texts["ssh_config"])
    (directory / "selected_entries.tsv").write_text(texts["entries"])
    (directory / "rankfile").write_text(texts["rankfile"])
    (directory / "rank_count.txt").write_text(str(texts["rank_count"]))


def is_local(label: str) -> bool:
    local = os.environ.get("MNNVL_LOCAL_LABEL") or socket.gethostname()
    short = label.split(".")[0]
    return short == "localhost" or short == local.split(".")[0]


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0 if argv else 1
    rack_yaml = Path(argv[0])
    rest = argv[1:]
    emit_dir = None
    if "--emit-dir" in rest:
        i = rest.index("--emit-dir")
        emit_dir = Path(rest[i + 1])
        del rest[i:i + 2]
    if not rack_yaml.is_file():
        raise SystemExit(f"error: cannot read {rack_yaml}")
    count_arg, selection = scan(rest)
    text = rack_yaml.read_text()
    total = racklib.parse_rack(text)["available_rank_count"]
    rank_count = int(count_arg) if count_arg else total
    if not 1 <= rank_count <= total:
        raise SystemExit(f"error: rank count {rank_count} must be between 1 and {total}")
    texts = racklib.launch_texts(text, rank_count, selection, os.environ.get("MNNVL_SSH_USER", ""),
                                 os.environ.get("MNNVL_SSH_IDENTITY", ""), os.environ.get("MNNVL_SSH_KNOWN_HOSTS", ""))
    plan = racklib.rank_plan(text, rank_count, selection)
    labels = sorted({t["host_label"] for t in plan})
    if emit_dir is not None:
        write_artefacts(emit_dir, texts)
        print(f"wrote launch artefacts to {emit_dir}")
    if not all(is_local(label) for label in labels):
        if emit_dir is None:
            emit_dir = Path(tempfile.mkdtemp(prefix="msharp_launch_"))
            write_artefacts(emit_dir, texts)
        print(f"error: the plan spans hosts {texts['hosts']}; this package starts ranks on one host only. "
              f"Launch artefacts for an external process manager are in {emit_dir}", file=sys.stderr)
        return 3
    exe = _build.build_native()["exe"]
    cmd = [str(exe), "--rack-config", str(rack_yaml.resolve())]
    if not count_arg:
        cmd += ["--rank-count", str(rank_count)]
    cmd += rest
    print(f"launching mnnvl_sharp_allreduce rank_count={rank_count} selection={selection} hosts={texts['hosts']}", flush=True)
    env = dict(os.environ)
    if len(labels) == 1 and labels[0].split(".")[0] != "localhost":
        env.setdefault("MNNVL_HOST_LABEL", labels[0])
    return subprocess.call(cmd, env=env)


if __name__ == "__main__":
    raise SystemExit(main())
