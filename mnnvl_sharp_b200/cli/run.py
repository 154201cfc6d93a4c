"""Launcher: one rank process per selected GPU, on one host or on every host of the plan.

    python -m mnnvl_sharp_b200.cli.run rack.yaml [--rank-count N] [--rank-selection balanced|prefix]
                                       [--emit-dir DIR] [--dry-run] [benchmark flags ...]

The job of the reference project's scripts/run_mnnvl_sharp.sh: build the native parts if
needed, derive the rank plan from the inventory, write the launch artefacts (host list,
ssh config, selected-entries table, rankfile, rank count; reference :184-216), prepare the
remote hosts (:222-244) and start the ranks (:252-263). All flags after the inventory are
passed to the binary unchanged, and --rank-count is appended when the user did not give it
(reference :246-250).

When every selected tray is this machine the ranks are started by the benchmark binary itself.
When the plan names other hosts, no mpirun is involved: the binary is started once per host
(over ssh with the generated config, or directly for this machine's tray) with that host's
tray label, each copy starts its own ranks, and all ranks meet at rank 0's TCP control socket
(the control hostname of rank 0's tray, port MSHARP_HUB_PORT, default 29431). Memory is then
shared with fabric handles, which needs IMEX between the hosts (`cli.preflight` checks it).

Environment (names and defaults of the reference launcher, :56-68): MNNVL_APP_DIR (directory of
this checkout on the remote hosts; default: the local path), MNNVL_SSH_USER, MNNVL_SSH_IDENTITY,
MNNVL_SSH_KNOWN_HOSTS, MNNVL_LOCAL_LABEL (this machine's tray label; default: short host name),
MNNVL_SKIP_REMOTE_BUILD (1: copy the built binary and library instead of building remotely).
Added: MNNVL_SSH_COMMAND / MNNVL_SCP_COMMAND (programs to use instead of ssh / scp),
MSHARP_HUB_PORT. Variables that start with MSHARP_ or MNNVL_DEBUG_ are handed to the remote ranks.
"""
from __future__ import annotations

import os
import shlex
import socket
import subprocess
import sys
import tempfile
import time
from pathlib import Path

from .. import _build
from ..utils import rack as racklib

REPO_ROOT = Path(__file__).resolve().parents[2]
BINARY_REL = Path("mnnvl_sharp_b200") / "_C" / "mnnvl_sharp_allreduce"
LIBRARY_REL = Path("mnnvl_sharp_b200") / "_C" / "libmsharp.so"


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


def local_label() -> str:
    return (os.environ.get("MNNVL_LOCAL_LABEL") or socket.gethostname()).split(".")[0]


def is_local(label: str) -> bool:
    short = label.split(".")[0]
    return short == "localhost" or short == local_label()


def forwarded_environment() -> dict[str, str]:
    return {k: v for k, v in os.environ.items() if k.startswith("MSHARP_") or k.startswith("MNNVL_DEBUG_")}


def host_commands(plan: list[dict], rack_path: str, flags: list[str], ssh_config: Path, app_dir: str,
                  hub: str) -> list[dict]:
    """One entry per host of the plan, in order of first appearance: how its launcher copy is started.
    `argv` is what this machine executes; for a remote host it is the ssh command line."""
    ssh = shlex.split(os.environ.get("MNNVL_SSH_COMMAND", "ssh"))
    seen: list[str] = []
    for target in plan:
        if target["host_label"] not in seen:
            seen.append(target["host_label"])
    commands = []
    for label in seen:
        env = dict(forwarded_environment(), MNNVL_HOST_LABEL=label, MSHARP_HUB_ADDR=hub)
        if is_local(label):
            argv = [str(REPO_ROOT / BINARY_REL), "--rack-config", rack_path] + flags
            commands.append({"label": label, "local": True, "argv": argv, "env": env})
        else:
            assignments = " ".join(f"{k}={shlex.quote(v)}" for k, v in sorted(env.items()))
            remote = (f"cd {shlex.quote(app_dir)} && {assignments} ./{BINARY_REL} --rack-config "
                      f"{shlex.quote(remote_rack_path(rack_path, app_dir))} " + " ".join(shlex.quote(f) for f in flags))
            commands.append({"label": label, "local": False, "argv": ssh + ["-F", str(ssh_config), label, remote], "env": {}})
    return commands


def remote_rack_path(rack_path: str, app_dir: str) -> str:
    """Where the inventory is read on a remote host: the copy that `prepare_remote` puts in the
    application directory (the reference copies it when the remote cannot read the local path, :229-233)."""
    return str(Path(app_dir) / ".launch_rack.yaml")


def prepare_remote(label: str, rack_path: str, ssh_config: Path, app_dir: str, dry_run: bool) -> list[list[str]]:
    """Commands that make a remote host ready: check the directory, copy the inventory, then build
    there or copy the built binary and library. Returns the commands (and runs them unless dry_run)."""
    ssh = shlex.split(os.environ.get("MNNVL_SSH_COMMAND", "ssh")) + ["-F", str(ssh_config)]
    scp = shlex.split(os.environ.get("MNNVL_SCP_COMMAND", "scp")) + ["-F", str(ssh_config)]
    steps = [ssh + [label, f"test -d {shlex.quote(app_dir)}"],
             scp + [rack_path, f"{label}:{remote_rack_path(rack_path, app_dir)}"]]
    if os.environ.get("MNNVL_SKIP_REMOTE_BUILD", "0") == "1":
        steps.append(ssh + [label, f"mkdir -p {shlex.quote(str(Path(app_dir) / BINARY_REL.parent))}"])
        for rel in (BINARY_REL, LIBRARY_REL):
            steps.append(scp + [str(REPO_ROOT / rel), f"{label}:{Path(app_dir) / rel}"])
    else:
        steps.append(ssh + [label, f"cd {shlex.quote(app_dir)} && python -m mnnvl_sharp_b200._build --no-torch"])
    if not dry_run:
        for step in steps:
            print("+ " + " ".join(shlex.quote(s) for s in step), flush=True)
            try:
                rc = subprocess.call(step)
            except FileNotFoundError:
                raise SystemExit(f"error: '{step[0]}' is not installed; it is needed to reach {label} "
                                 "(MNNVL_SSH_COMMAND / MNNVL_SCP_COMMAND name other programs)") from None
            if rc != 0:
                raise SystemExit(f"error: preparing {label} failed (exit {rc}): {' '.join(step)}")
    return steps


def run_hosts(commands: list[dict]) -> int:
    """Start every host's launcher copy, wait for all; when one fails, give the others a few
    seconds to notice through the control plane, then end them. Returns the first failure."""
    procs = []
    for c in commands:
        print(f"launching ranks of {c['label']}: " + " ".join(shlex.quote(a) for a in c["argv"]), flush=True)
        procs.append(subprocess.Popen(c["argv"], env=dict(os.environ, **c["env"])))
    result = 0
    grace_ends = None
    while any(p.poll() is None for p in procs):
        for p in procs:
            rc = p.poll()
            if rc not in (None, 0) and result == 0:
                result = rc
                grace_ends = time.time() + 5.0
        if grace_ends is not None and time.time() > grace_ends:
            for p in procs:
                if p.poll() is None:
                    p.terminate()
            grace_ends = time.time() + 3600.0
        time.sleep(0.05)
    for p in procs:
        if p.returncode != 0 and result == 0:
            result = p.returncode
    return result


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
        if i + 1 >= len(rest):
            raise SystemExit("error: --emit-dir requires a value")
        emit_dir = Path(rest[i + 1])
        del rest[i:i + 2]
    dry_run = "--dry-run" in rest
    if dry_run:
        rest.remove("--dry-run")
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
    flags = list(rest)
    if not count_arg:
        flags += ["--rank-count", str(rank_count)]

    if "--cpu-only" in flags or (len(labels) == 1 and is_local(labels[0])):
        # the host-only oracle needs no GPU and no other host: it always runs here
        exe = _build.build_native()["exe"] if not dry_run else REPO_ROOT / BINARY_REL
        cmd = [str(exe), "--rack-config", str(rack_yaml.resolve())] + flags
        print(f"launching mnnvl_sharp_allreduce rank_count={rank_count} selection={selection} hosts={texts['hosts']}", flush=True)
        env = dict(os.environ)
        if len(labels) == 1 and labels[0].split(".")[0] != "localhost":
            env.setdefault("MNNVL_HOST_LABEL", labels[0])
        if dry_run:
            print(" ".join(shlex.quote(c) for c in cmd))
            return 0
        return subprocess.call(cmd, env=env)

    # several hosts (or one host that is not this machine)
    if emit_dir is None:
        emit_dir = Path(tempfile.mkdtemp(prefix="msharp_launch_"))
        write_artefacts(emit_dir, texts)
    if not dry_run:
        _build.build_native()
    app_dir = os.environ.get("MNNVL_APP_DIR", str(REPO_ROOT))
    hub = f"{plan[0]['hostname']}:{os.environ.get('MSHARP_HUB_PORT', '29431')}"
    ssh_config = emit_dir / "ssh_config"
    print(f"launching mnnvl_sharp_allreduce rank_count={rank_count} selection={selection} hosts={texts['hosts']} hub={hub}",
          flush=True)
    commands = host_commands(plan, str(rack_yaml.resolve()), flags, ssh_config, app_dir, hub)
    for c in commands:
        if not c["local"]:
            for step in prepare_remote(c["label"], str(rack_yaml.resolve()), ssh_config, app_dir, dry_run):
                if dry_run:
                    print("+ " + " ".join(shlex.quote(s) for s in step))
    if dry_run:
        for c in commands:
            print("+ " + " ".join(shlex.quote(a) for a in c["argv"]))
        return 0
    return run_hosts(commands)


if __name__ == "__main__":
    raise SystemExit(main())
