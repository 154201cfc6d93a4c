"""Environment preflight: what a node needs before the all-reduce benchmark can run on it.

    python -m mnnvl_sharp_b200.cli.preflight                # this machine
    python -m mnnvl_sharp_b200.cli.preflight rack.yaml      # every tray of the inventory over SSH

Local mode reports the host name, GPU inventory and topology, the IMEX daemon and its channel
device (needed only for fabric handles across nodes; a single HGX box works with POSIX file
descriptors), the IMEX node list, and the CUDA capabilities this package relies on (virtual
memory management, shareable handle types, multicast). Rack mode runs the remote part of the
same checks per tray, warns when a tray's host name differs from its label, and compares the
IMEX node lists of all trays. Checks mirror the reference project's scripts/preflight_imex.sh
(local :33-69, rack :140-205). A missing tool is reported as a warning, never as a crash; the
exit code is 1 if a required check failed.
"""
from __future__ import annotations

import argparse
import difflib
import os
import shutil
import socket
import subprocess
import sys

from ..utils import rack as racklib

SSH_ENV = {
    "config": ("MNNVL_SSH_CONFIG", "/home/ubuntu/.ssh/config"),
    "identity": ("MNNVL_SSH_IDENTITY", "/home/ubuntu/.ssh/id_rsa"),
    "known_hosts": ("MNNVL_SSH_KNOWN_HOSTS", "/home/ubuntu/.ssh/known_hosts"),
    "user": ("MNNVL_SSH_USER", "ubuntu"),
}
IMEX_CHANNEL = "/dev/nvidia-caps-imex-channels/channel0"
IMEX_NODES = "/etc/nvidia-imex/nodes_config.cfg"

PARTITION_NOTE = """== nvlink partition reminder ==
Compute-node checks cannot prove NVSwitch partition membership. On an NVL72 rack ask the fabric
operator for `nv show sdn partition` (one healthy default partition holding all selected trays);
on a single HGX baseboard all eight GPUs share one NVSwitch domain."""


def ssh_setting(name: str) -> str:
    var, default = SSH_ENV[name]
    return os.environ.get(var, default)


def run(cmd: list[str], timeout: int = 30) -> tuple[int, str]:
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
        return proc.returncode, (proc.stdout + proc.stderr).strip()
    except FileNotFoundError:
        return 127, f"{cmd[0]}: not installed"
    except subprocess.TimeoutExpired:
        return 124, f"{' '.join(cmd)}: timed out"


def normalize_nodes_config(text: str) -> list[str]:
    """Comments and blank lines removed, inner blanks collapsed, sorted."""
    lines = []
    for line in text.splitlines():
        line = " ".join(line.split("#", 1)[0].split())
        if line:
            lines.append(line)
    return sorted(lines)


def section(title: str) -> None:
    print(f"== {title} ==", flush=True)


def cuda_capabilities() -> tuple[bool, list[str]]:
    """(ok, report lines) from the driver attributes of every visible GPU."""
    try:
        import ctypes

        cuda = ctypes.CDLL("libcuda.so.1")
    except OSError:
        return False, ["warning: libcuda.so.1 is not available; cannot query CUDA capabilities"]
    if cuda.cuInit(0) != 0:
        return False, ["error: cuInit failed"]
    count = ctypes.c_int()
    cuda.cuDeviceGetCount(ctypes.byref(count))
    attrs = {"vmm": 102, "posix_fd": 103, "fabric": 128, "multicast": 132, "host_numa_id": 134}
    lines, ok = [], count.value > 0
    for ordinal in range(count.value):
        dev = ctypes.c_int()
        cuda.cuDeviceGet(ctypes.byref(dev), ordinal)
        values = {}
        for name, attr in attrs.items():
            v = ctypes.c_int(-1)
            cuda.cuDeviceGetAttribute(ctypes.byref(v), attr, dev)
            values[name] = v.value
        lines.append(f"gpu {ordinal}: " + " ".join(f"{k}={v}" for k, v in values.items()))
        if not values["vmm"] or not (values["posix_fd"] or values["fabric"]):
            ok = False
        if count.value > 1 and not values["multicast"]:
            lines.append(f"warning: gpu {ordinal} reports no multicast support; the in-switch backends cannot run")
    return ok, lines


def local_checks() -> int:
    failures = 0
    section("local host")
    print(socket.gethostname())
    section("gpu inventory")
    rc, out = run(["nvidia-smi", "-L"])
    print(out)
    failures += rc != 0
    section("gpu topology")
    print(run(["nvidia-smi", "topo", "-m"])[1])
    section("cuda capabilities")
    ok, lines = cuda_capabilities()
    print("\n".join(lines))
    failures += not ok
    section("nvidia-imex service")
    rc, out = run(["systemctl", "is-active", "nvidia-imex"])
    if rc == 0:
        print(out)
    else:
        rc2, out2 = run(["pgrep", "-a", "nvidia-imex"])
        print(out2 if rc2 == 0 else "warning: nvidia-imex service state not visible in this container "
                                    "(needed for fabric handles across nodes only)")
    section("imex channels")
    if os.path.exists(IMEX_CHANNEL):
        print(run(["ls", "-la", os.path.dirname(IMEX_CHANNEL)])[1])
    else:
        print(f"warning: {IMEX_CHANNEL} is absent: fabric handles are unavailable, POSIX file descriptors are used")
    section("nodes_config.cfg")
    if os.path.exists(IMEX_NODES):
        print(open(IMEX_NODES).read().strip())
    else:
        print(f"warning: {IMEX_NODES} is absent")
    section("nvidia-imex-ctl -N")
    if shutil.which("nvidia-imex-ctl"):
        print(run(["nvidia-imex-ctl", "-N"])[1])
    else:
        print("warning: nvidia-imex-ctl is not installed in this container")
    print(PARTITION_NOTE)
    return 1 if failures else 0


def remote(port: int, host: str, command: str) -> tuple[int, str]:
    cmd = ["ssh", "-n", "-F", ssh_setting("config"), "-i", ssh_setting("identity"), "-o", "IdentitiesOnly=yes",
           "-o", "PasswordAuthentication=no", "-o", f"UserKnownHostsFile={ssh_setting('known_hosts')}",
           "-o", "StrictHostKeyChecking=accept-new", "-o", "BatchMode=yes", "-p", str(port),
           f"{ssh_setting('user')}@{host}", command]
    return run(cmd, timeout=60)


def rack_checks(path: str, runner=remote) -> int:
    inventory = racklib.load_rack(path)
    entries = inventory["entries"]
    if not 1 <= len(entries) <= 18:
        print("error: rack mode expects 1 to 18 rack entries", file=sys.stderr)
        return 1
    failures = 0
    first_nodes: list[str] | None = None
    for entry in entries:
        label, host, port = entry["host_label"], entry["hostname"], entry["port"]
        section(f"rack entry {label}")
        print(f"control_host: {host}\nssh_port: {port}\ndevices: {','.join(str(d) for d in entry['devices'])}")
        rc, name = runner(port, host, "hostname")
        print(f"hostname: {name}")
        if rc != 0:
            print(f"error: cannot reach {label} over ssh", file=sys.stderr)
            failures += 1
            continue
        if name.split(".")[0] != label.split(".")[0]:
            print("warning: hostname does not match rack key; launch with MNNVL_HOST_LABEL if intentional", file=sys.stderr)
        print("-- nvidia-imex service")
        print(runner(port, host, "systemctl is-active nvidia-imex 2>/dev/null || pgrep -a nvidia-imex || "
                                 "echo 'warning: nvidia-imex service state not visible in this container'")[1])
        print("-- imex channels")
        rc, out = runner(port, host, f"ls -la {os.path.dirname(IMEX_CHANNEL)} && test -e {IMEX_CHANNEL}")
        print(out if rc == 0 else f"warning: {IMEX_CHANNEL} is absent on {label}")
        print("-- gpu inventory")
        rc, out = runner(port, host, "nvidia-smi -L")
        print(out)
        failures += rc != 0
        print("-- imex health")
        print(runner(port, host, "if command -v nvidia-imex-ctl >/dev/null 2>&1; then nvidia-imex-ctl -N; else "
                                 "echo 'warning: nvidia-imex-ctl is not installed in this container'; fi")[1])
        rc, text = runner(port, host, f"cat {IMEX_NODES}")
        nodes = normalize_nodes_config(text) if rc == 0 else []
        print("-- normalized nodes_config.cfg")
        print("\n".join(nodes) if nodes else f"warning: {IMEX_NODES} is not readable on {label}")
        if first_nodes is None:
            first_nodes = nodes
        elif nodes != first_nodes:
            print("\n".join(difflib.unified_diff(first_nodes, nodes, "first tray", label, lineterm="")))
            failures += 1
    print("== remaining checks ==\nGPU-to-NUMA ids, CPU affinity, CUDA VMM, handle types and multicast are checked "
          "inside the benchmark binary.\n" + PARTITION_NOTE)
    return 1 if failures else 0


def main(argv: list[str] | None = None) -> int:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("rack_yaml", nargs="?")
    args = p.parse_args(argv)
    return rack_checks(args.rack_yaml) if args.rack_yaml else local_checks()


if __name__ == "__main__":
    raise SystemExit(main())
