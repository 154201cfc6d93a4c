"""Rack inventory, rank plan, launch artefacts and CLI parsing, backed by the native library
(one implementation for the binary, the launcher and the sweep scripts; the reference project
carries separate copies of this logic in src/rack_config.cc, scripts/run_mnnvl_sharp.sh:98-216,
scripts/preflight_imex.sh:73-107 and scripts/run_init_sweep.py:17-48).
"""
from __future__ import annotations

from pathlib import Path

from .. import _native as N


def load_rack(path: str | Path) -> dict:
    return N.as_json(N.lib.msharp_rack_from_file(str(path).encode()))


def parse_rack(yaml_text: str) -> dict:
    return N.as_json(N.lib.msharp_rack_from_yaml(yaml_text.encode()))


def available_rank_count(path: str | Path) -> int:
    return int(load_rack(path)["available_rank_count"])


def rank_plan(yaml_text: str, rank_count: int, selection: str = "balanced") -> list[dict]:
    return N.as_json(N.lib.msharp_plan_from_yaml(yaml_text.encode(), rank_count, selection.encode()))


def launch_texts(yaml_text: str, rank_count: int, selection: str = "balanced", ssh_user: str = "",
                 ssh_identity: str = "", ssh_known_hosts: str = "") -> dict:
    """Host list, Open MPI style rankfile, ssh config and selected-entries table as strings."""
    return N.as_json(N.lib.msharp_launch_texts(yaml_text.encode(), rank_count, selection.encode(), ssh_user.encode(),
                                                ssh_identity.encode(), ssh_known_hosts.encode()))


def parse_cpu_list(text: str) -> list[int]:
    return N.as_json(N.lib.msharp_parse_cpu_list(text.encode()))


def yaml_to_obj(yaml_text: str):
    """Parse the supported YAML subset into Python objects (scalars stay strings)."""
    return N.as_json(N.lib.msharp_yaml_to_json(yaml_text.encode()))


def parse_cli(args: list[str], prog: str = "mnnvl_sharp_allreduce") -> dict:
    """Validate benchmark flags exactly as the binary does; raises NativeError with its message."""
    argc, argv = N.argv([prog] + list(args))
    return N.as_json(N.lib.msharp_parse_config(argc, argv))


def usage(prog: str = "mnnvl_sharp_allreduce") -> str:
    return N.text(N.lib.msharp_usage(prog.encode()))


def run_cpu_only(args: list[str]) -> dict:
    """Host-only oracle run (the binary's --cpu-only mode) and its JSON summary."""
    argc, argv = N.argv(["mnnvl_sharp_allreduce"] + list(args) + ["--cpu-only"])
    return N.as_json(N.lib.msharp_run_cpu_only(argc, argv))


def single_host_yaml(device_count: int, label: str = "localhost") -> str:
    devices = ", ".join(str(d) for d in range(device_count))
    return f"rack:\n  - {label}:\n      - hostname: 127.0.0.1\n      - port: 4399\n      - device: [{devices}]\n"


CSV_HEADER = N.text(N.lib.msharp_init_latency_csv_header())
