"""Launcher, init-latency sweep, plot and preflight helpers (CPU only; the benchmark itself is
replaced by a stub process where one would be started)."""
import csv
import json
import sys
from pathlib import Path

import pytest

from mnnvl_sharp_b200.cli import init_sweep, plot_init_latency, preflight, run
from mnnvl_sharp_b200.utils import rack as racklib

RACK = """rack:
  - tray-a:
      - hostname: 10.0.0.11
      - device: [0, 1, 2, 3]
  - tray-b:
      - hostname: 10.0.0.12
      - port: 2222
      - device: [0, 1, 2, 3]
"""


def test_rank_count_selection_rules():
    assert init_sweep.parse_rank_counts("4, 8,16,") == [4, 8, 16]
    with pytest.raises(ValueError):
        init_sweep.parse_rank_counts("4,0")
    assert init_sweep.select_rank_counts([4, 8, 16, 32, 64, 72], 8) == [4, 8]
    assert init_sweep.select_rank_counts([4, 16], 8) == [4, 8]      # the inventory total is added
    assert init_sweep.select_rank_counts([1, 2, 4], 2) == [1, 2]    # ... but not below four devices
    assert init_sweep.select_rank_counts([16], 3) == []


def test_json_line_extraction_takes_the_last_object_line():
    out = 'launching ...\n{"peer_init_ms": 1}\nnoise\n {"peer_init_ms": 2} \ntrailer'
    assert init_sweep.extract_json_line(out) == {"peer_init_ms": 2}
    with pytest.raises(RuntimeError):
        init_sweep.extract_json_line("no json here\n{broken")


def test_sweep_writes_reference_schema_resumes_and_plots(tmp_path):
    rack_path = tmp_path / "rack.yaml"
    rack_path.write_text(RACK)
    stub = tmp_path / "stub.py"
    calls = tmp_path / "calls.txt"
    stub.write_text(
        "import sys, json\n"
        f"open({str(calls)!r}, 'a').write(' '.join(sys.argv[1:]) + '\\n')\n"
        "n = int(sys.argv[sys.argv.index('--rank-count') + 1])\n"
        "if n == 8 and '--fail8' in open(" + repr(str(tmp_path / 'mode.txt')) + ").read(): sys.exit(1)\n"
        "print('launching')\n"
        "print(json.dumps({'peer_init_ms': n * 1.5, 'peer_init_min_ms': n, 'peer_init_median_ms': n * 1.25,"
        " 'peer_init_p95_ms': n * 1.5, 'peer_init_max_ms': n * 1.5}))\n")
    (tmp_path / "mode.txt").write_text("--fail8")
    out_dir = tmp_path / "out"
    argv = [str(rack_path), "--rank-counts", "2,4,72", "--repeats", "2", "--out-dir", str(out_dir)]
    rc = init_sweep.main(argv, launcher=[sys.executable, str(stub)])
    assert rc == 1  # the 8-rank points failed, the others were kept
    rows = list(csv.DictReader((out_dir / "init_latency.csv").open()))
    assert list(rows[0]) == racklib.CSV_HEADER.split(",")
    assert [(r["rank_count"], r["repeat"]) for r in rows] == [("2", "0"), ("2", "1"), ("4", "0"), ("4", "1")]
    assert rows[2]["peer_init_ms"] == "6.0" and rows[2]["sharp_backend"] == "legacy"
    assert (out_dir / "rank_4_repeat_1.log").exists() and "--init-only --json" in calls.read_text()
    # second run: only the missing points are run
    (tmp_path / "mode.txt").write_text("")
    before = len(calls.read_text().splitlines())
    assert init_sweep.main(argv, launcher=[sys.executable, str(stub)]) == 0
    assert len(calls.read_text().splitlines()) - before == 2
    rows = list(csv.DictReader((out_dir / "init_latency.csv").open()))
    assert len(rows) == 6 and rows[-1]["rank_count"] == "8"
    assert (out_dir / "init_latency.png").exists() or (out_dir / "init_latency.svg").exists()


def test_svg_fallback_chart(tmp_path):
    svg = plot_init_latency.svg_chart({2: [1.0, 2.0, 3.0], 8: [4.0, 5.0, 9.0]})
    assert svg.startswith("<svg") and "rank count" in svg and "peer access initialization latency (ms)" in svg
    assert svg.count("<circle") == 2
    csv_path = tmp_path / "x.csv"
    csv_path.write_text(racklib.CSV_HEADER + "\n4,0,legacy,3.5,3,3.2,3.5,3.5\n")
    assert plot_init_latency.plot(csv_path, tmp_path / "p.png") is not None


def test_launcher_scans_flags_and_writes_artefacts(tmp_path, capsys):
    assert run.scan(["--json", "--rank-count", "4", "--rank-selection", "prefix"]) == ("4", "prefix")
    with pytest.raises(SystemExit):
        run.scan(["--rank-selection", "zigzag"])
    with pytest.raises(SystemExit):
        run.scan(["--rank-count"])
    rack_path = tmp_path / "rack.yaml"
    rack_path.write_text(RACK)
    emit = tmp_path / "emit"
    rc = run.main([str(rack_path), "--rank-count", "3", "--emit-dir", str(emit), "--json"])
    assert rc == 3  # two remote trays: artefacts only
    assert (emit / "hosts.txt").read_text() == "tray-a:2,tray-b:1"
    assert (emit / "rankfile").read_text().splitlines()[1] == "rank 1=tray-b slot=0"
    assert "Port 2222" in (emit / "ssh_config").read_text()
    assert (emit / "rank_count.txt").read_text() == "3"
    assert (emit / "selected_entries.tsv").read_text().splitlines()[1] == "tray-b\t10.0.0.12\t2222"
    with pytest.raises(SystemExit):
        run.main([str(rack_path), "--rank-count", "9"])


def test_preflight_helpers(tmp_path):
    text = "# comment\n10.0.0.1   # tray a\n\n  10.0.0.2\n10.0.0.1\n"
    assert preflight.normalize_nodes_config(text) == ["10.0.0.1", "10.0.0.1", "10.0.0.2"]
    rack_path = tmp_path / "rack.yaml"
    rack_path.write_text(RACK)
    answers = {"hostname": "tray-a", "cat": "10.0.0.11\n10.0.0.12"}

    def fake_remote(port, host, command):
        if command == "hostname":
            return 0, "tray-a" if host.endswith("11") else "other-name"
        if command.startswith("cat "):
            return 0, answers["cat"] if host.endswith("11") else "10.0.0.11"
        return 0, "ok"

    assert preflight.rack_checks(str(rack_path), runner=fake_remote) == 1  # node lists differ

    def unreachable(port, host, command):
        return 255, "ssh: connect refused"

    assert preflight.rack_checks(str(rack_path), runner=unreachable) == 1
