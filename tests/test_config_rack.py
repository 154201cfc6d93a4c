"""Command-line validation, YAML subset, rack inventory, rank plans, launch artefacts (CPU only).

The expected messages and plans are the reference project's (src/config.cc:111-179,
src/rack_config.cc:96-224, scripts/run_mnnvl_sharp.sh:184-216).
"""
import pytest

from mnnvl_sharp_b200._native import NativeError
from mnnvl_sharp_b200.utils import rack

BASE = ["--rack-config", "rack.yaml"]


def cli(*args):
    return rack.parse_cli(BASE + list(args))


def test_defaults_match_the_reference():
    c = cli()
    assert c["bytes"] == 1073741824 and c["warmup"] == 3 and c["iters"] == 20
    assert c["rank_selection"] == "balanced" and c["sharp_backend"] == "legacy" and c["datatype"] == "e4m3"
    assert c["reference_check_bytes"] == 16777216 and c["init_only"] is False and c["json"] is False
    assert c["rank_count"] is None and c["pattern"] == "reference"


def test_auto_type_follows_backend():
    assert cli("--sharp-backend", "tma_async")["datatype"] == "f16"
    assert cli("--sharp-backend", "pull")["datatype"] == "f16"
    assert cli("--sharp-backend", "sw_f32")["datatype"] == "e4m3"
    assert cli("--sharp-backend", "pull", "--types", "bf16")["datatype"] == "bf16"


def test_integers_accept_hex_and_octal_and_reject_garbage():
    assert cli("--bytes", "0x1000", "--reference-check-bytes", "010")["bytes"] == 4096
    assert cli("--bytes", "0x1000", "--reference-check-bytes", "010")["reference_check_bytes"] == 8
    for bad in ("12x", "", "1.5", "abc"):
        with pytest.raises(NativeError, match="invalid integer for --bytes"):
            cli("--bytes", bad)
    with pytest.raises(NativeError, match="invalid integer for --warmup: 3q"):
        cli("--warmup", "3q")


@pytest.mark.parametrize("args,message", [
    ([], None),
    (["--bytes", "0"], "--bytes must be nonzero and a multiple of 4"),
    (["--bytes", "6"], "--bytes must be nonzero and a multiple of 4"),
    (["--rank-count", "0"], "--rank-count must be >= 1"),
    (["--rank-selection", "random"], "--rank-selection must be balanced or prefix"),
    (["--reference-check-bytes", "0"], "--reference-check-bytes must be nonzero and a multiple of 4"),
    (["--reference-check-bytes", "7"], "--reference-check-bytes must be nonzero and a multiple of 4"),
    (["--bytes", "4096"], "--reference-check-bytes cannot exceed --bytes"),
    (["--warmup", "-1"], "--warmup must be >= 0"),
    (["--iters", "-2"], "--iters must be >= 0"),
    (["--types", "f16"], "--types f16 is not supported with --sharp-backend legacy"),
    (["--sharp-backend", "tma_async", "--types", "e4m3"], "--types e4m3 is not supported with --sharp-backend tma_async"),
    (["--sharp-backend", "tma_async", "--bytes", "16777224"], "--bytes must be a multiple of 16 for --sharp-backend tma_async"),
    (["--sharp-backend", "nccl"], "--sharp-backend must be legacy or tma_async"),
    (["--types", "fp4"], "--types must be auto, e4m3, or f16"),
    (["--bytes"], "missing value after --bytes"),
    (["--frobnicate"], "unknown argument: --frobnicate"),
    (["--pattern", "noise"], "--pattern must be reference, seeded, or tagged"),
    (["--acc", "f32"], "--acc f32 is not available in-switch for e4m3"),
    (["--block", "100"], "--block must be a multiple of 32"),
])
def test_validation_messages(args, message):
    if message is None:
        cli(*args)
        return
    with pytest.raises(NativeError) as err:
        cli(*args)
    assert message in str(err.value)


def test_missing_rack_config_and_help_print_usage():
    with pytest.raises(NativeError) as err:
        rack.parse_cli([])
    assert "--rack-config is required" in str(err.value) and "usage:" in str(err.value)
    with pytest.raises(NativeError) as err:
        rack.parse_cli(["--help"])
    assert str(err.value).startswith("usage: mnnvl_sharp_allreduce --rack-config rack.yaml [--rank-count N]")
    assert "[--rank-selection balanced|prefix] [--sharp-backend legacy|tma_async]" in rack.usage()


def test_extension_flags_are_parsed_and_listed_in_usage():
    cfg = rack.parse_cli(["--rack-config", "r.yaml", "--trace-phases", "--hub-address", "10.0.0.1:4000", "--session", "job7",
                          "--handle-type", "fabric", "--wait-timeout-ms", "500", "--no-pin"])
    assert cfg["trace_phases"] is True and cfg["hub_address"] == "10.0.0.1:4000" and cfg["session"] == "job7"
    assert cfg["handle_type"] == "fabric" and cfg["wait_timeout_ms"] == 500 and cfg["no_pin"] is True
    defaults = rack.parse_cli(["--rack-config", "r.yaml"])
    assert defaults["trace_phases"] is False and defaults["hub_address"] == "" and defaults["handle_type"] == "auto"
    for flag in ("--trace-phases", "--hub-address HOST:PORT", "--handle-type auto|posix_fd|fabric", "--cpu-only"):
        assert flag in rack.usage(), flag
    with pytest.raises(NativeError, match="--hub-address"):
        rack.parse_cli(["--rack-config", "r.yaml", "--hub-address"])


RACK_2X4 = """
# two trays
rack:
  - tray-a.example.com:
      - hostname: 10.0.0.11
      - port: 4399
      - device: [0, 1, 2, 3]
  - tray-b:
      hostname: "10.0.0.12"   # plain map body, default port
      device:
        - 3
        - 2
        - 1
        - 0
"""


def test_yaml_subset_shapes():
    obj = rack.yaml_to_obj(RACK_2X4)
    assert list(obj) == ["rack"] and len(obj["rack"]) == 2
    assert obj["rack"][0]["tray-a.example.com"][2] == {"device": ["0", "1", "2", "3"]}
    assert obj["rack"][1]["tray-b"]["device"] == ["3", "2", "1", "0"]
    assert rack.yaml_to_obj("a: 'it''s'\nb: \"x # not a comment\"  # comment\nc:\n- 1\n- {k: v, l: [1, 2]}\n") == {
        "a": "it's", "b": "x # not a comment", "c": ["1", {"k": "v", "l": ["1", "2"]}]}
    assert rack.yaml_to_obj("---\nkey: ~\n...\n") == {"key": None}
    for bad, why in [("a:\n\t- 1\n", "tab"), ("a: &x 1\n", "anchors"), ("a: [1, 2\n", "flow sequence"),
                     ("a: 1\na: 2\n", "duplicate mapping key"), ("a: 1\n   b: 2\n", "indentation"),
                     ("a: |\n  text\n", "block scalars")]:
        with pytest.raises(NativeError, match=why):
            rack.yaml_to_obj(bad)


def test_rack_fields_and_limits():
    r = rack.parse_rack(RACK_2X4)
    assert r["available_rank_count"] == 8
    a, b = r["entries"]
    assert (a["host_label"], a["hostname"], a["port"], a["devices"]) == ("tray-a.example.com", "10.0.0.11", 4399, [0, 1, 2, 3])
    assert (b["hostname"], b["port"], b["devices"]) == ("10.0.0.12", 4399, [3, 2, 1, 0])

    def one(body):
        return "rack:\n  - h1:\n" + "".join(f"      {line}\n" for line in body)

    cases = [
        ("racks: []\n", "top-level sequence named 'rack'"),
        ("rack:\n  - a: {hostname: x, device: [0]}\n    b: {hostname: y, device: [0]}\n", "single-key map"),
        (one(["hostname: x", "device: \"0,2\""]), "requires 'device' as a YAML sequence"),
        (one(["hostname: x", "device: 0"]), "requires 'device' as a YAML sequence"),
        (one(["device: [0]"]), "requires scalar field 'hostname'"),
        (one(["hostname: x", "device: [0, 0]"]), "duplicate CUDA device ordinals"),
        (one(["hostname: x", "device: [-1]"]), "negative CUDA device ordinal"),
        (one(["hostname: x", "device: [a]"]), "device entries must be scalar integers"),
        (one(["hostname: x", "device: []"]), "must list 1 to 8 CUDA device ordinals"),
        (one(["hostname: x", "device: [0,1,2,3,4,5,6,7,8]"]), "must list 1 to 8 CUDA device ordinals"),
        (one(["hostname: x", "port: 70000", "device: [0]"]), "invalid SSH port"),
        (one(["hostname: x", "port: 0", "device: [0]"]), "invalid SSH port"),
        ("rack:\n  - h.a:\n      hostname: x\n      device: [0]\n  - h.b:\n      hostname: y\n      device: [1]\n",
         "duplicate rack host label: h.b"),
    ]
    for text, message in cases:
        with pytest.raises(NativeError) as err:
            rack.parse_rack(text)
        assert message in str(err.value), (text, str(err.value))
    many = "rack:\n" + "".join(f"  - t{i}:\n      hostname: h{i}\n      device: [0]\n" for i in range(19))
    with pytest.raises(NativeError, match="1 to 18 rack entries"):
        rack.parse_rack(many)
    big = "rack:\n" + "".join(f"  - t{i}:\n      hostname: h{i}\n      device: [0,1,2,3,4,5,6,7]\n" for i in range(10))
    with pytest.raises(NativeError, match="more than 72 CUDA devices"):
        rack.parse_rack(big)
    with pytest.raises(NativeError, match="cannot read"):
        rack.load_rack("/nonexistent/rack.yaml")


def plan_pairs(count, selection):
    return [(t["host_label"].split(".")[0], t["gpu"]) for t in rack.rank_plan(RACK_2X4, count, selection)]


def test_rank_plans_for_two_trays_of_four():
    a, b = "tray-a", "tray-b"
    assert plan_pairs(2, "balanced") == [(a, 0), (b, 3)]
    assert plan_pairs(4, "balanced") == [(a, 0), (b, 3), (a, 1), (b, 2)]
    assert plan_pairs(8, "balanced") == [(a, 0), (b, 3), (a, 1), (b, 2), (a, 2), (b, 1), (a, 3), (b, 0)]
    assert plan_pairs(2, "prefix") == [(a, 0), (a, 1)]
    assert plan_pairs(4, "prefix") == [(a, 0), (a, 1), (a, 2), (a, 3)]
    assert plan_pairs(8, "prefix") == [(a, i) for i in range(4)] + [(b, 3), (b, 2), (b, 1), (b, 0)]
    plan = rack.rank_plan(RACK_2X4, 8, "balanced")
    assert [t["local_rank"] for t in plan] == [0, 0, 1, 1, 2, 2, 3, 3]
    assert [t["rack_index"] for t in plan] == [0, 1] * 4
    with pytest.raises(NativeError, match="rank_count 9 exceeds rack.yaml device count 8"):
        rack.rank_plan(RACK_2X4, 9, "balanced")
    with pytest.raises(NativeError, match="rank_count must be positive"):
        rack.rank_plan(RACK_2X4, 0, "balanced")
    with pytest.raises(NativeError, match="rank selection must be balanced or prefix"):
        rack.rank_plan(RACK_2X4, 2, "zigzag")


def test_uneven_trays_and_single_hgx_tray():
    text = "rack:\n  - a:\n      hostname: x\n      device: [0]\n  - b:\n      hostname: y\n      device: [4, 5, 6]\n"
    pairs = [(t["host_label"], t["gpu"]) for t in rack.rank_plan(text, 4, "balanced")]
    assert pairs == [("a", 0), ("b", 4), ("b", 5), ("b", 6)]
    hgx = rack.single_host_yaml(8)
    assert [t["gpu"] for t in rack.rank_plan(hgx, 8, "balanced")] == list(range(8))
    assert [t["gpu"] for t in rack.rank_plan(hgx, 3, "prefix")] == [0, 1, 2]


def test_launch_texts():
    t = rack.launch_texts(RACK_2X4, 3, "balanced", ssh_user="ops", ssh_identity="/k/id", ssh_known_hosts="/k/kh")
    assert t["hosts"] == "tray-a.example.com:2,tray-b:1"
    assert t["rankfile"] == "rank 0=tray-a.example.com slot=0\nrank 1=tray-b slot=0\nrank 2=tray-a.example.com slot=1\n"
    assert t["entries"] == "tray-a.example.com\t10.0.0.11\t4399\ntray-b\t10.0.0.12\t4399\n"
    block = ("Host tray-b\n  HostName 10.0.0.12\n  User ops\n  Port 4399\n  IdentityFile /k/id\n  IdentitiesOnly yes\n"
             "  PasswordAuthentication no\n  UserKnownHostsFile /k/kh\n  StrictHostKeyChecking accept-new\n  BatchMode yes\n\n")
    assert block in t["ssh_config"] and t["ssh_config"].count("Host ") == 2
    only_a = rack.launch_texts(RACK_2X4, 2, "prefix")
    assert only_a["hosts"] == "tray-a.example.com:2" and "tray-b" not in only_a["ssh_config"]
    assert "User ubuntu" in only_a["ssh_config"]


def test_cpu_list_parsing():
    assert rack.parse_cpu_list("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert rack.parse_cpu_list("") == []
    with pytest.raises(NativeError, match="invalid CPU range"):
        rack.parse_cpu_list("5-2")
    with pytest.raises(NativeError, match="invalid token"):
        rack.parse_cpu_list("a-b")


def test_cpu_only_oracle_run(tmp_path):
    path = tmp_path / "rack.yaml"
    path.write_text(RACK_2X4)
    out = rack.run_cpu_only(["--rack-config", str(path), "--rank-count", "8", "--bytes", "65536",
                             "--reference-check-bytes", "65536", "--pattern", "seeded"])
    assert out["mode"] == "cpu_only" and out["selected_rank_count"] == 8 and len(out["plan"]) == 8
    assert len(out["expected_f32_cast_hash"]) > 0 and out["cpu_reduce_f32_ms"] >= 0
    again = rack.run_cpu_only(["--rack-config", str(path), "--rank-count", "8", "--bytes", "65536",
                               "--reference-check-bytes", "65536", "--pattern", "seeded"])
    assert again["expected_f32_cast_hash"] == out["expected_f32_cast_hash"]


def test_cpu_only_binary_dumps_the_bitwise_expected_result(tmp_path):
    import json
    import subprocess

    import numpy as np

    from mnnvl_sharp_b200 import _build
    from mnnvl_sharp_b200.utils import numerics as nm

    exe = _build.build_native()["exe"]
    path = tmp_path / "rack.yaml"
    path.write_text(RACK_2X4)
    out = tmp_path / "expected.bin"
    for types, backend, dtype in (("e4m3", "legacy", "e4m3"), ("f16", "tma_async", "f16")):
        proc = subprocess.run([str(exe), "--rack-config", str(path), "--rank-count", "8", "--cpu-only", "--pattern", "seeded",
                               "--sharp-backend", backend, "--types", types, "--bytes", "65536",
                               "--reference-check-bytes", "65536", "--dump-expected", str(out)],
                              capture_output=True, text=True, timeout=120)
        assert proc.returncode == 0, proc.stderr
        summary = json.loads(proc.stdout.strip().splitlines()[-1])
        assert summary["datatype"] == dtype and summary["selected_rank_count"] == 8
        got = np.fromfile(out, dtype=nm.storage_dtype(dtype))
        assert np.array_equal(got, nm.reduce_f32_cast(dtype, "seeded", 8, got.size))
        assert int(summary["expected_f32_cast_hash"], 16) == nm.hash_words(got)
    with pytest.raises(NativeError, match="--dump-expected needs --cpu-only"):
        cli("--dump-expected", "x.bin")


def test_csv_header():
    assert rack.CSV_HEADER == ("rank_count,repeat,sharp_backend,peer_init_ms,peer_init_min_ms,peer_init_median_ms,"
                               "peer_init_p95_ms,peer_init_max_ms")


def _inventory_yaml(trays):
    lines = ["rack:"]
    for i, devices in enumerate(trays):
        lines += [f"  - tray{i:02d}:", f"      - hostname: 10.0.0.{i + 1}", f"      - device: {list(devices)}"]
    return "\n".join(lines) + "\n"


def test_rank_plan_invariants_over_random_inventories():
    """For any inventory and count: every selected (tray, device) pair is distinct and listed in the
    inventory; `prefix` fills trays in inventory order; `balanced` takes device slot s of every tray
    before slot s + 1 (so per-tray counts differ by at most one while trays still have devices)."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    trays_strategy = st.lists(
        st.lists(st.integers(min_value=0, max_value=15), min_size=1, max_size=8, unique=True), min_size=1, max_size=9)

    @settings(max_examples=150, deadline=None)
    @given(trays=trays_strategy, data=st.data())
    def check(trays, data):
        text = _inventory_yaml(trays)
        total = sum(len(t) for t in trays)
        count = data.draw(st.integers(min_value=1, max_value=total))
        for policy in ("prefix", "balanced"):
            plan = rack.rank_plan(text, count, policy)
            assert [t["rank"] for t in plan] == list(range(count))
            pairs = [(t["rack_index"], t["gpu"]) for t in plan]
            assert len(set(pairs)) == count
            assert all(gpu in trays[tray] for tray, gpu in pairs)
            per_tray = [sum(1 for tray, _ in pairs if tray == i) for i in range(len(trays))]
            for t in plan:  # local rank = position among the ranks of the same tray
                assert t["local_rank"] == [p for p in plan if p["rack_index"] == t["rack_index"]].index(t)
            if policy == "prefix":
                flat = [(i, g) for i, devices in enumerate(trays) for g in devices]
                assert pairs == flat[:count]
            else:
                slots = [(i, devices[s]) for s in range(8) for i, devices in enumerate(trays) if s < len(devices)]
                assert pairs == slots[:count]
                unfilled = [n for n, devices in zip(per_tray, trays) if n < len(devices)]
                if unfilled:
                    assert max(per_tray) - min(unfilled) <= 1
        with pytest.raises(NativeError):
            rack.rank_plan(text, total + 1, "balanced")

    check()
