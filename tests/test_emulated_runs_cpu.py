"""The whole benchmark flow among CPU processes: the binary with MSHARP_DRIVER=fake.

Ranks are real processes started by the binary's own launcher; the driver stand-in provides
shared host memory in place of GPUs and the collective is played through on the CPU. What is
checked is everything around the kernels: iteration loop, replica hashes, the comparison with
the oracle, the JSON line and the exit codes (0 ok, 2 result check failed, 1 error), which the
reference project can only exercise on a rack (its src/main.cc:389-486).
"""
import json
import os
import subprocess

import pytest

from mnnvl_sharp_b200 import _build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RACK = os.path.join(ROOT, "examples", "rack_hgx8.yaml")


def run_binary(*flags, env=None, ranks=4):
    exe = _build.build_native()["exe"]
    full_env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    full_env.update({"MSHARP_DRIVER": "fake", "MSHARP_BOOTSTRAP_TIMEOUT_MS": "20000"})
    full_env.update(env or {})
    cmd = [str(exe), "--rack-config", RACK, "--rank-count", str(ranks), "--no-pin", "--warmup", "1", "--iters", "2", *flags]
    return subprocess.run(cmd, env=full_env, capture_output=True, text=True, timeout=120)


def last_json(text):
    return json.loads([line for line in text.splitlines() if line.startswith("{")][-1])


@pytest.mark.parametrize("flags", [
    ["--sharp-backend", "legacy", "--pattern", "reference", "--bytes", "2097172"],
    ["--sharp-backend", "legacy", "--pattern", "seeded", "--bytes", "2097172"],
    ["--sharp-backend", "tma_async", "--pattern", "seeded", "--bytes", "2097168"],
    ["--sharp-backend", "pull", "--types", "bf16", "--pattern", "tagged", "--bytes", "2097156"],
    ["--sharp-backend", "sw_f32", "--pattern", "seeded", "--bytes", "4096"],
])
def test_full_run_reports_matching_replicas_and_exit_code_zero(flags):
    done = run_binary(*flags, "--json", "--reference-check-bytes", "4096")
    assert done.returncode == 0, done.stdout + done.stderr
    r = last_json(done.stdout)
    assert r["hashes_match"] is True and len(set(r["hashes"])) == 1 and len(r["hashes"]) == 4
    assert r["f32_requantized_mismatches"] == 0 and r["status"] == 0 and r["init_only"] is False
    assert r["kernel_variant"] == "host_emulation_f32_sum" and r["handle_type"] == "posix_fd"
    assert r["sharp_kernel_ms"]["max"] >= r["sharp_kernel_ms"]["min"] > 0
    assert len(r["host_mapping"]) == 4 and len(r["peer_init_local_ms_by_rank"]) == 4
    assert len(r["sharp_kernel_ms_median_by_rank"]) == 4 and max(r["sharp_kernel_ms_median_by_rank"]) <= r["sharp_kernel_ms"]["max"]
    assert r["link_bound_ms"] > 0 and r["link_bound_fraction"] == pytest.approx(r["link_bound_ms"] / r["sharp_kernel_ms"]["median"], rel=1e-3)


def test_a_corrupted_replica_gives_exit_code_two_on_the_whole_job():
    done = run_binary("--json", "--bytes", "1048576", "--reference-check-bytes", "4096", "--pattern", "seeded",
                      env={"MSHARP_FAKE_CORRUPT": "2:70000"})
    assert done.returncode == 2, done.stdout + done.stderr
    r = last_json(done.stdout)
    assert r["hashes_match"] is False and len(set(r["hashes"])) == 2 and r["status"] == 2
    assert r["f32_requantized_mismatches"] == 0  # the checked prefix (rank 0, first 4 KiB) is intact


def test_a_wrong_value_in_the_checked_prefix_is_counted_and_fails_the_run():
    done = run_binary("--json", "--bytes", "1048576", "--reference-check-bytes", "65536", "--pattern", "seeded",
                      env={"MSHARP_FAKE_CORRUPT": "0:100", "MNNVL_DEBUG_MISMATCH": "1"})
    assert done.returncode == 2
    r = last_json(done.stdout)
    assert r["f32_requantized_mismatches"] == 1 and r["semantic_exact_mismatches"] >= 1 and r["hashes_match"] is False
    assert "got" in done.stderr and "expected" in done.stderr  # the mismatch dump asked for by MNNVL_DEBUG_MISMATCH


def test_zero_iterations_still_produce_a_checked_result_and_init_only_stops_after_the_canary():
    # --iters 0: one unmeasured iteration runs so that the check has data (reference: src/main.cc:446-448)
    done = run_binary("--json", "--bytes", "65536", "--reference-check-bytes", "4096", "--iters", "0", "--warmup", "0", ranks=2)
    assert done.returncode == 0
    r = last_json(done.stdout)
    assert r["hashes_match"] is True and r["semantic_exact_mismatches"] == 0
    assert r["sharp_kernel_ms"] == {"min": 0, "median": 0, "p95": 0, "max": 0}
    # the default --reference-check-bytes (16 MiB) exceeds small --bytes: refused as in the reference (config.cc:159-161)
    done = run_binary("--bytes", "65536", "--init-only", ranks=2)
    assert done.returncode == 1 and "--reference-check-bytes cannot exceed --bytes" in done.stderr
    done = run_binary("--bytes", "65536", "--reference-check-bytes", "4096", "--init-only", ranks=2)
    assert done.returncode == 0
    assert "smoke_test: passed" in done.stdout and "sharp_allreduce: skipped" in done.stdout
    done = run_binary("--bytes", "65536", "--reference-check-bytes", "4096", "--init-only", "--json", ranks=2)
    r = last_json(done.stdout)
    assert r["init_only"] is True and r["hashes_match"] is None and r["hashes"] == [] and r["f32_max_abs_error"] is None


def test_human_report_of_a_full_run():
    done = run_binary("--bytes", "1048576", "--reference-check-bytes", "4096")
    assert done.returncode == 0
    text = done.stdout
    assert text.startswith("mnnvl_sharp_allreduce\n")
    for key in ("selected_rank_count: 4", "smoke_test: passed", "hashes_match: true", "semantic_exact_mismatches: 0",
                "sharp_kernel_ms:", "collective_wall_ms:", "effective_logical_bandwidth_gib_s_median:"):
        assert key in text, key


def test_an_error_on_one_rank_ends_the_job_with_exit_code_one():
    # rank-count 3 on an inventory whose label does not match this host and no override: every rank
    # fails topology discovery and says why
    done = run_binary("--json", "--bytes", "4096", "--reference-check-bytes", "4096", ranks=3,
                      env={"MNNVL_HOST_LABEL": "somewhere-else"})
    assert done.returncode == 1
    lines = done.stderr.splitlines()
    assert sorted(line.split(":")[0] for line in lines if line.startswith("rank ")) == ["rank 0 error", "rank 1 error", "rank 2 error"]
    assert all("MNNVL_HOST_LABEL 'somewhere-else' did not match rack.yaml" in line for line in lines if line.startswith("rank "))
