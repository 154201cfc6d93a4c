"""Headline benchmark: in-switch all-reduce bus bandwidth at 1 GiB per rank.

    python bench.py --gpus N --steps K --warmup W          # N == 1, or launched by torchrun for N > 1
    python bench.py --impl reference ...                   # the reference arm (see below)

One rank per GPU. Rank 0 prints one JSON line. `value` is the NCCL-convention bus bandwidth
algbw * 2 (N-1) / N of the FP8 E4M3 all-reduce (multimem.ld_reduce + multimem.st, the "legacy"
backend) over 1 GiB per rank, timed on the device as the maximum over ranks; for N == 1 the
factor is zero by definition, so the plain pass bandwidth is reported instead and the line
says so. The F16 figure of the same run (float32 accumulation in the switch) is in `f16`.
The buffers (1 GiB each) are larger than the 126 MB L2, so no flush is needed between steps.

The `e2e` block repeats the measurement through the package's public API with, per step, a
host-to-device copy of the step's input from pinned memory and a device-to-host read of the
step's result (the replica hash).

The reference arm cannot run here: the reference project is a CMake/MPI binary, not a Python
package (pip finds nothing to install), and its build needs CUDA 13.1, MPI and yaml-cpp, none
of which exist in this image; `--impl reference` therefore prints an `unavailable` line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

GIB = 1 << 30


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--bytes", type=int, default=GIB)
    p.add_argument("--check-bytes", type=int, default=16 << 20)
    return p.parse_args()


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.01):
        super().__init__(daemon=True)
        self.index = index
        self.period = period_s
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = 0
        self.power_w = 0.0
        self._stop_flag = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.dev = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.dev, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake",
        }
        while not self._stop_flag.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.dev, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.dev))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
                self.power_w = max(self.power_w, nv.nvmlDeviceGetPowerUsage(self.dev) / 1000.0)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self) -> dict:
        self._stop_flag.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {
            "sm_mhz": s[len(s) // 2] if s else None,
            "sm_max_mhz": self.max_mhz or None,
            "reasons": sorted(self.reasons),
            "samples": len(s),
            "power_w_max": round(self.power_w, 1),
        }


def busbw(nbytes: int, ms: float, n: int) -> float:
    alg = nbytes / (ms * 1e6)
    return alg if n == 1 else alg * 2.0 * (n - 1) / n


LINK_GB_S = 770.0  # measured peer-copy bandwidth per direction per GPU on this pool (nominal 900)


def roofline(nbytes: int, ms: float, n: int) -> dict:
    """Bound of the in-switch all-reduce: every GPU sends its buffer once into the switch (the
    reduce of the other ranks' slices) plus its reduced 1/N slice, and receives the same amount,
    so t >= S (1 + 1/N) / link. In bus-bandwidth terms that is link * 2 (N-1) / (N+1)."""
    if n == 1:
        return {"note": "one rank moves nothing over NVLink; no link bound applies"}
    bound_ms = nbytes * (1.0 + 1.0 / n) / (LINK_GB_S * 1e6)
    return {"link_gb_s_measured": LINK_GB_S, "bound_ms": round(bound_ms, 4),
            "bound_busbw_gb_s": round(LINK_GB_S * 2.0 * (n - 1) / (n + 1), 1),
            "fraction_of_measured": round(bound_ms / ms, 3)}


def run_ours(args) -> int:
    import numpy as np
    import torch

    from mnnvl_sharp_b200 import ops
    from mnnvl_sharp_b200.parallel import Bootstrap, Communicator
    from mnnvl_sharp_b200.utils import numerics as nm

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}; launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    nbytes = args.bytes
    steps, warmup = args.steps, max(args.warmup, 0)

    boot = Bootstrap.from_env()
    comm = Communicator(boot, local_rank, wait_timeout_ms=5000)
    buf = comm.alloc(nbytes, layout="single", multicast=True)
    buf.canary_check()
    launches = {"timed": 0}

    def sync_all():
        torch.cuda.synchronize()
        boot.barrier()

    def timed_region(fn, k: int) -> float:
        """barrier + sync, K steps between two events, sync + barrier; max over ranks, ms per step."""
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        sync_all()
        start.record()
        for _ in range(k):
            fn()
        stop.record()
        sync_all()
        comm.raise_if_failed("timed all-reduce")
        return boot.reduce_max(start.elapsed_time(stop)) / k

    results = {}
    checks = {}
    sampler = ClockSampler(local_rank) if rank == 0 else None
    for dtype, backend in (("e4m3", "legacy"), ("f16", "pull")):
        pattern = "seeded"
        # correctness first: one all-reduce of seeded inputs, compared with the host oracle
        ops.init_pattern(buf, dtype, pattern, rank, nbytes)
        sync_all()
        ops.all_reduce(comm, buf, dtype, backend=backend)
        sync_all()
        comm.raise_if_failed("all-reduce")
        got = buf.read(min(args.check_bytes, nbytes)).view(nm.storage_dtype(dtype))
        m = nm.compare(dtype, pattern, world, got)
        hashes = boot.allgather_array(np.array([ops.device_hash(buf.output_ptr(), nbytes)], dtype=np.uint64))
        ok = m.max_requantized_ulp_distance <= 1 and len(set(int(h) for h in hashes[:, 0])) == 1
        checks[dtype] = {"max_ulp_vs_f32": m.max_requantized_ulp_distance, "replicas_equal": len(set(int(h) for h in hashes[:, 0])) == 1}
        if not boot.all_true(ok):
            raise SystemExit(f"all-reduce {dtype} failed its check: {checks[dtype]}")
        step = lambda: ops.all_reduce(comm, buf, dtype, backend=backend)  # noqa: E731
        for _ in range(max(warmup, 3)):
            step()
        if sampler is not None and dtype == "e4m3":
            sampler.start()
        ms = timed_region(step, steps)
        if dtype == "e4m3":
            launches["timed"] = steps
            # The timed region lasts a few milliseconds, too short for more than a sample or two of
            # NVML: keep the same kernel running (untimed) for 0.4 s so that the clock record shows
            # the state of the GPU under this load. All ranks do it; the kernels wait for each other.
            t_end = time.time() + 0.4
            keep_going = True
            while keep_going:
                for _ in range(10):
                    step()
                torch.cuda.synchronize()
                keep_going = boot.all_true(time.time() < t_end)
            if sampler is not None:
                clocks = sampler.stop()
                clocks["window"] = "timed region plus 0.4 s of the same kernel"
        results[dtype] = ms
    if sampler is None:
        clocks = {}

    # end to end through the public API: pinned host input -> device, all-reduce, result -> host
    dtype, backend = "e4m3", "legacy"
    host_in = torch.from_numpy(nm.generate(dtype, "seeded", rank, min(nbytes, 64 << 20))).repeat(
        max(1, nbytes // min(nbytes, 64 << 20)))[:nbytes].contiguous().pin_memory()
    dev_view = buf.tensor(torch.uint8)
    hash_dev = torch.zeros(1, dtype=torch.int64, device="cuda")
    hash_host = torch.zeros(1, dtype=torch.int64).pin_memory()
    from mnnvl_sharp_b200 import _native as N

    def e2e_step():
        dev_view.copy_(host_in, non_blocking=True)
        ops.all_reduce(comm, buf, dtype, backend=backend)
        N.check(N.lib.msharp_hash_device(buf.output_ptr(), nbytes, hash_dev.data_ptr(),
                                         int(torch.cuda.current_stream().cuda_stream)))
        hash_host.copy_(hash_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the step's result is on the host

    for _ in range(2):
        e2e_step()
    e2e_ms = timed_region(e2e_step, max(1, min(steps, 10)))

    if rank == 0:
        ms = results["e4m3"]
        line = {
            "metric": "allreduce_busbw_gb_s_1GiB_fp8_e4m3",
            "value": round(busbw(nbytes, ms, world), 3),
            "unit": "GB/s",
            "n_gpus": world,
            "steps": steps,
            "warmup": max(warmup, 3),
            "ms_per_step": round(ms, 6),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "fp8_e4m3 (fp16 accumulate in switch); f16 in `f16`",
            "data": "synthetic seeded uniform[-2,2)->e4m3 and ~N(0,1)->f16, generated on device",
            "impl": "ours",
            "config": {
                "model": "allreduce_sum_inplace",
                "global_batch": world,
                "seq_len": nbytes,
                "bytes_per_rank": nbytes,
                "parallelism": f"dp{world}",
                "backend": "legacy(e4m3)+pull(f16)",
                "l2": "inputs (1 GiB per rank) exceed the 126 MB L2; no flush between steps",
                "n1_note": "busbw factor 2(N-1)/N is 0 at N=1; value is the local pass bandwidth there" if world == 1 else "",
                "handle_type": buf.info["handle_type"],
                "peer_init_ms": buf.info["peer_init_ms"],
            },
            "algbw_gb_s": round(nbytes / (ms * 1e6), 3),
            "aggregate_logical_gb_s": round(world * nbytes / (ms * 1e6), 3),
            "f16": {"ms_per_step": round(results["f16"], 6), "busbw_gb_s": round(busbw(nbytes, results["f16"], world), 3),
                    "algbw_gb_s": round(nbytes / (results["f16"] * 1e6), 3)},
            "roofline": roofline(nbytes, ms, world),
            "scaling_note": "bus bandwidth is normalised per GPU (ideal: flat in N, at the link bound); the whole-job "
                            "figure is aggregate_logical_gb_s = N * bytes / time",
            "checks": checks,
            "clocks": clocks,
            "e2e": {"value": round(busbw(nbytes, e2e_ms, world), 3), "unit": "GB/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": 8},
            "gpu_launches": launches["timed"],
        }
        print(json.dumps(line), flush=True)
    sync_all()
    del dev_view
    comm.close()
    boot.close()
    return 0


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return 0  # launched once per GPU: one line for the job, from rank 0
        print(json.dumps({
            "impl": "reference",
            "unavailable": "reference is a CMake+MPI+yaml-cpp binary needing CUDA 13.1 (none in this image); "
                           "pip finds no setup.py/pyproject.toml in it, so nothing can be installed or run",
        }), flush=True)
        return 0
    if args.gpus > 1 and "RANK" not in os.environ:
        # convenience: start the ranks ourselves when not under torchrun
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 1000), os.path.abspath(__file__)] + sys.argv[1:]
        return subprocess.call(cmd)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
