"""Shared helpers of the command-line tools that run as one process per GPU."""
from __future__ import annotations

import os

import torch

from ..parallel import Bootstrap, Communicator


def init_rank(wait_timeout_ms: int = 5000):
    """Bind this process to its GPU and connect the control plane (RANK / WORLD_SIZE / LOCAL_RANK)."""
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local_rank)
    boot = Bootstrap.from_env()
    comm = Communicator(boot, local_rank, wait_timeout_ms=wait_timeout_ms)
    return boot, comm


def time_steps(boot, comm, fn, iters: int, warmup: int = 3, graph: bool = False) -> float:
    """Milliseconds per call of `fn`, device-timed over `iters` back-to-back calls, max over ranks.

    With graph=True the `iters` calls are captured once into a CUDA graph and the replay is
    timed, which removes the host's launch cost from the figure (the kernels keep their barrier
    epochs in device memory, so a captured launch can be replayed any number of times).
    """
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    # fail fast: a kernel that gave up waiting for a peer would do so again in every timed call
    if not boot.all_true(comm.status().ok):
        comm.raise_if_failed("warm-up")
        raise RuntimeError("a device-side wait failed on another rank during warm-up")
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    runner = None
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                fn()
        runner = g.replay
        runner()  # one untimed replay
        torch.cuda.synchronize()
    boot.barrier()
    start.record()
    if runner is not None:
        runner()
    else:
        for _ in range(iters):
            fn()
    stop.record()
    torch.cuda.synchronize()
    boot.barrier()
    comm.raise_if_failed("timed kernel")
    return boot.reduce_max(start.elapsed_time(stop)) / iters


def busbw(nbytes: int, ms: float, world: int) -> float:
    alg = nbytes / (ms * 1e6)
    return alg * 2.0 * (world - 1) / world if world > 1 else alg
