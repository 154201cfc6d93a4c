"""Shared scaffolding of the multi-process CPU tests: start one process per rank, collect one
result per rank through a queue, and never leave a process behind."""
import multiprocessing as mp
import os
import time

CTX = mp.get_context("spawn")


def run_processes(target, world, args=(), timeout=60, prefix="t"):
    """Run target(rank, world, session, queue, *args) in `world` processes. Every process puts
    (rank, value) on the queue; returns {rank: value} of those that did so before the deadline."""
    session = f"{prefix}{os.getpid()}_{time.monotonic_ns()}"
    q = CTX.Queue()
    procs = [CTX.Process(target=target, args=(r, world, session, q) + tuple(args)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    deadline = time.time() + timeout
    while len(results) < world and time.time() < deadline:
        try:
            rank, value = q.get(timeout=0.5)
            results[rank] = value
        except Exception:  # queue.Empty
            if all(not p.is_alive() for p in procs) and q.empty():
                break
    for p in procs:
        p.join(timeout=10)
        if p.is_alive():
            p.kill()
    return results
