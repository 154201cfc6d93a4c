"""Control plane and symmetric-memory set-up among CPU processes (no GPU).

The ranks are real processes; device memory is replaced by the host-memory fake driver, whose
allocations are memfd files, so exported handles really travel between processes and the
canary of every rank is really read by every other rank. Failures are injected on the host:
a rank that never joins, a rank that dies, a stranger on the socket, a driver call that fails.
"""
import os
import socket
import struct
import time

import numpy as np
import pytest

from _procs import run_processes

CUDA_ERROR_NOT_SUPPORTED = 801
CUDA_ERROR_NOT_PERMITTED = 800
CUDA_ERROR_OUT_OF_MEMORY = 2


def _run(target, world, *args, timeout=60):
    """Run target(rank, world, session, queue, *args) in `world` processes; return results by rank."""
    return run_processes(target, world, args, timeout, prefix="test")


def _collectives(rank, world, session, q):
    from mnnvl_sharp_b200.parallel import Bootstrap

    try:
        with Bootstrap(rank, world, session, timeout_ms=20000) as b:
            b.barrier()
            gathered = b.allgather_bytes(bytes([rank]) * 64)
            arr = b.allgather_array(np.array([rank * 1.5, rank], dtype=np.float64))
            root_value = b.broadcast_bytes(b"R%d" % rank, root=world - 1)
            mx = b.reduce_max(float(rank))
            all_ok = b.all_true(rank != 1)
            # descriptor passing: every rank shares a pipe's read end; everyone writes to everyone
            rd, wr = os.pipe()
            os.write(wr, b"from%d" % rank)
            fds = b.allgather_fd(rd)
            seen = [os.read(fd, 16) for fd in fds] if rank == 0 else None
            b.barrier()
            for fd in fds:
                os.close(fd)
            q.put((rank, dict(gathered=[g[0] for g in gathered], arr=arr.tolist(), root=root_value, mx=mx, all_ok=all_ok,
                              seen=seen)))
    except Exception as ex:  # noqa: BLE001
        q.put((rank, repr(ex)))


@pytest.mark.parametrize("world", [1, 2, 4])
def test_collectives(world):
    res = _run(_collectives, world)
    assert sorted(res) == list(range(world)), res
    for rank, r in res.items():
        assert isinstance(r, dict), r
        assert r["gathered"] == list(range(world))
        assert r["arr"] == [[k * 1.5, float(k)] for k in range(world)]
        assert r["root"] == b"R%d" % (world - 1)
        assert r["mx"] == world - 1
        assert r["all_ok"] == (world < 2)
    if world > 1:
        assert sorted(res[0]["seen"]) == sorted(b"from%d" % k for k in range(world))


def _missing_rank(rank, world, session, q):
    from mnnvl_sharp_b200.parallel import Bootstrap

    if rank == world - 1:
        q.put((rank, "stayed away"))
        return
    t0 = time.time()
    try:
        Bootstrap(rank, world, session, timeout_ms=1500)
        q.put((rank, "connected?!"))
    except Exception as ex:  # noqa: BLE001
        q.put((rank, (str(ex), time.time() - t0)))


def test_rank_that_never_joins_times_out_everyone():
    res = _run(_missing_rank, 3)
    msg0, dt0 = res[0]
    assert "timed out waiting for rank(s) 2 to join" in msg0 and dt0 < 5
    msg1, dt1 = res[1]
    assert ("timed out" in msg1 or "lost the connection" in msg1) and dt1 < 8


def _dies_midway(rank, world, session, q):
    from mnnvl_sharp_b200.parallel import Bootstrap

    b = Bootstrap(rank, world, session, timeout_ms=5000)
    b.barrier()
    if rank == 1:
        os._exit(0)  # leaves between two collectives without saying goodbye
    t0 = time.time()
    try:
        b.barrier()
        q.put((rank, "passed?!"))
    except Exception as ex:  # noqa: BLE001
        q.put((rank, (str(ex), time.time() - t0)))


def test_rank_that_exits_is_reported_by_name_without_waiting_for_the_deadline():
    res = _run(_dies_midway, 3)
    msg0, dt0 = res[0]
    assert "lost the connection to rank 1" in msg0 and dt0 < 3
    msg2, dt2 = res[2]
    assert "rank 1" in msg2 and dt2 < 3


def _abort(rank, world, session, q):
    from mnnvl_sharp_b200.parallel import Bootstrap

    b = Bootstrap(rank, world, session, timeout_ms=5000)
    b.barrier()
    if rank == 2:
        b.abort("GPU 2 lacks multicast")
        q.put((rank, "aborted"))
        return
    try:
        b.barrier()
        q.put((rank, "passed?!"))
    except Exception as ex:  # noqa: BLE001
        q.put((rank, str(ex)))


def test_abort_reaches_every_rank_with_its_reason():
    res = _run(_abort, 3)
    assert "rank 2 aborted: GPU 2 lacks multicast" in res[0]
    assert "rank 2 aborted: GPU 2 lacks multicast" in res[1]


def _mismatch(rank, world, session, q):
    from mnnvl_sharp_b200.parallel import Bootstrap

    b = Bootstrap(rank, world, session, timeout_ms=3000)
    try:
        if rank == 0:
            b.barrier()
        else:
            b.allgather_bytes(b"x" * 8)
        q.put((rank, "passed?!"))
    except Exception as ex:  # noqa: BLE001
        q.put((rank, str(ex)))


def test_collective_mismatch_is_an_error_not_a_hang():
    res = _run(_mismatch, 2)
    assert "collective mismatch" in res[0]
    assert "collective mismatch" in res[1] or "lost the connection" in res[1] or "rank 0" in res[1]


def _hub_with_stranger(rank, world, session, q):
    from mnnvl_sharp_b200.parallel import Bootstrap

    if rank == 1:
        # a stranger connects first and sends garbage; the hub must drop it and still accept rank 1
        time.sleep(0.3)
        s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        s.connect("\0msharp." + session)
        s.sendall(struct.pack("<IIIiQ", 0xBAD, 1, 0, 1, 2))
        time.sleep(0.2)
        s.close()
    with Bootstrap(rank, world, session, timeout_ms=8000) as b:
        b.barrier()
        q.put((rank, "ok"))


def test_hub_ignores_a_stranger_with_a_bad_hello():
    assert _run(_hub_with_stranger, 2) == {0: "ok", 1: "ok"}


# ------------------------------------------------------------------------------- symmetric memory
def _symm(rank, world, session, q, fail_call, fail_rank, fail_nth, fail_code, multicast):
    from mnnvl_sharp_b200 import _native as N
    from mnnvl_sharp_b200.parallel import Bootstrap, Communicator

    N.lib.msharp_fake_driver_reset(8)
    if not multicast:
        N.lib.msharp_fake_driver_set_attribute(132, 0)  # CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED
    out = {}
    try:
        with Bootstrap(rank, world, session, timeout_ms=20000) as b:
            comm = Communicator(b, rank, fake_driver=True)
            out["info"] = comm.info()
            if fail_call and rank == fail_rank:
                N.lib.msharp_fake_driver_fail_call(fail_call.encode(), fail_nth, fail_code)
            try:
                buf = comm.alloc(3 << 20, layout="input_output")
                out["symm"] = buf.info
                out["slots"] = [buf.input_ptr(r) - buf.input_ptr(0) for r in range(world)]
                buf.canary_check()
                # peers' memory is really shared: read what rank r wrote into its own slot
                buf.write(np.full(64, 100 + rank, dtype=np.uint8), offset=4096, region="output")
                b.barrier()
                out["peer_bytes"] = [int(buf.read(1, offset=4096, slot_rank=r)[0]) for r in range(world)]
                b.barrier()
                buf.free()
            except Exception as ex:  # noqa: BLE001
                out["alloc_error"] = str(ex)
            comm.close()
            leaks = (N.ctypes.c_int * 4)()
            N.lib.msharp_fake_driver_leaks(leaks)
            out["leaks"] = list(leaks)
            out["log"] = N.as_json(N.lib.msharp_fake_driver_log())
    except Exception as ex:  # noqa: BLE001
        out["error"] = repr(ex)
    q.put((rank, out))


@pytest.mark.parametrize("world", [1, 2, 4])
def test_symmetric_memory_set_up_and_teardown(world):
    res = _run(_symm, world, "", 0, 0, 0, True)
    assert sorted(res) == list(range(world))
    for rank, r in res.items():
        assert "error" not in r and "alloc_error" not in r, r
        s = r["symm"]
        assert s["payload_bytes"] == 3 << 20 and s["allocation_bytes"] == 8 << 20  # two regions of 4 MiB
        assert s["input_offset"] == 0 and s["output_offset"] == 4 << 20
        assert s["handle_type"] == ("none" if world == 1 else "posix_fd")
        assert s["multicast_bytes"] == (0 if world == 1 else 4 << 20) and s["multicast_bound"] == (world > 1)
        assert len(s["peer_init_local_ms_by_rank"]) == world and s["peer_init_ms"] == max(s["peer_init_local_ms_by_rank"])
        assert r["slots"] == [k * (8 << 20) for k in range(world)]
        assert r["peer_bytes"] == [100 + k for k in range(world)]
        assert r["leaks"] == [0, 0, 0, 0], r["leaks"]
        names = [line.split("(")[0] for line in r["log"]]
        data = names[names.index("cuMemCreate", names.index("cuMemCreate") + 1):]  # calls of the data buffer
        # the reference's order: create, (timed) export / import / reserve / map+access per slot, then multicast
        assert data[0] == "cuMemCreate"
        if world > 1:
            assert data.index("cuMemExportToShareableHandle") < data.index("cuMemImportFromShareableHandle")
            assert data.index("cuMemImportFromShareableHandle") < data.index("cuMemAddressReserve") < data.index("cuMemMap")
            assert data.count("cuMemImportFromShareableHandle") >= world - 1
            assert data.index("cuMulticastAddDevice") < data.index("cuMulticastBindMem")
            tail = data[data.index("cuMulticastBindMem"):]
            # teardown: alias unmapped, unbound, slots unmapped, imported handles and own handle released
            assert tail.index("cuMulticastUnbind") < len(tail) - 1 - tail[::-1].index("cuMemRelease")
            assert tail.index("cuMemUnmap") < tail.index("cuMulticastUnbind")


@pytest.mark.parametrize("call,nth,code,expect", [
    ("cuMemImportFromShareableHandle", 1, CUDA_ERROR_NOT_SUPPORTED, "cuMemImportFromShareableHandle"),
    ("cuMemExportToShareableHandle", 1, CUDA_ERROR_NOT_PERMITTED, "cuMemExportToShareableHandle"),
    ("cuMulticastBindMem", 1, CUDA_ERROR_OUT_OF_MEMORY, "multicast bind"),
    ("cuMemMap", 2, CUDA_ERROR_OUT_OF_MEMORY, "peer mapping"),
    ("cuMulticastCreate", 1, CUDA_ERROR_NOT_SUPPORTED, "multicast"),
])
def test_a_driver_failure_on_one_rank_fails_all_ranks_together_and_leaks_nothing(call, nth, code, expect):
    fail_rank = 0 if call == "cuMulticastCreate" else 1
    res = _run(_symm, 3, call, fail_rank, nth, code, True)
    assert sorted(res) == [0, 1, 2], res
    for rank, r in res.items():
        assert "error" not in r, r
        assert "alloc_error" in r, (rank, r)
        assert r["leaks"] == [0, 0, 0, 0], (rank, r["leaks"])
    assert expect in res[fail_rank]["alloc_error"]
    others = [res[k]["alloc_error"] for k in res if k != fail_rank]
    assert all("another rank" in e or "rank 0 could not" in e or "shared no handle" in e or expect in e for e in others), others


def test_no_multicast_support_still_gives_unicast_slots():
    res = _run(_symm, 2, "", 0, 0, 0, False)
    for r in res.values():
        assert "alloc_error" not in r and "error" not in r, r
        assert r["info"]["multicast"] is False and r["symm"]["multicast_bytes"] == 0
        assert r["peer_bytes"] == [100, 101]
