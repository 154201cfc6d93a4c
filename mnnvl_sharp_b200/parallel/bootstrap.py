"""Control plane between the rank processes (socket hub in the native library): Unix-domain
sockets on one host, TCP to rank 0 when an address is given (jobs that span hosts).

It does what MPI does for the reference project (handle exchange, barriers, small reductions;
call sites listed in the reference at src/fabric_memory.cc:111-169 and src/main.cc:91-195) and
can pass file descriptors between processes of one host, which the POSIX-FD memory handles need
(over TCP `can_pass_fds` is false and symmetric memory uses fabric handles).
Every call is collective, has a deadline, and raises `NativeError` naming the rank that failed.
"""
from __future__ import annotations

import ctypes

import numpy as np

from .. import _native as N


class Bootstrap:
    def __init__(self, rank: int, world: int, session: str = "default", timeout_ms: int = 30000,
                 address: str | None = None):
        self.rank = rank
        self.world = world
        self.session = session
        self.address = address or ""
        self._h = N.pointer(N.lib.msharp_bootstrap_connect_address(rank, world, session.encode(),
                                                                   self.address.encode(), timeout_ms))

    @classmethod
    def from_env(cls, timeout_ms: int = 60000) -> "Bootstrap":
        """Rank and world size as exported by torchrun (RANK / WORLD_SIZE), mpirun, a PMI launcher or
        srun; session from MSHARP_SESSION, else MASTER_PORT, else the Slurm / Open MPI job id.
        MSHARP_HUB_ADDR=host:port selects TCP (rank 0 listens on that port; needed only when the
        ranks are on more than one host). The rules live in the native library so that the
        benchmark binary and this package agree."""
        opt = N.as_json(N.lib.msharp_bootstrap_env_options())
        return cls(opt["rank"], opt["world"], opt["session"], timeout_ms, opt["address"] or None)

    @classmethod
    def from_process_group(cls, group=None, timeout_ms: int = 60000, address: str | None = None) -> "Bootstrap":
        """Join through an initialised `torch.distributed` process group (any backend; gloo on CPU
        hosts): rank 0 of the group picks a fresh session name and broadcasts it, so nothing has
        to be agreed out of band. `address` as in the constructor."""
        import uuid

        import torch.distributed as dist

        rank = dist.get_rank(group)
        world = dist.get_world_size(group)
        box = [uuid.uuid4().hex[:16] if rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls(rank, world, "pg" + box[0], timeout_ms, address)

    @classmethod
    def reform(cls, session: str, old_rank: int, old_world: int, hub_old_rank: int = 0, census_ms: int = 2000,
               timeout_ms: int = 30000, address: str | None = None) -> "Bootstrap":
        """Re-form the control plane among the ranks that are left after a failure.

        Every survivor calls this with the same NEW session name (for instance the old one plus a
        generation number) and its old rank. The survivor with old rank `hub_old_rank` takes a census
        for `census_ms` milliseconds (or until all `old_world` ranks have joined); those who joined get
        dense new ranks (the hub 0, then by old rank) and the new world size, available as `.rank` /
        `.world` of the result. Communicators and symmetric buffers of the old job are not carried
        over: build new ones on the new control plane (the old ones refer to the lost rank's memory)."""
        self = cls.__new__(cls)
        new_rank = ctypes.c_int(-1)
        new_world = ctypes.c_int(0)
        self.session = session
        self.address = address or ""
        self._h = N.pointer(N.lib.msharp_bootstrap_reform(session.encode(), self.address.encode(), old_rank, old_world,
                                                          hub_old_rank, census_ms, timeout_ms, ctypes.byref(new_rank),
                                                          ctypes.byref(new_world)))
        self.rank = new_rank.value
        self.world = new_world.value
        return self

    @property
    def can_pass_fds(self) -> bool:
        return bool(N.lib.msharp_bootstrap_can_pass_fds(self._h))

    @property
    def handle(self) -> int:
        return self._h

    def barrier(self) -> None:
        N.check(N.lib.msharp_bootstrap_barrier(self._h))

    def allgather_bytes(self, payload: bytes) -> list[bytes]:
        send = ctypes.create_string_buffer(payload, len(payload))
        recv = ctypes.create_string_buffer(len(payload) * self.world)
        N.check(N.lib.msharp_bootstrap_allgather(self._h, send, recv, len(payload)))
        raw = recv.raw
        return [raw[i * len(payload):(i + 1) * len(payload)] for i in range(self.world)]

    def allgather_array(self, value: np.ndarray) -> np.ndarray:
        value = np.ascontiguousarray(value)
        out = np.empty((self.world,) + value.shape, dtype=value.dtype)
        N.check(N.lib.msharp_bootstrap_allgather(self._h, value.ctypes.data, out.ctypes.data, value.nbytes))
        return out

    def allgather_float(self, value: float) -> list[float]:
        return [float(v) for v in self.allgather_array(np.array([value], dtype=np.float64))[:, 0]]

    def reduce_max(self, value: float) -> float:
        return max(self.allgather_float(value))

    def all_true(self, value: bool) -> bool:
        return all(v != 0.0 for v in self.allgather_float(1.0 if value else 0.0))

    def broadcast_bytes(self, payload: bytes, root: int = 0) -> bytes:
        buf = ctypes.create_string_buffer(payload, len(payload))
        N.check(N.lib.msharp_bootstrap_broadcast(self._h, buf, len(payload), root))
        return buf.raw

    def allgather_fd(self, fd: int) -> list[int]:
        out = (ctypes.c_int * self.world)()
        N.check(N.lib.msharp_bootstrap_allgather_fd(self._h, fd, out))
        return list(out)

    def abort(self, reason: str) -> None:
        if self._h:
            N.lib.msharp_bootstrap_abort(self._h, reason.encode())

    def close(self) -> None:
        if self._h:
            N.lib.msharp_bootstrap_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        if exc is not None:
            self.abort(str(exc))
        self.close()
