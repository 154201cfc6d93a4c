"""All-reduce a symmetric tensor in the NVSwitch, one process per GPU.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/allreduce_torchrun.py

Every rank fills its copy of a symmetric FP16 buffer with its rank number + 1, the in-switch
all-reduce sums the copies in place, and every rank ends up with world * (world + 1) / 2
everywhere. The kernel synchronises with its peers on the device, so the only host-side
synchronisation here is the one that makes the inputs visible before the launch.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mnnvl_sharp_b200 import ops  # noqa: E402
from mnnvl_sharp_b200.parallel import Bootstrap, Communicator  # noqa: E402


def main() -> int:
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    boot = Bootstrap.from_env()                      # RANK / WORLD_SIZE / MASTER_PORT from torchrun
    comm = Communicator(boot, local_rank)
    buf = comm.alloc(64 << 20)                       # 64 MiB per rank, with a multicast alias when world > 1
    x = buf.tensor(torch.float16)                    # zero-copy view of this rank's copy
    x.fill_(float(comm.rank + 1))
    torch.cuda.synchronize()
    boot.barrier()                                   # every rank's input is in place

    ops.all_reduce(comm, buf, "f16", backend="pull")  # one kernel on the current stream
    torch.cuda.synchronize()
    comm.raise_if_failed("all-reduce")               # a peer that never arrived shows up here, not as a hang

    want = comm.world * (comm.world + 1) / 2
    ok = bool((x == want).all().item())
    print(f"rank {comm.rank}: {'ok' if ok else 'WRONG'} (every element == {want})", flush=True)
    boot.barrier()
    del x
    comm.close()
    boot.close()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
