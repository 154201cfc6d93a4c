"""Data-parallel gradient averaging on symmetric memory.

Gradients are packed into one symmetric bucket (BF16 or FP16), summed in place with the
in-switch all-reduce (float32 accumulation inside the NVSwitch) and unpacked, scaled by
1 / world. The collective is one kernel launch per bucket on the current stream, so it
overlaps with whatever runs on other streams. The reference project provides only the
collective; this is the data-parallel use it is the primitive for.
"""
from __future__ import annotations

import torch

from ..ops.all_reduce import all_reduce_pull
from ..parallel.symmetric import Communicator


class GradientAllReducer:
    def __init__(self, comm: Communicator, params, dtype: torch.dtype = torch.bfloat16, bucket_bytes: int | None = None):
        self.comm = comm
        self.params = [p for p in params if p.requires_grad]
        self.dtype = dtype
        self.code = {torch.bfloat16: "bf16", torch.float16: "f16"}[dtype]
        total = sum(p.numel() for p in self.params)
        nbytes = ((total * 2 + 15) // 16) * 16
        self.nbytes = max(nbytes, 16) if bucket_bytes is None else max(bucket_bytes, nbytes)
        self.bucket = comm.alloc(self.nbytes, layout="single", multicast=True)
        self.flat = self.bucket.tensor(dtype)[: self.nbytes // 2]
        self.flat.zero_()

    @torch.no_grad()
    def step(self) -> None:
        """Average `.grad` of all parameters over the ranks (in place)."""
        offset = 0
        for p in self.params:
            n = p.numel()
            if p.grad is None:
                self.flat[offset:offset + n].zero_()
            else:
                self.flat[offset:offset + n].copy_(p.grad.reshape(-1))
            offset += n
        all_reduce_pull(self.comm, self.bucket, self.code, nbytes=self.nbytes)
        offset = 0
        scale = 1.0 / self.comm.world
        for p in self.params:
            n = p.numel()
            if p.grad is not None:
                p.grad.copy_((self.flat[offset:offset + n].float() * scale).reshape(p.grad.shape))
            offset += n

    def free(self) -> None:
        self.flat = None
        self.bucket.free()
