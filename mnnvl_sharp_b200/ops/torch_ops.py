"""The `torch.ops.msharp.*` operator library (csrc/torch/ops.cpp): the same kernels as the
ctypes path, registered with PyTorch's dispatcher so that they can be called from TorchScript-
free Python, captured in CUDA graphs, and found by tools that walk `torch.ops`."""
from __future__ import annotations

from pathlib import Path

import torch

_LIB = Path(__file__).resolve().parent.parent / "_C" / "msharp_torch_ops.so"
_loaded = False


def load() -> None:
    """Load (building it first when missing) the operator library. Idempotent."""
    global _loaded
    if _loaded:
        return
    if not _LIB.exists():
        from .. import _build

        _build.build_native()
        _build.build_torch_ops()
    torch.ops.load_library(str(_LIB))
    _loaded = True


def all_reduce_pull(comm, buf, dtype: str, nbytes: int | None = None, offset: int = 0, acc_f32: bool | None = None,
                    grid: int = 0, block: int = 0, unroll: int = 0) -> None:
    load()
    torch.ops.msharp.all_reduce_pull(comm.handle, buf.handle, dtype, dtype != "e4m3" if acc_f32 is None else acc_f32, offset,
                                     buf.payload_bytes if nbytes is None else nbytes, grid, block, unroll)


def all_reduce_sw_f32(comm, buf, nbytes: int | None = None, offset: int = 0, in_scales=None, out_scale: float = 1.0,
                      grid: int = 0, block: int = 0) -> None:
    load()
    torch.ops.msharp.all_reduce_sw_f32(comm.handle, buf.handle, offset, buf.payload_bytes if nbytes is None else nbytes,
                                       in_scales, out_scale, grid, block)


def all_reduce_bulk_push(comm, buf, dtype: str = "f16", nbytes: int | None = None, offset: int = 0, grid: int = 0) -> None:
    load()
    torch.ops.msharp.all_reduce_bulk_push(comm.handle, buf.handle, dtype, offset,
                                          buf.payload_bytes if nbytes is None else nbytes, grid)


def gemm_allreduce(comm, out_buf, a, a_scales, w, w_scales, reducer_ctas: int = 0) -> None:
    load()
    torch.ops.msharp.gemm_allreduce(comm.handle, out_buf.handle, a, a_scales, w, w_scales, reducer_ctas)


def tensor_from_ptr(ptr: int, nbytes: int, device: int) -> torch.Tensor:
    load()
    return torch.ops.msharp.tensor_from_ptr(ptr, nbytes, device)
