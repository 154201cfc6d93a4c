"""Zero-copy torch tensors over raw device pointers (symmetric memory is allocated by the
driver's virtual memory API, not by torch's caching allocator)."""
from __future__ import annotations

import torch

_TYPESTR = {
    torch.uint8: "|u1", torch.int8: "|i1", torch.float16: "<f2", torch.float32: "<f4", torch.int32: "<i4",
    torch.int64: "<i8", torch.uint16: "<u2",
}


class _CudaArray:
    def __init__(self, ptr: int, nbytes: int, owner):
        self.owner = owner  # keeps the allocation alive as long as the tensor
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


def device_tensor(ptr: int, nbytes: int, dtype: torch.dtype, device: int, owner=None) -> torch.Tensor:
    raw = torch.as_tensor(_CudaArray(ptr, nbytes, owner), device=torch.device("cuda", device))
    return raw.view(dtype)


def host_tensor(ptr: int, nbytes: int, dtype: torch.dtype, owner=None) -> torch.Tensor:
    """The same for communicators on the host-memory driver stand-in, whose "device" pointers are
    host pointers: a CPU tensor over that memory, without a copy."""
    import ctypes

    array = (ctypes.c_uint8 * nbytes).from_address(ptr)
    array._owner = owner  # torch keeps `array` alive as long as any view of the storage; it keeps the allocation
    return torch.frombuffer(array, dtype=torch.uint8).view(dtype)
