"""The allocation-free replica hash (msharp_hash_no_alloc), called through its exported C symbol.

The function exists for callers that may not allocate device memory while they run: a process
whose memory is entirely owned by its own pool, or a checker running beside a job in flight that
must not make the device wait. The test therefore prepares every buffer up front with PyTorch
(input, the two result words) and then only passes pointers; the function under test gets no
chance to allocate on the caller's behalf. It is compared with the regular entry point
(msharp_hash_device), whose hash must be identical bit for bit, on two calls in a row with
different data, so that state left in the built-in scratch array by the first call would show.
This file sorts last on purpose: a failure here stops a `-x` run only after everything else ran.
"""
import ctypes

import pytest

from mnnvl_sharp_b200 import _native as N

lib = N.lib
lib.msharp_hash_no_alloc.restype = ctypes.c_int
lib.msharp_hash_no_alloc.argtypes = [ctypes.c_uint64, ctypes.c_size_t, ctypes.c_uint64, ctypes.c_uint64]
lib.msharp_no_alloc_last_error.restype = ctypes.c_char_p
MAX_BYTES = 4 << 30


def test_refuses_bad_arguments_before_touching_the_gpu():
    assert lib.msharp_hash_no_alloc(0x1000, MAX_BYTES + 4, 0x2000, 0) != 0
    assert b"exceed" in lib.msharp_no_alloc_last_error()
    assert lib.msharp_hash_no_alloc(0x1000, 6, 0x2000, 0) != 0
    assert b"multiple of 4" in lib.msharp_no_alloc_last_error()
    assert lib.msharp_hash_no_alloc(0x1008, 64, 0x2000, 0) != 0
    assert b"aligned" in lib.msharp_no_alloc_last_error()
    assert lib.msharp_hash_no_alloc(0, 64, 0x2000, 0) != 0


@pytest.mark.gpu
def test_matches_the_regular_hash_on_two_calls_in_a_row():
    import torch

    from mnnvl_sharp_b200.utils import numerics as nm

    torch.cuda.set_device(0)
    stream = int(torch.cuda.current_stream().cuda_stream)
    sizes = [(48 << 20) + 20, 4096]  # many blocks with a ragged tail, then a single block
    gen = torch.Generator(device="cuda").manual_seed(7)
    inputs = [torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda", generator=gen) for n in sizes]
    expected = torch.zeros(len(sizes), dtype=torch.int64, device="cuda")
    got = torch.full((len(sizes),), -1, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    for i, x in enumerate(inputs):
        N.check(lib.msharp_hash_device(x.data_ptr(), x.numel(), expected[i:].data_ptr(), stream))
    # two calls in a row on the same stream, no synchronisation in between
    for i, x in enumerate(inputs):
        rc = lib.msharp_hash_no_alloc(x.data_ptr(), x.numel(), got[i:].data_ptr(), stream)
        assert rc == 0, lib.msharp_no_alloc_last_error()
    torch.cuda.synchronize()
    assert got.tolist() == expected.tolist()
    host = nm.hash_words(inputs[1].cpu().numpy())
    assert (int(got[1].item()) & 0xFFFFFFFFFFFFFFFF) == host
    # and once more after a synchronisation: the array was left ready for reuse
    got.fill_(-1)
    rc = lib.msharp_hash_no_alloc(inputs[0].data_ptr(), inputs[0].numel(), got.data_ptr(), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(got[0].item()) == int(expected[0].item())
