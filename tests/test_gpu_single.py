"""Single-GPU tests of the native kernels against the host oracle (world of one rank)."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def comm():
    import torch

    from mnnvl_sharp_b200.parallel import Bootstrap, Communicator

    torch.cuda.set_device(0)
    boot = Bootstrap(0, 1, session=f"t{os.getpid()}")
    c = Communicator(boot, 0)
    yield c
    c.close()
    boot.close()


@pytest.mark.parametrize("dtype", ["e4m3", "f16", "bf16"])
@pytest.mark.parametrize("pattern", ["reference", "seeded", "tagged"])
@pytest.mark.parametrize("nbytes", [4096, 65540, 1 << 20])
def test_device_init_matches_host_generator(comm, dtype, pattern, nbytes):
    import torch

    from mnnvl_sharp_b200 import ops
    from mnnvl_sharp_b200.utils import numerics as nm

    buf = comm.alloc(nbytes)
    ops.poison_fill(buf.output_ptr(), nbytes)
    ops.init_pattern(buf, dtype, pattern, 3, nbytes, seed=77)
    torch.cuda.synchronize()
    got = buf.read(nbytes).view(nm.storage_dtype(dtype))
    want = nm.generate(dtype, pattern, 3, got.size, seed=77)
    assert np.array_equal(got, want)
    assert ops.device_hash(buf.output_ptr(), nbytes) == nm.hash_words(want)
    buf.free()


@pytest.mark.parametrize("backend,dtype,layout", [("legacy", "e4m3", "single"), ("pull", "f16", "single"),
                                                  ("pull", "bf16", "single"), ("sw_f32", "e4m3", "single"),
                                                  ("tma_async", "f16", "input_output"),
                                                  ("tma_async", "bf16", "input_output")])
@pytest.mark.parametrize("nbytes", [16, 4096, 100000 * 16, (8 << 20) + 16])
def test_single_rank_allreduce_is_identity(comm, backend, dtype, layout, nbytes):
    import torch

    from mnnvl_sharp_b200 import ops
    from mnnvl_sharp_b200.utils import numerics as nm

    buf = comm.alloc(nbytes, layout=layout)
    buf.canary_check()
    ops.poison_fill(buf.output_ptr(), nbytes)
    ops.init_pattern(buf, dtype, "seeded", 0, nbytes)
    ops.all_reduce(comm, buf, dtype, backend=backend)
    torch.cuda.synchronize()
    comm.raise_if_failed(backend)
    got = buf.read(nbytes).view(nm.storage_dtype(dtype))
    m = nm.compare(dtype, "seeded", 1, got)
    assert m.max_requantized_ulp_distance == 0 and m.max_abs_error == 0.0
    buf.free()


def test_sw_f32_scales(comm):
    import torch

    from mnnvl_sharp_b200 import ops
    from mnnvl_sharp_b200.utils import numerics as nm

    nbytes = 1 << 16
    buf = comm.alloc(nbytes)
    ops.init_pattern(buf, "e4m3", "seeded", 0, nbytes)
    scales = torch.tensor([0.5], dtype=torch.float32, device="cuda")
    ops.all_reduce_sw_f32(comm, buf, in_scales=scales, out_scale=0.25)
    torch.cuda.synchronize()
    got = nm.decode("e4m3", buf.read(nbytes))
    x = nm.decode("e4m3", nm.generate("e4m3", "seeded", 0, nbytes))
    want = nm.decode("e4m3", nm.encode("e4m3", (x * np.float32(0.5)) * np.float32(4.0)))
    assert np.array_equal(got, want)
    buf.free()


def test_tensor_view_roundtrip(comm):
    import torch

    buf = comm.alloc(1 << 16)
    t = buf.tensor(torch.float16)
    t.copy_(torch.arange(t.numel(), dtype=torch.float32, device="cuda").remainder(100).to(torch.float16))
    torch.cuda.synchronize()
    host = buf.read(1 << 16).view(np.float16)
    assert host[5] == 5 and host[199] == 99
    del t
    buf.free()
