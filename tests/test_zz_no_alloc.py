"""iomb_sumsq_static: the sum of squares for callers that may not allocate.

Some hosts of the library cannot hand over scratch memory: an IOM backend hook
is admitted with a {0,1} workspace requirement and the contract forbids native
allocation after device set-up. The static entry point must give the same
result as iomb_sumsq with caller scratch, call after call, although every call
reuses one built-in array that still holds the previous call's partials.
This file is collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

from iom_b200.tensor import DataType
from gpu_support import gpu, upload  # noqa: F401
from support import HostTensor, abi, oracle, random_payload

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_caller_scratch_on_repeated_calls(gpu):
    device, queue = gpu
    lib = device._lib
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(77)
    result = torch.zeros(4, dtype=torch.float32, device=device.torch_device)
    scratch = torch.full((int(lib.iomb_sumsq_scratch_bytes()),), 0x3C, dtype=torch.uint8,
                         device=device.torch_device)
    shapes = [((3, 100, 700), DataType.BF16), ((512, 2048), DataType.BF16), ((17, 33), DataType.F32)]
    for shape, dtype in shapes:
        host = HostTensor(shape, dtype).poison(0xA5)
        host.view().copy_from_host(random_payload(rng, shape, dtype, "normal"))
        dev = upload(device, host)
        view = dev.view().as_abi()
        assert lib.iomb_sumsq(ctypes.byref(view), scratch.data_ptr(), result.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        expected = float(result[0])
        truth = oracle().iomo_sumsq(abi(host.view()))
        assert abs(expected - truth) <= 1e-6 * truth
        # two calls in a row: the second one finds the first one's partials in the array
        for slot in (1, 2):
            rc = lib.iomb_sumsq_static(ctypes.byref(view), result.data_ptr() + 4 * slot, stream)
            assert rc == 0, lib.iomb_last_error()
        torch.cuda.synchronize()
        first, second = float(result[1]), float(result[2])
        assert abs(first - expected) <= 1e-6 * abs(expected)
        assert abs(second - expected) <= 1e-6 * abs(expected)
        assert first == second == expected       # same kernel, same order: identical bits


def test_static_scratch_rejects_oversized_views(gpu):
    device, _ = gpu
    lib = device._lib
    small = device.create_tensor(HostTensor((16, 16), DataType.BF16).spec)
    view = small.view().as_abi()
    # Metadata only: a view of 2^33 elements (nothing is launched for it).
    view.dims[0], view.dims[1] = 1 << 17, 1 << 16
    view.storage_bytes = (1 << 33) * 2
    out = torch.zeros(1, dtype=torch.float32, device=device.torch_device)
    rc = lib.iomb_sumsq_static(ctypes.byref(view), out.data_ptr(),
                               torch.cuda.current_stream().cuda_stream)
    assert rc == 1
    assert b"2^32" in lib.iomb_last_error()
    torch.cuda.synchronize()
