"""GPU parity: iomb_rope against the oracle, bit-exact.

The angle table is built on the host with the C library's powf / sinf / cosf (the
reference CPU backend's expression), so the CUDA path, the oracle and the reference
CPU backend agree on every bit when they run on the same host."""
import ctypes

import numpy as np
import pytest

from iom_b200.tensor import DataType
from gpu_support import download, gpu, like, run, upload  # noqa: F401
from support import HostTensor, SPECIAL_BF16, SPECIAL_F32, abi, oracle, random_payload

pytestmark = pytest.mark.gpu


def seeded(shape, dtype, rng, specials=True):
    t = HostTensor(shape, dtype).poison()
    payload = random_payload(rng, shape, dtype, "normal")
    if specials:
        special = SPECIAL_F32 if dtype == DataType.F32 else SPECIAL_BF16
        flat = payload.reshape(-1).view(special.dtype)
        count = min(flat.size, special.size)
        flat[:count] = special[:count]
    t.view().copy_from_host(payload)
    return t


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
@pytest.mark.parametrize("shape,a", [
    ((2, 3, 5, 64), 0),            # position 0 row is copied raw
    ((4, 17, 128), 7),
    ((1, 2, 33, 34), 2040),        # half not a multiple of 16: the per-pair kernel
    ((2, 1, 1, 6), 123456),
    ((3, 40, 96), 1),              # half = 48: whole tiles, three per half
    ((2, 8, 512, 64), 1536),       # prefill-like: 16 heads x 512 rows
])
@pytest.mark.parametrize("theta", [10000.0, 500000.0])
def test_rope_parity(gpu, dtype, shape, a, theta):
    device, queue = gpu
    rng = np.random.default_rng(a + len(shape))
    x, out = seeded(shape, dtype, rng), seeded(shape, dtype, rng, specials=False)
    dx, do = upload(device, x), upload(device, out)
    run(queue, queue.rope(dx.view(), do.view(), a, theta))
    assert oracle().iomo_rope(abi(x.view()), abi(out.view()), a, theta) == 0
    assert np.array_equal(download(do), out.storage)
    assert np.array_equal(download(dx), x.storage)


def test_rope_angle_table_equals_the_oracle(gpu):
    device, _ = gpu
    width, rows, first, theta = 64, 40, 2030, 10000.0
    table = np.empty((rows, width // 2, 2), dtype=np.float32)
    assert device._lib.iomb_rope_angles(table.ctypes.data, first, rows, width, theta) == 0
    sine, cosine = ctypes.c_float(), ctypes.c_float()
    for r in (0, 1, 17, rows - 1):
        for c in (0, 1, 15, 31):
            oracle().iomo_rope_angle(c, width, first + r, np.float32(theta), ctypes.byref(sine),
                                     ctypes.byref(cosine))
            assert table[r, c, 0] == np.float32(cosine.value)
            assert table[r, c, 1] == np.float32(sine.value)


def test_rope_views_and_rejections(gpu):
    device, queue = gpu
    rng = np.random.default_rng(43)
    x = seeded((3, 2, 9, 32), DataType.BF16, rng)
    out = seeded((2, 3, 9, 32), DataType.BF16, rng, specials=False)
    xv = x.view().permute([1, 0])
    dx, do = upload(device, x), upload(device, out)
    run(queue, queue.rope(like(xv, dx), do.view(), 5, 10000.0))
    assert oracle().iomo_rope(abi(xv), abi(out.view()), 5, 10000.0) == 0
    assert np.array_equal(download(do), out.storage)
    assert queue.rope(dx.view(), dx.view(), 0, 10000.0) == -1                 # in place
    assert queue.rope(like(xv, dx), do.view(), 0, 0.5) == -1                  # theta below one
    assert queue.rope(like(xv, dx), do.view(), (1 << 24) - 5, 10000.0) == -1  # position bound
    odd = device.create_tensor(HostTensor((2, 4, 33), DataType.BF16).spec)
    odd2 = device.create_tensor(HostTensor((2, 4, 33), DataType.BF16).spec)
    assert queue.rope(odd.view(), odd2.view(), 0, 10000.0) == -1              # odd width
    flat = device.create_tensor(HostTensor((4, 32), DataType.BF16).spec)
    flat2 = device.create_tensor(HostTensor((4, 32), DataType.BF16).spec)
    assert queue.rope(flat.view(), flat2.view(), 0, 10000.0) == -1            # rank two
    i32 = device.create_tensor(HostTensor((2, 4, 32), DataType.I32).spec)
    j32 = device.create_tensor(HostTensor((2, 4, 32), DataType.I32).spec)
    assert queue.rope(i32.view(), j32.view(), 0, 10000.0) == -2               # leaf not served
