"""GPU parity: iomb_silu / iomb_silu_mul against the oracle.

BF16: bit-identical to the oracle on BOTH carriers (FP32 = the reference CPU
backend, FP64 = the reference GPU backends) for every one of the 65 536 codes.
F32: the kernel evaluates on the FP64 carrier; bit-identical to the oracle's FP64
carrier except where the device's and the C library's double exp differ in their
last bit (at most one F32 ulp, and on well under one element in ten thousand), and
within 4 F32 ulp of the FP32 carrier (the spread between the reference's own CPU
and GPU backends).
"""
import numpy as np
import pytest

from iom_b200.tensor import DataType
from gpu_support import download, gpu, like, run, upload  # noqa: F401
from support import HostTensor, SPECIAL_BF16, SPECIAL_F32, abi, oracle, random_payload

pytestmark = pytest.mark.gpu


def seeded(shape, dtype, rng, scale=4.0, poison=0xA5):
    t = HostTensor(shape, dtype).poison(poison)
    payload = random_payload(rng, shape, dtype, "normal")
    if dtype == DataType.F32:
        payload = (payload * np.float32(scale)).astype(np.float32)
    t.view().copy_from_host(payload)
    return t


def test_silu_every_bf16_code(gpu):
    device, queue = gpu
    codes = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    x = HostTensor((256, 256), DataType.BF16).poison()
    x.view().copy_from_host(codes)
    y = HostTensor((256, 256), DataType.BF16).poison()
    dx, dy = upload(device, x), upload(device, y)
    run(queue, queue.silu(dx.view(), dy.view()))
    got = download(dy)
    for carrier in (0, 1):
        assert oracle().iomo_silu(abi(x.view()), abi(y.view()), carrier) == 0
        assert np.array_equal(got, y.storage), f"carrier {carrier}"
    assert np.array_equal(download(dx), x.storage)


@pytest.mark.parametrize("fused", [False, True])
def test_silu_every_bf16_code_through_the_staged_table(gpu, fused):
    """A request large enough for the shared-memory table path (16 MiB), holding
    every BF16 code 128 times."""
    device, queue = gpu
    codes = np.tile(np.arange(65536, dtype=np.uint16), 128).reshape(8192, 1024)
    x = HostTensor((8192, 1024), DataType.BF16).poison()
    x.view().copy_from_host(codes)
    y = HostTensor((8192, 1024), DataType.BF16).poison()
    dx, dy = upload(device, x), upload(device, y)
    assert oracle().iomo_silu(abi(x.view()), abi(y.view()), 0) == 0
    if not fused:
        run(queue, queue.silu(dx.view(), dy.view()))
        assert np.array_equal(download(dy), y.storage)
        return
    rng = np.random.default_rng(5)
    up = seeded((8192, 1024), DataType.BF16, rng)
    out = HostTensor((8192, 1024), DataType.BF16).poison()
    du, do = upload(device, up), upload(device, out)
    run(queue, queue.silu_mul(dx.view(), du.view(), do.view(), dy.view()))
    assert np.array_equal(download(dy), y.storage)
    assert oracle().iomo_binary(1, abi(y.view()), abi(up.view()), abi(out.view()), 0) == 0
    assert np.array_equal(download(do), out.storage)


@pytest.mark.parametrize("shape", [(1, 1), (15, 17), (17, 33), (2, 3, 16, 31), (64, 2048),
                                   (2, 2, 1, 2, 1, 2, 17, 48), (4096, 2064), (16, 512, 1024)])
def test_silu_bf16_shapes(gpu, shape):
    """Ragged, multi-plane, dense-small (table through L1) and dense-large (table in
    shared memory) requests; padding and other planes stay untouched."""
    device, queue = gpu
    rng = np.random.default_rng(len(shape) * 1000 + shape[-1])
    x, y = seeded(shape, DataType.BF16, rng), seeded(shape, DataType.BF16, rng)
    dx, dy = upload(device, x), upload(device, y)
    run(queue, queue.silu(dx.view(), dy.view()))
    assert oracle().iomo_silu(abi(x.view()), abi(y.view()), 0) == 0
    assert np.array_equal(download(dy), y.storage)


@pytest.mark.parametrize("shape", [(17, 33), (2, 3, 16, 31), (256, 1024)])
def test_silu_f32(gpu, shape):
    device, queue = gpu
    rng = np.random.default_rng(shape[-1])
    x, y = seeded(shape, DataType.F32, rng, scale=8.0), seeded(shape, DataType.F32, rng)
    dx, dy = upload(device, x), upload(device, y)
    run(queue, queue.silu(dx.view(), dy.view()))
    got = download(dy).view(np.uint32).astype(np.int64)
    assert oracle().iomo_silu(abi(x.view()), abi(y.view()), 1) == 0
    fp64 = y.storage.view(np.uint32).astype(np.int64)
    differs = np.abs(got - fp64)
    assert differs.max() <= 1
    assert np.count_nonzero(differs) <= max(1, got.size // 10000)
    assert oracle().iomo_silu(abi(x.view()), abi(y.view()), 0) == 0
    fp32 = y.storage.view(np.uint32).astype(np.int64)
    assert np.abs(got - fp32).max() <= 4


def test_silu_f32_special_values(gpu):
    device, queue = gpu
    extra = np.array([-104.0, -103.0, -90.0, -88.0, -20.0, -1e-30, 1e-30, 20.0, 88.0, 89.0, 3e38,
                      -3e38, 1e-45, -1e-45], dtype=np.float32).view(np.uint32)
    values = np.concatenate([SPECIAL_F32, extra])
    n = values.size
    x = HostTensor((1, n), DataType.F32).poison()
    x.view().copy_from_host(values.reshape(1, n))
    y = HostTensor((1, n), DataType.F32).poison()
    dx, dy = upload(device, x), upload(device, y)
    run(queue, queue.silu(dx.view(), dy.view()))
    assert oracle().iomo_silu(abi(x.view()), abi(y.view()), 1) == 0
    got = download(dy).view(np.uint32).astype(np.int64)
    want = y.storage.view(np.uint32).astype(np.int64)
    assert np.abs(got - want).max() <= 1
    # NaN, infinities and zeros are exact classes, not approximations
    magnitude = want & 0x7FFFFFFF
    exact = (magnitude == 0) | (magnitude >= 0x7F800000)
    assert np.array_equal(got[exact], want[exact])


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
def test_silu_views_and_rejections(gpu, dtype):
    device, queue = gpu
    rng = np.random.default_rng(3)
    x = seeded((3, 2, 17, 33), dtype, rng)
    y = seeded((2, 3, 17, 33), dtype, rng)
    xv = x.view().permute([1, 0])
    yv = y.view()
    dx, dy = upload(device, x), upload(device, y)
    run(queue, queue.silu(like(xv, dx), like(yv, dy)))
    assert oracle().iomo_silu(abi(xv), abi(yv), 1) == 0
    got, want = download(dy), y.storage
    if dtype == DataType.BF16:
        assert np.array_equal(got, want)
    else:
        assert np.abs(got.view(np.uint32).astype(np.int64) - want.view(np.uint32).astype(np.int64)).max() <= 1
    assert queue.silu(dx.view(), dx.view()) == -1                           # in place
    assert queue.silu(dx.view().slice(0, 0, 1), dx.view().slice(0, 1, 1)) == -1   # same owner
    assert queue.silu(dx.view(), dy.view()) == -1                           # shapes differ
    other = device.create_tensor(HostTensor((3, 2, 17, 33), DataType.I32).spec)
    assert queue.silu(other.view(), other.view()) == -1
    i32 = device.create_tensor(HostTensor((3, 2, 17, 33), DataType.I32).spec)
    assert queue.silu(other.view(), i32.view()) == -2                       # leaf not served


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
@pytest.mark.parametrize("shape", [(17, 33), (2, 48, 64), (2048, 5632)])
@pytest.mark.parametrize("store_activated", [False, True])
def test_silu_mul_equals_silu_then_mul(gpu, dtype, shape, store_activated):
    """The fused gate equals iomb_silu followed by iomb_binary(MUL) bit for bit."""
    device, queue = gpu
    rng = np.random.default_rng(shape[-1] + int(dtype))
    x, up = seeded(shape, dtype, rng), seeded(shape, dtype, rng)
    act, out = seeded(shape, dtype, rng), seeded(shape, dtype, rng)
    dx, du = upload(device, x), upload(device, up)
    da, do = upload(device, act), upload(device, out)
    run(queue, queue.silu_mul(dx.view(), du.view(), do.view(), da.view() if store_activated else None))
    da2, do2 = upload(device, act), upload(device, out)
    run(queue, queue.silu(dx.view(), da2.view()))
    run(queue, queue.mul(da2.view(), du.view(), do2.view()))
    assert np.array_equal(download(do), download(do2))
    if store_activated:
        assert np.array_equal(download(da), download(da2))
    else:
        assert np.array_equal(download(da), act.storage)        # untouched
    if dtype == DataType.BF16:
        assert oracle().iomo_silu(abi(x.view()), abi(act.view()), 0) == 0
        assert oracle().iomo_binary(1, abi(act.view()), abi(up.view()), abi(out.view()), 0) == 0
        assert np.array_equal(download(do), out.storage)
    # an output that shares an operand's owner is rejected
    assert queue.silu_mul(dx.view(), du.view(), dx.view()) == -1
    assert queue.silu_mul(dx.view(), du.view(), do.view(), du.view()) == -1
