"""GPU parity: iomb_binary against the oracle, bit-exact on physical storage."""
import numpy as np
import pytest

from iom_b200.tensor import DataType
from gpu_support import download, gpu, like, run, upload  # noqa: F401
from support import (HostTensor, SPECIAL_BF16, SPECIAL_F32, abi, oracle, random_payload)

pytestmark = pytest.mark.gpu
OPS = {"add": 0, "mul": 1, "sub": 2, "div": 3}
DTYPES = [DataType.I32, DataType.U32, DataType.F32, DataType.BF16,
          # per-element kernel: the other byte-multiple integers and F16
          DataType.I8, DataType.U8, DataType.I16, DataType.U16, DataType.I64, DataType.U64, DataType.F16,
          DataType.F8_E4M3FN, DataType.F8_E5M2,
          # one thread per tile row: the leaves narrower than a byte
          DataType.I2, DataType.U2, DataType.I4, DataType.U4, DataType.F4_E2M1, DataType.F6_E2M3,
          DataType.F6_E3M2]
INTEGERS = (DataType.I8, DataType.U8, DataType.I16, DataType.U16, DataType.I32, DataType.U32,
            DataType.I64, DataType.U64, DataType.I2, DataType.U2, DataType.I4, DataType.U4)

CASES = [
    ((2, 17, 33), (2, 17, 33), (2, 17, 33)),
    ((2, 1, 33), (1, 17, 1), (2, 17, 33)),
    ((64, 256), (64, 256), (64, 256)),
    ((4, 32, 48), (4, 32, 48), (4, 32, 48)),
    ((32, 48), (1, 48), (32, 48)),
    ((32, 48), (32, 1), (32, 48)),
    ((1, 1), (3, 20, 35), (3, 20, 35)),
    ((2, 3, 16, 16), (3, 1, 16), (2, 3, 16, 16)),
    ((5, 31), (1, 1), (5, 31)),
    ((1, 15), (1, 15), (1, 15)),
    ((17, 1), (17, 1), (17, 1)),
    ((2, 1, 2, 1, 2, 1, 16, 17), (1, 3, 1, 2, 1, 2, 1, 17), (2, 3, 2, 2, 2, 2, 16, 17)),
    # tile-multiple extents with one broadcast row / column plane: the linear-stream
    # broadcast kernel (power-of-two and other tile-column counts, either operand
    # small, several result planes, chunk tails).
    ((64, 128), (1, 128), (64, 128)),
    ((64, 128), (64, 1), (64, 128)),
    ((1, 48), (160, 48), (160, 48)),
    ((160, 1), (160, 48), (160, 48)),
    ((3, 48, 80), (1, 80), (3, 48, 80)),
    ((3, 48, 80), (48, 1), (3, 48, 80)),
    ((1, 1, 256), (5, 32, 256), (5, 32, 256)),
    ((1, 32, 1), (5, 32, 256), (5, 32, 256)),
    ((2, 2, 32, 32), (1, 32), (2, 2, 32, 32)),
    ((528, 512), (1, 512), (528, 512)),
    ((528, 512), (528, 1), (528, 512)),
]


def check(queue, device, op, lhs, rhs, out, lv=None, rv=None, ov=None):
    lv = lv or lhs.view()
    rv = rv or rhs.view()
    ov = ov or out.view()
    dl, dr, do = upload(device, lhs), upload(device, rhs), upload(device, out)
    run(queue, getattr(queue, op)(like(lv, dl), like(rv, dr), like(ov, do)))
    assert oracle().iomo_binary(OPS[op], abi(lv), abi(rv), abi(ov), 0) == 0
    assert np.array_equal(download(do), out.storage)
    # inputs untouched
    assert np.array_equal(download(dl), lhs.storage)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("op", ["add", "mul", "sub", "div"])
@pytest.mark.parametrize("shapes", CASES)
def test_binary_parity(gpu, dtype, op, shapes):
    device, queue = gpu
    if op == "div" and dtype in INTEGERS:
        pytest.skip("integer division is rejected (test_binary_rejections)")
    rng = np.random.default_rng(abs(hash((int(dtype), op, shapes))) & 0xFFFF)
    tensors = []
    for shape in shapes:
        t = HostTensor(shape, dtype).poison(0xA5)
        t.view().copy_from_host(random_payload(rng, shape, dtype))
        tensors.append(t)
    check(queue, device, op, *tensors)


@pytest.mark.parametrize("dtype,specials", [(DataType.F32, SPECIAL_F32), (DataType.BF16, SPECIAL_BF16)])
@pytest.mark.parametrize("op", ["add", "mul", "sub", "div"])
def test_binary_special_values(gpu, dtype, op, specials):
    device, queue = gpu
    n = len(specials)
    lhs, rhs, out = (HostTensor((n, n), dtype).poison(0x5A) for _ in range(3))
    lhs.view().copy_from_host(np.repeat(specials, n).reshape(n, n))
    rhs.view().copy_from_host(np.tile(specials, n).reshape(n, n))
    check(queue, device, op, lhs, rhs, out)


def test_binary_exhaustive_bf16_pairs(gpu):
    """Every BF16 code against 512 boundary-rich codes, all four operations."""
    device, queue = gpu
    a = np.arange(65536, dtype=np.uint16)
    mant = np.array([0, 1, 2, 0x3F, 0x40, 0x41, 0x7E, 0x7F], dtype=np.uint16)
    exps = np.array([0, 1, 2, 63, 64, 126, 127, 128, 129, 191, 192, 253, 254, 255, 120, 134],
                    dtype=np.uint16)
    b = np.array([(s << 15) | (e << 7) | m for s in (0, 1) for e in exps for m in mant],
                 dtype=np.uint16)
    b = np.concatenate([b, b])[:512]
    lhs = HostTensor((65536, 512), DataType.BF16)
    rhs = HostTensor((65536, 512), DataType.BF16)
    out = HostTensor((65536, 512), DataType.BF16)
    lhs.view().copy_from_host(np.repeat(a, 512).reshape(65536, 512))
    rhs.view().copy_from_host(np.tile(b, 65536).reshape(65536, 512))
    for op in ("add", "mul", "sub", "div"):
        dl, dr, do = upload(device, lhs), upload(device, rhs), upload(device, out)
        run(queue, getattr(queue, op)(dl.view(), dr.view(), do.view()))
        assert oracle().iomo_binary(OPS[op], abi(lhs.view()), abi(rhs.view()), abi(out.view()), 1) == 0
        assert np.array_equal(download(do), out.storage)
        for t in (dl, dr, do):
            t.close()


def test_binary_exhaustive_f16_pairs(gpu):
    """Every F16 code against 192 boundary-rich codes, all four operations."""
    device, queue = gpu
    a = np.arange(65536, dtype=np.uint16)
    mant = np.array([0, 1, 2, 0x1FF, 0x200, 0x201, 0x3FE, 0x3FF], dtype=np.uint16)
    exps = np.array([0, 1, 2, 14, 15, 16, 29, 30, 31, 10, 20, 25], dtype=np.uint16)
    b = np.array([(s << 15) | (e << 10) | m for s in (0, 1) for e in exps for m in mant],
                 dtype=np.uint16)
    lhs = HostTensor((65536, 192), DataType.F16)
    rhs = HostTensor((65536, 192), DataType.F16)
    out = HostTensor((65536, 192), DataType.F16)
    lhs.view().copy_from_host(np.repeat(a, 192).reshape(65536, 192))
    rhs.view().copy_from_host(np.tile(b, 65536).reshape(65536, 192))
    for op in ("add", "mul", "sub", "div"):
        dl, dr, do = upload(device, lhs), upload(device, rhs), upload(device, out)
        run(queue, getattr(queue, op)(dl.view(), dr.view(), do.view()))
        assert oracle().iomo_binary(OPS[op], abi(lhs.view()), abi(rhs.view()), abi(out.view()), 1) == 0
        assert np.array_equal(download(do), out.storage)
        for t in (dl, dr, do):
            t.close()


@pytest.mark.parametrize("dtype", [DataType.F8_E4M3FN, DataType.F8_E5M2])
def test_binary_every_f8_pair(gpu, dtype):
    """All 65 536 pairs of an 8-bit floating leaf, all four operations, against the codec."""
    device, queue = gpu
    codes = np.arange(256, dtype=np.uint8)
    lhs, rhs, out = (HostTensor((256, 256), dtype) for _ in range(3))
    lhs.view().copy_from_host(np.repeat(codes, 256).reshape(256, 256))
    rhs.view().copy_from_host(np.tile(codes, 256).reshape(256, 256))
    for op in ("add", "mul", "sub", "div"):
        dl, dr, do = upload(device, lhs), upload(device, rhs), upload(device, out)
        run(queue, getattr(queue, op)(dl.view(), dr.view(), do.view()))
        assert oracle().iomo_binary(OPS[op], abi(lhs.view()), abi(rhs.view()), abi(out.view()), 0) == 0
        assert np.array_equal(download(do), out.storage), op
        for t in (dl, dr, do):
            t.close()


def test_binary_views_and_alias(gpu):
    device, queue = gpu
    rng = np.random.default_rng(7)
    lhs = HostTensor((4, 3, 17, 33), DataType.F32).poison()
    rhs = HostTensor((3, 4, 17, 33), DataType.F32).poison()
    out = HostTensor((2, 3, 17, 33), DataType.F32).poison()
    for t in (lhs, rhs, out):
        t.view().copy_from_host(random_payload(rng, t.spec.shape, DataType.F32))
    lv = lhs.view().slice(0, 1, 2, 2)
    rv = rhs.view().permute([1, 0]).slice(0, 0, 2, 1)
    check(queue, device, "add", lhs, rhs, out, lv, rv, out.view())
    # exact in-place alias
    dl, dr = upload(device, lhs), upload(device, rhs)
    big = lhs.view()
    run(queue, queue.mul(like(big, dl), like(rhs.view().permute([1, 0]), dr), like(big, dl)))
    assert oracle().iomo_binary(1, abi(big), abi(rhs.view().permute([1, 0])), abi(big), 0) == 0
    assert np.array_equal(download(dl), lhs.storage)


@pytest.mark.parametrize("dtype", [DataType.F32, DataType.BF16])
def test_binary_broadcast_stream_views(gpu, dtype):
    """Bias add / per-row scale over windows: a dense plane range (offset, unit
    stride) streams linearly, a strided one does not; both must match, and the
    in-place form must leave every plane outside the window untouched."""
    device, queue = gpu
    rng = np.random.default_rng(11 + int(dtype))
    big = HostTensor((6, 32, 64), dtype).poison()
    out = HostTensor((6, 32, 64), dtype).poison()
    row = HostTensor((2, 1, 64), dtype).poison()
    col = HostTensor((32, 1), dtype).poison()
    for t in (big, out, row, col):
        t.view().copy_from_host(random_payload(rng, t.spec.shape, dtype))
    window = big.view().slice(0, 2, 3, 1)
    strided = big.view().slice(0, 0, 3, 2)
    one_row = row.view().slice(0, 1, 1, 1)
    check(queue, device, "add", big, row, out, window, one_row, out.view().slice(0, 1, 3, 1))
    check(queue, device, "mul", col, big, out, col.view(), window, out.view().slice(0, 3, 3, 1))
    check(queue, device, "add", big, row, out, strided, one_row, out.view().slice(0, 0, 3, 2))
    # in place: out is the big operand's own window
    db, dr = upload(device, big), upload(device, row)
    run(queue, queue.add(like(window, db), like(one_row, dr), like(window, db)))
    assert oracle().iomo_binary(0, abi(window), abi(one_row), abi(window), 0) == 0
    assert np.array_equal(download(db), big.storage)


def test_binary_rejections(gpu):
    device, queue = gpu
    a = device.create_tensor(HostTensor((4, 16, 16), DataType.F32).spec)
    b = device.create_tensor(HostTensor((3, 16, 16), DataType.F32).spec)
    c = device.create_tensor(HostTensor((4, 16, 16), DataType.BF16).spec)
    assert queue.add(a.view(), b.view(), a.view()) == -1          # not broadcast compatible
    assert queue.add(a.view(), a.view(), c.view()) == -1          # dtype mismatch
    assert queue.add(a.view().slice(0, 0, 2), a.view().slice(0, 1, 2), a.view().slice(0, 0, 2)) == -1
    flag = device.create_tensor(HostTensor((16, 16), DataType.BOOL).spec)
    assert queue.add(flag.view(), flag.view(), flag.view()) < 0   # not a numeric leaf
    i32 = device.create_tensor(HostTensor((16, 16), DataType.I32).spec)
    assert queue.div(i32.view(), i32.view(), i32.view()) == -2    # no integer division
    assert queue.sub(i32.view(), i32.view(), i32.view()) > 0
    i8 = device.create_tensor(HostTensor((16, 16), DataType.I8).spec)
    assert queue.div(i8.view(), i8.view(), i8.view()) == -2
    f8 = device.create_tensor(HostTensor((16, 16), DataType.F8_E5M2).spec)
    assert queue.div(f8.view(), f8.view(), f8.view()) > 0         # a floating leaf: division exists
    e8 = device.create_tensor(HostTensor((16, 16), DataType.F8_E8M0).spec)
    assert queue.add(e8.view(), e8.view(), e8.view()) == -2       # not a numeric leaf
    with pytest.raises(ValueError):
        queue.wait(12345)


@pytest.mark.parametrize("op,numpy_op", [("add", np.add), ("mul", np.multiply), ("sub", np.subtract),
                                         ("div", np.divide)])
def test_binary_f64(gpu, op, numpy_op):
    """F64 runs on an IEEE binary64 carrier, as the reference's GPU kernels do
    (src/shared/standard_tiled_add.inl:110-116): equal to numpy's correctly rounded result with
    NaNs canonical. The reference CPU backend's x87 carrier rounds twice; the oracle restates
    that carrier, and the two may differ by one code in the last place."""
    device, queue = gpu
    rng = np.random.default_rng(17)
    shape = (3, 37, 50)
    specials = np.array([0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, np.nan, 5e-324, -5e-324,
                         1.7976931348623157e308, 2.2250738585072014e-308, 1.0000000000000002])
    def payload(s):
        values = rng.standard_normal(s) * np.exp(rng.uniform(-40, 40, size=s))
        flat = values.reshape(-1)
        picks = rng.integers(0, flat.size, size=specials.size * 4)
        flat[picks] = np.tile(specials, 4)
        return values
    a_values, b_values = payload(shape), payload((1, 37, 1))
    a = HostTensor(shape, DataType.F64).poison()
    b = HostTensor((1, 37, 1), DataType.F64).poison()
    out = HostTensor(shape, DataType.F64).poison()
    a.view().copy_from_host(a_values)
    b.view().copy_from_host(b_values)
    da, db, do = upload(device, a), upload(device, b), upload(device, out)
    run(queue, getattr(queue, op)(da.view(), db.view(), do.view()))
    got = HostTensor(shape, DataType.F64, fill=None)
    got.storage[:] = download(do)
    got_bits = got.view().copy_to_host().view(np.uint64).reshape(shape)
    with np.errstate(all="ignore"):
        expect = numpy_op(a_values, b_values)
    expect_bits = expect.view(np.uint64).copy()
    expect_bits[np.isnan(expect)] = 0x7FF8000000000000
    assert np.array_equal(got_bits, expect_bits)
    # padding untouched
    code = {"add": 0, "mul": 1, "sub": 2, "div": 3}[op]
    assert oracle().iomo_binary(code, abi(a.view()), abi(b.view()), abi(out.view()), 0) == 0
    oracle_bits = out.view().copy_to_host().view(np.uint64).reshape(shape)
    differing = got_bits != oracle_bits
    # one code at most between the binary64 carrier and the x87 carrier's double rounding
    delta = np.abs(got_bits[differing].astype(np.int64) - oracle_bits[differing].astype(np.int64))
    assert np.all(delta <= 1)
    mask = HostTensor(shape, DataType.F64).poison(0)
    mask.view().copy_from_host(np.full(shape, -1, dtype=np.int64))
    outside = mask.storage == 0
    assert np.array_equal(got.storage[outside], out.storage[outside])


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
def test_binary_bf16_every_pair_equals_one_rounded_binary32_operation(gpu, op):
    """All 2^32 pairs of BF16 codes: the kernel's result (packed BF16 instructions for ADD,
    SUB and MUL) equals RNE(binary32 operation) with every NaN canonical, which is what the
    reference's codec computes (src/shared/scalar_binary_codec.hpp:45-178; equality of the
    codec with one binary32 operation is shown on the CPU in test_layout_and_codec.py).
    The binary32 side is evaluated by torch on the device, block by block: 2048 left codes
    against all 65 536 right codes at a time, laid over the raw storage of tile-multiple
    tensors (elementwise work pairs equal storage positions, whatever the tile map)."""
    import torch

    device, queue = gpu
    block = 2048
    spec = HostTensor((block, 65536), DataType.BF16, fill=None).spec
    dl, dr, do = (device.create_tensor(spec) for _ in range(3))
    right = torch.arange(65536, dtype=torch.int32, device=device.torch_device).to(torch.int16)
    dr.storage().view(torch.int16).view(block, 65536).copy_(right.expand(block, 65536))
    fn = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div}[op]
    for first in range(0, 65536, block):
        left = torch.arange(first, first + block, dtype=torch.int32, device=device.torch_device).to(torch.int16)
        dl.storage().view(torch.int16).view(block, 65536).copy_(left.unsqueeze(1).expand(block, 65536))
        torch.cuda.synchronize()      # the fills ran on torch's stream, the operation uses the queue's
        run(queue, getattr(queue, op)(dl.view(), dr.view(), do.view()))
        torch.cuda.synchronize()
        a = dl.storage().view(torch.bfloat16).view(block, 65536).float()
        b = dr.storage().view(torch.bfloat16).view(block, 65536).float()
        want = fn(a, b).to(torch.bfloat16).view(torch.int16)
        want = torch.where(torch.isnan(fn(a, b)), torch.full_like(want, 0x7FC0), want)
        got = do.storage().view(torch.int16).view(block, 65536)
        mismatches = int((got != want).sum().item())
        assert mismatches == 0, f"{op}: {mismatches} pairs differ in the block of left codes {first}.."
    for t in (dl, dr, do):
        t.close()
