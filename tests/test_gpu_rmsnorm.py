"""GPU parity: iomb_rmsnorm / iomb_add_rmsnorm against the oracle.

LANES16 order must be bit-identical to the oracle's order 0 (the reference's
AVX-512 BF16 build) and SEQUENTIAL to order 1 (the portable build), for BF16 and
(SEQUENTIAL) for F32: those are the orders the reference has, and the ones the
operation facade picks. Across orders the BF16 outputs may differ by at most one
code. F32 in the lane order has no reference counterpart; it is held to 2e-6
relative against an FP64 evaluation of the same formula (the portable order's own
distance from that evaluation grows with the row length and passes 2e-6 near
8192 values, so it cannot be the yardstick for another order at that bar).
"""
import numpy as np
import pytest

from iom_b200.device import RMS_LANES16, RMS_SEQUENTIAL
from iom_b200.tensor import DataType
from gpu_support import download, gpu, like, run, upload  # noqa: F401
from support import (HostTensor, SPECIAL_BF16, SPECIAL_F32, abi, bf16_bits_to_f32, logical,
                     oracle, random_payload)

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1), (15, 17), (16, 16), (17, 33), (2, 3, 16, 31), (33, 15), (4, 256),
          (64, 2048), (40, 8192), (3, 5000), (2, 2, 1, 2, 1, 2, 17, 48),
          # long rows: whole bands streamed by one CTA (more bands than SMs, a band
          # longer than shared memory, ragged last band in every plane)
          (4800, 2064), (4000, 8200), (2, 170, 3000), (7, 20000), (3, 40000), (2400, 4096),
          # groups of two rows with two chains (rows too long for taller groups)
          (320, 12288),
          # a row beyond every staging capacity: the unstaged kernel
          (3, 100000)]


def seeded(shape, dtype, rng, kind="normal", poison=0xA5):
    t = HostTensor(shape, dtype).poison(poison)
    t.view().copy_from_host(random_payload(rng, shape, dtype, kind))
    return t


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("order", [RMS_LANES16, RMS_SEQUENTIAL])
def test_rmsnorm_parity(gpu, dtype, shape, order):
    device, queue = gpu
    rng = np.random.default_rng(abs(hash((int(dtype), shape))) & 0xFFFF)
    x = seeded(shape, dtype, rng)
    w = seeded((1, shape[-1]), dtype, rng)
    out = seeded(shape, dtype, rng)
    dx, dw, do = upload(device, x), upload(device, w), upload(device, out)
    for eps in (1e-5, 0.0):
        run(queue, queue.rmsnorm(dx.view(), dw.view(), do.view(), eps, order=order))
        # The oracle's order 0 applies lanes to BF16 only; F32 LANES16 has no
        # reference counterpart and is checked by tolerance below.
        if dtype == DataType.BF16 or order == RMS_SEQUENTIAL:
            assert oracle().iomo_rmsnorm(abi(x.view()), abi(w.view()), abi(out.view()), eps, order) == 0
            assert np.array_equal(download(do), out.storage)
        else:
            assert oracle().iomo_rmsnorm(abi(x.view()), abi(w.view()), abi(out.view()), eps, 1) == 0
            got = HostTensor(shape, dtype, fill=None)
            got.storage[:] = download(do)
            xs = logical(x.view()).astype(np.float64)
            ws = logical(w.view()).astype(np.float64)
            inv = 1.0 / np.sqrt(np.mean(xs * xs, axis=-1, keepdims=True) + np.float64(np.float32(eps)))
            truth = xs * inv * ws
            err = np.abs(logical(got.view()).astype(np.float64) - truth)
            assert np.all(err <= 2e-6 * np.abs(truth) + 1e-30)
            # padding and everything outside the logical window stay untouched
            mask = HostTensor(shape, dtype).poison(0)
            mask.view().copy_from_host(np.full(shape, 0xFFFFFFFF, dtype=np.uint32))
            outside = mask.storage == 0
            assert np.array_equal(got.storage[outside], out.storage[outside])
    assert np.array_equal(download(dx), x.storage)


def test_rmsnorm_orders_within_one_bf16_code(gpu):
    device, queue = gpu
    rng = np.random.default_rng(5)
    x = seeded((256, 2048), DataType.BF16, rng)
    w = seeded((1, 2048), DataType.BF16, rng)
    outs = []
    dx, dw = upload(device, x), upload(device, w)
    for order in (RMS_LANES16, RMS_SEQUENTIAL):
        do = device.create_tensor(x.spec)
        run(queue, queue.rmsnorm(dx.view(), dw.view(), do.view(), 1e-5, order=order))
        outs.append(download(do).view(np.uint16).astype(np.int32))
    assert np.max(np.abs(outs[0] - outs[1])) <= 1


@pytest.mark.parametrize("dtype,specials", [(DataType.F32, SPECIAL_F32), (DataType.BF16, SPECIAL_BF16)])
@pytest.mark.parametrize("order", [RMS_LANES16, RMS_SEQUENTIAL])
def test_rmsnorm_special_rows(gpu, dtype, specials, order):
    device, queue = gpu
    rng = np.random.default_rng(3)
    n = len(specials)
    base = random_payload(rng, (n + 2, 40), dtype, "normal")
    raw = base.view(np.uint32 if dtype == DataType.F32 else np.uint16)
    for i, code in enumerate(specials):
        raw[i, (3 * i) % 40] = code
    raw[n, :] = specials[4]
    raw[n + 1, :] = specials[8]
    scale = random_payload(rng, (1, 40), dtype, "normal")
    sraw = scale.view(np.uint32 if dtype == DataType.F32 else np.uint16)
    sraw[0, 5] = specials[10]
    sraw[0, 6] = specials[12]
    x = HostTensor((n + 2, 40), dtype).poison()
    w = HostTensor((1, 40), dtype).poison()
    out = HostTensor((n + 2, 40), dtype).poison()
    x.view().copy_from_host(base)
    w.view().copy_from_host(scale)
    dx, dw, do = upload(device, x), upload(device, w), upload(device, out)
    for eps in (0.0, 1e-5, float(np.finfo(np.float32).max), float(np.finfo(np.float32).smallest_subnormal)):
        run(queue, queue.rmsnorm(dx.view(), dw.view(), do.view(), eps, order=order))
        oracle_order = order if dtype == DataType.BF16 else 1
        assert oracle().iomo_rmsnorm(abi(x.view()), abi(w.view()), abi(out.view()), eps, oracle_order) == 0
        got = download(do)
        if dtype == DataType.BF16 or order == RMS_SEQUENTIAL:
            assert np.array_equal(got, out.storage)
        else:
            a = got.view(np.uint32)
            b = out.storage.view(np.uint32)
            nan_a = (a & 0x7FFFFFFF) > 0x7F800000
            nan_b = (b & 0x7FFFFFFF) > 0x7F800000
            assert np.array_equal(nan_a, nan_b)
            af, bf = a.view(np.float32).astype(np.float64), b.view(np.float32).astype(np.float64)
            fin = np.isfinite(bf) & ~nan_b
            assert np.array_equal(a[~fin], b[~fin])
            assert np.all(np.abs(af[fin] - bf[fin]) <= 2e-6 * np.abs(bf[fin]) + 1e-44)


@pytest.mark.parametrize("dtype,order", [(DataType.BF16, RMS_LANES16), (DataType.BF16, RMS_SEQUENTIAL),
                                         (DataType.F32, RMS_SEQUENTIAL)])
@pytest.mark.parametrize("features,rows", [(4100, 40), (8192, 40),
                                           # enough bands for groups of 8 and of 16 rows, whose
                                           # chain threads own two columns and use packed
                                           # arithmetic (a packed product feeding a packed sum
                                           # must not be contracted)
                                           (4100, 1200), (2064, 2400)])
def test_rmsnorm_long_rows_special_values(gpu, dtype, order, features, rows):
    """Rows that defeat the clean-row shortcut, at lengths served by the band kernel:
    all-zero rows with eps 0, infinities, NaNs, overflowing and vanishing sums,
    and a scale row holding a NaN and an infinity."""
    device, queue = gpu
    rng = np.random.default_rng(features + int(dtype) + order)
    payload = random_payload(rng, (rows, features), dtype, "normal")
    bits = payload.view(np.uint16 if dtype == DataType.BF16 else np.uint32)
    code = (lambda v: np.float32(v).view(np.uint32) >> 16) if dtype == DataType.BF16 \
        else (lambda v: np.float32(v).view(np.uint32))
    bits[0, :] = 0
    bits[1, 17] = code(np.inf)
    bits[2, features - 1] = code(np.nan)
    bits[3, :] = code(3e38)
    bits[4, :] = code(1e-30)
    bits[5, 5] = code(-np.inf)
    bits[5, 6] = code(np.inf)
    bits[17, :] = code(-0.0)
    # squares that are subnormal in FP32: a fused multiply-add would keep bits the
    # reference's separately rounded product drops
    bits[6, 0::3] = code(3.3e-21)
    bits[6, 1::3] = code(-1.7e-21)
    bits[6, 2::3] = code(2.9e-22)
    x = HostTensor((rows, features), dtype).poison()
    x.view().copy_from_host(payload)
    out = HostTensor((rows, features), dtype).poison()
    scale_payload = random_payload(rng, (1, features), dtype, "normal")
    for poisoned_scale in (False, True):
        if poisoned_scale:
            sbits = scale_payload.view(bits.dtype)
            sbits[0, 3] = code(np.nan)
            sbits[0, features - 2] = code(np.inf)
        w = HostTensor((1, features), dtype).poison()
        w.view().copy_from_host(scale_payload)
        dx, dw, do = upload(device, x), upload(device, w), upload(device, out)
        for eps in (0.0, 1e-5):
            run(queue, queue.rmsnorm(dx.view(), dw.view(), do.view(), eps, order=order))
            assert oracle().iomo_rmsnorm(abi(x.view()), abi(w.view()), abi(out.view()), eps, order) == 0
            assert np.array_equal(download(do), out.storage)


@pytest.mark.parametrize("features,rows", [(2304, 2400), (4100, 1200), (2064, 2400), (8192, 640)])
def test_f32_lane_order_does_not_depend_on_the_group_height(gpu, features, rows):
    """F32 in the lane order has no reference build to compare with bit for bit, so its own
    consistency is pinned: many rows (tall groups, whose chain threads own two columns and add
    with a packed instruction) give, row by row, the bits of the same rows run as a small
    tensor (groups of one row, scalar arithmetic). A product contracted into the sum would
    show here: F32 squares are not exact."""
    device, queue = gpu
    rng = np.random.default_rng(features)
    x = seeded((rows, features), DataType.F32, rng)
    w = seeded((1, features), DataType.F32, rng)
    out = seeded((rows, features), DataType.F32, rng)
    dx, dw, do = upload(device, x), upload(device, w), upload(device, out)
    run(queue, queue.rmsnorm(dx.view(), dw.view(), do.view(), 1e-6, order=RMS_LANES16))
    tall = HostTensor((rows, features), DataType.F32, fill=None)
    tall.storage[:] = download(do)
    tall_rows = tall.view().copy_to_host().view(np.uint32).reshape(rows, features)
    few = 32
    values = x.view().copy_to_host().view(np.uint32).reshape(rows, features)
    small_x = HostTensor((few, features), DataType.F32).poison()
    small_x.view().copy_from_host(values[:few].copy())
    small_out = HostTensor((few, features), DataType.F32).poison()
    dsx, dso = upload(device, small_x), upload(device, small_out)
    run(queue, queue.rmsnorm(dsx.view(), dw.view(), dso.view(), 1e-6, order=RMS_LANES16))
    got = HostTensor((few, features), DataType.F32, fill=None)
    got.storage[:] = download(dso)
    small_rows = got.view().copy_to_host().view(np.uint32).reshape(few, features)
    assert np.array_equal(tall_rows[:few], small_rows)


def test_rmsnorm_rejections(gpu):
    device, queue = gpu
    x = device.create_tensor(HostTensor((16, 32), DataType.BF16).spec)
    w = device.create_tensor(HostTensor((1, 32), DataType.BF16).spec)
    w2 = device.create_tensor(HostTensor((2, 32), DataType.BF16).spec)
    o = device.create_tensor(HostTensor((16, 32), DataType.BF16).spec)
    assert queue.rmsnorm(x.view(), w.view(), x.view(), 1e-5) == -1     # output shares input owner
    assert queue.rmsnorm(x.view(), w2.view(), o.view(), 1e-5) == -1    # scale not [1,F]
    for eps in (-1.0, float("inf"), float("nan")):
        assert queue.rmsnorm(x.view(), w.view(), o.view(), eps) == -1
    i32 = device.create_tensor(HostTensor((16, 32), DataType.I32).spec)
    wi = device.create_tensor(HostTensor((1, 32), DataType.I32).spec)
    oi = device.create_tensor(HostTensor((16, 32), DataType.I32).spec)
    assert queue.rmsnorm(i32.view(), wi.view(), oi.view(), 1e-5) == -2


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
@pytest.mark.parametrize("shape", [(17, 33), (64, 2048), (3, 16, 8192), (2, 3, 5, 100),
                                   # long rows: the pipelined kernel (more units than SMs,
                                   # ragged last band and last tile, several planes)
                                   (1200, 8200), (2, 170, 3000), (7, 20000), (3, 40000), (2, 100000),
                                   # fused groups of 4 and of 8 rows (one chain), and of one
                                   # row with two chains
                                   (640, 4096), (2400, 2304), (320, 12288)])
@pytest.mark.parametrize("order", [RMS_LANES16, RMS_SEQUENTIAL])
def test_add_rmsnorm_equals_add_then_rmsnorm(gpu, dtype, shape, order):
    """The fused entry stores the rounded sum and normalises the rounded value."""
    device, queue = gpu
    rng = np.random.default_rng(abs(hash((int(dtype), shape, order))) & 0xFFFF)
    x = seeded(shape, dtype, rng)
    r = seeded(shape, dtype, rng)
    w = seeded((1, shape[-1]), dtype, rng)
    s = seeded(shape, dtype, rng)
    out = seeded(shape, dtype, rng)
    dx, dr, dw, ds, do = (upload(device, t) for t in (x, r, w, s, out))
    run(queue, queue.add_rmsnorm(dx.view(), dr.view(), dw.view(), ds.view(), do.view(), 1e-5, order=order))
    # unfused on the device: must be bit-identical to the fused result
    ds2, do2 = upload(device, s), upload(device, out)
    run(queue, queue.add(dx.view(), dr.view(), ds2.view()))
    run(queue, queue.rmsnorm(ds2.view(), dw.view(), do2.view(), 1e-5, order=order))
    assert np.array_equal(download(ds), download(ds2))
    assert np.array_equal(download(do), download(do2))
    # and the stored sum equals the oracle's ADD
    assert oracle().iomo_binary(0, abi(x.view()), abi(r.view()), abi(s.view()), 0) == 0
    assert np.array_equal(download(ds), s.storage)
    if dtype == DataType.BF16 or order == RMS_SEQUENTIAL:
        assert oracle().iomo_rmsnorm(abi(s.view()), abi(w.view()), abi(out.view()), 1e-5, order) == 0
        assert np.array_equal(download(do), out.storage)
    # in-place residual update: sum aliases x exactly
    dx3, do3 = upload(device, x), upload(device, out)
    run(queue, queue.add_rmsnorm(dx3.view(), dr.view(), dw.view(), dx3.view(), do3.view(), 1e-5, order=order))
    assert np.array_equal(download(dx3), download(ds))
    assert np.array_equal(download(do3), download(do))


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
@pytest.mark.parametrize("features", [2100, 8192])
def test_long_rows_through_transformed_views(gpu, dtype, features):
    """Long rows behind sliced, permuted views with different strides per operand:
    every plane of the window is normalised, the planes in between keep their poison."""
    device, queue = gpu
    order = RMS_LANES16 if dtype == DataType.BF16 else RMS_SEQUENTIAL
    rng = np.random.default_rng(features)
    x = seeded((5, 3, 20, features), dtype, rng)
    r = seeded((3, 4, 20, features), dtype, rng)
    w = seeded((1, features), dtype, rng)
    s = seeded((2, 3, 20, features), dtype, rng)
    out = seeded((3, 2, 20, features), dtype, rng, poison=0x5A)
    xv = x.view().slice(0, 1, 2, 2)                              # planes 1 and 3 of five: [2,3,...]
    rv = r.view().slice(1, 1, 2, 2).permute([1, 0])              # [2,3,...] with swapped strides
    sv = s.view()
    ov = out.view().permute([1, 0])                              # [2,3,...] over a [3,2,...] owner
    dx, dr, dw, ds, do = (upload(device, t) for t in (x, r, w, s, out))
    run(queue, queue.add_rmsnorm(like(xv, dx), like(rv, dr), dw.view(), like(sv, ds), like(ov, do),
                                 1e-6, order=order))
    assert oracle().iomo_binary(0, abi(xv), abi(rv), abi(sv), 0) == 0
    assert oracle().iomo_rmsnorm(abi(sv), abi(w.view()), abi(ov), 1e-6, order) == 0
    assert np.array_equal(download(ds), s.storage)
    assert np.array_equal(download(do), out.storage)
    # unfused, reading the strided window directly
    out2 = seeded((3, 2, 20, features), dtype, rng, poison=0x33)
    do2 = upload(device, out2)
    ov2 = out2.view().permute([1, 0])
    run(queue, queue.rmsnorm(like(xv, dx), dw.view(), like(ov2, do2), 1e-6, order=order))
    assert oracle().iomo_rmsnorm(abi(xv), abi(w.view()), abi(ov2), 1e-6, order) == 0
    assert np.array_equal(download(do2), out2.storage)


def test_zz_no_long_row_wait_gave_up(gpu):
    """The long-row kernels bound their waits for asynchronous copies; a wait that gives up
    is counted on the device. After every case above the counter is still zero."""
    import ctypes

    import torch
    device, _ = gpu
    torch.cuda.synchronize()
    count = ctypes.c_uint(123)
    assert device._lib.iomb_rmsnorm_copy_timeouts(ctypes.byref(count)) == 0
    assert count.value == 0
