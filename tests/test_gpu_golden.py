"""GPU kernels against the golden vectors recorded from the unmodified
reference (no oracle in between)."""
import numpy as np
import pytest

from iom_b200.device import RMS_LANES16, RMS_SEQUENTIAL
from iom_b200.tensor import DataType
from gpu_support import download, gpu, like, run, upload  # noqa: F401
from support import HostTensor
from test_golden import GOLDEN, SMALL_FLOATS, host_from, split_shapes, view_from

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [DataType.I32, DataType.F32, DataType.BF16])
@pytest.mark.parametrize("op", ["add", "mul", "sub", "div"])
def test_binary_golden_gpu(gpu, dtype, op):
    device, queue = gpu
    if op == "div" and dtype == DataType.I32:
        pytest.skip("the reference admits no integer division")
    for case in range(5):
        key = f"binary_{op}_{dtype.name}_{case}"
        ls, rs, os_ = split_shapes(GOLDEN[key + "_shapes"])
        dl = upload(device, host_from(GOLDEN[key + "_lhs"], ls, dtype))
        dr = upload(device, host_from(GOLDEN[key + "_rhs"], rs, dtype))
        do = upload(device, host_from(GOLDEN[key + "_out_before"], os_, dtype))
        run(queue, getattr(queue, op)(dl.view(), dr.view(), do.view()))
        assert np.array_equal(download(do), GOLDEN[key + "_out"]), key


@pytest.mark.parametrize("dtype,n", SMALL_FLOATS)
def test_every_pair_of_the_small_floats_golden_gpu(gpu, dtype, n):
    """Every pair of codes of the 8-, 6- and 4-bit floating leaves against the reference's record."""
    device, queue = gpu
    for op in ("add", "mul", "sub", "div"):
        key = f"pairs_{op}_{dtype.name}"
        dl = upload(device, host_from(GOLDEN[key + "_lhs"], (n, n), dtype))
        dr = upload(device, host_from(GOLDEN[key + "_rhs"], (n, n), dtype))
        do = upload(device, HostTensor((n, n), dtype))
        run(queue, getattr(queue, op)(dl.view(), dr.view(), do.view()))
        assert np.array_equal(download(do), GOLDEN[key + "_out"]), key
        for t in (dl, dr, do):
            t.close()


@pytest.mark.parametrize("build,order", [("portable", RMS_SEQUENTIAL), ("avx512", RMS_LANES16)])
def test_rmsnorm_golden_gpu(gpu, build, order):
    device, queue = gpu
    for dtype in (DataType.BF16, DataType.F32):
        if dtype == DataType.F32 and order == RMS_LANES16:
            continue   # the reference has no lane-ordered F32 path
        for case in range(6):
            key = f"rmsnorm_{build}_{dtype.name}_{case}"
            shape = tuple(int(v) for v in GOLDEN[key + "_shape"])
            dx = upload(device, host_from(GOLDEN[key + "_x"], shape, dtype))
            dw = upload(device, host_from(GOLDEN[key + "_w"], (1, shape[-1]), dtype))
            do = upload(device, host_from(GOLDEN[key + "_out_before"], shape, dtype))
            run(queue, queue.rmsnorm(dx.view(), dw.view(), do.view(), 1e-5, order=order))
            assert np.array_equal(download(do), GOLDEN[key + "_out"]), key


def test_movers_golden_gpu(gpu):
    device, queue = gpu
    src = host_from(GOLDEN["copy_src"], (3, 4, 17, 33), DataType.BF16)
    dst = host_from(GOLDEN["copy_dst_before"], (4, 3, 17, 33), DataType.BF16)
    ds, dd = upload(device, src), upload(device, dst)
    run(queue, queue.copy(like(view_from(src, GOLDEN["copy_src_view"], 4), ds),
                          like(view_from(dst, GOLDEN["copy_dst_view"], 4), dd)))
    assert np.array_equal(download(dd), GOLDEN["copy_dst"])

    dt = upload(device, host_from(GOLDEN["embedding_table"], (50, 37), DataType.BF16))
    di = upload(device, host_from(GOLDEN["embedding_ids"], (2, 1, 19), DataType.U32))
    do = upload(device, host_from(GOLDEN["embedding_out_before"], (2, 19, 37), DataType.BF16))
    ws = device.create_workspace(32)
    run(queue, queue.embedding(dt.view(), di.view(), do.view(), ws.view()))
    assert np.array_equal(download(do), GOLDEN["embedding_out"])

    for a in (0, 5, 29):
        s = upload(device, host_from(GOLDEN[f"append_{a}_src"], (2, 3, 3, 40), DataType.BF16))
        d = upload(device, host_from(GOLDEN[f"append_{a}_dst_before"], (2, 3, 32, 40), DataType.BF16))
        run(queue, queue.cache_append(s.view(), d.view(), a))
        assert np.array_equal(download(d), GOLDEN[f"append_{a}_dst"])

    host = host_from(GOLDEN["transfer_before"], (3, 2, 17, 35), DataType.F32)
    dev = upload(device, host)
    view = like(view_from(host, GOLDEN["transfer_view"], 4), dev)
    staging = device.create_workspace(GOLDEN["transfer_payload"].nbytes + 32)
    view.copy_from_host(GOLDEN["transfer_payload"], staging.view())
    assert np.array_equal(download(dev), GOLDEN["transfer_after"])


def test_silu_golden_gpu(gpu):
    """The CUDA path against the reference CPU backend's stored outputs: BF16 bit for
    bit on every code; F32 within 4 ulp (the kernel evaluates on the FP64 carrier of
    the reference's GPU backends, the stored outputs come from its FP32 CPU carrier)."""
    device, queue = gpu
    codes = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    x = HostTensor((256, 256), DataType.BF16).poison(0xA5)
    x.view().copy_from_host(codes)
    y = HostTensor((256, 256), DataType.BF16).poison(0xA5)
    y.view().copy_from_host(np.zeros((256, 256), dtype=np.uint16))
    dx, dy = upload(device, x), upload(device, y)
    run(queue, queue.silu(dx.view(), dy.view()))
    assert np.array_equal(download(dy), GOLDEN["silu_portable_BF16_out"])
    assert np.array_equal(download(dy), GOLDEN["silu_avx512_BF16_out"])
    xf = upload(device, host_from(GOLDEN["silu_portable_F32_x"], (2, 17, 35), DataType.F32))
    yf = upload(device, host_from(GOLDEN["silu_portable_F32_out_before"], (2, 17, 35), DataType.F32))
    run(queue, queue.silu(xf.view(), yf.view()))
    got = download(yf).view(np.uint32).astype(np.int64)
    want = GOLDEN["silu_portable_F32_out"].view(np.uint32).astype(np.int64)
    assert np.abs(got - want).max() <= 4
    before = GOLDEN["silu_portable_F32_out_before"].view(np.uint32).astype(np.int64)
    untouched = want == before        # padding and nothing else (payloads are random)
    assert np.array_equal(got[untouched], want[untouched])


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
def test_rope_golden_gpu(gpu, dtype):
    """The CUDA path against the reference CPU backend's stored RoPE outputs, bit for bit
    (both builds stored the same bytes)."""
    from test_golden import ROPE_CASES
    device, queue = gpu
    for case, (shape, a, theta) in enumerate(ROPE_CASES):
        key = f"rope_portable_{dtype.name}_{case}"
        dx = upload(device, host_from(GOLDEN[key + "_x"], shape, dtype))
        do = upload(device, host_from(GOLDEN[key + "_out_before"], shape, dtype))
        run(queue, queue.rope(dx.view(), do.view(), a, theta))
        assert np.array_equal(download(do), GOLDEN[key + "_out"]), key
        assert np.array_equal(GOLDEN[key + "_out"], GOLDEN[f"rope_avx512_{dtype.name}_{case}_out"])
