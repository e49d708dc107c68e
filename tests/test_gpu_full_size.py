"""GPU: the operations at the full sizes of the benchmark configurations, checked
through properties that do not need a CPU pass over gigabytes:

* replication: rows (planes) are independent, so a tensor built from copies of a small
  pattern must produce copies of the pattern's result, and the pattern's result is
  checked against the oracle;
* algebra that is exact in the leaf: x * 1 == x, x + 0 == x, a + b == b + a,
  (a + b) - b == a for wrapping integers;
* a sum of squares whose value is an exactly representable integer.

Comparisons of whole tensors run on the device (torch.equal on the storage bytes)."""
import ctypes
import re

import numpy as np
import pytest
import torch

from iom_b200.device import DeviceMemoryConfig, make_b200_device
from iom_b200.tensor import DataType, TensorSpec
from support import HostTensor, abi, f32_to_bf16_bits, oracle, random_payload

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def big():
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    device = make_b200_device(0, DeviceMemoryConfig(26 << 30))
    queue = device.create_ops()
    yield device, queue
    queue.close()


def run(queue, token):
    assert token > 0, f"operation rejected with oid {token}"
    queue.wait(token)


def replicate(device, pattern: HostTensor, copies: int, shape):
    """Device tensor of `shape` whose storage is `copies` repetitions of the pattern's
    storage (valid whenever the pattern is a whole number of 16-row bands / planes)."""
    tensor = device.create_tensor(TensorSpec(shape, pattern.spec.data_type))
    piece = torch.from_numpy(pattern.storage.copy()).to(device.torch_device)
    assert tensor.storage_nbytes == copies * piece.numel()
    tensor.storage().view(copies, piece.numel()).copy_(piece.unsqueeze(0).expand(copies, -1))
    return tensor, piece


def test_fused_add_rmsnorm_at_the_benchmark_size(big):
    """BF16 [16, 8192, 2048] (the bench workload): 16 identical planes in, 16 planes out
    that all equal the oracle's result for one plane; fused == add then rmsnorm."""
    device, queue = big
    rng = np.random.default_rng(101)
    plane = (8192, 2048)
    hx, hr, hs, ho = (HostTensor(plane, DataType.BF16) for _ in range(4))
    hx.view().copy_from_host(random_payload(rng, plane, DataType.BF16, "normal"))
    hr.view().copy_from_host(random_payload(rng, plane, DataType.BF16, "normal"))
    hw = HostTensor((1, 2048), DataType.BF16)
    hw.view().copy_from_host(f32_to_bf16_bits((1.0 + 0.02 * rng.standard_normal((1, 2048))).astype(np.float32)))
    shape = (16, 8192, 2048)
    x, _ = replicate(device, hx, 16, shape)
    r, _ = replicate(device, hr, 16, shape)
    w = device.create_tensor(hw.spec)
    w.storage().copy_(torch.from_numpy(hw.storage.copy()))
    total, out, total2, out2 = (device.create_tensor(TensorSpec(shape, DataType.BF16)) for _ in range(4))
    torch.cuda.synchronize()      # the fills ran on torch's stream, the operations use the queue's
    run(queue, queue.add_rmsnorm(x.view(), r.view(), w.view(), total.view(), out.view(), 1e-5))
    assert oracle().iomo_binary(0, abi(hx.view()), abi(hr.view()), abi(hs.view()), 0) == 0
    assert oracle().iomo_rmsnorm(abi(hs.view()), abi(hw.view()), abi(ho.view()), 1e-5, 0) == 0
    want_sum = torch.from_numpy(hs.storage.copy()).to(device.torch_device)
    want_out = torch.from_numpy(ho.storage.copy()).to(device.torch_device)
    for p in range(16):
        assert torch.equal(total.storage().view(16, -1)[p], want_sum), f"sum plane {p}"
        assert torch.equal(out.storage().view(16, -1)[p], want_out), f"out plane {p}"
    run(queue, queue.add(x.view(), r.view(), total2.view()))
    run(queue, queue.rmsnorm(total2.view(), w.view(), out2.view(), 1e-5))
    assert torch.equal(total.storage(), total2.storage())
    assert torch.equal(out.storage(), out2.storage())
    for t in (x, r, w, total, out, total2, out2):
        t.close()


def test_rmsnorm_at_the_sharded_size(big):
    """BF16 [32768, 8192] (one eighth of [262144, 8192]), eps 1e-6: 128 copies of a
    256-row pattern; every copy must equal the oracle's result for the pattern, in
    both accumulation orders."""
    device, queue = big
    rng = np.random.default_rng(102)
    pattern = (256, 8192)
    hx, ho = HostTensor(pattern, DataType.BF16), HostTensor(pattern, DataType.BF16)
    hx.view().copy_from_host(random_payload(rng, pattern, DataType.BF16, "normal"))
    hw = HostTensor((1, 8192), DataType.BF16)
    hw.view().copy_from_host(f32_to_bf16_bits((1.0 + 0.02 * rng.standard_normal((1, 8192))).astype(np.float32)))
    x, _ = replicate(device, hx, 128, (32768, 8192))
    w = device.create_tensor(hw.spec)
    w.storage().copy_(torch.from_numpy(hw.storage.copy()))
    out = device.create_tensor(TensorSpec((32768, 8192), DataType.BF16))
    torch.cuda.synchronize()
    for order in (0, 1):
        run(queue, queue.rmsnorm(x.view(), w.view(), out.view(), 1e-6, order=order))
        assert oracle().iomo_rmsnorm(abi(hx.view()), abi(hw.view()), abi(ho.view()), 1e-6, order) == 0
        want = torch.from_numpy(ho.storage.copy()).to(device.torch_device)
        got = out.storage().view(128, -1)
        assert torch.equal(got, want.unsqueeze(0).expand(128, -1)), f"order {order}"
    # whole-tensor sum of squares of all ones: 2^28, exact in FP32
    ones = device.create_tensor(TensorSpec((32768, 8192), DataType.BF16))
    ones.storage().view(torch.int16).fill_(0x3F80)
    scratch = device.create_workspace(int(device._lib.iomb_sumsq_scratch_bytes()))
    cell = device.create_workspace(32)
    torch.cuda.synchronize()
    run(queue, queue.sumsq(ones.view(), scratch.view(), cell.view().address()))
    value = cell.tensor()[:4].view(torch.float32).item()
    assert value == float(1 << 28)
    for t in (x, w, out, ones):
        t.close()
    scratch.close()
    cell.close()


def test_long_rows_issued_as_several_launches(big):
    """BF16 [81920 + 16, 8192], eps 1e-6: more row groups than one launch of the long-row
    kernel takes per SM, so the call is issued as several launches (the fused form with its
    half-height groups as more of them). 320 copies of a 256-row pattern plus one ragged
    16-row band: every copy must equal the oracle's result for the pattern, and the fused
    entry must equal add then rmsnorm on the whole tensor."""
    device, queue = big
    rng = np.random.default_rng(103)
    pattern, copies = (256, 8192), 320
    hx, hr, hs, ho = (HostTensor(pattern, DataType.BF16) for _ in range(4))
    hx.view().copy_from_host(random_payload(rng, pattern, DataType.BF16, "normal"))
    hr.view().copy_from_host(random_payload(rng, pattern, DataType.BF16, "normal"))
    hw = HostTensor((1, 8192), DataType.BF16)
    hw.view().copy_from_host(f32_to_bf16_bits((1.0 + 0.02 * rng.standard_normal((1, 8192))).astype(np.float32)))
    rows = copies * 256 + 16
    shape = (rows, 8192)
    band = 16 * 8192 * 2

    def replicated(host):
        tensor = device.create_tensor(TensorSpec(shape, DataType.BF16))
        piece = torch.from_numpy(host.storage.copy()).to(device.torch_device)
        body = tensor.storage()[:copies * piece.numel()]
        body.view(copies, piece.numel()).copy_(piece.unsqueeze(0).expand(copies, -1))
        tensor.storage()[copies * piece.numel():].copy_(piece[:band])     # the last band: rows 0..15
        return tensor

    x, r = replicated(hx), replicated(hr)
    w = device.create_tensor(hw.spec)
    w.storage().copy_(torch.from_numpy(hw.storage.copy()))
    total, out, total2, out2 = (device.create_tensor(TensorSpec(shape, DataType.BF16)) for _ in range(4))
    torch.cuda.synchronize()
    run(queue, queue.add_rmsnorm(x.view(), r.view(), w.view(), total.view(), out.view(), 1e-6))
    launched = (device._lib.iomb_last_launch() or b"").decode()
    assert "rmsnorm_long_kernel" in launched, launched
    assert int(re.search(r"(\d+) launch\(es\)", launched).group(1)) > 1, launched
    assert oracle().iomo_binary(0, abi(hx.view()), abi(hr.view()), abi(hs.view()), 0) == 0
    assert oracle().iomo_rmsnorm(abi(hs.view()), abi(hw.view()), abi(ho.view()), 1e-6, 0) == 0
    for got, host in ((total, hs), (out, ho)):
        want = torch.from_numpy(host.storage.copy()).to(device.torch_device)
        body = got.storage()[:copies * want.numel()].view(copies, -1)
        assert torch.equal(body, want.unsqueeze(0).expand(copies, -1))
        assert torch.equal(got.storage()[copies * want.numel():], want[:band])
    run(queue, queue.add(x.view(), r.view(), total2.view()))
    run(queue, queue.rmsnorm(total2.view(), w.view(), out2.view(), 1e-6))
    assert torch.equal(total.storage(), total2.storage())
    assert torch.equal(out.storage(), out2.storage())
    count = ctypes.c_uint(1)
    assert device._lib.iomb_rmsnorm_copy_timeouts(ctypes.byref(count)) == 0 and count.value == 0
    for t in (x, r, w, total, out, total2, out2):
        t.close()


@pytest.mark.parametrize("dtype,op", [(DataType.F32, "mul"), (DataType.I32, "add"), (DataType.BF16, "add")])
def test_elementwise_at_two_to_the_thirty(big, dtype, op):
    """2^30 elements per tensor ([524288, 2048]), full shape and both broadcast forms."""
    device, queue = big
    m, n = 524288, 2048
    width = 2 if dtype == DataType.BF16 else 4
    x, y, o, o2 = (device.create_tensor(TensorSpec((m, n), dtype)) for _ in range(4))
    row, col = device.create_tensor(TensorSpec((1, n), dtype)), device.create_tensor(TensorSpec((m, 1), dtype))
    generator = torch.Generator(device=device.torch_device).manual_seed(7)
    count = x.storage_nbytes // width
    if dtype == DataType.I32:
        for t in (x, y):
            t.storage().view(torch.int32).copy_(torch.randint(-(1 << 30), 1 << 30, (count,), generator=generator,
                                                              device=device.torch_device, dtype=torch.int32))
        identity = 0
    else:
        for t in (x, y):
            values = torch.randn(count, generator=generator, device=device.torch_device) + 3.0   # no -0, no NaN
            if dtype == DataType.BF16:
                t.storage().view(torch.bfloat16).copy_(values.to(torch.bfloat16))
            else:
                t.storage().view(torch.float32).copy_(values)
        identity = 1.0 if op == "mul" else 0.0
    torch_type = {DataType.I32: torch.int32, DataType.F32: torch.float32, DataType.BF16: torch.bfloat16}[dtype]
    row.storage().view(torch_type).fill_(identity)
    col.storage().view(torch_type).fill_(identity)
    fn = getattr(queue, op)
    torch.cuda.synchronize()      # the fills ran on torch's stream, the operations use the queue's
    # the operation is commutative bit for bit
    run(queue, fn(x.view(), y.view(), o.view()))
    run(queue, fn(y.view(), x.view(), o2.view()))
    assert torch.equal(o.storage(), o2.storage())
    # spot parity: first and last 16-row bands against torch on the device
    band = 16 * n * width
    for start in (0, x.storage_nbytes - band):
        a = x.storage()[start:start + band].view(torch_type)
        b = y.storage()[start:start + band].view(torch_type)
        want = (a * b) if op == "mul" else (a + b)
        assert torch.equal(o.storage()[start:start + band].view(torch_type), want)
    # the identity element through a row and a column broadcast leaves x unchanged
    run(queue, fn(x.view(), row.view(), o.view()))
    assert torch.equal(o.storage(), x.storage())
    run(queue, fn(col.view(), x.view(), o2.view()))
    assert torch.equal(o2.storage(), x.storage())
    if dtype == DataType.I32:
        run(queue, queue.add(x.view(), y.view(), o.view()))
        run(queue, queue.sub(o.view(), y.view(), o2.view()))       # wraps back exactly
        assert torch.equal(o2.storage(), x.storage())
    for t in (x, y, o, o2, row, col):
        t.close()


def test_decode_step_data_movement_at_full_geometry(big):
    """TinyLlama decode geometry: 64 ids from the [32000, 2048] table, and the
    [64, 32000] logits cast to F32, against the oracle."""
    device, queue = big
    rng = np.random.default_rng(104)
    table = HostTensor((32000, 2048), DataType.BF16)
    table.view().copy_from_host(f32_to_bf16_bits((0.02 * rng.standard_normal((32000, 2048))).astype(np.float32)))
    ids = HostTensor((1, 64), DataType.U32)
    ids.view().copy_from_host(rng.integers(0, 32000, size=(1, 64)).astype(np.uint32))
    out = HostTensor((64, 2048), DataType.BF16).poison()
    tensors = []
    for host in (table, ids, out):
        t = device.create_tensor(host.spec)
        t.storage().copy_(torch.from_numpy(host.storage.copy()))
        tensors.append(t)
    dt, di, do = tensors
    workspace = device.create_workspace(32)
    torch.cuda.synchronize()
    run(queue, queue.embedding(dt.view(), di.view(), do.view(), workspace.view()))
    status = ctypes.c_uint32(9)
    assert oracle().iomo_embedding(abi(table.view()), abi(ids.view()), abi(out.view()),
                                   ctypes.byref(status)) == 0
    assert status.value == 0
    assert np.array_equal(do.storage().cpu().numpy(), out.storage)
    logits = HostTensor((64, 32000), DataType.BF16)
    logits.view().copy_from_host(random_payload(rng, (64, 32000), DataType.BF16, "normal"))
    wide = HostTensor((64, 32000), DataType.F32).poison()
    dl, dw = device.create_tensor(logits.spec), device.create_tensor(wide.spec)
    dl.storage().copy_(torch.from_numpy(logits.storage.copy()))
    dw.storage().copy_(torch.from_numpy(wide.storage.copy()))
    torch.cuda.synchronize()
    run(queue, queue.cast(dl.view(), dw.view()))
    assert oracle().iomo_cast(abi(logits.view()), abi(wide.view())) == 0
    assert np.array_equal(dw.storage().cpu().numpy(), wide.storage)
    for t in (dt, di, do, dl, dw):
        t.close()
    workspace.close()
