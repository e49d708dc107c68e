"""GPU parity: copy, cast, embedding, cache_append, sumsq and host transfers."""
import ctypes

import numpy as np
import pytest
import torch

from iom_b200.tensor import DataType
from gpu_support import download, gpu, like, run, upload  # noqa: F401
from support import (HostTensor, NUMPY_OF, SPECIAL_BF16, SPECIAL_F32, abi, oracle,
                     random_payload)

pytestmark = pytest.mark.gpu


def seeded(shape, dtype, rng, poison=0xA5, kind="uniform"):
    t = HostTensor(shape, dtype).poison(poison)
    t.view().copy_from_host(random_payload(rng, shape, dtype, kind))
    return t


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32, DataType.U8, DataType.I64, DataType.F16,
                                   DataType.I2, DataType.U4, DataType.F4_E2M1, DataType.F6_E2M3])
def test_copy_parity(gpu, dtype):
    device, queue = gpu
    rng = np.random.default_rng(11)
    src = seeded((3, 4, 17, 33), dtype, rng)
    dst = seeded((4, 3, 17, 33), dtype, rng)
    sv = src.view().slice(1, 0, 2, 2)
    dv = dst.view().permute([1, 0]).slice(1, 1, 2, 2)
    ds, dd = upload(device, src), upload(device, dst)
    run(queue, queue.copy(like(sv, ds), like(dv, dd)))
    assert oracle().iomo_copy(abi(sv), abi(dv)) == 0
    assert np.array_equal(download(dd), dst.storage)
    # dense tile-multiple owners take the linear stream
    a = seeded((5, 32, 64), dtype, rng)
    b = seeded((5, 32, 64), dtype, rng)
    da, db = upload(device, a), upload(device, b)
    run(queue, queue.copy(da.view(), db.view()))
    assert np.array_equal(download(db), a.storage)
    # identical window: accepted no-op
    run(queue, queue.copy(da.view(), da.view()))
    assert np.array_equal(download(da), a.storage)
    # different specification: rejected
    assert queue.copy(da.view(), dd.view()) == -1


@pytest.mark.parametrize("shape", [(17, 33), (64, 128), (2, 3, 16, 31), (3, 32, 32)])
def test_cast_parity(gpu, shape):
    device, queue = gpu
    rng = np.random.default_rng(29)
    half = seeded(shape, DataType.BF16, rng)
    wide = seeded(shape, DataType.F32, rng)
    # plant special values
    hp = random_payload(rng, shape, DataType.BF16).reshape(-1)
    hp[:len(SPECIAL_BF16)] = SPECIAL_BF16[:hp.size]
    half.view().copy_from_host(hp.reshape(shape))
    wp = random_payload(rng, shape, DataType.F32).reshape(-1).view(np.uint32)
    wp[:len(SPECIAL_F32)] = SPECIAL_F32[:wp.size]
    extra = np.array([0x3F808000, 0x3F818000, 0x3F808001, 0x7F7FFFFF, 0x7F7F8000, 0x00008000,
                      0x00018000, 0x80008001], dtype=np.uint32)   # ties, overflow, subnormal ties
    if wp.size >= len(SPECIAL_F32) + len(extra):
        wp[len(SPECIAL_F32):len(SPECIAL_F32) + len(extra)] = extra
    wide.view().copy_from_host(wp.reshape(shape))
    dh, dw = upload(device, half), upload(device, wide)
    out_w = seeded(shape, DataType.F32, rng)
    out_h = seeded(shape, DataType.BF16, rng)
    dow, doh = upload(device, out_w), upload(device, out_h)
    run(queue, queue.cast(dh.view(), dow.view()))
    run(queue, queue.cast(dw.view(), doh.view()))
    assert oracle().iomo_cast(abi(half.view()), abi(out_w.view())) == 0
    assert oracle().iomo_cast(abi(wide.view()), abi(out_h.view())) == 0
    assert np.array_equal(download(dow), out_w.storage)
    assert np.array_equal(download(doh), out_h.storage)


def test_cast_all_bf16_codes(gpu):
    device, queue = gpu
    codes = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    half = HostTensor((256, 256), DataType.BF16)
    half.view().copy_from_host(codes)
    wide = HostTensor((256, 256), DataType.F32)
    dh, dw = upload(device, half), upload(device, wide)
    run(queue, queue.cast(dh.view(), dw.view()))
    assert oracle().iomo_cast(abi(half.view()), abi(wide.view())) == 0
    assert np.array_equal(download(dw), wide.storage)
    back = HostTensor((256, 256), DataType.BF16)
    db = upload(device, back)
    run(queue, queue.cast(dw.view(), db.view()))
    assert oracle().iomo_cast(abi(wide.view()), abi(back.view())) == 0
    assert np.array_equal(download(db), back.storage)


@pytest.mark.parametrize("index_dtype", [DataType.U32, DataType.I64, DataType.U8, DataType.I16])
@pytest.mark.parametrize("payload", [DataType.BF16, DataType.F32, DataType.U8, DataType.U4, DataType.F6_E2M3,
                                     DataType.I2])
def test_embedding_parity(gpu, index_dtype, payload):
    device, queue = gpu
    rng = np.random.default_rng(13)
    vocab, feat, run_len = 50, 37, 19
    table = seeded((vocab, feat), payload, rng)
    ids = rng.integers(0, vocab, size=(2, 1, run_len)).astype(NUMPY_OF[index_dtype])
    idx = HostTensor((2, 1, run_len), index_dtype).poison()
    idx.view().copy_from_host(ids)
    out = seeded((2, run_len, feat), payload, rng)
    dt, di, do = upload(device, table), upload(device, idx), upload(device, out)
    ws = device.create_workspace(32)
    run(queue, queue.embedding(dt.view(), di.view(), do.view(), ws.view()))
    status = ctypes.c_uint32(9)
    assert oracle().iomo_embedding(abi(table.view()), abi(idx.view()), abi(out.view()),
                                   ctypes.byref(status)) == 0
    assert np.array_equal(download(do), out.storage)
    # invalid ids: retained failure on wait, valid rows only are written
    bad = ids.copy()
    bad[1, 0, 3] = vocab
    if index_dtype in (DataType.I64, DataType.I16):
        bad[0, 0, 5] = -1
    idx.view().copy_from_host(bad)
    di2 = upload(device, idx)
    token = queue.embedding(dt.view(), di2.view(), do.view(), ws.view())
    assert token > 0
    with pytest.raises(ValueError):
        queue.wait(token)
    with pytest.raises(ValueError):
        queue.wait(token)   # retained failures are rethrown on every wait
    # the next valid call resets the status word
    run(queue, queue.embedding(dt.view(), di.view(), do.view(), ws.view()))
    assert np.array_equal(download(do), out.storage)


def pack_lsb_first(values, bits):
    """Logical payload of a leaf narrower than a byte: codes packed LSB first, row-major."""
    flat = np.asarray(values, dtype=np.uint64).reshape(-1)
    out = np.zeros((flat.size * bits + 7) // 8, dtype=np.uint8)
    for i, code in enumerate(flat):
        bit = i * bits
        out[bit >> 3] |= np.uint8((int(code) << (bit & 7)) & 0xFF)
    return out


@pytest.mark.parametrize("index_dtype,bits,signed", [(DataType.U2, 2, False), (DataType.I2, 2, True),
                                                     (DataType.U4, 4, False), (DataType.I4, 4, True)])
@pytest.mark.parametrize("payload", [DataType.BF16, DataType.U4])
def test_embedding_index_leaves_narrower_than_a_byte(gpu, index_dtype, bits, signed, payload):
    """Ids of 2 and 4 bits (src/device_ops_embedding.cpp:27-46 admits every integer leaf):
    compared at full width, a set sign bit is a negative id."""
    device, queue = gpu
    rng = np.random.default_rng(bits * 10 + signed)
    largest = (1 << (bits - 1)) - 1 if signed else (1 << bits) - 1
    vocab, feat, run_len = largest, 37, 21         # the largest positive code is out of range
    table = seeded((vocab, feat), payload, rng)
    ids = rng.integers(0, vocab, size=(2, 1, run_len))
    idx = HostTensor((2, 1, run_len), index_dtype).poison()
    idx.view().copy_from_host(pack_lsb_first(ids, bits))
    out = seeded((2, run_len, feat), payload, rng)
    dt, di, do = upload(device, table), upload(device, idx), upload(device, out)
    ws = device.create_workspace(32)
    run(queue, queue.embedding(dt.view(), di.view(), do.view(), ws.view()))
    status = ctypes.c_uint32(9)
    assert oracle().iomo_embedding(abi(table.view()), abi(idx.view()), abi(out.view()),
                                   ctypes.byref(status)) == 0
    assert status.value == 0
    assert np.array_equal(download(do), out.storage)
    for bad_code in ([vocab] + ([(1 << bits) - 1] if signed else [])):   # too large; negative
        bad = ids.copy()
        bad[1, 0, 4] = bad_code
        idx.view().copy_from_host(pack_lsb_first(bad, bits))
        di2 = upload(device, idx)
        token = queue.embedding(dt.view(), di2.view(), do.view(), ws.view())
        assert token > 0
        with pytest.raises(ValueError):
            queue.wait(token)


def test_embedding_decode_shape(gpu):
    """TinyLlama decode geometry: [32000,2048] BF16 table, 64 ids."""
    device, queue = gpu
    rng = np.random.default_rng(4)
    table = HostTensor((32000, 2048), DataType.BF16)
    table.storage[:] = rng.integers(0, 256, size=table.storage.size, dtype=np.uint8)
    ids = rng.integers(0, 32000, size=(1, 64)).astype(np.uint32)
    idx = HostTensor((1, 64), DataType.U32)
    idx.view().copy_from_host(ids)
    out = HostTensor((64, 2048), DataType.BF16).poison()
    dt, di, do = upload(device, table), upload(device, idx), upload(device, out)
    ws = device.create_workspace(32)
    run(queue, queue.embedding(dt.view(), di.view(), do.view(), ws.view()))
    status = ctypes.c_uint32()
    assert oracle().iomo_embedding(abi(table.view()), abi(idx.view()), abi(out.view()),
                                   ctypes.byref(status)) == 0
    assert np.array_equal(download(do), out.storage)


@pytest.mark.parametrize("a", [0, 5, 29])
@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32, DataType.U8, DataType.U4, DataType.F6_E3M2,
                                   DataType.I2])
def test_cache_append_parity(gpu, a, dtype):
    device, queue = gpu
    rng = np.random.default_rng(17)
    src = seeded((2, 3, 3, 40), dtype, rng)
    dst = seeded((2, 3, 32, 40), dtype, rng)
    ds, dd = upload(device, src), upload(device, dst)
    run(queue, queue.cache_append(ds.view(), dd.view(), a))
    assert oracle().iomo_cache_append(abi(src.view()), abi(dst.view()), a) == 0
    assert np.array_equal(download(dd), dst.storage)
    assert queue.cache_append(ds.view(), dd.view(), 30) == -1
    assert queue.cache_append(ds.view(), dd.view(), 33) == -1


def test_cache_append_batched_equals_per_sequence_calls(gpu):
    """Decode geometry: K [64,4,1,64] into caches [64,4,2048,64] at per-sequence positions."""
    device, queue = gpu
    rng = np.random.default_rng(21)
    src = seeded((64, 4, 1, 64), DataType.BF16, rng)
    dst = seeded((64, 4, 2048, 64), DataType.BF16, rng)
    positions = rng.integers(0, 2047, size=64).astype(np.uint32)
    ds, dd = upload(device, src), upload(device, dst)
    pos = torch.from_numpy(positions.view(np.int32)).to(device.torch_device)
    status = torch.ones(1, dtype=torch.int32, device=device.torch_device)
    s, d = ds.view().as_abi(), dd.view().as_abi()
    rc = device._lib.iomb_cache_append_batched(ctypes.byref(s), ctypes.byref(d), pos.data_ptr(),
                                               status.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for b in range(64):
        assert oracle().iomo_cache_append(abi(src.view().select(0, b)),
                                          abi(dst.view().select(0, b)), int(positions[b])) == 0
    assert np.array_equal(download(dd), dst.storage)
    # the contract form: 64 calls on select(0, b) views
    dd2 = upload(device, seeded((64, 4, 2048, 64), DataType.BF16, np.random.default_rng(21)))
    # (same seed would differ in payload order; compare against a fresh oracle run instead)
    host2 = HostTensor((64, 4, 2048, 64), DataType.BF16, fill=None)
    host2.storage[:] = download(dd2)
    for b in range(64):
        token = queue.cache_append(ds.view().select(0, b), dd2.view().select(0, b), int(positions[b]))
        assert token > 0
        assert oracle().iomo_cache_append(abi(src.view().select(0, b)),
                                          abi(host2.view().select(0, b)), int(positions[b])) == 0
    queue.wait(token)
    assert np.array_equal(download(dd2), host2.storage)
    # an overrunning position sets the status word and skips that sequence
    positions[7] = 2048
    pos = torch.from_numpy(positions.view(np.int32)).to(device.torch_device)
    before = download(dd)
    rc = device._lib.iomb_cache_append_batched(ctypes.byref(s), ctypes.byref(d), pos.data_ptr(),
                                               status.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    after = download(dd)
    plane_bytes = 4 * 2048 * 64 * 2
    assert np.array_equal(after[7 * plane_bytes:8 * plane_bytes], before[7 * plane_bytes:8 * plane_bytes])


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
@pytest.mark.parametrize("shape", [(17, 33), (512, 2048), (3, 100, 700)])
def test_sumsq(gpu, dtype, shape):
    device, queue = gpu
    rng = np.random.default_rng(31)
    x = seeded(shape, dtype, rng, kind="normal")
    dx = upload(device, x)
    scratch = torch.full((device._lib.iomb_sumsq_scratch_bytes(),), 0x5A, dtype=torch.uint8,
                         device=device.torch_device)
    result = torch.zeros(2, dtype=torch.float32, device=device.torch_device)
    v = dx.view().as_abi()
    values = []
    for _ in range(2):
        rc = device._lib.iomb_sumsq(ctypes.byref(v), scratch.data_ptr(), result.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        values.append(result[0].item())
    truth = oracle().iomo_sumsq(abi(x.view()))
    assert values[0] == values[1]                      # run-to-run identical
    assert abs(values[0] - truth) <= 1e-6 * truth     # FP32 vs FP64 evaluation


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32, DataType.U8, DataType.I64,
                                   DataType.U2, DataType.I4, DataType.F6_E3M2])
def test_host_transfers(gpu, dtype):
    device, queue = gpu
    rng = np.random.default_rng(23)
    host = seeded((3, 2, 17, 35), dtype, rng)
    dev = upload(device, host)
    hv = host.view().permute([1, 0]).slice(1, 1, 2, 1)
    dv = like(hv, dev)
    need = dv.copy_to_host_workspace_requirements()
    ws = device.create_workspace(need.bytes + 32)
    assert np.array_equal(dv.copy_to_host(None, ws.view()), hv.copy_to_host())
    payload = random_payload(rng, hv.spec.shape, dtype)
    hv.copy_from_host(payload)
    dv.copy_from_host(payload, ws.view())
    assert np.array_equal(download(dev), host.storage)
    with pytest.raises(ValueError):
        dv.copy_from_host(payload, None)      # the staging workspace is mandatory
    # aligned rows take the vector path
    big = seeded((2, 64, 128), dtype, rng)
    dbig = upload(device, big)
    ws2 = device.create_workspace(big.spec.logical_nbytes() + 32)
    p2 = random_payload(rng, big.spec.shape, dtype)
    big.view().copy_from_host(p2)
    dbig.view().copy_from_host(p2, ws2.view())
    assert np.array_equal(download(dbig), big.storage)
    assert np.array_equal(dbig.view().copy_to_host(None, ws2.view()), big.view().copy_to_host())
