"""Pins the plain-C oracle against the unmodified reference CPU backend.

Each case seeds identical physical storage on both sides (including poisoned
padding), runs the operation through the reference's own DeviceOps facade and
through the oracle, and compares every byte of the owners' tiled storage.
"""
import ctypes

import numpy as np
import pytest

from iom_b200.tensor import DataType
from support import (HostTensor, SPECIAL_BF16, SPECIAL_F32, abi, oracle, random_payload,
                     reference_or_skip)

OPS = {"add": 0, "mul": 1, "sub": 2, "div": 3}


@pytest.fixture(scope="module", params=["portable", "avx512"])
def ref(request):
    reference = reference_or_skip(request.param)
    yield reference
    reference.close()


def mirror(ref, shape, dtype, rng, poison=0xA5, payload=None, kind="uniform"):
    """Creates the same owner on both sides: poisoned storage + seeded logical payload."""
    host = HostTensor(shape, dtype).poison(poison)
    theirs = ref.tensor(shape, dtype)
    theirs.storage[:] = poison
    if payload is None:
        payload = random_payload(rng, shape, dtype, kind)
    host.view().copy_from_host(payload)
    theirs.view().from_host(payload)
    assert np.array_equal(host.storage, theirs.storage), "scatter differs from the reference"
    return host, theirs


def apply(view, ref_view, steps):
    for name, args in steps:
        view = getattr(view, name)(*args)
        ref_view = getattr(ref_view, name)(*args)
    dims, offset, strides, _ = ref_view.describe()
    assert dims == view.spec.shape and offset == view.plane_offset
    assert strides == view.plane_strides
    return view, ref_view


BINARY_CASES = [
    # (lhs shape, rhs shape, out shape)
    ((2, 17, 33), (2, 17, 33), (2, 17, 33)),
    ((2, 1, 33), (1, 17, 1), (2, 17, 33)),
    ((32, 48), (1, 48), (32, 48)),
    ((32, 48), (32, 1), (32, 48)),
    ((1, 1), (3, 20, 35), (3, 20, 35)),
    ((2, 3, 16, 16), (3, 1, 16), (2, 3, 16, 16)),
    ((5, 31), (1, 1), (5, 31)),
]


@pytest.mark.parametrize("dtype", [DataType.I32, DataType.U32, DataType.F32, DataType.BF16,
                                   DataType.I8, DataType.U8, DataType.I16, DataType.U16,
                                   DataType.I64, DataType.U64, DataType.F16,
                                   DataType.F8_E4M3FN, DataType.F8_E5M2,
                                   DataType.I2, DataType.U2, DataType.I4, DataType.U4,
                                   DataType.F4_E2M1, DataType.F6_E2M3, DataType.F6_E3M2])
@pytest.mark.parametrize("op", ["add", "mul", "sub", "div"])
@pytest.mark.parametrize("shapes", BINARY_CASES)
def test_binary_matches_reference(ref, dtype, op, shapes):
    if op == "div" and dtype not in (DataType.F32, DataType.BF16, DataType.F16, DataType.F8_E4M3FN,
                                     DataType.F8_E5M2, DataType.F4_E2M1, DataType.F6_E2M3,
                                     DataType.F6_E3M2):
        pytest.skip("the reference admits no integer division")
    rng = np.random.default_rng(hash((int(dtype), op, shapes)) & 0xFFFF)
    lhs, rlhs = mirror(ref, shapes[0], dtype, rng)
    rhs, rrhs = mirror(ref, shapes[1], dtype, rng)
    out, rout = mirror(ref, shapes[2], dtype, rng)
    token = ref.lib.iomref_binary(ref.queue, OPS[op], rlhs.view().handle, rrhs.view().handle,
                                  rout.view().handle)
    assert ref.run(token) == 0, ref.error()
    for ieee in (0, 1):
        mine = out.clone()
        assert oracle().iomo_binary(OPS[op], abi(lhs.view()), abi(rhs.view()),
                                    abi(mine.view()), ieee) == 0
        assert np.array_equal(mine.storage, rout.storage), f"ieee={ieee}"


@pytest.mark.parametrize("dtype,specials", [(DataType.F32, SPECIAL_F32), (DataType.BF16, SPECIAL_BF16)])
@pytest.mark.parametrize("op", ["add", "mul"])
def test_binary_special_values(ref, dtype, op, specials):
    n = len(specials)
    a = np.repeat(specials, n).reshape(n, n)
    b = np.tile(specials, n).reshape(n, n)
    rng = np.random.default_rng(0)
    lhs, rlhs = mirror(ref, (n, n), dtype, rng, payload=a)
    rhs, rrhs = mirror(ref, (n, n), dtype, rng, payload=b)
    out, rout = mirror(ref, (n, n), dtype, rng)
    token = ref.lib.iomref_binary(ref.queue, OPS[op], rlhs.view().handle, rrhs.view().handle,
                                  rout.view().handle)
    assert ref.run(token) == 0
    for ieee in (0, 1):
        mine = out.clone()
        assert oracle().iomo_binary(OPS[op], abi(lhs.view()), abi(rhs.view()),
                                    abi(mine.view()), ieee) == 0
        assert np.array_equal(mine.storage, rout.storage)


def test_binary_sliced_views_and_alias(ref):
    rng = np.random.default_rng(7)
    lhs, rlhs = mirror(ref, (4, 3, 17, 33), DataType.F32, rng)
    rhs, rrhs = mirror(ref, (3, 4, 17, 33), DataType.F32, rng)
    out, rout = mirror(ref, (2, 3, 17, 33), DataType.F32, rng)
    lv, rlv = apply(lhs.view(), rlhs.view(), [("slice", (0, 1, 2, 2))])
    rv, rrv = apply(rhs.view(), rrhs.view(), [("permute", ([1, 0],)), ("slice", (0, 0, 2, 1))])
    ov, rov = out.view(), rout.view()
    token = ref.lib.iomref_binary(ref.queue, 0, rlv.handle, rrv.handle, rov.handle)
    assert ref.run(token) == 0, ref.error()
    assert oracle().iomo_binary(0, abi(lv), abi(rv), abi(ov), 0) == 0
    assert np.array_equal(out.storage, rout.storage)
    # exact in-place alias: out is lhs
    token = ref.lib.iomref_binary(ref.queue, 1, rov.handle, rrv.handle, rov.handle)
    assert ref.run(token) == 0, ref.error()
    assert oracle().iomo_binary(1, abi(ov), abi(rv), abi(ov), 1) == 0
    assert np.array_equal(out.storage, rout.storage)


RMS_SHAPES = [(1, 1), (15, 17), (16, 16), (17, 33), (2, 3, 16, 31), (33, 15), (4, 256)]


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
@pytest.mark.parametrize("shape", RMS_SHAPES)
@pytest.mark.parametrize("eps", [0.0, 1e-5, 1e-6])
def test_rmsnorm_matches_reference(ref, dtype, shape, eps):
    rng = np.random.default_rng(hash((int(dtype), shape)) & 0xFFFF)
    x, rx = mirror(ref, shape, dtype, rng, kind="normal")
    w, rw = mirror(ref, (1, shape[-1]), dtype, rng, kind="normal")
    out, rout = mirror(ref, shape, dtype, rng)
    token = ref.lib.iomref_rmsnorm(ref.queue, rx.view().handle, rw.view().handle,
                                   rout.view().handle, eps)
    assert ref.run(token) == 0, ref.error()
    order = 0 if ref.kind == "avx512" else 1
    assert oracle().iomo_rmsnorm(abi(x.view()), abi(w.view()), abi(out.view()), eps, order) == 0
    assert np.array_equal(out.storage, rout.storage)


@pytest.mark.parametrize("dtype,specials", [(DataType.F32, SPECIAL_F32), (DataType.BF16, SPECIAL_BF16)])
def test_rmsnorm_special_rows(ref, dtype, specials):
    """Rows holding inf / NaN / subnormals / huge values; non-finite scale."""
    rng = np.random.default_rng(3)
    n = len(specials)
    base = random_payload(rng, (n + 2, 40), dtype, "normal")
    raw = base.view(np.uint32 if dtype == DataType.F32 else np.uint16)
    for i, code in enumerate(specials):
        raw[i, (3 * i) % 40] = code
    raw[n, :] = specials[4]          # every element max finite: accumulator overflow
    raw[n + 1, :] = specials[8]      # every element min subnormal: accumulator underflow
    scale = random_payload(rng, (1, 40), dtype, "normal")
    sraw = scale.view(np.uint32 if dtype == DataType.F32 else np.uint16)
    sraw[0, 5] = specials[10]
    sraw[0, 6] = specials[12]
    x, rx = mirror(ref, (n + 2, 40), dtype, rng, payload=base)
    w, rw = mirror(ref, (1, 40), dtype, rng, payload=scale)
    out, rout = mirror(ref, (n + 2, 40), dtype, rng)
    for eps in (0.0, 1e-5, float(np.finfo(np.float32).max)):
        token = ref.lib.iomref_rmsnorm(ref.queue, rx.view().handle, rw.view().handle,
                                       rout.view().handle, eps)
        assert ref.run(token) == 0, ref.error()
        order = 0 if ref.kind == "avx512" else 1
        assert oracle().iomo_rmsnorm(abi(x.view()), abi(w.view()), abi(out.view()), eps, order) == 0
        assert np.array_equal(out.storage, rout.storage)


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32, DataType.U8, DataType.I64,
                                   DataType.I2, DataType.U4, DataType.F4_E2M1, DataType.F6_E2M3])
def test_copy_matches_reference(ref, dtype):
    rng = np.random.default_rng(11)
    src, rsrc = mirror(ref, (3, 4, 17, 33), dtype, rng)
    dst, rdst = mirror(ref, (4, 3, 17, 33), dtype, rng)
    sv, rsv = apply(src.view(), rsrc.view(), [("slice", (1, 0, 2, 2))])
    dv, rdv = apply(dst.view(), rdst.view(), [("permute", ([1, 0],)), ("slice", (1, 1, 2, 2))])
    token = ref.lib.iomref_copy(ref.queue, rsv.handle, rdv.handle)
    assert ref.run(token) == 0, ref.error()
    assert oracle().iomo_copy(abi(sv), abi(dv)) == 0
    assert np.array_equal(dst.storage, rdst.storage)


def test_silu_every_bf16_code_matches_reference(ref):
    """All 65 536 BF16 codes through the reference CPU backend's SiLU (portable and
    AVX-512 builds run the same FP32 evaluation) against the oracle's FP32 carrier."""
    codes = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    x, rx = mirror(ref, (256, 256), DataType.BF16, np.random.default_rng(1), payload=codes)
    y, ry = mirror(ref, (256, 256), DataType.BF16, np.random.default_rng(2))
    assert ref.run(ref.lib.iomref_silu(ref.queue, rx.view().handle, ry.view().handle)) == 0, ref.error()
    assert oracle().iomo_silu(abi(x.view()), abi(y.view()), 0) == 0
    assert np.array_equal(y.storage, ry.storage)


@pytest.mark.parametrize("dtype", [DataType.F32, DataType.BF16, DataType.F16])
def test_silu_views_and_ragged_extents_match_reference(ref, dtype):
    rng = np.random.default_rng(21)
    payload = random_payload(rng, (3, 2, 17, 33), dtype, "normal") if dtype != DataType.F16 \
        else rng.integers(0, 1 << 16, size=(3, 2, 17, 33), dtype=np.uint16)
    if dtype == DataType.F32:
        payload = (payload * np.float32(6.0)).astype(np.float32)
        flat = payload.reshape(-1).view(np.uint32)
        flat[:SPECIAL_F32.size] = SPECIAL_F32
        flat[100:104] = np.array([-90.0, -104.0, 88.0, -0.0], dtype=np.float32).view(np.uint32)
    x, rx = mirror(ref, (3, 2, 17, 33), dtype, rng, payload=payload)
    y, ry = mirror(ref, (2, 3, 17, 33), dtype, rng)
    xv, rxv = apply(x.view(), rx.view(), [("permute", ([1, 0],))])
    yv, ryv = y.view(), ry.view()
    assert ref.run(ref.lib.iomref_silu(ref.queue, rxv.handle, ryv.handle)) == 0, ref.error()
    assert oracle().iomo_silu(abi(xv), abi(yv), 0) == 0
    assert np.array_equal(y.storage, ry.storage)
    # in-place and cross-shape requests are rejected by the reference; the oracle agrees
    assert ref.lib.iomref_silu(ref.queue, rx.view().handle, rx.view().handle) == -1
    assert oracle().iomo_silu(abi(x.view()), abi(x.view()), 0) == 1


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
@pytest.mark.parametrize("shape,a", [((2, 3, 5, 64), 0), ((4, 17, 128), 7), ((1, 2, 33, 34), 2040),
                                     ((2, 1, 1, 6), 123456)])
@pytest.mark.parametrize("theta", [10000.0, 500000.0, 1.0])
def test_rope_matches_reference(ref, dtype, shape, a, theta):
    """Split-half RoPE: both reference CPU builds against the oracle, including the
    raw-copy row at position 0, ragged widths and transformed leading views."""
    rng = np.random.default_rng(41 + len(shape))
    payload = random_payload(rng, shape, dtype, "normal")
    if dtype == DataType.F32:
        flat = payload.reshape(-1).view(np.uint32)
        count = min(flat.size, SPECIAL_F32.size)
        flat[:count] = SPECIAL_F32[:count]
    else:
        flat = payload.reshape(-1)
        count = min(flat.size, SPECIAL_BF16.size)
        flat[:count] = SPECIAL_BF16[:count]
    x, rx = mirror(ref, shape, dtype, rng, payload=payload)
    out, rout = mirror(ref, shape, dtype, rng)
    token = ref.lib.iomref_rope(ref.queue, rx.view().handle, rout.view().handle, a, theta)
    assert ref.run(token) == 0, ref.error()
    assert oracle().iomo_rope(abi(x.view()), abi(out.view()), a, theta) == 0
    assert np.array_equal(out.storage, rout.storage)


def test_rope_views_and_rejections_match_reference(ref):
    rng = np.random.default_rng(43)
    x, rx = mirror(ref, (3, 2, 9, 32), DataType.BF16, rng, kind="normal")
    out, rout = mirror(ref, (2, 3, 9, 32), DataType.BF16, rng)
    xv, rxv = apply(x.view(), rx.view(), [("permute", ([1, 0],))])
    assert ref.run(ref.lib.iomref_rope(ref.queue, rxv.handle, rout.view().handle, 5, 10000.0)) == 0
    assert oracle().iomo_rope(abi(xv), abi(out.view()), 5, 10000.0) == 0
    assert np.array_equal(out.storage, rout.storage)
    # in place, odd width, rank two and theta below one are rejected by both
    assert ref.lib.iomref_rope(ref.queue, rx.view().handle, rx.view().handle, 0, 10000.0) == -1
    assert oracle().iomo_rope(abi(x.view()), abi(x.view()), 0, 10000.0) == 1
    assert ref.lib.iomref_rope(ref.queue, rxv.handle, rout.view().handle, 0, 0.5) == -1
    assert oracle().iomo_rope(abi(xv), abi(out.view()), 0, 0.5) == 1
    odd, rodd = mirror(ref, (2, 4, 33), DataType.BF16, rng)
    odd2, rodd2 = mirror(ref, (2, 4, 33), DataType.BF16, rng)
    assert ref.lib.iomref_rope(ref.queue, rodd.view().handle, rodd2.view().handle, 0, 10000.0) == -1
    assert oracle().iomo_rope(abi(odd.view()), abi(odd2.view()), 0, 10000.0) == 1


@pytest.mark.parametrize("payload", [DataType.BF16, DataType.U4, DataType.F6_E2M3, DataType.I2])
@pytest.mark.parametrize("index_dtype", [DataType.U32, DataType.I64, DataType.U8, DataType.I16])
def test_embedding_matches_reference(ref, index_dtype, payload):
    rng = np.random.default_rng(13)
    vocab, feat, run = 50, 37, 19
    table, rtable = mirror(ref, (vocab, feat), payload, rng)
    ids = rng.integers(0, vocab, size=(2, 1, run)).astype(
        {DataType.U32: np.uint32, DataType.I64: np.int64, DataType.U8: np.uint8,
         DataType.I16: np.int16}[index_dtype])
    idx, ridx = mirror(ref, (2, 1, run), index_dtype, rng, payload=ids)
    out, rout = mirror(ref, (2, run, feat), payload, rng)
    token = ref.lib.iomref_embedding(ref.queue, rtable.view().handle, ridx.view().handle,
                                     rout.view().handle)
    assert ref.run(token) == 0, ref.error()
    status = ctypes.c_uint32(9)
    assert oracle().iomo_embedding(abi(table.view()), abi(idx.view()), abi(out.view()),
                                   ctypes.byref(status)) == 0
    assert status.value == 0
    assert np.array_equal(out.storage, rout.storage)
    # an out-of-range id is a retained invalid_argument in the reference, status 1 here
    ids[1, 0, 3] = vocab
    idx.view().copy_from_host(ids)
    ridx.view().from_host(ids)
    before = out.storage.copy()
    token = ref.lib.iomref_embedding(ref.queue, rtable.view().handle, ridx.view().handle,
                                     rout.view().handle)
    assert token > 0 and ref.run(token) == 1
    assert oracle().iomo_embedding(abi(table.view()), abi(idx.view()), abi(out.view()),
                                   ctypes.byref(status)) == 0
    assert status.value == 1
    assert np.array_equal(out.storage, before) and np.array_equal(rout.storage, before)


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.U4, DataType.F6_E3M2, DataType.I2])
@pytest.mark.parametrize("a", [0, 5, 29])
def test_cache_append_matches_reference(ref, a, dtype):
    rng = np.random.default_rng(17)
    src, rsrc = mirror(ref, (2, 3, 3, 40), dtype, rng)
    dst, rdst = mirror(ref, (2, 3, 32, 40), dtype, rng)
    token = ref.lib.iomref_cache_append(ref.queue, rsrc.view().handle, rdst.view().handle, a)
    assert ref.run(token) == 0, ref.error()
    assert oracle().iomo_cache_append(abi(src.view()), abi(dst.view()), a) == 0
    assert np.array_equal(dst.storage, rdst.storage)


def test_cache_append_rejects_overrun(ref):
    rng = np.random.default_rng(19)
    src, rsrc = mirror(ref, (2, 3, 3, 40), DataType.BF16, rng)
    dst, rdst = mirror(ref, (2, 3, 32, 40), DataType.BF16, rng)
    assert ref.lib.iomref_cache_append(ref.queue, rsrc.view().handle, rdst.view().handle, 30) == -1
    assert oracle().iomo_cache_append(abi(src.view()), abi(dst.view()), 30) == 1


def test_host_transfer_matches_reference(ref):
    rng = np.random.default_rng(23)
    for dtype in (DataType.BF16, DataType.F32, DataType.U8, DataType.I64):
        host, theirs = mirror(ref, (3, 2, 17, 35), dtype, rng)
        hv, rv = apply(host.view(), theirs.view(), [("permute", ([1, 0],)), ("slice", (1, 1, 2, 1))])
        assert np.array_equal(hv.copy_to_host(), rv.to_host())
        payload = random_payload(rng, hv.spec.shape, dtype)
        hv.copy_from_host(payload)
        rv.from_host(payload)
        assert np.array_equal(host.storage, theirs.storage)
