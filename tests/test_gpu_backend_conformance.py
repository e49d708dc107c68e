"""The C++ B200 backend behind the reference's own DeviceOps facade, side by
side with the reference CPU backend: identical calls, identical physical bytes.

Both devices live in oracle/_ref/libiomref_b200.so (reference common + CPU
sources compiled unmodified, iom_b200/backend/b200_backend.cpp, the shim). The
candidate's storage is seeded and observed with plain cudaMemcpy, independent
of the code under test, as the reference's CUDA storage oracle does.
"""
import numpy as np
import pytest

from iom_b200.tensor import DataType
from support import NUMPY_OF, REF_LIBS, Reference, SPECIAL_BF16, SPECIAL_F32, random_payload

pytestmark = pytest.mark.gpu
POISON = 0xA5


@pytest.fixture(scope="module")
def pair():
    if not REF_LIBS["b200"].exists():
        pytest.skip("libiomref_b200.so is not built (make -C oracle b200)")
    cpu = Reference("b200")
    gpu = Reference("b200", accelerator=True, arena_bytes=1 << 30)
    yield cpu, gpu
    gpu.close()
    cpu.close()


def both(pair, shape, dtype, rng, payload=None, kind="uniform"):
    """The same poisoned owner with the same logical payload on both devices."""
    if payload is None:
        payload = random_payload(rng, shape, dtype, kind)
    owners = []
    for ref in pair:
        tensor = ref.tensor(shape, dtype)
        tensor.write(np.full(tensor.nbytes, POISON, dtype=np.uint8))
        tensor.view().from_host(payload)
        owners.append(tensor)
    # the candidate's host transfer must produce the reference's physical bytes
    assert np.array_equal(owners[0].read(), owners[1].read()), "copy_from_host differs"
    return owners


def views(owners, steps=()):
    result = []
    for owner in owners:
        view = owner.view()
        for name, args in steps:
            view = getattr(view, name)(*args)
        result.append(view)
    return result


def same(owners):
    assert np.array_equal(owners[0].read(), owners[1].read())


@pytest.mark.parametrize("dtype", [DataType.I32, DataType.U32, DataType.F32, DataType.BF16,
                                   DataType.I8, DataType.U16, DataType.I64, DataType.F16,
                                   DataType.F8_E4M3FN, DataType.F8_E5M2, DataType.U4,
                                   DataType.F6_E2M3])
@pytest.mark.parametrize("op", [0, 1, 2, 3])
@pytest.mark.parametrize("shapes", [
    ((2, 17, 33), (2, 17, 33), (2, 17, 33)), ((2, 1, 33), (1, 17, 1), (2, 17, 33)),
    ((64, 256), (1, 256), (64, 256)), ((32, 48), (32, 1), (32, 48)), ((1, 1), (3, 20, 35), (3, 20, 35)),
])
def test_binary(pair, dtype, op, shapes):
    rng = np.random.default_rng(5)
    lhs, rhs, out = (both(pair, s, dtype, rng) for s in shapes)
    integer_division = op == 3 and dtype not in (DataType.F32, DataType.BF16, DataType.F16,
                                                 DataType.F8_E4M3FN, DataType.F8_E5M2, DataType.F6_E2M3)
    for i, ref in enumerate(pair):
        token = ref.lib.iomref_binary(ref.queue, op, lhs[i].view().handle, rhs[i].view().handle,
                                      out[i].view().handle)
        if integer_division:
            assert token == -2          # both backends: UnsupportedOperation at admission
            continue
        assert ref.run(token) == 0, ref.error()
    same(out)
    same(lhs)


def test_binary_views_alias_and_rejections(pair):
    rng = np.random.default_rng(6)
    lhs = both(pair, (4, 3, 17, 33), DataType.F32, rng)
    rhs = both(pair, (3, 4, 17, 33), DataType.F32, rng)
    out = both(pair, (2, 3, 17, 33), DataType.F32, rng)
    lv = views(lhs, [("slice", (0, 1, 2, 2))])
    rv = views(rhs, [("permute", ([1, 0],)), ("slice", (0, 0, 2, 1))])
    ov = views(out)
    other = views(lhs, [("slice", (0, 0, 2, 2))])   # same owner as lv, another window
    for i, ref in enumerate(pair):
        assert ref.run(ref.lib.iomref_binary(ref.queue, 0, lv[i].handle, rv[i].handle, ov[i].handle)) == 0
        # exact in-place alias
        assert ref.run(ref.lib.iomref_binary(ref.queue, 1, ov[i].handle, rv[i].handle, ov[i].handle)) == 0
        # the facade's own rejections arrive unchanged through the new backend
        assert ref.lib.iomref_binary(ref.queue, 0, ov[i].handle, other[i].handle, lv[i].handle) == -1
    same(out)
    # leaves no backend serves: explicit rejection, never a fallback
    cpu, gpu = pair
    flag = gpu.tensor((16, 16), DataType.BOOL)
    assert gpu.lib.iomref_binary(gpu.queue, 0, flag.view().handle, flag.view().handle,
                                 flag.view().handle) < 0
    # a view of the other device is rejected by device identity
    foreign = cpu.tensor((2, 3, 17, 33), DataType.F32)
    assert gpu.lib.iomref_binary(gpu.queue, 0, foreign.view().handle, rv[1].handle, ov[1].handle) == -1


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
@pytest.mark.parametrize("shape", [(15, 17), (17, 33), (2, 3, 16, 31), (64, 2048)])
def test_rmsnorm_within_contract_tolerance(pair, dtype, shape):
    """Through the facade the candidate runs the lane order (bit-identical to the
    reference's AVX-512 BF16 build); against this portable CPU build the contract
    allows one BF16 code / 2e-6 relative."""
    rng = np.random.default_rng(8)
    x = both(pair, shape, dtype, rng, kind="normal")
    w = both(pair, (1, shape[-1]), dtype, rng, kind="normal")
    out = both(pair, shape, dtype, rng)
    for i, ref in enumerate(pair):
        token = ref.lib.iomref_rmsnorm(ref.queue, x[i].view().handle, w[i].view().handle,
                                       out[i].view().handle, 1e-5)
        assert ref.run(token) == 0, ref.error()
        assert ref.lib.iomref_rmsnorm(ref.queue, x[i].view().handle, w[i].view().handle,
                                      x[i].view().handle, 1e-5) == -1   # output shares input
    a, b = out[0].read(), out[1].read()
    if dtype == DataType.BF16:
        assert np.max(np.abs(a.view(np.uint16).astype(np.int32) - b.view(np.uint16).astype(np.int32))) <= 1
    else:
        fa, fb = a.view(np.float32).astype(np.float64), b.view(np.float32).astype(np.float64)
        logical = np.abs(fa) < 1e30          # poisoned padding (0xA5A5A5A5) is identical anyway
        assert np.array_equal(a.view(np.uint32)[~logical], b.view(np.uint32)[~logical])
        assert np.all(np.abs(fa[logical] - fb[logical]) <= 2e-6 * np.abs(fa[logical]) + 1e-30)


def test_copy_embedding_cache_append(pair):
    rng = np.random.default_rng(9)
    src = both(pair, (3, 4, 17, 33), DataType.BF16, rng)
    dst = both(pair, (4, 3, 17, 33), DataType.BF16, rng)
    sv = views(src, [("slice", (1, 0, 2, 2))])
    dv = views(dst, [("permute", ([1, 0],)), ("slice", (1, 1, 2, 2))])
    for i, ref in enumerate(pair):
        assert ref.run(ref.lib.iomref_copy(ref.queue, sv[i].handle, dv[i].handle)) == 0
    same(dst)

    table = both(pair, (50, 37), DataType.BF16, rng)
    ids = rng.integers(0, 50, size=(2, 1, 19)).astype(np.uint32)
    idx = both(pair, (2, 1, 19), DataType.U32, rng, payload=ids)
    out = both(pair, (2, 19, 37), DataType.BF16, rng)
    for i, ref in enumerate(pair):
        token = ref.lib.iomref_embedding(ref.queue, table[i].view().handle, idx[i].view().handle,
                                         out[i].view().handle)
        assert ref.run(token) == 0, ref.error()
    same(out)
    bad = ids.copy()
    bad[1, 0, 3] = 50
    for i, ref in enumerate(pair):
        idx[i].view().from_host(bad)
        token = ref.lib.iomref_embedding(ref.queue, table[i].view().handle, idx[i].view().handle,
                                         out[i].view().handle)
        assert token > 0
        assert ref.run(token) == 1          # retained invalid_argument on wait
        assert ref.run(token) == 1          # ... on every wait

    for a in (0, 5, 29):
        s = both(pair, (2, 3, 3, 40), DataType.BF16, rng)
        d = both(pair, (2, 3, 32, 40), DataType.BF16, rng)
        for i, ref in enumerate(pair):
            assert ref.run(ref.lib.iomref_cache_append(ref.queue, s[i].view().handle,
                                                       d[i].view().handle, a)) == 0
            assert ref.lib.iomref_cache_append(ref.queue, s[i].view().handle, d[i].view().handle, 30) == -1
        same(d)

    # the leaves of 2, 4 and 6 bits: copy through transformed views and cache_append
    for dtype in (DataType.U4, DataType.F6_E2M3, DataType.I2):
        src = both(pair, (3, 4, 17, 33), dtype, rng)
        dst = both(pair, (4, 3, 17, 33), dtype, rng)
        sv = views(src, [("slice", (1, 0, 2, 2))])
        dv = views(dst, [("permute", ([1, 0],)), ("slice", (1, 1, 2, 2))])
        s = both(pair, (2, 3, 3, 40), dtype, rng)
        d = both(pair, (2, 3, 32, 40), dtype, rng)
        for i, ref in enumerate(pair):
            assert ref.run(ref.lib.iomref_copy(ref.queue, sv[i].handle, dv[i].handle)) == 0
            assert ref.run(ref.lib.iomref_cache_append(ref.queue, s[i].view().handle,
                                                       d[i].view().handle, 7)) == 0
        same(dst)
        same(d)
        table = both(pair, (50, 37), dtype, rng)
        idx = both(pair, (2, 1, 19), DataType.U32, rng, payload=ids)
        out = both(pair, (2, 19, 37), dtype, rng)
        for i, ref in enumerate(pair):
            token = ref.lib.iomref_embedding(ref.queue, table[i].view().handle, idx[i].view().handle,
                                             out[i].view().handle)
            assert ref.run(token) == 0, ref.error()
        same(out)


def test_silu_and_fused_gate(pair):
    """SiLU behind the facade: BF16 equals the reference CPU backend on every code;
    F32 stays within 4 ulp (FP64 against FP32 evaluation, as between the reference's
    own GPU and CPU backends). The fused gate extension equals silu then mul."""
    rng = np.random.default_rng(31)
    codes = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    x = both(pair, (256, 256), DataType.BF16, rng, payload=codes)
    y = both(pair, (256, 256), DataType.BF16, rng)
    for i, ref in enumerate(pair):
        assert ref.run(ref.lib.iomref_silu(ref.queue, x[i].view().handle, y[i].view().handle)) == 0, ref.error()
    same(y)
    xf = both(pair, (3, 17, 33), DataType.F32, rng, kind="normal")
    yf = both(pair, (3, 17, 33), DataType.F32, rng)
    for i, ref in enumerate(pair):
        assert ref.run(ref.lib.iomref_silu(ref.queue, xf[i].view().handle, yf[i].view().handle)) == 0, ref.error()
    a, b = (o.read().view(np.uint32).astype(np.int64) for o in yf)
    assert np.abs(a - b).max() <= 4
    cpu, gpu = pair
    # rejections arrive unchanged: in place, and a leaf outside the SiLU set
    assert gpu.lib.iomref_silu(gpu.queue, x[1].view().handle, x[1].view().handle) == -1
    i32 = gpu.tensor((16, 16), DataType.I32)
    j32 = gpu.tensor((16, 16), DataType.I32)
    assert gpu.lib.iomref_silu(gpu.queue, i32.view().handle, j32.view().handle) == -2
    # fused gate on the candidate equals its own silu followed by mul
    up = gpu.tensor((256, 256), DataType.BF16)
    up.view().from_host(random_payload(rng, (256, 256), DataType.BF16, "normal"))
    act, out, out2 = (gpu.tensor((256, 256), DataType.BF16) for _ in range(3))
    token = gpu.lib.iomref_silu_mul(gpu.queue, x[1].view().handle, up.view().handle,
                                    act.view().handle, out.view().handle)
    assert gpu.run(token) == 0, gpu.error()
    assert gpu.run(gpu.lib.iomref_binary(gpu.queue, 1, y[1].view().handle, up.view().handle,
                                         out2.view().handle)) == 0
    assert np.array_equal(act.read(), y[1].read())
    assert np.array_equal(out.read(), out2.read())
    token = gpu.lib.iomref_silu_mul(gpu.queue, x[1].view().handle, up.view().handle, None,
                                    out.view().handle)
    assert gpu.run(token) == 0, gpu.error()
    assert np.array_equal(out.read(), out2.read())


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
@pytest.mark.parametrize("shape,a", [((2, 3, 5, 64), 0), ((4, 17, 128), 7), ((1, 2, 33, 34), 2040)])
def test_rope(pair, dtype, shape, a):
    """RoPE behind the facade, candidate and reference CPU backend side by side, bit for
    bit; a second call at a later position grows the candidate's rotary cache."""
    rng = np.random.default_rng(51)
    x = both(pair, shape, dtype, rng, kind="normal")
    out = both(pair, shape, dtype, rng)
    for position in (a, a + 3000):
        for i, ref in enumerate(pair):
            token = ref.lib.iomref_rope(ref.queue, x[i].view().handle, out[i].view().handle,
                                        position, 10000.0)
            assert ref.run(token) == 0, ref.error()
        same(out)
    same(x)
    cpu, gpu = pair
    assert gpu.lib.iomref_rope(gpu.queue, x[1].view().handle, x[1].view().handle, 0, 10000.0) == -1
    assert gpu.lib.iomref_rope(gpu.queue, x[1].view().handle, out[1].view().handle, 0, 0.5) == -1


def test_extension_entries_of_the_cpp_backend(pair):
    """cast, batched cache_append and sumsq through the C++ backend's extension functions:
    cast against the oracle's codec, the batched append against one reference CPU
    cache_append per sequence, the sum of squares against FP64."""
    import ctypes
    from support import HostTensor, abi, oracle
    cpu, gpu = pair
    rng = np.random.default_rng(61)
    payload = random_payload(rng, (3, 17, 40), DataType.BF16, "normal")
    narrow = gpu.tensor((3, 17, 40), DataType.BF16)
    narrow.view().from_host(payload)
    wide = gpu.tensor((3, 17, 40), DataType.F32)
    assert gpu.run(gpu.lib.iomref_cast(gpu.queue, narrow.view().handle, wide.view().handle)) == 0, gpu.error()
    host_narrow, host_wide = HostTensor((3, 17, 40), DataType.BF16), HostTensor((3, 17, 40), DataType.F32)
    host_narrow.view().copy_from_host(payload)
    assert oracle().iomo_cast(abi(host_narrow.view()), abi(host_wide.view())) == 0
    assert np.array_equal(wide.read(), host_wide.storage)
    back = gpu.tensor((3, 17, 40), DataType.BF16)
    assert gpu.run(gpu.lib.iomref_cast(gpu.queue, wide.view().handle, back.view().handle)) == 0
    assert np.array_equal(back.read(), narrow.read())

    # batched append: 6 sequences, 2 heads, one new row each, per-sequence positions
    source = both(pair, (6, 2, 1, 48), DataType.BF16, rng, kind="normal")
    cache = both(pair, (6, 2, 40, 48), DataType.BF16, rng, kind="normal")
    positions = np.array([0, 39, 7, 16, 15, 31], dtype=np.uint32)
    status = ctypes.c_uint32(9)
    token = gpu.lib.iomref_cache_append_batched(
        gpu.queue, source[1].view().handle, cache[1].view().handle,
        positions.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), 6, ctypes.byref(status))
    assert token > 0 and status.value == 0
    for b in range(6):
        sv = source[0].view().select(0, b)
        cv = cache[0].view().select(0, b)
        assert cpu.run(cpu.lib.iomref_cache_append(cpu.queue, sv.handle, cv.handle, int(positions[b]))) == 0
    same(cache)
    positions[2] = 40                         # overruns: reported, that sequence skipped
    before = cache[1].read().copy()
    token = gpu.lib.iomref_cache_append_batched(
        gpu.queue, source[1].view().handle, cache[1].view().handle,
        positions.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), 6, ctypes.byref(status))
    assert token > 0 and status.value == 1
    assert np.array_equal(cache[1].read(), before)   # the other rows were rewritten with the same bytes

    x = gpu.tensor((5, 33, 70), DataType.F32)
    values = rng.standard_normal((5, 33, 70)).astype(np.float32)
    x.view().from_host(values)
    result = ctypes.c_float(0.0)
    assert gpu.lib.iomref_sumsq(gpu.queue, x.view().handle, ctypes.byref(result)) > 0
    truth = float(np.sum(values.astype(np.float64) ** 2))
    assert abs(result.value - truth) <= 1e-6 * truth


def test_attention_stage_extensions_of_the_cpp_backend(pair):
    """The attention stages through the C++ backend's extension functions: two launches and
    the fused one against the oracle (scores bit for bit up to NaN payloads, probabilities
    within one BF16 code), the fused stage equal to the two launches, and the output
    canonicalisation against its rule (-0 to +0, every NaN to 0x7FC0)."""
    import ctypes
    import torch
    from sdpa_stage_cases import random_case
    cpu, gpu = pair
    geometry = (2, 4, 2, 37, 64, 16, 5, 45)
    host = random_case(31, *geometry)
    raw_scores = host.scores.copy()
    packed = (ctypes.c_uint64 * 8)(*geometry)

    score_bytes = (raw_scores.nbytes + 31) // 32 * 32
    probability_codes = host.probability.astype(np.uint16)

    class Segments:
        """Scores and probabilities inside one workspace of the device, as the backend's
        attention path would place them."""

        def __init__(self):
            address = ctypes.c_void_p()
            self.owner = gpu.lib.iomref_workspace_create(
                gpu.device, score_bytes + probability_codes.nbytes, ctypes.byref(address))
            assert self.owner, gpu.error()
            self.scores = address.value
            self.probability = address.value + score_bytes
            source = raw_scores.copy()
            assert gpu.lib.iomref_memcpy_b200(self.scores, source.ctypes.data, source.nbytes, 1) == 0
            assert gpu.lib.iomref_memcpy_b200(self.probability, probability_codes.ctypes.data,
                                              probability_codes.nbytes, 1) == 0

        def stage(self, number):
            return gpu.lib.iomref_sdpa_stage_b200(gpu.queue, number, self.scores, self.probability,
                                                  packed, None, self.owner)

        def read(self):
            scores = np.empty_like(raw_scores)
            codes = np.empty_like(probability_codes)
            assert gpu.lib.iomref_memcpy_b200(scores.ctypes.data, self.scores, scores.nbytes, 0) == 0
            assert gpu.lib.iomref_memcpy_b200(codes.ctypes.data, self.probability, codes.nbytes, 0) == 0
            return scores, codes

    two = Segments()
    for stage in (0, 1):
        assert two.stage(stage) > 0
    kept = Segments()
    assert kept.stage(3) > 0
    read_only = Segments()
    assert read_only.stage(2) > 0
    s2, p2 = two.read()
    s1, p1 = kept.read()
    s0, p0 = read_only.read()
    assert np.array_equal(p1, p2) and np.array_equal(p0, p2)
    assert np.array_equal(s1.view(np.uint32), s2.view(np.uint32))
    assert np.array_equal(s0.view(np.uint32), raw_scores.view(np.uint32))   # only read
    host.scale_mask().softmax()
    same = (s2.view(np.uint32) == host.scores.view(np.uint32)) | (np.isnan(s2) & np.isnan(host.scores))
    assert same.all()
    distance = np.abs(p2.astype(np.int32) - host.probability.astype(np.int32))
    assert distance.max() <= 1 and (distance != 0).mean() <= 2e-3

    rng = np.random.default_rng(32)
    codes = rng.integers(0, 65536, size=(3, 19, 40), dtype=np.uint16)
    codes[0, 0, :4] = [0x8000, 0x7FFF, 0xFF81, 0x3F80]
    out = gpu.tensor((3, 19, 40), DataType.BF16)
    out.view().from_host(codes)
    assert gpu.lib.iomref_sdpa_stage_b200(gpu.queue, 4, None, None, packed, out.view().handle, None) > 0
    got = out.view().to_host()
    expected = codes.copy()
    zero = (codes & 0x7FFF) == 0
    nan = ((codes & 0x7F80) == 0x7F80) & ((codes & 0x007F) != 0)
    expected[zero] = 0
    expected[nan] = 0x7FC0
    assert np.array_equal(np.asarray(got).view(np.uint16).reshape(codes.shape), expected)


def test_host_transfers_and_fused_extension(pair):
    cpu, gpu = pair
    rng = np.random.default_rng(10)
    for dtype in (DataType.BF16, DataType.F32, DataType.U8, DataType.I64):
        owners = both(pair, (3, 2, 17, 35), dtype, rng)
        tv = views(owners, [("permute", ([1, 0],)), ("slice", (1, 1, 2, 1))])
        assert np.array_equal(tv[0].to_host(), tv[1].to_host())
        payload = random_payload(rng, (2, 2, 17, 35), dtype)
        for v in tv:
            v.from_host(payload)
        same(owners)
    # fused residual ADD + RMSNorm equals add then rmsnorm on the candidate itself
    shape = (40, 2048)
    x = gpu.tensor(shape, DataType.BF16)
    r = gpu.tensor(shape, DataType.BF16)
    w = gpu.tensor((1, 2048), DataType.BF16)
    s1, s2, n1, n2 = (gpu.tensor(shape, DataType.BF16) for _ in range(4))
    x.view().from_host(random_payload(rng, shape, DataType.BF16, "normal"))
    r.view().from_host(random_payload(rng, shape, DataType.BF16, "normal"))
    w.view().from_host(random_payload(rng, (1, 2048), DataType.BF16, "normal"))
    token = gpu.lib.iomref_add_rmsnorm(gpu.queue, x.view().handle, r.view().handle, w.view().handle,
                                       s1.view().handle, n1.view().handle, 1e-5)
    assert gpu.run(token) == 0, gpu.error()
    assert gpu.run(gpu.lib.iomref_binary(gpu.queue, 0, x.view().handle, r.view().handle, s2.view().handle)) == 0
    assert gpu.run(gpu.lib.iomref_rmsnorm(gpu.queue, s2.view().handle, w.view().handle, n2.view().handle, 1e-5)) == 0
    assert np.array_equal(s1.read(), s2.read())
    assert np.array_equal(n1.read(), n2.read())
    # the CPU reference computes the same stored sum
    cx = cpu.tensor(shape, DataType.BF16)
    cr = cpu.tensor(shape, DataType.BF16)
    cs = cpu.tensor(shape, DataType.BF16)
    cx.view().from_host(x.view().to_host())
    cr.view().from_host(r.view().to_host())
    assert cpu.run(cpu.lib.iomref_binary(cpu.queue, 0, cx.view().handle, cr.view().handle, cs.view().handle)) == 0
    assert np.array_equal(cs.read(), s1.read())


def test_queue_limits_and_tokens(pair):
    _, gpu = pair
    queues = []
    for _ in range(3):                       # one queue already exists: four is the cap
        handle = gpu.lib.iomref_queue_create(gpu.device)
        assert handle, gpu.error()
        queues.append(handle)
    assert not gpu.lib.iomref_queue_create(gpu.device)      # the fifth is bad_alloc
    for handle in queues:
        gpu.lib.iomref_queue_destroy(handle)
    assert gpu.lib.iomref_wait(gpu.queue, 12345) == 1       # foreign / never submitted token
    assert gpu.lib.iomref_wait(gpu.queue, -1) == 1
