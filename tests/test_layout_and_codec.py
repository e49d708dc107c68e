"""Known-answer tests the reference's own suites hold for the tile map and the
scalar codec, applied to the oracle (and to the Python/ABI layout helpers)."""
import ctypes

import numpy as np
import pytest

from iom_b200.tensor import DataType, plane_slot
from support import HostTensor, oracle

ADD, MUL, SUB, DIV = 0, 1, 2, 3


def slot(shape, coords):
    rows, cols = shape[-2], shape[-1]
    plane = 0
    for extent, c in zip(shape[:-2], coords[:-2]):
        plane = plane * extent + c
    return plane_slot(rows, cols, plane, coords[-2], coords[-1])


def test_tile_map_known_answers():
    # test/test_iom.cpp:614-655
    assert slot((32, 32), (0, 16)) == 256
    assert slot((32, 32), (16, 0)) == 512
    assert slot((32, 32), (31, 31)) == 3 * 256 + 255
    assert slot((2, 8, 31, 33), (0, 1, 0, 0)) == 6 * 256
    assert slot((20, 35), (0, 34)) == 2 * 256 + 2


def test_physical_placement_known_answer():
    # test/cpu/test_cpu.cpp:760-795: F32 [1,32], logical element 16 lives at byte
    # 1024 and byte 64 keeps the sentinel.
    t = HostTensor((1, 32), DataType.F32).poison(0xAA)
    payload = np.arange(32, dtype=np.float32)
    t.view().copy_from_host(payload)
    assert t.storage[1024:1028].view(np.float32)[0] == 16.0
    assert t.storage[64] == 0xAA
    assert t.storage[0:64].view(np.float32).tolist() == list(range(16))


def binary(op, dtype, a, b):
    return oracle().iomo_scalar_binary(op, int(dtype), a, b)


def test_codec_known_answers():
    # test/backend/test_scalar_add.cpp:40-61
    assert binary(MUL, DataType.U64, 0xFFFFFFFFFFFFFFFF, 3) == 0xFFFFFFFFFFFFFFFD
    assert binary(MUL, DataType.I32, 0x80000000, 3) == 0x80000000
    assert binary(SUB, DataType.U16, 0, 1) == 0xFFFF
    assert binary(SUB, DataType.I64, 0, 1) == 0xFFFFFFFFFFFFFFFF
    assert binary(MUL, DataType.F32, 0x7F800000, 0) == 0x7FC00000
    assert binary(SUB, DataType.F32, 0x7F800000, 0x7F800000) == 0x7FC00000
    assert binary(DIV, DataType.F32, 0, 0) == 0x7FC00000
    assert binary(DIV, DataType.F32, 0x80000000, 1) == 0x80000000
    assert binary(DIV, DataType.F32, 0x80000000, 0x80000000) == 0x7FC00000
    assert binary(DIV, DataType.F32, 0x3F800000, 0x7F800000) == 0
    assert binary(ADD, DataType.F16, 0x7C00, 0xFC00) == 0x7E00
    assert binary(ADD, DataType.F32, 0x80000000, 0) == 0
    assert binary(ADD, DataType.F32, 0x3F800000, 0x3F800000) == 0x40000000


@pytest.mark.parametrize("dtype,maximum,two,half,infinity,sign", [
    (DataType.F8_E5M2, 0x7B, 0x40, 0x38, 0x7C, 0x80),
    (DataType.F16, 0x7BFF, 0x4000, 0x3800, 0x7C00, 0x8000),
    (DataType.BF16, 0x7F7F, 0x4000, 0x3F00, 0x7F80, 0x8000),
    (DataType.F32, 0x7F7FFFFF, 0x40000000, 0x3F000000, 0x7F800000, 0x80000000),
    (DataType.F64, 0x7FEFFFFFFFFFFFFF, 0x4000000000000000, 0x3FE0000000000000,
     0x7FF0000000000000, 0x8000000000000000),
])
def test_codec_overflow_known_answers(dtype, maximum, two, half, infinity, sign):
    # test/backend/test_scalar_add.cpp:63-132
    assert binary(ADD, dtype, maximum, maximum) == infinity
    assert binary(MUL, dtype, maximum, two) == infinity
    assert binary(SUB, dtype, maximum, maximum | sign) == infinity
    assert binary(DIV, dtype, maximum, half) == infinity
    assert binary(ADD, dtype, maximum | sign, maximum | sign) == infinity | sign
    assert binary(MUL, dtype, maximum | sign, two) == infinity | sign
    assert binary(SUB, dtype, maximum | sign, maximum) == infinity | sign


@pytest.mark.parametrize("dtype,maximum,two,sign", [
    (DataType.F4_E2M1, 0x7, 0x4, 0x8), (DataType.F6_E2M3, 0x1F, 0x10, 0x20),
    (DataType.F6_E3M2, 0x1F, 0x10, 0x20), (DataType.F8_E4M3FN, 0x77, 0x40, 0x80),
])
def test_codec_finite_only_saturates(dtype, maximum, two, sign):
    # test/backend/test_scalar_add.cpp:134-152
    assert binary(MUL, dtype, maximum, two) == maximum
    assert binary(MUL, dtype, maximum | sign, two) == maximum | sign


def boundary_bf16():
    mant = [0, 1, 2, 0x3F, 0x40, 0x41, 0x7E, 0x7F]
    exps = list(range(0, 4)) + list(range(60, 68)) + list(range(118, 138)) + list(range(186, 194)) \
        + list(range(250, 256))
    codes = [(s << 15) | (e << 7) | m for s in (0, 1) for e in exps for m in mant]
    return np.array(codes, dtype=np.uint16)


@pytest.mark.parametrize("op", [ADD, MUL, SUB, DIV])
def test_ieee_form_equals_codec_bf16(op):
    """Every BF16 code against a boundary-rich set: the arithmetic the kernels
    implement (binary32 op, RNE, canonical NaN) equals the reference codec."""
    a = np.arange(65536, dtype=np.uint16)
    b = boundary_bf16()
    mismatches = oracle().iomo_codec_mismatches(op, int(DataType.BF16), a.ctypes.data, a.size,
                                                b.ctypes.data, b.size)
    assert mismatches == 0


@pytest.mark.parametrize("op", [ADD, MUL, SUB, DIV])
def test_ieee_form_equals_codec_f16(op):
    """Every F16 code against a boundary-rich set: a binary32 operation followed by one
    RNE narrowing to binary16 equals the reference codec (24 >= 2 * 11 + 2)."""
    a = np.arange(65536, dtype=np.uint16)
    mant = np.array([0, 1, 2, 0x1FF, 0x200, 0x201, 0x3FE, 0x3FF], dtype=np.uint16)
    exps = np.array([0, 1, 2, 14, 15, 16, 29, 30, 31, 10, 20, 25], dtype=np.uint16)
    b = np.array([(s << 15) | (e << 10) | m for s in (0, 1) for e in exps for m in mant],
                 dtype=np.uint16)
    mismatches = oracle().iomo_codec_mismatches(op, int(DataType.F16), a.ctypes.data, a.size,
                                                b.ctypes.data, b.size)
    assert mismatches == 0


@pytest.mark.parametrize("dtype", [DataType.F8_E4M3FN, DataType.F8_E5M2])
@pytest.mark.parametrize("op", [ADD, MUL, SUB, DIV])
def test_ieee_form_equals_codec_f8_every_pair(op, dtype):
    """All 65 536 pairs of the 8-bit floating leaves: exact decode, one binary32 operation and
    one encode by the codec's rules equal the reference codec's long double evaluation."""
    codes = np.arange(256, dtype=np.uint8)
    assert oracle().iomo_codec_mismatches(op, int(dtype), codes.ctypes.data, 256, codes.ctypes.data, 256) == 0


@pytest.mark.parametrize("dtype,bits", [(DataType.F4_E2M1, 4), (DataType.F6_E2M3, 6), (DataType.F6_E3M2, 6),
                                        (DataType.I2, 2), (DataType.U2, 2), (DataType.I4, 4), (DataType.U4, 4)])
@pytest.mark.parametrize("op", [ADD, MUL, SUB, DIV])
def test_ieee_form_equals_codec_every_pair_of_the_narrow_leaves(op, dtype, bits):
    """Every pair of codes of the leaves narrower than a byte. The small floats have no NaN
    and no infinity: such a result encodes to the largest value (a NaN to the positive one)."""
    if op == DIV and dtype in (DataType.I2, DataType.U2, DataType.I4, DataType.U4):
        pytest.skip("the reference admits no integer division")
    codes = np.arange(1 << bits, dtype=np.uint8)
    assert oracle().iomo_codec_mismatches(op, int(dtype), codes.ctypes.data, codes.size,
                                          codes.ctypes.data, codes.size) == 0


def test_narrow_float_known_codes():
    assert binary(DIV, DataType.F4_E2M1, 0x0, 0x0) == 0x7        # 0 / 0: NaN -> +6, the largest value
    assert binary(DIV, DataType.F4_E2M1, 0xA, 0x0) == 0xF        # -1 / 0: -inf -> -6
    assert binary(ADD, DataType.F4_E2M1, 0x7, 0x7) == 0x7        # 6 + 6 saturates
    assert binary(ADD, DataType.F4_E2M1, 0x1, 0x1) == 0x2        # 0.5 + 0.5 = 1
    assert binary(MUL, DataType.F6_E3M2, 0x01, 0x01) == 0x00     # 2^-8 rounds to zero
    assert binary(SUB, DataType.I4, 0x0, 0x1) == 0xF             # wraps


def test_f8_known_codes():
    """The codec's reading of the two formats (src/shared/scalar_binary_codec.hpp:30-108):
    E4M3FN has no infinities and every all-ones exponent is NaN, so 240 (0x77) is the largest
    value and the overflow code; E5M2 overflows to its infinities."""
    e4, e5 = int(DataType.F8_E4M3FN), int(DataType.F8_E5M2)
    assert binary(ADD, DataType.F8_E4M3FN, 0x77, 0x77) == 0x77          # 240 + 240 saturates
    assert binary(ADD, DataType.F8_E4M3FN, 0x78, 0x00) == 0x7F          # exponent 15 reads as NaN
    assert binary(MUL, DataType.F8_E4M3FN, 0x01, 0x01) == 0x00          # 2^-18 rounds to zero
    assert binary(SUB, DataType.F8_E4M3FN, 0x38, 0x38) == 0x00          # 1 - 1 = +0
    assert binary(ADD, DataType.F8_E5M2, 0x7B, 0x7B) == 0x7C            # 57344 * 2 -> +inf
    assert binary(SUB, DataType.F8_E5M2, 0x7C, 0x7C) == 0x7E            # inf - inf -> NaN
    assert binary(DIV, DataType.F8_E5M2, 0x3C, 0x80) == 0xFC            # 1 / -0 -> -inf
    assert e4 == 16 and e5 == 17


@pytest.mark.parametrize("op", [ADD, MUL, SUB, DIV])
def test_ieee_form_equals_codec_f32(op):
    rng = np.random.default_rng(9)
    exps = np.array([0, 1, 2, 23, 24, 25, 100, 126, 127, 128, 149, 150, 151, 230, 253, 254, 255],
                    dtype=np.uint32)
    mant = np.array([0, 1, 2, 0x3FFFFF, 0x400000, 0x400001, 0x7FFFFE, 0x7FFFFF], dtype=np.uint32)
    grid = np.array([(s << 31) | (e << 23) | m for s in (0, 1) for e in exps for m in mant],
                    dtype=np.uint32)
    rand = rng.integers(0, 1 << 32, size=1500, dtype=np.uint64).astype(np.uint32)
    values = np.concatenate([grid, rand])
    mismatches = oracle().iomo_codec_mismatches(op, int(DataType.F32), values.ctypes.data,
                                                values.size, values.ctypes.data, values.size)
    assert mismatches == 0


def test_cast_semantics():
    lib = oracle()
    bf16, f32 = int(DataType.BF16), int(DataType.F32)
    assert lib.iomo_decode_encode(bf16, f32, 0x3F80) == 0x3F800000
    assert lib.iomo_decode_encode(bf16, f32, 0x8001) == 0x80010000          # subnormal, exact
    assert lib.iomo_decode_encode(bf16, f32, 0xFFC1) == 0x7FC00000          # NaN: sign, payload dropped
    assert lib.iomo_decode_encode(f32, bf16, 0x3F808000) == 0x3F80          # tie to even (down)
    assert lib.iomo_decode_encode(f32, bf16, 0x3F818000) == 0x3F82          # tie to even (up)
    assert lib.iomo_decode_encode(f32, bf16, 0x3F808001) == 0x3F81
    assert lib.iomo_decode_encode(f32, bf16, 0x7F7FFFFF) == 0x7F80          # overflow to infinity
    assert lib.iomo_decode_encode(f32, bf16, 0x00008000) == 0x0000          # subnormal tie to even
    assert lib.iomo_decode_encode(f32, bf16, 0x00018000) == 0x0002
    assert lib.iomo_decode_encode(f32, bf16, 0xFF800001) == 0x7FC0
