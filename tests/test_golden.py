"""The oracle against the golden vectors recorded from the unmodified reference
(tests/golden/reference_vectors.npz, made by tests/golden/generate.py)."""
import ctypes
from pathlib import Path

import numpy as np
import pytest

from iom_b200.tensor import DataType, TensorView
from support import HostTensor, abi, oracle

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_vectors.npz")
BINARY_SHAPES = 5


def host_from(storage, shape, dtype):
    tensor = HostTensor(shape, dtype, fill=None)
    assert tensor.storage.size == storage.size
    tensor.storage[:] = storage
    return tensor


def split_shapes(packed):
    shapes, i = [], 0
    for _ in range(3):
        n = int(packed[i])
        shapes.append(tuple(int(v) for v in packed[i + 1:i + 1 + n]))
        i += 1 + n
    return shapes


def view_from(tensor, described, rank):
    dims = tuple(int(v) for v in described[:rank])
    offset = int(described[rank])
    strides = tuple(int(v) for v in described[rank + 1:])
    from iom_b200.tensor import TensorSpec
    return TensorView(tensor, TensorSpec(dims, tensor.spec.data_type), offset, strides)


OP_CODES = {"add": 0, "mul": 1, "sub": 2, "div": 3}


@pytest.mark.parametrize("dtype", [DataType.I32, DataType.F32, DataType.BF16])
@pytest.mark.parametrize("op", ["add", "mul", "sub", "div"])
@pytest.mark.parametrize("case", range(BINARY_SHAPES))
@pytest.mark.parametrize("ieee", [0, 1])
def test_binary_golden(dtype, op, case, ieee):
    if op == "div" and dtype == DataType.I32:
        pytest.skip("the reference admits no integer division")
    key = f"binary_{op}_{dtype.name}_{case}"
    ls, rs, os_ = split_shapes(GOLDEN[key + "_shapes"])
    lhs = host_from(GOLDEN[key + "_lhs"], ls, dtype)
    rhs = host_from(GOLDEN[key + "_rhs"], rs, dtype)
    out = host_from(GOLDEN[key + "_out_before"], os_, dtype)
    assert oracle().iomo_binary(OP_CODES[op], abi(lhs.view()), abi(rhs.view()),
                                abi(out.view()), ieee) == 0
    assert np.array_equal(out.storage, GOLDEN[key + "_out"])


@pytest.mark.parametrize("dtype", [DataType.F32, DataType.BF16])
@pytest.mark.parametrize("op", ["add", "mul", "sub", "div"])
def test_special_values_golden(dtype, op):
    key = f"special_{op}_{dtype.name}"
    n = int(round((GOLDEN[key + "_out"].size / (4 if dtype == DataType.F32 else 2)) ** 0.5))
    n = {DataType.F32: 18, DataType.BF16: 20}[dtype]
    lhs = host_from(GOLDEN[key + "_lhs"], (n, n), dtype)
    rhs = host_from(GOLDEN[key + "_rhs"], (n, n), dtype)
    for ieee in (0, 1):
        out = HostTensor((n, n), dtype).poison(0xA5)
        out.view().copy_from_host(np.zeros((n, n), dtype=np.uint32 if dtype == DataType.F32 else np.uint16))
        assert oracle().iomo_binary(OP_CODES[op], abi(lhs.view()), abi(rhs.view()),
                                    abi(out.view()), ieee) == 0
        assert np.array_equal(out.storage, GOLDEN[key + "_out"])


SMALL_FLOATS = [(DataType.F8_E4M3FN, 256), (DataType.F8_E5M2, 256), (DataType.F6_E2M3, 64),
                (DataType.F6_E3M2, 64), (DataType.F4_E2M1, 16)]


@pytest.mark.parametrize("dtype,n", SMALL_FLOATS)
@pytest.mark.parametrize("op", ["add", "mul", "sub", "div"])
def test_every_pair_of_the_small_floats_golden(dtype, n, op):
    """Every pair of codes, recorded from the reference CPU backend: the oracle's codec and
    its binary32 form both reproduce it."""
    key = f"pairs_{op}_{dtype.name}"
    lhs = host_from(GOLDEN[key + "_lhs"], (n, n), dtype)
    rhs = host_from(GOLDEN[key + "_rhs"], (n, n), dtype)
    for ieee in (0, 1):
        out = HostTensor((n, n), dtype)
        assert oracle().iomo_binary(OP_CODES[op], abi(lhs.view()), abi(rhs.view()),
                                    abi(out.view()), ieee) == 0
        assert np.array_equal(out.storage, GOLDEN[key + "_out"])


@pytest.mark.parametrize("build,order", [("portable", 1), ("avx512", 0)])
@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
@pytest.mark.parametrize("case", range(6))
def test_rmsnorm_golden(build, order, dtype, case):
    key = f"rmsnorm_{build}_{dtype.name}_{case}"
    shape = tuple(int(v) for v in GOLDEN[key + "_shape"])
    x = host_from(GOLDEN[key + "_x"], shape, dtype)
    w = host_from(GOLDEN[key + "_w"], (1, shape[-1]), dtype)
    out = host_from(GOLDEN[key + "_out_before"], shape, dtype)
    assert oracle().iomo_rmsnorm(abi(x.view()), abi(w.view()), abi(out.view()), 1e-5, order) == 0
    assert np.array_equal(out.storage, GOLDEN[key + "_out"])


def test_copy_golden():
    src = host_from(GOLDEN["copy_src"], (3, 4, 17, 33), DataType.BF16)
    dst = host_from(GOLDEN["copy_dst_before"], (4, 3, 17, 33), DataType.BF16)
    sv = view_from(src, GOLDEN["copy_src_view"], 4)
    dv = view_from(dst, GOLDEN["copy_dst_view"], 4)
    assert oracle().iomo_copy(abi(sv), abi(dv)) == 0
    assert np.array_equal(dst.storage, GOLDEN["copy_dst"])


def test_embedding_golden():
    table = host_from(GOLDEN["embedding_table"], (50, 37), DataType.BF16)
    ids = host_from(GOLDEN["embedding_ids"], (2, 1, 19), DataType.U32)
    out = host_from(GOLDEN["embedding_out_before"], (2, 19, 37), DataType.BF16)
    status = ctypes.c_uint32(7)
    assert oracle().iomo_embedding(abi(table.view()), abi(ids.view()), abi(out.view()),
                                   ctypes.byref(status)) == 0
    assert status.value == 0
    assert np.array_equal(out.storage, GOLDEN["embedding_out"])


@pytest.mark.parametrize("a", [0, 5, 29])
def test_cache_append_golden(a):
    src = host_from(GOLDEN[f"append_{a}_src"], (2, 3, 3, 40), DataType.BF16)
    dst = host_from(GOLDEN[f"append_{a}_dst_before"], (2, 3, 32, 40), DataType.BF16)
    assert oracle().iomo_cache_append(abi(src.view()), abi(dst.view()), a) == 0
    assert np.array_equal(dst.storage, GOLDEN[f"append_{a}_dst"])


def test_host_transfer_golden():
    host = host_from(GOLDEN["transfer_before"], (3, 2, 17, 35), DataType.F32)
    view = view_from(host, GOLDEN["transfer_view"], 4)
    view.copy_from_host(GOLDEN["transfer_payload"])
    assert np.array_equal(host.storage, GOLDEN["transfer_after"])


@pytest.mark.parametrize("build", ["portable", "avx512"])
def test_silu_golden(build):
    """Oracle (FP32 carrier) against the reference CPU backend's stored outputs:
    every BF16 code, and a ragged F32 case with special values."""
    codes = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    x = HostTensor((256, 256), DataType.BF16).poison(0xA5)
    x.view().copy_from_host(codes)
    y = HostTensor((256, 256), DataType.BF16).poison(0xA5)
    y.view().copy_from_host(np.zeros((256, 256), dtype=np.uint16))
    assert oracle().iomo_silu(abi(x.view()), abi(y.view()), 0) == 0
    assert np.array_equal(y.storage, GOLDEN[f"silu_{build}_BF16_out"])
    # the FP64 carrier of the reference's GPU backends agrees on every BF16 code
    assert oracle().iomo_silu(abi(x.view()), abi(y.view()), 1) == 0
    assert np.array_equal(y.storage, GOLDEN[f"silu_{build}_BF16_out"])
    xf = host_from(GOLDEN[f"silu_{build}_F32_x"], (2, 17, 35), DataType.F32)
    yf = host_from(GOLDEN[f"silu_{build}_F32_out_before"], (2, 17, 35), DataType.F32)
    assert oracle().iomo_silu(abi(xf.view()), abi(yf.view()), 0) == 0
    assert np.array_equal(yf.storage, GOLDEN[f"silu_{build}_F32_out"])


ROPE_CASES = [((2, 3, 5, 64), 0, 10000.0), ((4, 17, 128), 7, 10000.0), ((1, 2, 33, 34), 2040, 500000.0)]


@pytest.mark.parametrize("build", ["portable", "avx512"])
@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
@pytest.mark.parametrize("case", range(len(ROPE_CASES)))
def test_rope_golden(build, dtype, case):
    """Oracle against the reference CPU backend's stored RoPE outputs. The angles go
    through this host's powf / sinf / cosf, as they did when the vectors were made
    (same image, same C library)."""
    shape, a, theta = ROPE_CASES[case]
    key = f"rope_{build}_{dtype.name}_{case}"
    x = host_from(GOLDEN[key + "_x"], shape, dtype)
    out = host_from(GOLDEN[key + "_out_before"], shape, dtype)
    assert oracle().iomo_rope(abi(x.view()), abi(out.view()), a, theta) == 0
    assert np.array_equal(out.storage, GOLDEN[key + "_out"])
