"""The C-ABI library loads, exports every symbol include/iom_b200.h declares,
serves its device-free helpers, rejects bad arguments before touching CUDA, and
reports a device error (never a CPU result) when no GPU is present."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

from iom_b200 import _abi
from iom_b200.tensor import DataType, TensorSpec, leaf_bits, plane_slot
from support import HostTensor, oracle

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    header = (ROOT / "include" / "iom_b200.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return sorted(set(re.findall(r"\b(iomb_[a-z0-9_]+)\s*\(", header)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = _abi.load_library()
    names = declared_symbols()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), f"{name} is declared but not exported"
        assert name in _abi.PROTOTYPES, f"{name} has no ctypes prototype"
    assert set(_abi.PROTOTYPES) == set(names)


def test_view_struct_matches_header_layout():
    assert ctypes.sizeof(_abi.IombView) == 8 + 8 + 4 + 4 + 8 * 8 + 8 + 6 * 8


def test_layout_helpers_agree_with_oracle_and_python():
    lib = _abi.load_library()
    assert lib.iomb_abi_version() >= 1
    for dtype in DataType:
        assert lib.iomb_dtype_bits(int(dtype)) == leaf_bits(dtype) == oracle().iomo_leaf_bits(int(dtype))
    assert lib.iomb_dtype_bits(99) == 0
    rng = np.random.default_rng(0)
    for _ in range(200):
        rows, cols = (int(v) for v in rng.integers(1, 70, size=2))
        plane, row, col = int(rng.integers(0, 5)), int(rng.integers(0, rows)), int(rng.integers(0, cols))
        expect = plane_slot(rows, cols, plane, row, col)
        assert lib.iomb_plane_slot(rows, cols, plane, row, col) == expect
        assert oracle().iomo_plane_slot(rows, cols, plane, row, col) == expect
    for shape, dtype in (((2, 17, 33), DataType.BF16), ((1, 1), DataType.I4), ((3, 16, 16), DataType.F64),
                         ((5, 31), DataType.F6_E2M3)):
        spec = TensorSpec(shape, dtype)
        dims = (ctypes.c_uint64 * len(shape))(*shape)
        out = ctypes.c_uint64()
        assert lib.iomb_tiled_storage_nbytes(dims, len(shape), int(dtype), ctypes.byref(out)) == 0
        assert out.value == spec.tiled_storage_nbytes()
        assert lib.iomb_logical_nbytes(dims, len(shape), int(dtype), ctypes.byref(out)) == 0
        assert out.value == spec.logical_nbytes()
    huge = (ctypes.c_uint64 * 2)(1 << 40, 1 << 40)
    assert lib.iomb_tiled_storage_nbytes(huge, 2, int(DataType.F32), ctypes.byref(out)) == 3
    assert lib.iomb_tiled_storage_nbytes(huge, 1, int(DataType.F32), ctypes.byref(out)) == 1


def test_admission_rejects_before_any_device_work():
    lib = _abi.load_library()
    a = HostTensor((4, 16, 16), DataType.F32)
    b = HostTensor((3, 16, 16), DataType.F32)
    c = HostTensor((4, 16, 16), DataType.BF16)
    va, vb, vc = a.view().as_abi(), b.view().as_abi(), c.view().as_abi()
    assert lib.iomb_binary(0, ctypes.byref(va), ctypes.byref(vb), ctypes.byref(va), None) == 1
    assert "broadcast" in _abi.last_error()
    assert lib.iomb_binary(0, ctypes.byref(va), ctypes.byref(va), ctypes.byref(vc), None) == 1
    assert lib.iomb_binary(7, ctypes.byref(va), ctypes.byref(va), ctypes.byref(va), None) == 1   # unknown operation
    assert lib.iomb_binary(0, None, ctypes.byref(va), ctypes.byref(va), None) == 1
    bad = a.view().as_abi()
    bad.storage_bytes = 100                       # view exceeds its owner
    assert lib.iomb_copy(ctypes.byref(bad), ctypes.byref(va), None) == 1
    bad = a.view().as_abi()
    bad.base = bad.base + 8                       # not 32-byte aligned
    assert lib.iomb_copy(ctypes.byref(bad), ctypes.byref(va), None) == 1
    bad = a.view().as_abi()
    bad.plane_strides[0] = 0
    assert lib.iomb_copy(ctypes.byref(bad), ctypes.byref(va), None) == 1
    assert lib.iomb_cast(ctypes.byref(va), ctypes.byref(va), None) == 2
    assert lib.iomb_rmsnorm(ctypes.byref(vc), ctypes.byref(vc), ctypes.byref(vc),
                            ctypes.c_float(1e-5), 0, None) == 1


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    lib = _abi.load_library()
    a = HostTensor((16, 16), DataType.F32)
    out = HostTensor((16, 16), DataType.F32).poison(0x11)
    va, vo = a.view().as_abi(), out.view().as_abi()
    assert lib.iomb_binary(0, ctypes.byref(va), ctypes.byref(va), ctypes.byref(vo), None) == 5
    assert np.all(out.storage == 0x11)            # nothing was computed on the host
    from iom_b200.device import DeviceMemoryConfig, make_b200_device
    with pytest.raises(RuntimeError):
        make_b200_device(0, DeviceMemoryConfig(1 << 20))
