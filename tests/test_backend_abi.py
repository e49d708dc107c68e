"""The C++ backend's shared library loads, exports every symbol its C driver header
(include/iom_b200_backend_c.h) declares, and the ctypes wrapper binds exactly those. No
device work: creating a device without a GPU must fail with a message, never fall back."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

from iom_b200 import backend_driver as bd

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    header = (ROOT / "include" / "iom_b200_backend_c.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return sorted(set(re.findall(r"\b(iomb_backend_[a-z0-9_]+)\s*\(", header)))


def library():
    if not bd.available():
        pytest.skip("libiom_b200_backend.so is built against a reference checkout "
                    "(python -m iom_b200.build --backend=<checkout>), none was available")
    return bd.load_library()


def test_every_declared_symbol_is_exported_and_bound():
    lib = library()
    names = declared_symbols()
    assert len(names) >= 17
    for name in names:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert set(bd.PROTOTYPES) == set(names)


def test_operation_record_matches_the_header():
    header = (ROOT / "include" / "iom_b200_backend_c.h").read_text()
    opcodes = dict(re.findall(r"IOMB_BACKEND_([A-Z_]+) = (\d+)", header))
    for name in ("ADD", "MUL", "SUB", "DIV", "RMSNORM", "ADD_RMSNORM", "COPY", "EMBEDDING", "CACHE_APPEND",
                 "CACHE_APPEND_BATCHED", "SILU", "SILU_MUL", "ROPE", "CAST", "SUMSQ", "FROM_HOST", "TO_HOST",
                 "WAIT"):
        assert int(opcodes[name]) == getattr(bd, name), name
    assert ctypes.sizeof(bd.Timing) >= 3 * 8


@pytest.mark.skipif(torch.cuda.is_available(), reason="needs a box without a GPU")
def test_no_device_means_an_error_not_a_fallback():
    lib = library()
    assert not lib.iomb_backend_device_create(0, 1 << 20, 0)
    assert (lib.iomb_backend_last_error() or b"") != b""
    with pytest.raises(RuntimeError):
        bd.Backend(0, 1 << 20)
