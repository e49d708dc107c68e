"""Shared test infrastructure: the CPU oracle, the reference shim, host tensors.

Everything here is checker-side code. It loads oracle/libiom_oracle.so (the
plain-C restatement, built on demand with gcc) and, when present, the shim
around the unmodified reference CPU backend under oracle/_ref/.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

from iom_b200._abi import IombSdpaStages, IombView
from iom_b200.tensor import DataType, TensorSpec, TensorView, dense_plane_strides, leaf_bits

REPO = Path(__file__).resolve().parent.parent
ORACLE_DIR = REPO / "oracle"
ORACLE_LIB = ORACLE_DIR / "libiom_oracle.so"
REF_LIBS = {
    "portable": ORACLE_DIR / "_ref" / "libiomref_portable.so",
    "avx512": ORACLE_DIR / "_ref" / "libiomref_avx512.so",
    # reference CPU backend + the C++ B200 backend behind the same facade
    "b200": ORACLE_DIR / "_ref" / "libiomref_b200.so",
}

_VIEW = ctypes.POINTER(IombView)
_oracle = None


def oracle() -> ctypes.CDLL:
    global _oracle
    if _oracle is None:
        source_time = max((ORACLE_DIR / name).stat().st_mtime
                          for name in ("iom_oracle.c", "iom_oracle.h"))
        if not ORACLE_LIB.exists() or ORACLE_LIB.stat().st_mtime < source_time:
            subprocess.run(["make", "-C", str(ORACLE_DIR), "oracle"], check=True,
                           capture_output=True)
        lib = ctypes.CDLL(str(ORACLE_LIB))
        u64 = ctypes.c_uint64
        lib.iomo_leaf_bits.restype = ctypes.c_uint32
        lib.iomo_leaf_bits.argtypes = [ctypes.c_uint32]
        lib.iomo_plane_slot.restype = u64
        lib.iomo_plane_slot.argtypes = [u64] * 5
        lib.iomo_scalar_binary.restype = u64
        lib.iomo_scalar_binary.argtypes = [ctypes.c_int, ctypes.c_uint32, u64, u64]
        lib.iomo_scalar_binary_ieee.restype = u64
        lib.iomo_scalar_binary_ieee.argtypes = [ctypes.c_int, ctypes.c_uint32, u64, u64]
        lib.iomo_decode_encode.restype = u64
        lib.iomo_decode_encode.argtypes = [ctypes.c_uint32, ctypes.c_uint32, u64]
        lib.iomo_codec_mismatches.restype = u64
        lib.iomo_codec_mismatches.argtypes = [ctypes.c_int, ctypes.c_uint32,
                                              ctypes.c_void_p, u64, ctypes.c_void_p, u64]
        lib.iomo_binary.restype = ctypes.c_int
        lib.iomo_binary.argtypes = [ctypes.c_int, _VIEW, _VIEW, _VIEW, ctypes.c_int]
        lib.iomo_rmsnorm.restype = ctypes.c_int
        lib.iomo_rmsnorm.argtypes = [_VIEW, _VIEW, _VIEW, ctypes.c_float, ctypes.c_int]
        lib.iomo_copy.restype = ctypes.c_int
        lib.iomo_copy.argtypes = [_VIEW, _VIEW]
        lib.iomo_rope.restype = ctypes.c_int
        lib.iomo_rope.argtypes = [_VIEW, _VIEW, ctypes.c_uint64, ctypes.c_double]
        lib.iomo_rope_angle.restype = None
        lib.iomo_rope_angle.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float,
                                        ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_float)]
        lib.iomo_silu.restype = ctypes.c_int
        lib.iomo_silu.argtypes = [_VIEW, _VIEW, ctypes.c_int]
        lib.iomo_scalar_silu.restype = ctypes.c_uint64
        lib.iomo_scalar_silu.argtypes = [ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int]
        lib.iomo_cast.restype = ctypes.c_int
        lib.iomo_cast.argtypes = [_VIEW, _VIEW]
        lib.iomo_embedding.restype = ctypes.c_int
        lib.iomo_embedding.argtypes = [_VIEW, _VIEW, _VIEW, ctypes.POINTER(ctypes.c_uint32)]
        lib.iomo_cache_append.restype = ctypes.c_int
        lib.iomo_cache_append.argtypes = [_VIEW, _VIEW, u64]
        lib.iomo_sumsq.restype = ctypes.c_double
        lib.iomo_sumsq.argtypes = [_VIEW]
        lib.iomo_scatter.restype = ctypes.c_int
        lib.iomo_scatter.argtypes = [_VIEW, ctypes.c_void_p]
        lib.iomo_gather.restype = ctypes.c_int
        lib.iomo_gather.argtypes = [_VIEW, ctypes.c_void_p]
        lib.iomo_sdpa_scale_mask.restype = ctypes.c_int
        lib.iomo_sdpa_scale_mask.argtypes = [ctypes.POINTER(IombSdpaStages)]
        lib.iomo_sdpa_softmax.restype = ctypes.c_int
        lib.iomo_sdpa_softmax.argtypes = [ctypes.POINTER(IombSdpaStages)]
        lib.iomo_sdpa_canonicalize_output.restype = ctypes.c_int
        lib.iomo_sdpa_canonicalize_output.argtypes = [_VIEW]
        _oracle = lib
    return _oracle


class HostStages:
    """Host copies of the attention stage workspace: FP32 scores and BF16 probabilities,
    both [planes, Hq, pad16(R), pad16(L)], for the oracle's stage functions."""

    def __init__(self, planes, Hq, Hkv, R, C, D, a, L, score_fill=777.0, probability_fill=0xA5A5):
        self.geometry = (planes, Hq, Hkv, R, C, D, a, L)
        self.Rp, self.Lp = (R + 15) // 16 * 16, (L + 15) // 16 * 16
        shape = (planes, Hq, self.Rp, self.Lp)
        self.scores = np.full(shape, score_fill, dtype=np.float32)
        self.probability = np.full(shape, probability_fill, dtype=np.uint16)

    def visible(self, row: int) -> int:
        _, _, _, _, _, _, a, L = self.geometry
        return min(L, a + row + 1)

    def visible_mask(self) -> np.ndarray:
        """Boolean [Rp, Lp]: the cells the causal prefix rule lets row r see."""
        _, _, _, R, _, _, a, L = self.geometry
        rows = np.arange(self.Rp)[:, None]
        tokens = np.arange(self.Lp)[None, :]
        return (rows < R) & (tokens < L) & (tokens <= a + rows)

    def request(self) -> "IombSdpaStages":
        return IombSdpaStages(self.scores.ctypes.data, self.probability.ctypes.data, *self.geometry)

    def scale_mask(self):
        assert oracle().iomo_sdpa_scale_mask(ctypes.byref(self.request())) == 0
        return self

    def softmax(self):
        assert oracle().iomo_sdpa_softmax(ctypes.byref(self.request())) == 0
        return self


_sdpa_reference = None


def sdpa_reference_stages_or_skip() -> ctypes.CDLL:
    """The reference's own CUDA stage kernels (oracle/_ref/libiomref_sdpa_stages.so, built by
    `make -C oracle cudastages` where the reference checkout is present)."""
    global _sdpa_reference
    path = ORACLE_DIR / "_ref" / "libiomref_sdpa_stages.so"
    if _sdpa_reference is None:
        if not path.exists():
            import pytest
            pytest.skip("reference stage kernels are not built (make -C oracle cudastages)")
        lib = ctypes.CDLL(str(path))
        u64, u64p = ctypes.c_uint64, ctypes.POINTER(ctypes.c_uint64)
        lib.iomref_sdpa_stage.restype = ctypes.c_int
        lib.iomref_sdpa_stage.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                          u64, u64, u64p, ctypes.c_uint32, u64p,
                                          u64, u64, u64, u64, u64, u64, u64, ctypes.c_void_p]
        lib.iomref_sdpa_error.restype = ctypes.c_char_p
        _sdpa_reference = lib
    return _sdpa_reference


# ---- numpy <-> leaf encodings ------------------------------------------------

NUMPY_OF = {
    DataType.I8: np.int8, DataType.U8: np.uint8, DataType.I16: np.int16, DataType.U16: np.uint16,
    DataType.I32: np.int32, DataType.U32: np.uint32, DataType.I64: np.int64,
    DataType.U64: np.uint64, DataType.F16: np.uint16, DataType.BF16: np.uint16,
    DataType.F32: np.float32, DataType.F64: np.float64, DataType.BOOL: np.uint8,
    DataType.F8_E4M3FN: np.uint8, DataType.F8_E5M2: np.uint8, DataType.F8_E8M0: np.uint8,
}


def f32_to_bf16_bits(values: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> BF16 codes (NaN -> 0x7FC0)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    rounded[np.isnan(values)] = 0x7FC0
    return rounded


def bf16_bits_to_f32(codes: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(codes, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


class HostTensor:
    """A host copy of one owner's tiled storage (zero-filled like create_tensor)."""

    device = None

    def __init__(self, shape, data_type: DataType, fill: int | None = 0):
        self.spec = TensorSpec(shape, data_type)
        self.storage_nbytes = self.spec.tiled_storage_nbytes()
        # 64-byte aligned backing store.
        raw = np.empty(self.storage_nbytes + 64, dtype=np.uint8)
        offset = (-raw.ctypes.data) % 64
        self.storage = raw[offset:offset + self.storage_nbytes]
        self._raw = raw
        if fill is not None:
            self.storage[:] = fill

    def storage_address(self) -> int:
        return self.storage.ctypes.data

    def view(self) -> TensorView:
        return TensorView(self, self.spec, 0, dense_plane_strides(self.spec.shape))

    def poison(self, value: int = 0xA5) -> "HostTensor":
        self.storage[:] = value
        return self

    def clone(self) -> "HostTensor":
        other = HostTensor(self.spec.shape, self.spec.data_type, fill=None)
        other.storage[:] = self.storage
        return other

    def region_from_host(self, view: TensorView, source, workspace=None) -> None:
        payload = np.ascontiguousarray(source).view(np.uint8).reshape(-1)
        assert payload.size == view.spec.logical_nbytes(), "payload size mismatch"
        abi = view.as_abi()
        assert oracle().iomo_scatter(ctypes.byref(abi), payload.ctypes.data) == 0

    def region_to_host(self, view: TensorView, destination=None, workspace=None):
        out = np.zeros(view.spec.logical_nbytes(), dtype=np.uint8)
        abi = view.as_abi()
        assert oracle().iomo_gather(ctypes.byref(abi), out.ctypes.data) == 0
        return out

    def host_transfer_workspace_requirements(self, nbytes):
        return (0, 1)


def logical(view: TensorView) -> np.ndarray:
    """Logical payload of a host view as a typed numpy array of the view's shape."""
    raw = view.copy_to_host()
    return raw.view(NUMPY_OF[view.spec.data_type]).reshape(view.spec.shape)


def abi(view: TensorView):
    return ctypes.byref(view.as_abi())


# ---- the real reference through its shim ---------------------------------------

class Reference:
    """ctypes access to oracle/_ref/libiomref_<kind>.so (see oracle/ref_driver.cpp)."""

    def __init__(self, kind: str, accelerator: bool = False, arena_bytes: int = 1 << 30):
        path = REF_LIBS[kind]
        if not path.exists():
            raise FileNotFoundError(path)
        lib = ctypes.CDLL(str(path))
        vp, u64, u32 = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32
        u64p = ctypes.POINTER(u64)
        spec = {
            "iomref_last_error": (ctypes.c_char_p, []),
            "iomref_avx512_bf16_active": (ctypes.c_int, []),
            "iomref_device_create": (vp, []),
            "iomref_device_destroy": (None, [vp]),
            "iomref_tensor_create": (vp, [vp, u64p, u32, u32]),
            "iomref_tensor_destroy": (None, [vp]),
            "iomref_tensor_storage": (vp, [vp]),
            "iomref_tensor_storage_nbytes": (u64, [vp]),
            "iomref_view_full": (vp, [vp]),
            "iomref_view_slice": (vp, [vp, u64, u64, u64, u64]),
            "iomref_view_select": (vp, [vp, u64, u64]),
            "iomref_view_permute": (vp, [vp, u64p, u32]),
            "iomref_view_reshape_leading": (vp, [vp, u64p, u32]),
            "iomref_view_destroy": (None, [vp]),
            "iomref_view_describe": (ctypes.c_int, [vp, ctypes.POINTER(u32), u64p, u64p, u64p,
                                                    ctypes.POINTER(u32)]),
            "iomref_view_logical_nbytes": (u64, [vp]),
            "iomref_view_from_host": (ctypes.c_int, [vp, vp, u64]),
            "iomref_view_to_host": (ctypes.c_int, [vp, vp, u64]),
            "iomref_queue_create": (vp, [vp]),
            "iomref_queue_destroy": (None, [vp]),
            "iomref_binary": (ctypes.c_int64, [vp, ctypes.c_int, vp, vp, vp]),
            "iomref_rmsnorm": (ctypes.c_int64, [vp, vp, vp, vp, ctypes.c_float]),
            "iomref_copy": (ctypes.c_int64, [vp, vp, vp]),
            "iomref_silu": (ctypes.c_int64, [vp, vp, vp]),
            "iomref_rope": (ctypes.c_int64, [vp, vp, vp, ctypes.c_uint64, ctypes.c_double]),
            "iomref_embedding": (ctypes.c_int64, [vp, vp, vp, vp]),
            "iomref_cache_append": (ctypes.c_int64, [vp, vp, vp, u64]),
            "iomref_wait": (ctypes.c_int, [vp, ctypes.c_int64]),
        }
        if kind == "b200":
            spec.update({
                "iomref_device_create_b200": (vp, [u32, u64]),
                "iomref_tensor_upload": (ctypes.c_int, [vp, vp, u64]),
                "iomref_tensor_download": (ctypes.c_int, [vp, vp, u64]),
                "iomref_add_rmsnorm": (ctypes.c_int64, [vp, vp, vp, vp, vp, vp, ctypes.c_float]),
                "iomref_silu_mul": (ctypes.c_int64, [vp, vp, vp, vp, vp]),
                "iomref_cast": (ctypes.c_int64, [vp, vp, vp]),
                "iomref_cache_append_batched": (ctypes.c_int64, [vp, vp, vp, ctypes.POINTER(ctypes.c_uint32),
                                                                 ctypes.c_uint32,
                                                                 ctypes.POINTER(ctypes.c_uint32)]),
                "iomref_sumsq": (ctypes.c_int64, [vp, vp, ctypes.POINTER(ctypes.c_float)]),
                "iomref_sdpa_stage_b200": (ctypes.c_int64, [vp, ctypes.c_int, vp, vp,
                                                            ctypes.POINTER(ctypes.c_uint64), vp, vp]),
                "iomref_workspace_create": (vp, [vp, u64, ctypes.POINTER(vp)]),
                "iomref_memcpy_b200": (ctypes.c_int, [vp, vp, u64, ctypes.c_int]),
                "iomref_inject_fault_b200": (None, [ctypes.c_int]),
                "iomref_quarantined_events_b200": (u64, [vp]),
                "iomref_capture_begin_b200": (ctypes.c_int, [vp]),
                "iomref_capture_end_b200": (vp, [vp]),
                "iomref_replay_b200": (ctypes.c_int64, [vp, vp]),
                "iomref_recording_destroy_b200": (None, [vp]),
            })
        for name, (restype, argtypes) in spec.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        self.lib = lib
        self.kind = kind
        self.accelerator = accelerator
        self.device = (lib.iomref_device_create_b200(0, arena_bytes) if accelerator
                       else lib.iomref_device_create())
        assert self.device, self.error()
        self.queue = lib.iomref_queue_create(self.device)
        assert self.queue, self.error()
        self._tensors = []

    def error(self) -> str:
        return (self.lib.iomref_last_error() or b"").decode()

    def close(self) -> None:
        if self.queue:
            self.lib.iomref_queue_destroy(self.queue)
            self.queue = None
        for tensor in self._tensors:
            tensor.close()
        self._tensors = []
        if self.device:
            self.lib.iomref_device_destroy(self.device)
            self.device = None

    def tensor(self, shape, data_type: DataType) -> "RefTensor":
        tensor = RefTensor(self, shape, data_type)
        self._tensors.append(tensor)
        return tensor

    def run(self, token: int) -> int:
        """Waits for a token; returns 0 or the failure class. Negative oids pass through."""
        if token < 0:
            return int(token)
        return self.lib.iomref_wait(self.queue, token)


class RefView:
    def __init__(self, ref: Reference, handle):
        assert handle, ref.error()
        self.ref = ref
        self.handle = handle

    def _wrap(self, handle):
        if not handle:
            raise ValueError(self.ref.error())
        return RefView(self.ref, handle)

    def slice(self, dim, first, count, step=1):
        return self._wrap(self.ref.lib.iomref_view_slice(self.handle, dim, first, count, step))

    def select(self, dim, index):
        return self._wrap(self.ref.lib.iomref_view_select(self.handle, dim, index))

    def permute(self, order):
        arr = (ctypes.c_uint64 * len(order))(*order)
        return self._wrap(self.ref.lib.iomref_view_permute(self.handle, arr, len(order)))

    def reshape_leading(self, dims):
        arr = (ctypes.c_uint64 * max(len(dims), 1))(*dims)
        return self._wrap(self.ref.lib.iomref_view_reshape_leading(self.handle, arr, len(dims)))

    def describe(self):
        rank = ctypes.c_uint32()
        dtype = ctypes.c_uint32()
        dims = (ctypes.c_uint64 * 8)()
        strides = (ctypes.c_uint64 * 6)()
        offset = ctypes.c_uint64()
        assert self.ref.lib.iomref_view_describe(
            self.handle, ctypes.byref(rank), dims, ctypes.byref(offset), strides,
            ctypes.byref(dtype)) == 0
        n = rank.value
        return (tuple(dims[:n]), offset.value, tuple(strides[:n - 2]), DataType(dtype.value))

    def from_host(self, payload) -> None:
        data = np.ascontiguousarray(payload).view(np.uint8).reshape(-1)
        rc = self.ref.lib.iomref_view_from_host(self.handle, data.ctypes.data, data.size)
        assert rc == 0, self.ref.error()

    def to_host(self) -> np.ndarray:
        n = self.ref.lib.iomref_view_logical_nbytes(self.handle)
        out = np.zeros(n, dtype=np.uint8)
        rc = self.ref.lib.iomref_view_to_host(self.handle, out.ctypes.data, n)
        assert rc == 0, self.ref.error()
        return out


class RefTensor:
    def __init__(self, ref: Reference, shape, data_type: DataType):
        dims = (ctypes.c_uint64 * len(shape))(*shape)
        self.ref = ref
        self.handle = ref.lib.iomref_tensor_create(ref.device, dims, len(shape), int(data_type))
        assert self.handle, ref.error()
        self.nbytes = ref.lib.iomref_tensor_storage_nbytes(self.handle)
        if ref.accelerator:
            self.storage = None     # device memory: use write() / read()
        else:
            address = ref.lib.iomref_tensor_storage(self.handle)
            self.storage = np.ctypeslib.as_array(
                ctypes.cast(address, ctypes.POINTER(ctypes.c_uint8)), shape=(self.nbytes,))

    def write(self, raw) -> None:
        """Sets the owner's complete physical storage."""
        data = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
        assert data.size == self.nbytes
        if self.ref.accelerator:
            rc = self.ref.lib.iomref_tensor_upload(self.handle, data.ctypes.data, data.size)
            assert rc == 0, self.ref.error()
        else:
            self.storage[:] = data

    def read(self) -> np.ndarray:
        """The owner's complete physical storage."""
        if self.ref.accelerator:
            out = np.empty(self.nbytes, dtype=np.uint8)
            rc = self.ref.lib.iomref_tensor_download(self.handle, out.ctypes.data, out.size)
            assert rc == 0, self.ref.error()
            return out
        return self.storage.copy()

    def view(self) -> RefView:
        return RefView(self.ref, self.ref.lib.iomref_view_full(self.handle))

    def close(self) -> None:
        if self.handle:
            self.ref.lib.iomref_tensor_destroy(self.handle)
            self.handle = None


def reference_or_skip(kind: str = "portable") -> Reference:
    import pytest
    if not REF_LIBS[kind].exists():
        pytest.skip(f"reference shim {REF_LIBS[kind].name} is not built (make -C oracle ref)")
    return Reference(kind)


# ---- seeded data ------------------------------------------------------------------

def random_payload(rng: np.random.Generator, shape, data_type: DataType, kind: str = "uniform"):
    """Logical payload as a numpy array in the leaf's raw representation."""
    if data_type in (DataType.I32, DataType.U32):
        values = rng.integers(-(1 << 20), 1 << 20, size=shape, dtype=np.int64)
        return values.astype(np.int32).view(NUMPY_OF[data_type])
    if data_type in (DataType.F32, DataType.BF16):
        if kind == "normal":
            values = rng.standard_normal(size=shape, dtype=np.float32)
        else:
            values = rng.uniform(-1.0, 1.0, size=shape).astype(np.float32)
        return values if data_type == DataType.F32 else f32_to_bf16_bits(values)
    if leaf_bits(data_type) < 8:
        # narrower than a byte: the logical payload is packed LSB first; every bit pattern is a value
        return rng.integers(0, 256, size=TensorSpec(shape, data_type).logical_nbytes(), dtype=np.uint8)
    info = np.iinfo(NUMPY_OF[data_type])
    return rng.integers(info.min, info.max, size=shape, dtype=NUMPY_OF[data_type], endpoint=True)


SPECIAL_F32 = np.array(
    [0x00000000, 0x80000000, 0x3F800000, 0xBF800000, 0x7F7FFFFF, 0xFF7FFFFF, 0x00800000,
     0x007FFFFF, 0x00000001, 0x80000001, 0x7F800000, 0xFF800000, 0x7FC00001, 0xFFC00000,
     0x7F800001, 0x33800000, 0x4B800000, 0x3F7FFFFF], dtype=np.uint32)

SPECIAL_BF16 = np.array(
    [0x0000, 0x8000, 0x3F80, 0xBF80, 0x7F7F, 0xFF7F, 0x0080, 0x007F, 0x0001, 0x8001, 0x7F80,
     0xFF80, 0x7FC1, 0xFFC0, 0x7F81, 0x3F7F, 0x4000, 0x3F00, 0x0040, 0x3B80], dtype=np.uint16)
