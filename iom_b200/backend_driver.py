"""ctypes binding of libiom_b200_backend.so: the C++ B200 backend (an iom::Device behind
the reference's own facade) driven through include/iom_b200_backend_c.h.

The library is built by `python -m iom_b200.build --backend=<reference checkout>`. It is
what a program links that uses IOM's C++ interface; this module exists so that the
benchmark and the tests can issue facade operations from C++ (iomb_backend_run) and time
them on the queue's stream without an interpreter between two submissions.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
LIBRARY_PATH = PACKAGE_DIR / "libiom_b200_backend.so"

(ADD, MUL, SUB, DIV, RMSNORM, ADD_RMSNORM, COPY, EMBEDDING, CACHE_APPEND, CACHE_APPEND_BATCHED,
 SILU, SILU_MUL, ROPE, CAST, SUMSQ, FROM_HOST, TO_HOST, WAIT) = range(18)
EAGER, WAIT_EACH, RECORDED = 0, 1, 2


class Op(ctypes.Structure):
    """struct iomb_backend_op."""

    _fields_ = [
        ("opcode", ctypes.c_uint32), ("reserved", ctypes.c_uint32),
        ("views", ctypes.c_void_p * 5),
        ("workspace", ctypes.c_void_p),
        ("host", ctypes.c_void_p), ("host_bytes", ctypes.c_uint64),
        ("a", ctypes.c_uint64), ("theta", ctypes.c_double),
        ("eps", ctypes.c_float), ("reserved2", ctypes.c_float),
    ]


class Timing(ctypes.Structure):
    """struct iomb_backend_timing."""

    _fields_ = [
        ("host_seconds", ctypes.c_double), ("submit_seconds", ctypes.c_double),
        ("device_ms", ctypes.c_float), ("reserved", ctypes.c_uint32),
        ("operations", ctypes.c_uint64),
    ]


_vp, _u64, _u32 = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32
PROTOTYPES = {
    "iomb_backend_last_error": (ctypes.c_char_p, []),
    "iomb_backend_device_create": (_vp, [_u32, _u64, _u32]),
    "iomb_backend_device_destroy": (None, [_vp]),
    "iomb_backend_queue_create": (_vp, [_vp]),
    "iomb_backend_queue_destroy": (None, [_vp]),
    "iomb_backend_tensor_create": (_vp, [_vp, ctypes.POINTER(_u64), _u32, _u32]),
    "iomb_backend_tensor_destroy": (None, [_vp]),
    "iomb_backend_tensor_address": (_vp, [_vp]),
    "iomb_backend_tensor_nbytes": (_u64, [_vp]),
    "iomb_backend_workspace_create": (_vp, [_vp, _u64]),
    "iomb_backend_workspace_destroy": (None, [_vp]),
    "iomb_backend_workspace_address": (_vp, [_vp]),
    "iomb_backend_view_full": (_vp, [_vp]),
    "iomb_backend_view_select": (_vp, [_vp, _u64, _u64]),
    "iomb_backend_view_slice": (_vp, [_vp, _u64, _u64, _u64, _u64]),
    "iomb_backend_view_destroy": (None, [_vp]),
    "iomb_backend_run": (ctypes.c_int, [_vp, ctypes.POINTER(Op), _u32, _u32, _u32, _u32,
                                        ctypes.POINTER(Timing)]),
}

_library = None


def available() -> bool:
    return LIBRARY_PATH.exists()


def load_library() -> ctypes.CDLL:
    global _library
    if _library is None:
        if not LIBRARY_PATH.exists():
            raise RuntimeError(
                f"{LIBRARY_PATH} is missing: build it with "
                "`python -m iom_b200.build --backend=<reference checkout>`")
        library = ctypes.CDLL(str(LIBRARY_PATH))
        for name, (restype, argtypes) in PROTOTYPES.items():
            function = getattr(library, name)
            function.restype = restype
            function.argtypes = argtypes
        _library = library
    return _library


class _DeviceMemory:
    """A device address range as an object torch can wrap without copying."""

    def __init__(self, address: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 3,
            "strides": None,
        }


class Backend:
    """One device of the C++ backend with one queue; handles are released by close()."""

    def __init__(self, ordinal: int, arena_bytes: int, max_in_flight: int = 0):
        self.lib = load_library()
        self.device = self.lib.iomb_backend_device_create(ordinal, arena_bytes // 32 * 32, max_in_flight)
        if not self.device:
            raise RuntimeError(f"make_b200_device failed: {self.error()}")
        self.queue = self.lib.iomb_backend_queue_create(self.device)
        if not self.queue:
            raise RuntimeError(f"create_ops failed: {self.error()}")
        self._tensors, self._views, self._workspaces = [], [], []

    def error(self) -> str:
        return (self.lib.iomb_backend_last_error() or b"").decode()

    def tensor(self, shape, data_type) -> int:
        dims = (ctypes.c_uint64 * len(shape))(*shape)
        handle = self.lib.iomb_backend_tensor_create(self.device, dims, len(shape), int(data_type))
        if not handle:
            raise MemoryError(f"create_tensor{tuple(shape)} failed: {self.error()}")
        self._tensors.append(handle)
        return handle

    def storage(self, tensor: int):
        """The owner's tiled storage as a uint8 torch tensor on the device (no copy)."""
        import torch
        address = self.lib.iomb_backend_tensor_address(tensor)
        nbytes = self.lib.iomb_backend_tensor_nbytes(tensor)
        return torch.as_tensor(_DeviceMemory(address, nbytes), device="cuda")

    def view(self, tensor: int) -> int:
        handle = self.lib.iomb_backend_view_full(tensor)
        if not handle:
            raise RuntimeError(self.error())
        self._views.append(handle)
        return handle

    def select(self, view: int, dim: int, index: int) -> int:
        handle = self.lib.iomb_backend_view_select(view, dim, index)
        if not handle:
            raise RuntimeError(self.error())
        self._views.append(handle)
        return handle

    def workspace(self, nbytes: int) -> int:
        handle = self.lib.iomb_backend_workspace_create(self.device, nbytes)
        if not handle:
            raise MemoryError(f"create_workspace({nbytes}) failed: {self.error()}")
        self._workspaces.append(handle)
        return handle

    def workspace_memory(self, workspace: int, nbytes: int):
        import torch
        address = self.lib.iomb_backend_workspace_address(workspace)
        return torch.as_tensor(_DeviceMemory(address, nbytes), device="cuda")

    @staticmethod
    def op(opcode: int, views=(), workspace=None, host=None, host_bytes=0, a=0, theta=0.0, eps=0.0) -> Op:
        record = Op()
        record.opcode = opcode
        for i, view in enumerate(views):
            record.views[i] = view
        record.workspace = workspace
        record.host = host
        record.host_bytes = host_bytes
        record.a = a
        record.theta = theta
        record.eps = eps
        return record

    def run(self, program, passes: int = 1, warmup: int = 0, mode: int = EAGER, queue=None) -> Timing:
        """Runs the list of Op records `passes` times after `warmup` untimed passes."""
        array = (Op * len(program))(*program)
        timing = Timing()
        status = self.lib.iomb_backend_run(queue or self.queue, array, len(program), warmup, passes,
                                           mode, ctypes.byref(timing))
        if status != 0:
            raise RuntimeError(f"iomb_backend_run failed (class {status}): {self.error()}")
        return timing

    def close(self) -> None:
        for handle in self._views:
            self.lib.iomb_backend_view_destroy(handle)
        self._views = []
        if self.queue:
            self.lib.iomb_backend_queue_destroy(self.queue)
            self.queue = None
        for handle in self._tensors:
            self.lib.iomb_backend_tensor_destroy(handle)
        for handle in self._workspaces:
            self.lib.iomb_backend_workspace_destroy(handle)
        self._tensors, self._workspaces = [], []
        if self.device:
            self.lib.iomb_backend_device_destroy(self.device)
            self.device = None
