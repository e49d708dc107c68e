"""B200 device, tensors, workspaces and the in-order operation queue.

Python mirror of the reference's backend contract for the CUDA backend it
replaces (include/iom/device.hpp:57-131, include/iom/iom.hpp:105-373,
src/cuda/device.cpp:349-432): one device owns one fixed data arena reserved at
construction, tensors and workspaces are 32-byte-aligned suballocations of it,
an operation queue is one CUDA stream, every operation returns an `oid`
(negative = synchronous error, positive = accepted token) and `wait` observes
completion and rethrows retained failures. All device work goes through the C
ABI of libiom_b200.so; torch supplies device memory, streams and events only.
"""
from __future__ import annotations

import collections
import ctypes
import threading
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import _abi
from .tensor import DataType, TensorSpec, TensorView, dense_plane_strides

# OidError (include/iom/oid.hpp:16-23)
OID_INVALID_ARGUMENT = -1
OID_UNSUPPORTED = -2
OID_OVERFLOW = -3
OID_RESOURCE_EXHAUSTED = -4
OID_DEVICE_ERROR = -5
OID_INTERNAL_ERROR = -6

ADD, MUL, SUB, DIV = 0, 1, 2, 3
RMS_LANES16, RMS_SEQUENTIAL = 0, 1


def facade_order(data_type) -> int:
    """Accumulation order an operation takes when the caller names none."""
    return RMS_SEQUENTIAL if data_type == DataType.F32 else RMS_LANES16

_ALIGNMENT = 256          # arena suballocation granularity (the contract needs 32)
_MAX_QUEUES = 4           # src/device_ops.cpp:210-218
_SEQUENCE_BITS = 55       # token = (queue_id << 55) | sequence
# Returned by operations issued while a queue records a CapturedSequence: accepted,
# but completed (and waited for) only through the replay's own token.
OID_CAPTURED = (1 << 62) - 1


class UnsupportedOperation(Exception):
    """detail::UnsupportedOperation -> OidError::Unsupported."""


class DeviceError(RuntimeError):
    """A CUDA runtime failure reported by the kernel library."""


@dataclass(frozen=True)
class QueueConfig:
    max_in_flight_per_queue: int = 16

    def __post_init__(self):
        if self.max_in_flight_per_queue <= 0:
            raise ValueError("QueueConfig max_in_flight_per_queue must be nonzero")


@dataclass(frozen=True)
class DeviceMemoryConfig:
    tensor_arena_bytes: int = 0


@dataclass(frozen=True)
class WorkspaceRequirements:
    bytes: int = 0
    alignment: int = 1


def compute_staging_size(logical_nbytes: int) -> int:
    """gpu_algorithm::compute_staging_size (include/iom/gpu_algorithm.hpp:10-20)."""
    return logical_nbytes + (4 - logical_nbytes % 4) % 4


def _status_to_exception(status: int) -> Exception:
    text = _abi.last_error()
    if status == 1:
        return ValueError(text)
    if status == 2:
        return UnsupportedOperation(text)
    if status == 3:
        return OverflowError(text)
    if status == 4:
        return MemoryError(text)
    if status == 5:
        return DeviceError(text)
    return RuntimeError(text)


def _exception_to_oid(error: BaseException) -> int:
    """map_failure (src/device_ops.cpp:422-439)."""
    if isinstance(error, UnsupportedOperation):
        return OID_UNSUPPORTED
    if isinstance(error, MemoryError):
        return OID_RESOURCE_EXHAUSTED
    if isinstance(error, OverflowError):
        return OID_OVERFLOW
    if isinstance(error, (ValueError, IndexError)):
        return OID_INVALID_ARGUMENT
    if isinstance(error, DeviceError):
        return OID_DEVICE_ERROR
    return OID_DEVICE_ERROR


class _Arena:
    """First-fit free list with coalescing over one device allocation
    (the role of ListAllocator, include/iom/alloc.hpp:52-80).

    `release` may be called from a finalizer, which the garbage collector can
    run in the middle of `alloc` on the same thread. It therefore never takes
    the lock: it only queues the range (deque.append is atomic) and the next
    `alloc` folds the queue into the free list.
    """

    def __init__(self, capacity: int):
        self.capacity = capacity
        self.free = [(0, capacity)]
        self.lock = threading.Lock()
        self.pending = collections.deque()

    def _drain(self) -> None:
        changed = False
        while True:
            try:
                self.free.append(self.pending.popleft())
                changed = True
            except IndexError:
                break
        if changed:
            self.free.sort()
            merged = []
            for start, length in self.free:
                if merged and merged[-1][0] + merged[-1][1] == start:
                    merged[-1] = (merged[-1][0], merged[-1][1] + length)
                else:
                    merged.append((start, length))
            self.free = merged

    def alloc(self, size: int) -> int:
        size = (size + _ALIGNMENT - 1) // _ALIGNMENT * _ALIGNMENT
        with self.lock:
            self._drain()
            for i, (offset, length) in enumerate(self.free):
                if length >= size:
                    if length == size:
                        del self.free[i]
                    else:
                        self.free[i] = (offset + size, length - size)
                    return offset
        raise MemoryError("device tensor arena is exhausted")

    def release(self, offset: int, size: int) -> None:
        size = (size + _ALIGNMENT - 1) // _ALIGNMENT * _ALIGNMENT
        self.pending.append((offset, size))


class RawWorkspaceView:
    """Checked byte range over one live workspace (include/iom/tensor.hpp:186-241)."""

    def __init__(self, owner: Optional["RawWorkspace"] = None, offset: int = 0, nbytes: int = 0):
        self.owner = owner
        self.offset = offset
        self.nbytes = nbytes

    def empty(self) -> bool:
        return self.owner is None

    def byte_size(self) -> int:
        return self.nbytes

    def address(self) -> int:
        return 0 if self.owner is None else self.owner.address + self.offset

    def subrange(self, offset: int, nbytes: int) -> "RawWorkspaceView":
        if self.owner is None:
            raise ValueError("empty workspace view has no subrange")
        if offset % 32 != 0:
            raise ValueError("workspace subrange offset must stay 32-byte aligned")
        if offset > self.owner.nbytes or nbytes > self.owner.nbytes - offset:
            raise ValueError("workspace subrange exceeds the owner range")
        return RawWorkspaceView(self.owner, offset, nbytes)


class RawWorkspace:
    """Explicitly owned raw device scratch, an arena suballocation."""

    def __init__(self, device: "B200Device", nbytes: int):
        self.device = device
        self.nbytes = nbytes
        self._offset = device._arena.alloc(nbytes) if nbytes else None
        self.address = device._arena_address + self._offset if nbytes else 0
        device._live_workspaces.add(self)

    def view(self) -> RawWorkspaceView:
        return RawWorkspaceView(self if self.nbytes else None, 0, self.nbytes)

    def tensor(self) -> torch.Tensor:
        return self.device._arena_tensor[self._offset:self._offset + self.nbytes]

    def close(self) -> None:
        if self in self.device._live_workspaces:
            self.device._live_workspaces.discard(self)
            if self.nbytes:
                self.device._arena.release(self._offset, self.nbytes)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class B200Tensor:
    """Tensor owner: zero-filled tiled storage inside the device arena
    (src/cuda/device_tensor.cpp:81-103)."""

    def __init__(self, device: "B200Device", spec: TensorSpec):
        self.device = device
        self.spec = spec
        self.storage_nbytes = spec.tiled_storage_nbytes()
        self._offset = device._arena.alloc(self.storage_nbytes)
        self._address = device._arena_address + self._offset
        self._view = TensorView(self, spec, 0, dense_plane_strides(spec.shape))
        self._closed = False
        self.storage().zero_()
        torch.cuda.current_stream(device.torch_device).synchronize()

    def storage(self) -> torch.Tensor:
        """The owner's raw tiled bytes as a uint8 device tensor."""
        return self.device._arena_tensor[self._offset:self._offset + self.storage_nbytes]

    def storage_address(self) -> int:
        return self._address

    def view(self) -> TensorView:
        return self._view

    def host_transfer_workspace_requirements(self, logical_nbytes: int) -> WorkspaceRequirements:
        return WorkspaceRequirements(compute_staging_size(logical_nbytes), 32)

    def _staging(self, view: TensorView, workspace: Optional[RawWorkspaceView]) -> RawWorkspaceView:
        need = self.host_transfer_workspace_requirements(view.spec.logical_nbytes())
        if workspace is None or workspace.empty():
            raise ValueError("host transfer requires a staging workspace")
        if workspace.owner.device is not self.device or workspace.owner not in self.device._live_workspaces:
            raise ValueError("host transfer workspace belongs to another device or is dead")
        if workspace.byte_size() < need.bytes or workspace.address() % need.alignment != 0:
            raise ValueError("host transfer workspace is too small or misaligned")
        return workspace

    def region_from_host(self, view: TensorView, source, workspace=None) -> None:
        """Tensor::region_from_host (src/cuda/device_tensor.cpp:140-158): synchronous."""
        payload = np.ascontiguousarray(source).view(np.uint8).reshape(-1)
        if payload.size != view.spec.logical_nbytes():
            raise ValueError("host source must hold exactly logical_nbytes bytes")
        if view.spec.data_type == DataType.BOOL and payload.size and payload.max() > 1:
            raise ValueError("BOOL host bytes must contain zero or one")
        staging = self._staging(view, workspace)
        with self.device._transfer_lock:
            stream = torch.cuda.current_stream(self.device.torch_device)
            target = staging.owner.tensor()[staging.offset:staging.offset + payload.size]
            target.copy_(torch.from_numpy(payload), non_blocking=True)
            abi_view = view.as_abi()
            status = self.device._lib.iomb_scatter(
                ctypes.byref(abi_view), staging.address(), stream.cuda_stream)
            if status != 0:
                raise _status_to_exception(status)
            stream.synchronize()

    def region_to_host(self, view: TensorView, destination=None, workspace=None):
        nbytes = view.spec.logical_nbytes()
        staging = self._staging(view, workspace)
        with self.device._transfer_lock:
            stream = torch.cuda.current_stream(self.device.torch_device)
            abi_view = view.as_abi()
            status = self.device._lib.iomb_gather(
                ctypes.byref(abi_view), staging.address(), stream.cuda_stream)
            if status != 0:
                raise _status_to_exception(status)
            device_bytes = staging.owner.tensor()[staging.offset:staging.offset + nbytes]
            if destination is not None:
                out = np.asarray(destination).view(np.uint8).reshape(-1)
                if out.size != nbytes:
                    raise ValueError("host destination must hold exactly logical_nbytes bytes")
                torch.from_numpy(out).copy_(device_bytes, non_blocking=True)
                stream.synchronize()
                return destination
            return device_bytes.cpu().numpy()

    def close(self) -> None:
        if not self._closed:
            self._closed = True
            self.device._arena.release(self._offset, self.storage_nbytes)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class B200Device:
    """One CUDA device ordinal with a fixed tensor arena."""

    def __init__(self, ordinal: int, memory: DeviceMemoryConfig, queue_config: QueueConfig):
        if memory.tensor_arena_bytes == 0 or memory.tensor_arena_bytes % 32 != 0:
            raise ValueError("tensor_arena_bytes must be nonzero and divisible by 32")
        self._lib = _abi.load_library()          # raises when the kernels are not built
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: the B200 backend has no CPU fallback")
        if ordinal < 0 or ordinal >= torch.cuda.device_count():
            raise ValueError("invalid CUDA device ordinal")
        self.ordinal = ordinal
        self.torch_device = torch.device("cuda", ordinal)
        self.queue_config = queue_config
        try:
            self._arena_tensor = torch.empty(memory.tensor_arena_bytes, dtype=torch.uint8,
                                             device=self.torch_device)
        except torch.OutOfMemoryError as error:
            raise MemoryError(str(error)) from None
        self._arena_address = self._arena_tensor.data_ptr()
        self._arena = _Arena(memory.tensor_arena_bytes)
        self._live_workspaces = set()
        self._live_queues = 0
        self._next_queue_id = 1
        self._transfer_lock = threading.Lock()
        self._lock = threading.RLock()   # finalizers may re-enter on the same thread
        # Rotary caches: (theta as binary32 bits, width) -> device table of (cos, sin)
        # for positions 0 .. rows-1, grown by doubling; replaced tables stay alive
        # because work already queued may still read them.
        self._rope_tables = {}
        self._rope_retired = []

    def backend_kind(self) -> str:
        return "CUDA"

    def backend_device(self) -> int:
        return self.ordinal

    def supported_data_types(self):
        return tuple(DataType)

    def create_tensor(self, spec: TensorSpec) -> B200Tensor:
        with torch.cuda.device(self.torch_device):
            return B200Tensor(self, spec)

    def create_workspace(self, nbytes: int) -> RawWorkspace:
        return RawWorkspace(self, nbytes)

    def owns_workspace(self, workspace: RawWorkspace) -> bool:
        return workspace in self._live_workspaces

    def rope_table(self, theta: float, width: int, positions: int) -> torch.Tensor:
        """Device table [rows, width/2, 2] of (cos, sin) covering at least `positions`
        positions from 0. The angles are computed on the host by iomb_rope_angles (the
        reference CPU backend's expression with this host's powf / sinf / cosf)."""
        import struct
        key = (struct.unpack("<I", struct.pack("<f", theta))[0], width)
        with self._lock:
            table = self._rope_tables.get(key)
            if table is not None and table.shape[0] >= positions:
                return table
            rows = 256
            while rows < positions:
                rows *= 2
            host = torch.empty((rows, width // 2, 2), dtype=torch.float32).pin_memory()
            status = self._lib.iomb_rope_angles(host.data_ptr(), 0, rows, width, float(theta))
            if status != 0:
                raise _status_to_exception(status)
            if table is not None:
                self._rope_retired.append(table)
            table = host.to(self.torch_device)
            self._rope_tables[key] = table
            return table

    def create_ops(self) -> "B200Queue":
        with self._lock:
            if self._live_queues >= _MAX_QUEUES:
                raise MemoryError("device queue capacity is exhausted")
            self._live_queues += 1
            queue_id = self._next_queue_id
            self._next_queue_id += 1
        return B200Queue(self, queue_id)


def make_b200_device(ordinal: int, memory: DeviceMemoryConfig,
                     queue_config: QueueConfig = QueueConfig()) -> B200Device:
    """Factory with the signature of make_cuda_device (include/iom/cuda/device.hpp:22-24)."""
    return B200Device(ordinal, memory, queue_config)


class SdpaStages:
    """The two workspace segments of the attention stages that are not matrix products,
    laid out as the reference's CUDA backend does (src/cuda/sdpa_nonmatrix_request.hpp:22-49):
    FP32 scores [planes, Hq, pad16(R), pad16(L)] at the start of the workspace range, the
    BF16 probabilities of the same extents behind them, each segment rounded up to 32 bytes."""

    def __init__(self, workspace: RawWorkspaceView, planes: int, Hq: int, Hkv: int, R: int,
                 C: int, D: int, a: int, L: int):
        for name, value in (("planes", planes), ("Hq", Hq), ("Hkv", Hkv), ("R", R), ("C", C),
                            ("D", D), ("a", a), ("L", L)):
            if not 0 <= value < 1 << 64:
                raise ValueError(f"sdpa stages: {name} is out of range")
        self.workspace = workspace
        self.planes, self.Hq, self.Hkv, self.R, self.C, self.D, self.a, self.L = \
            planes, Hq, Hkv, R, C, D, a, L
        self.Rp, self.Lp = (R + 15) // 16 * 16, (L + 15) // 16 * 16
        self.cells = planes * Hq * self.Rp * self.Lp
        self.score_bytes = (self.cells * 4 + 31) // 32 * 32
        self.probability_bytes = (self.cells * 2 + 31) // 32 * 32
        if workspace is None or workspace.empty() or \
                workspace.byte_size() < self.score_bytes + self.probability_bytes:
            raise ValueError("sdpa stages: the workspace is smaller than workspace_bytes()")

    @staticmethod
    def workspace_bytes(planes: int, Hq: int, R: int, L: int) -> int:
        cells = planes * Hq * ((R + 15) // 16 * 16) * ((L + 15) // 16 * 16)
        return (cells * 4 + 31) // 32 * 32 + (cells * 2 + 31) // 32 * 32

    def scores_address(self) -> int:
        return self.workspace.address()

    def probability_address(self) -> int:
        return self.workspace.address() + self.score_bytes

    def as_abi(self) -> "_abi.IombSdpaStages":
        return _abi.IombSdpaStages(self.scores_address(), self.probability_address(), self.planes,
                                   self.Hq, self.Hkv, self.R, self.C, self.D, self.a, self.L)


class SubmissionFaults:
    """Host-side fault table of one queue, for failure-path tests (the role of the
    reference's test-only failure latches, src/cpu/queue.cpp:51-87,128-160): a named
    point of the submission path is armed to fail once, after `skip` passages.
    Nothing here touches the device: every fault is an error code or an exception
    raised on the host, the context stays usable.

      "launch"    the kernel library's entry point is not called; the wrapper reports
                  IOMB_ERR_DEVICE -> the operation returns OidError::DeviceError
      "record"    the completion event cannot be recorded after an accepted launch ->
                  the stream is drained instead (the reference's second proof of
                  completion) and the operation still returns a token
      "complete"  the accepted operation is reported failed when its completion is
                  observed -> retained failure, rethrown by every wait on the token
    """

    POINTS = ("launch", "record", "complete")

    def __init__(self):
        self._armed = {}

    def arm(self, point: str, skip: int = 0) -> None:
        if point not in self.POINTS:
            raise ValueError(f"unknown fault point {point!r}")
        self._armed[point] = int(skip)

    def clear(self) -> None:
        self._armed.clear()

    def take(self, point: str) -> bool:
        """True exactly once per arming, on the passage the arming named."""
        left = self._armed.get(point)
        if left is None:
            return False
        if left > 0:
            self._armed[point] = left - 1
            return False
        del self._armed[point]
        return True


class CapturedSequence:
    """A run of queue operations recorded once and replayed as one CUDA graph launch:
    the launch-bound inner loop of a decode step (embedding, norms, cache appends,
    gate) costs one submission instead of one per kernel.

        with queue.capture() as step:
            queue.embedding(...); queue.rmsnorm(...); queue.cache_append_batched(...)
        token = step.replay()        # an ordinary token of the queue
        queue.wait(token)
    """

    def __init__(self, queue: "B200Queue"):
        self._queue = queue
        self._graph = torch.cuda.CUDAGraph()
        self._context = None
        self._owners = []
        self._status_cells = []
        self._rejected = []
        self._operations = 0
        self._ready = False
        # Pinned status cells are reserved before the capture starts (pinning memory
        # is not a capturable call): one per status-bearing operation.
        self._cell_pool = torch.zeros(self.MAX_STATUS_OPERATIONS, dtype=torch.int32).pin_memory()
        # The queue keeps every sequence alive until close(): a graph or pinned cell
        # released by the garbage collector while another sequence is being recorded
        # would invalidate that capture.
        queue._sequences.append(self)

    MAX_STATUS_OPERATIONS = 64

    def _take_cell(self):
        index = len(self._status_cells)
        if index >= self.MAX_STATUS_OPERATIONS:
            raise ValueError("a captured sequence holds at most 64 status-bearing operations")
        cell = self._cell_pool[index:index + 1]
        self._status_cells.append(cell)
        return cell

    def __enter__(self) -> "CapturedSequence":
        queue = self._queue
        queue._stream.synchronize()
        queue._capture = self
        # Only this thread's unsafe calls invalidate the capture (other threads may
        # allocate freely meanwhile).
        self._context = torch.cuda.graph(self._graph, stream=queue._stream,
                                         capture_error_mode="thread_local")
        try:
            self._context.__enter__()
        except BaseException:
            queue._capture = None
            raise
        return self

    def __exit__(self, kind, value, trace) -> bool:
        queue = self._queue
        try:
            self._context.__exit__(kind, value, trace)
        finally:
            queue._capture = None
        if kind is None:
            if self._rejected:
                raise self._rejected[0]
            self._ready = True
        return False

    @property
    def operations(self) -> int:
        return self._operations

    def close(self) -> None:
        """Releases the graph; not while the queue is recording."""
        queue = self._queue
        if queue._capture is not None:
            raise RuntimeError("a sequence cannot be released while the queue records another")
        queue._stream.synchronize()
        self._ready = False
        if self in queue._sequences:
            queue._sequences.remove(self)

    def replay(self) -> int:
        """Launches the recorded graph on the queue's stream; returns a token."""
        if not self._ready:
            raise RuntimeError("the sequence was not recorded successfully")
        queue = self._queue
        if queue._capture is not None:
            raise RuntimeError("a sequence cannot be replayed while the queue records another")

        def launch(_stream):
            with torch.cuda.stream(queue._stream):
                self._graph.replay()
            return 0
        token = queue._submit(launch, tuple(self._owners))
        if token > 0 and self._status_cells:
            sequence = token & ((1 << _SEQUENCE_BITS) - 1)
            event, owners, _ = queue._records[sequence]
            queue._records[sequence] = (event, owners, self._status_cells)
        return token


class B200Queue:
    """DeviceOps: one in-order asynchronous queue = one CUDA stream."""

    def __init__(self, device: B200Device, queue_id: int):
        self._device = device
        self._lib = device._lib
        self._queue_id = queue_id
        self._stream = torch.cuda.Stream(device=device.torch_device)
        self._sequence = 0
        self._records = {}        # sequence -> (event, owners, status cell or None)
        self._failures = {}       # sequence -> exception
        self._completed = 0
        self._closed = False
        self._capture = None      # the CapturedSequence being recorded, if any
        self.faults = SubmissionFaults()
        self._sequences = []      # every recorded sequence, kept alive until closed
        # Queue-owned pinned cells for status read-backs, one per in-flight credit
        # (the reference keeps one pinned cell per queue, src/cuda/device.cpp:165-200).
        self._status_cells = torch.zeros(device.queue_config.max_in_flight_per_queue,
                                         dtype=torch.int32).pin_memory()

    # -- plumbing -----------------------------------------------------------
    def device(self) -> B200Device:
        return self._device

    @property
    def stream(self) -> torch.cuda.Stream:
        return self._stream

    def close(self) -> None:
        if not self._closed:
            self._closed = True
            self._stream.synchronize()
            self._records.clear()
            self._sequences.clear()
            with self._device._lock:
                self._device._live_queues -= 1

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check_view(self, view: TensorView, what: str) -> None:
        owner = view.owner_identity()
        if owner is None or getattr(owner, "device", None) is not self._device:
            raise ValueError(f"{what} view owner belongs to another device")

    def _retire(self, limit: int) -> None:
        """Bounds in-flight work to the configured credit count."""
        while len(self._records) >= limit:
            oldest = min(self._records)
            self._finish(oldest)

    def _finish(self, sequence: int) -> None:
        record = self._records.pop(sequence, None)
        if record is None:
            return
        event, _owners, status_cell = record
        if event is None:
            self._stream.synchronize()      # no event could be recorded: drain the stream
        else:
            event.synchronize()
        if self.faults.take("complete"):
            self._failures[sequence] = DeviceError("injected completion failure")
            return
        cells = status_cell if isinstance(status_cell, list) else \
            ([] if status_cell is None else [status_cell])
        if any(int(cell.item()) != 0 for cell in cells):
            self._failures[sequence] = ValueError("embedding index is negative or out of range")

    def _submit(self, launch, owners, status_cell=None) -> int:
        if self._capture is not None:
            return self._submit_captured(launch, owners, status_cell)
        try:
            self._retire(self._device.queue_config.max_in_flight_per_queue)
            with torch.cuda.device(self._device.torch_device):
                if self.faults.take("launch"):
                    raise DeviceError("injected launch failure")
                status = launch(self._stream.cuda_stream)
                if status != 0:
                    raise _status_to_exception(status)
                event = None
                if not self.faults.take("record"):
                    event = torch.cuda.Event()
                    event.record(self._stream)
                pinned = None
                if status_cell is not None:
                    slot = (self._sequence + 1) % self._status_cells.numel()
                    pinned = self._status_cells[slot:slot + 1]
                    with torch.cuda.stream(self._stream):
                        pinned.copy_(status_cell, non_blocking=True)
                    event = torch.cuda.Event()
                    event.record(self._stream)
            self._sequence += 1
            self._records[self._sequence] = (event, owners, pinned)
            return (self._queue_id << _SEQUENCE_BITS) | self._sequence
        except BaseException as error:  # the facade is noexcept: map to an oid
            return _exception_to_oid(error)

    # -- CUDA graph capture ---------------------------------------------------
    def _submit_captured(self, launch, owners, status_cell) -> int:
        """One operation inside capture(): the launch is recorded into the graph; no
        event, no sequence number. Status words are copied to a pinned cell of the
        sequence by a captured copy and checked after every replay."""
        try:
            with torch.cuda.device(self._device.torch_device):
                status = launch(self._stream.cuda_stream)
                if status != 0:
                    raise _status_to_exception(status)
                if status_cell is not None:
                    pinned = self._capture._take_cell()
                    pinned.copy_(status_cell, non_blocking=True)
            self._capture._owners.extend(owners)
            self._capture._operations += 1
            return OID_CAPTURED
        except BaseException as error:
            self._capture._rejected.append(error)
            return _exception_to_oid(error)

    def capture(self) -> "CapturedSequence":
        """Context manager: records the operations issued on this queue inside the
        block into one CUDA graph instead of running them. The C ABI entry points
        neither allocate nor synchronise, so they are capture-safe as they are;
        run the same sequence once eagerly first (one-time set-up such as the SiLU
        table build does synchronise). The views' storage is baked into the graph:
        replays read whatever the same tensors hold at that time."""
        if self._capture is not None:
            raise RuntimeError("this queue is already recording a sequence")
        return CapturedSequence(self)

    def wait(self, token: int) -> None:
        """DeviceOps::wait (src/device_ops.cpp:536-568)."""
        if token == OID_CAPTURED:
            raise ValueError("a captured operation completes with its sequence's replay token")
        if token <= 0 or (token >> _SEQUENCE_BITS) != self._queue_id:
            raise ValueError("wait token is not an accepted token of this queue")
        sequence = token & ((1 << _SEQUENCE_BITS) - 1)
        if sequence == 0 or sequence > self._sequence:
            raise ValueError("wait token was never submitted")
        for pending in sorted(s for s in self._records if s <= sequence):
            self._finish(pending)
        if sequence in self._failures:
            raise self._failures[sequence]

    # -- operations -----------------------------------------------------------
    def _binary(self, op: int, lhs: TensorView, rhs: TensorView, out: TensorView) -> int:
        try:
            for view, what in ((lhs, "lhs"), (rhs, "rhs"), (out, "out")):
                self._check_view(view, what)
            a, b, c = lhs.as_abi(), rhs.as_abi(), out.as_abi()
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(
            lambda stream: self._lib.iomb_binary(op, ctypes.byref(a), ctypes.byref(b),
                                                 ctypes.byref(c), stream),
            (lhs.owner, rhs.owner, out.owner))

    def add(self, lhs: TensorView, rhs: TensorView, out: TensorView, workspace=None) -> int:
        return self._binary(ADD, lhs, rhs, out)

    def mul(self, lhs: TensorView, rhs: TensorView, out: TensorView, workspace=None) -> int:
        return self._binary(MUL, lhs, rhs, out)

    def sub(self, lhs: TensorView, rhs: TensorView, out: TensorView, workspace=None) -> int:
        return self._binary(SUB, lhs, rhs, out)

    def div(self, lhs: TensorView, rhs: TensorView, out: TensorView, workspace=None) -> int:
        return self._binary(DIV, lhs, rhs, out)

    def rmsnorm(self, x: TensorView, scale: TensorView, out: TensorView, eps: float,
                workspace: Optional[RawWorkspaceView] = None, order: Optional[int] = None) -> int:
        """`order` None takes the facade's choice: the lane order for BF16 (the reference's
        AVX-512 BF16 build, bit for bit), the sequential order for F32 (the only F32 order
        the reference has, src/cpu/queue.cpp:1187-1196, bit for bit)."""
        try:
            for view, what in ((x, "x"), (scale, "scale"), (out, "out")):
                self._check_view(view, what)
            if order is None:
                order = facade_order(x.spec.data_type)
            if workspace is not None and not workspace.empty():
                raise ValueError("rmsnorm takes no workspace")
            a, b, c = x.as_abi(), scale.as_abi(), out.as_abi()
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(
            lambda stream: self._lib.iomb_rmsnorm(ctypes.byref(a), ctypes.byref(b),
                                                  ctypes.byref(c), eps, order, stream),
            (x.owner, scale.owner, out.owner))

    def add_rmsnorm(self, x: TensorView, residual: TensorView, scale: TensorView,
                    total: TensorView, out: TensorView, eps: float,
                    order: Optional[int] = None) -> int:
        """Extension: residual ADD fused into the following RMSNorm."""
        try:
            views = (x, residual, scale, total, out)
            for view in views:
                self._check_view(view, "add_rmsnorm")
            if order is None:
                order = facade_order(x.spec.data_type)
            abis = [v.as_abi() for v in views]
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(
            lambda stream: self._lib.iomb_add_rmsnorm(*[ctypes.byref(v) for v in abis], eps,
                                                      order, stream),
            tuple(v.owner for v in views))

    def copy(self, source: TensorView, destination: TensorView) -> int:
        try:
            self._check_view(source, "source")
            self._check_view(destination, "destination")
            if source.spec != destination.spec:
                raise ValueError("copy views must have identical shape, leaf type, and quantization")
            a, b = source.as_abi(), destination.as_abi()
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(
            lambda stream: self._lib.iomb_copy(ctypes.byref(a), ctypes.byref(b), stream),
            (source.owner, destination.owner))

    def cast(self, source: TensorView, destination: TensorView) -> int:
        """Extension: BF16<->F32 conversion."""
        try:
            self._check_view(source, "source")
            self._check_view(destination, "destination")
            a, b = source.as_abi(), destination.as_abi()
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(
            lambda stream: self._lib.iomb_cast(ctypes.byref(a), ctypes.byref(b), stream),
            (source.owner, destination.owner))

    def embedding_workspace_requirements(self, table, indices, out) -> WorkspaceRequirements:
        return WorkspaceRequirements(32, 32)

    def embedding(self, table: TensorView, indices: TensorView, out: TensorView,
                  workspace: Optional[RawWorkspaceView] = None) -> int:
        try:
            for view, what in ((table, "table"), (indices, "indices"), (out, "out")):
                self._check_view(view, what)
            if workspace is None or workspace.empty() or workspace.byte_size() < 32 \
                    or workspace.address() % 32 != 0 \
                    or not self._device.owns_workspace(workspace.owner):
                raise ValueError("embedding requires a live {32,32} workspace of this device")
            a, b, c = table.as_abi(), indices.as_abi(), out.as_abi()
            cell = workspace.owner.tensor()[workspace.offset:workspace.offset + 4].view(torch.int32)
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(
            lambda stream: self._lib.iomb_embedding(ctypes.byref(a), ctypes.byref(b),
                                                    ctypes.byref(c), workspace.address(), stream),
            (table.owner, indices.owner, out.owner, workspace.owner), status_cell=cell)

    def cache_append(self, source: TensorView, destination: TensorView, a: int,
                     workspace=None) -> int:
        try:
            self._check_view(source, "source")
            self._check_view(destination, "destination")
            if a < 0 or a >= 1 << 64:
                raise ValueError("cache_append offset is out of range")
            s, d = source.as_abi(), destination.as_abi()
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(
            lambda stream: self._lib.iomb_cache_append(ctypes.byref(s), ctypes.byref(d), a, stream),
            (source.owner, destination.owner))

    def cache_append_batched(self, source: TensorView, destination: TensorView,
                             positions: int, status: int) -> int:
        """Extension: one row offset per index of the first leading axis.
        `positions` / `status` are device addresses (uint32[dims[0]] / uint32)."""
        try:
            self._check_view(source, "source")
            self._check_view(destination, "destination")
            s, d = source.as_abi(), destination.as_abi()
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(
            lambda stream: self._lib.iomb_cache_append_batched(
                ctypes.byref(s), ctypes.byref(d), positions, status, stream),
            (source.owner, destination.owner))

    def upload(self, view: TensorView, source, workspace: RawWorkspaceView) -> int:
        """Extension: the host-to-device transfer of Tensor::region_from_host as an
        asynchronous operation of this queue. `source` holds the view's logical bytes
        (row-major) in pinned host memory and must stay untouched until the returned
        token completes; `workspace` is the {logical bytes, 32} staging range, private
        to this queue while the token is pending. Two queues uploading and downloading
        alternate slices keep both PCIe directions busy."""
        try:
            self._check_view(view, "view")
            payload = np.ascontiguousarray(source).view(np.uint8).reshape(-1)
            if payload.size != view.spec.logical_nbytes():
                raise ValueError("host source must hold exactly logical_nbytes bytes")
            staging = view.owner._staging(view, workspace)
            host = torch.from_numpy(payload)
            target = staging.owner.tensor()[staging.offset:staging.offset + payload.size]
            abi_view = view.as_abi()
        except BaseException as error:
            return _exception_to_oid(error)

        def launch(stream):
            with torch.cuda.stream(self._stream):
                target.copy_(host, non_blocking=True)
            return self._lib.iomb_scatter(ctypes.byref(abi_view), staging.address(), stream)
        return self._submit(launch, (view.owner, staging.owner, host))

    def download(self, view: TensorView, destination, workspace: RawWorkspaceView) -> int:
        """Extension: Tensor::region_to_host as an asynchronous operation of this queue;
        `destination` (pinned host memory, logical_nbytes bytes) is valid once the
        returned token completes."""
        try:
            self._check_view(view, "view")
            out = np.asarray(destination).view(np.uint8).reshape(-1)
            if out.size != view.spec.logical_nbytes() or not out.flags.writeable:
                raise ValueError("host destination must hold exactly logical_nbytes writable bytes")
            staging = view.owner._staging(view, workspace)
            host = torch.from_numpy(out)
            source = staging.owner.tensor()[staging.offset:staging.offset + out.size]
            abi_view = view.as_abi()
        except BaseException as error:
            return _exception_to_oid(error)

        def launch(stream):
            status = self._lib.iomb_gather(ctypes.byref(abi_view), staging.address(), stream)
            if status == 0:
                with torch.cuda.stream(self._stream):
                    host.copy_(source, non_blocking=True)
            return status
        return self._submit(launch, (view.owner, staging.owner, host))

    def sumsq(self, x: TensorView, scratch: RawWorkspaceView, result: int) -> int:
        """Extension: whole-view FP32 sum of squares into the device float at `result`."""
        try:
            self._check_view(x, "x")
            need = int(self._lib.iomb_sumsq_scratch_bytes())
            if scratch is None or scratch.empty() or scratch.byte_size() < need:
                raise ValueError("sumsq requires a scratch workspace of iomb_sumsq_scratch_bytes()")
            view = x.as_abi()
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(
            lambda stream: self._lib.iomb_sumsq(ctypes.byref(view), scratch.address(), result,
                                                stream),
            (x.owner, scratch.owner))

    # The remaining operations of the contract are not part of this backend.
    def silu_workspace_requirements(self, x, y) -> WorkspaceRequirements:
        return WorkspaceRequirements(0, 1)

    def silu(self, x: TensorView, y: TensorView, workspace=None) -> int:
        try:
            self._check_view(x, "x")
            self._check_view(y, "y")
            a, b = x.as_abi(), y.as_abi()
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(
            lambda stream: self._lib.iomb_silu(ctypes.byref(a), ctypes.byref(b), stream),
            (x.owner, y.owner))

    def silu_mul(self, x: TensorView, up: TensorView, out: TensorView,
                 activated: Optional[TensorView] = None) -> int:
        """Extension: out = silu(x) * up in one pass; `activated` receives silu(x) when given."""
        try:
            views = [x, up, out] + ([activated] if activated is not None else [])
            for view in views:
                self._check_view(view, "silu_mul")
            a, b, c = x.as_abi(), up.as_abi(), out.as_abi()
            d = activated.as_abi() if activated is not None else None
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(
            lambda stream: self._lib.iomb_silu_mul(
                ctypes.byref(a), ctypes.byref(b), ctypes.byref(d) if d is not None else None,
                ctypes.byref(c), stream),
            tuple(view.owner for view in views))

    def linear(self, *args, **kwargs) -> int:
        return OID_UNSUPPORTED

    def rope_workspace_requirements(self, x, out, a, theta) -> WorkspaceRequirements:
        return WorkspaceRequirements(0, 1)

    def rope(self, x: TensorView, out: TensorView, a: int, theta: float, workspace=None) -> int:
        """DeviceOps::rope (include/iom/iom.hpp): split-half rotary embedding of
        [..., H, R, W] with row r at position a + r."""
        try:
            self._check_view(x, "x")
            self._check_view(out, "out")
            if a < 0 or a >= 1 << 64:
                raise ValueError("rope position offset is out of range")
            xv, ov = x.as_abi(), out.as_abi()
            rows, width = x.spec.shape[-2], x.spec.shape[-1]
            if x.spec.rank < 3 or width % 2 != 0 or a + rows - 1 >= 1 << 24:
                raise ValueError("rope requires rank >= 3, an even width and positions below 2^24")
            if not (1.0 <= theta <= 3.4028234663852886e38):
                raise ValueError("rope theta must be finite in [1,float_max]")
            table = self._device.rope_table(theta, width, a + rows)
            first = table.data_ptr() + a * (width // 2) * 8
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(
            lambda stream: self._lib.iomb_rope(ctypes.byref(xv), ctypes.byref(ov), a, first, stream),
            (x.owner, out.owner, table))

    def sdpa(self, *args, **kwargs) -> int:
        return OID_UNSUPPORTED

    # The stages of attention that are not matrix products (the backend-private launches
    # of src/cuda/sdpa_nonmatrix.hpp:15-28), offered on their own until the QK and PV
    # products exist here.
    def _sdpa_stage(self, stages: "SdpaStages", call) -> int:
        try:
            if not isinstance(stages, SdpaStages):
                raise ValueError("sdpa stage requires an SdpaStages description")
            request = stages.as_abi()
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(lambda stream: call(ctypes.byref(request), stream),
                            (stages.workspace.owner,))

    def sdpa_scale_mask(self, stages: "SdpaStages") -> int:
        """launch_sdpa_scale_mask: visible scores times 1/sqrt(D), zero products as +0."""
        return self._sdpa_stage(stages, self._lib.iomb_sdpa_scale_mask)

    def sdpa_softmax(self, stages: "SdpaStages") -> int:
        """launch_sdpa_softmax: BF16 probabilities of the visible tokens, +0 up to L."""
        return self._sdpa_stage(stages, self._lib.iomb_sdpa_softmax)

    def sdpa_scale_mask_softmax(self, stages: "SdpaStages", keep_scores: bool = False) -> int:
        """Extension: both stages in one pass; the scaled scores are stored only on request."""
        keep = 1 if keep_scores else 0
        return self._sdpa_stage(
            stages, lambda request, stream: self._lib.iomb_sdpa_scale_mask_softmax(request, keep, stream))

    def sdpa_canonicalize_output(self, out: TensorView) -> int:
        """launch_sdpa_canonicalize_output: -0 to +0 and every NaN to 0x7FC0 in the merged
        BF16 output [B..., R, Hq*D]."""
        try:
            self._check_view(out, "out")
            view = out.as_abi()
        except BaseException as error:
            return _exception_to_oid(error)
        return self._submit(
            lambda stream: self._lib.iomb_sdpa_canonicalize_output(ctypes.byref(view), stream),
            (out.owner,))
