"""Host-side tensor metadata: the reference's core tensor contract in Python.

Mirrors include/iom/tensor.hpp (TensorSpec :111-124, TensorView :302-366) and
src/tensor_view.cpp of the reference: a view is an owner plus a plane offset
and plane strides counted in whole planes; transforms touch leading axes only
and never relocate storage. Exception categories follow the reference:
std::invalid_argument -> ValueError, std::out_of_range -> IndexError,
std::overflow_error -> OverflowError, std::bad_alloc -> MemoryError.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Sequence

from ._abi import IombView, MAX_LEADING, MAX_RANK

TILE = 16
_SIZE_MAX = (1 << 64) - 1


class DataType(enum.IntEnum):
    """iom::DataType ordinals (include/iom/tensor.hpp:10-32)."""

    BOOL = 0
    I2 = 1
    U2 = 2
    I4 = 3
    U4 = 4
    I8 = 5
    U8 = 6
    I16 = 7
    U16 = 8
    I32 = 9
    U32 = 10
    I64 = 11
    U64 = 12
    F4_E2M1 = 13
    F6_E2M3 = 14
    F6_E3M2 = 15
    F8_E4M3FN = 16
    F8_E5M2 = 17
    F8_E8M0 = 18
    F16 = 19
    BF16 = 20
    F32 = 21
    F64 = 22


_LEAF_BITS = {
    DataType.BOOL: 8, DataType.I2: 2, DataType.U2: 2, DataType.I4: 4, DataType.U4: 4,
    DataType.I8: 8, DataType.U8: 8, DataType.I16: 16, DataType.U16: 16,
    DataType.I32: 32, DataType.U32: 32, DataType.I64: 64, DataType.U64: 64,
    DataType.F4_E2M1: 4, DataType.F6_E2M3: 6, DataType.F6_E3M2: 6,
    DataType.F8_E4M3FN: 8, DataType.F8_E5M2: 8, DataType.F8_E8M0: 8,
    DataType.F16: 16, DataType.BF16: 16, DataType.F32: 32, DataType.F64: 64,
}


def leaf_bits(data_type: DataType) -> int:
    """detail::leaf_bits (src/tensor.cpp:107-134)."""
    try:
        return _LEAF_BITS[DataType(data_type)]
    except (KeyError, ValueError):
        raise ValueError("unknown DataType value") from None


def _checked_mul(a: int, b: int, what: str) -> int:
    value = a * b
    if value > _SIZE_MAX:
        raise OverflowError(what)
    return value


def _checked_add(a: int, b: int, what: str) -> int:
    value = a + b
    if value > _SIZE_MAX:
        raise OverflowError(what)
    return value


def plane_slot(rows: int, columns: int, plane: int, row: int, column: int) -> int:
    """detail::standard_plane_slot (src/tensor.cpp:136-164)."""
    tile_rows = (rows + TILE - 1) // TILE
    tile_columns = (columns + TILE - 1) // TILE
    tile = plane * tile_rows * tile_columns + (row // TILE) * tile_columns + column // TILE
    return tile * TILE * TILE + (row % TILE) * TILE + column % TILE


@dataclass(frozen=True)
class TensorSpec:
    """Full shape (rank two through eight) plus leaf type."""

    shape: tuple
    data_type: DataType

    def __init__(self, shape: Sequence[int], data_type: DataType):
        dims = tuple(int(d) for d in shape)
        if len(dims) < 2:
            raise ValueError("tensor shape requires rank of at least two")
        if len(dims) > MAX_RANK:
            raise ValueError("tensor shape requires rank of at most eight")
        if any(d <= 0 for d in dims):
            raise ValueError("tensor dimensions must be nonzero")
        object.__setattr__(self, "shape", dims)
        object.__setattr__(self, "data_type", DataType(data_type))

    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def rows(self) -> int:
        return self.shape[-2]

    @property
    def columns(self) -> int:
        return self.shape[-1]

    def element_count(self) -> int:
        count = 1
        for extent in self.shape:
            count = _checked_mul(count, extent, "tensor element count overflows")
        return count

    def standard_padded_shape(self) -> tuple:
        padded = list(self.shape)
        for axis in (-2, -1):
            padded[axis] = _checked_add(padded[axis], TILE - 1, "padded dimension overflows") \
                // TILE * TILE
        return tuple(padded)

    def logical_nbytes(self) -> int:
        bits = _checked_mul(self.element_count(), leaf_bits(self.data_type),
                            "logical bit count overflows")
        return (bits + 7) // 8

    def tiled_storage_nbytes(self) -> int:
        count = 1
        for extent in self.standard_padded_shape():
            count = _checked_mul(count, extent, "tiled bit count overflows")
        bits = _checked_mul(count, leaf_bits(self.data_type), "tiled bit count overflows")
        return (bits + 7) // 8

    def plane_count(self) -> int:
        planes = 1
        for extent in self.shape[:-2]:
            planes = _checked_mul(planes, extent, "plane count overflows")
        return planes


def dense_plane_strides(shape: Sequence[int]) -> tuple:
    """Row-major plane strides of a dense owner (src/tensor_view.cpp:32-44)."""
    leading = len(shape) - 2
    strides = [1] * leading
    for i in range(leading - 1, 0, -1):
        strides[i - 1] = _checked_mul(strides[i], shape[i], "dense plane stride overflows")
    return tuple(strides)


class TensorView:
    """Non-owning operand over one owner (include/iom/tensor.hpp:302-366).

    `owner` is any object exposing `storage_address()` (an integer address),
    `storage_nbytes` and `device`.
    """

    __slots__ = ("_owner", "_spec", "_plane_offset", "_plane_strides")

    def __init__(self, owner, spec: TensorSpec, plane_offset: int, plane_strides: Sequence[int]):
        self._owner = owner
        self._spec = spec
        self._plane_offset = int(plane_offset)
        self._plane_strides = tuple(int(s) for s in plane_strides)

    @property
    def spec(self) -> TensorSpec:
        return self._spec

    @property
    def owner(self):
        return self._owner

    def owner_identity(self):
        return self._owner

    @property
    def device(self):
        return self._owner.device

    @property
    def plane_offset(self) -> int:
        return self._plane_offset

    @property
    def plane_strides(self) -> tuple:
        return self._plane_strides

    def native_handle(self) -> int:
        return self._owner.storage_address()

    def _leading(self) -> list:
        return list(self._spec.shape[:-2])

    def _with_leading(self, dims, offset, strides) -> "TensorView":
        spec = TensorSpec(tuple(dims) + self._spec.shape[-2:], self._spec.data_type)
        return TensorView(self._owner, spec, offset, strides)

    def slice(self, dim: int, first: int, count: int, step: int = 1) -> "TensorView":
        leading_rank = self._spec.rank - 2
        if dim >= leading_rank or dim < 0:
            raise IndexError("slice dimension is not a leading dimension")
        if count == 0:
            raise ValueError("slice count must be nonzero")
        if step == 0:
            raise ValueError("slice step must be nonzero")
        last = _checked_add(first, _checked_mul(count - 1, step, "slice last index overflows"),
                            "slice last index overflows")
        if last >= self._spec.shape[dim]:
            raise IndexError("slice last selected index exceeds the dimension")
        dims = self._leading()
        dims[dim] = count
        strides = list(self._plane_strides)
        stride = strides[dim]
        strides[dim] = _checked_mul(stride, step, "sliced plane stride overflows")
        offset = _checked_add(self._plane_offset,
                              _checked_mul(first, stride, "slice plane offset overflows"),
                              "slice plane offset overflows")
        return self._with_leading(dims, offset, strides)

    def select(self, dim: int, index: int) -> "TensorView":
        leading_rank = self._spec.rank - 2
        if dim >= leading_rank or dim < 0:
            raise IndexError("select dimension is not a leading dimension")
        if index >= self._spec.shape[dim]:
            raise IndexError("select index exceeds the dimension")
        dims = self._leading()
        strides = list(self._plane_strides)
        stride = strides[dim]
        del dims[dim]
        del strides[dim]
        offset = _checked_add(self._plane_offset,
                              _checked_mul(index, stride, "select plane offset overflows"),
                              "select plane offset overflows")
        return self._with_leading(dims, offset, strides)

    def permute(self, leading_order: Sequence[int]) -> "TensorView":
        leading_rank = self._spec.rank - 2
        order = list(leading_order)
        if len(order) != leading_rank:
            raise ValueError("permutation must cover exactly the leading dimensions")
        seen = set()
        for axis in order:
            if axis >= leading_rank or axis < 0:
                raise ValueError("permutation index exceeds the leading rank")
            if axis in seen:
                raise ValueError("duplicate permutation index")
            seen.add(axis)
        dims = [self._spec.shape[a] for a in order]
        strides = [self._plane_strides[a] for a in order]
        return self._with_leading(dims, self._plane_offset, strides)

    def reshape_leading(self, leading_dimensions: Sequence[int]) -> "TensorView":
        new_dims = [int(d) for d in leading_dimensions]
        if len(new_dims) + 2 > MAX_RANK:
            raise ValueError("reshape result rank exceeds the rank-eight limit")
        planes = 1
        for extent in self._spec.shape[:-2]:
            planes = _checked_mul(planes, extent, "leading plane count overflows")
        new_planes = 1
        for extent in new_dims:
            if extent == 0:
                raise ValueError("reshape dimension must be nonzero")
            new_planes = _checked_mul(new_planes, extent, "reshaped plane count overflows")
        if new_planes != planes:
            raise ValueError("reshape changes the leading plane count")
        expected = 1
        for i in range(self._spec.rank - 3, -1, -1):
            extent = self._spec.shape[i]
            if extent > 1:
                if self._plane_strides[i] != expected:
                    raise ValueError("reshape requires a contiguous view")
                expected = _checked_mul(expected, extent, "reshape contiguity overflows")
        strides = [0] * len(new_dims)
        stride = 1
        for i in range(len(new_dims) - 1, -1, -1):
            strides[i] = stride
            stride = _checked_mul(stride, new_dims[i], "reshaped plane stride overflows")
        return self._with_leading(new_dims, self._plane_offset, strides)

    def as_abi(self) -> IombView:
        """The value snapshot the C ABI takes (struct iomb_view)."""
        view = IombView()
        view.base = self._owner.storage_address()
        view.storage_bytes = self._owner.storage_nbytes
        view.dtype = int(self._spec.data_type)
        view.rank = self._spec.rank
        for i, extent in enumerate(self._spec.shape):
            view.dims[i] = extent
        view.plane_offset = self._plane_offset
        for i, stride in enumerate(self._plane_strides[:MAX_LEADING]):
            view.plane_strides[i] = stride
        return view

    # Host transfers are provided by the owning device tensor.
    def copy_from_host(self, source, workspace=None) -> None:
        self._owner.region_from_host(self, source, workspace)

    def copy_to_host(self, destination=None, workspace=None):
        return self._owner.region_to_host(self, destination, workspace)

    def copy_from_host_workspace_requirements(self):
        return self._owner.host_transfer_workspace_requirements(self._spec.logical_nbytes())

    def copy_to_host_workspace_requirements(self):
        return self._owner.host_transfer_workspace_requirements(self._spec.logical_nbytes())
