"""The Python TensorView transforms against the reference's own TensorView."""
import numpy as np
import pytest

from iom_b200.tensor import DataType, TensorSpec
from support import HostTensor, reference_or_skip


@pytest.fixture(scope="module")
def ref():
    reference = reference_or_skip("portable")
    yield reference
    reference.close()


def test_random_transform_chains_match(ref):
    rng = np.random.default_rng(42)
    for _ in range(200):
        leading = [int(v) for v in rng.integers(1, 5, size=int(rng.integers(1, 5)))]
        shape = tuple(leading) + (17, 33)
        mine = HostTensor(shape, DataType.BF16).view()
        theirs = ref.tensor(shape, DataType.BF16).view()
        for _ in range(int(rng.integers(1, 5))):
            lead = len(mine.spec.shape) - 2
            if lead == 0:
                break
            choice = rng.integers(0, 4)
            if choice == 0:
                dim = int(rng.integers(0, lead))
                extent = mine.spec.shape[dim]
                first = int(rng.integers(0, extent))
                step = int(rng.integers(1, 3))
                count = int(rng.integers(1, (extent - first - 1) // step + 2))
                args = ("slice", (dim, first, count, step))
            elif choice == 1:
                dim = int(rng.integers(0, lead))
                args = ("select", (dim, int(rng.integers(0, mine.spec.shape[dim]))))
            elif choice == 2:
                args = ("permute", ([int(v) for v in rng.permutation(lead)],))
            else:
                total = int(np.prod(mine.spec.shape[:-2]))
                args = ("reshape_leading", ([total],))
            try:
                theirs_next = getattr(theirs, args[0])(*args[1])
            except ValueError:
                with pytest.raises((ValueError, IndexError)):
                    getattr(mine, args[0])(*args[1])
                continue
            mine = getattr(mine, args[0])(*args[1])
            theirs = theirs_next
            dims, offset, strides, dtype = theirs.describe()
            assert dims == mine.spec.shape
            assert offset == mine.plane_offset
            assert strides == mine.plane_strides
            assert dtype == mine.spec.data_type


def test_spec_sizes_and_rank_limits():
    spec = TensorSpec((2, 8, 31, 33), DataType.F6_E2M3)
    assert spec.standard_padded_shape() == (2, 8, 32, 48)
    assert spec.logical_nbytes() == (2 * 8 * 31 * 33 * 6 + 7) // 8
    assert spec.tiled_storage_nbytes() == 2 * 8 * 32 * 48 * 6 // 8
    with pytest.raises(ValueError):
        TensorSpec((4,), DataType.F32)
    with pytest.raises(ValueError):
        TensorSpec((1,) * 9, DataType.F32)
    with pytest.raises(ValueError):
        TensorSpec((4, 0), DataType.F32)
    view = HostTensor((3, 4, 16, 16), DataType.F32).view()
    with pytest.raises(IndexError):
        view.slice(2, 0, 1)
    with pytest.raises(IndexError):
        view.slice(0, 2, 2)
    with pytest.raises(ValueError):
        view.slice(0, 0, 0)
    with pytest.raises(ValueError):
        view.permute([0, 0])
    with pytest.raises(ValueError):
        view.slice(0, 0, 2, 2).reshape_leading([8])
    with pytest.raises(ValueError):
        view.reshape_leading([2, 2, 3, 1, 1, 1, 1])
