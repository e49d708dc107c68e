"""Helpers for the GPU parity tests: mirror a host tensor onto the device,
run an operation through the C ABI, and compare physical storage bytes."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from iom_b200.device import DeviceMemoryConfig, make_b200_device
from iom_b200.tensor import TensorView
from support import HostTensor


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    device = make_b200_device(0, DeviceMemoryConfig(2 << 30))
    queue = device.create_ops()
    yield device, queue
    queue.close()


def upload(device, host: HostTensor):
    """Device owner holding exactly the host owner's physical bytes."""
    tensor = device.create_tensor(host.spec)
    tensor.storage().copy_(torch.from_numpy(host.storage.copy()))
    torch.cuda.synchronize()
    return tensor


def download(tensor) -> np.ndarray:
    torch.cuda.synchronize()
    return tensor.storage().cpu().numpy()


def like(view: TensorView, tensor) -> TensorView:
    """The same window (shape, offset, strides) over another owner."""
    return TensorView(tensor, view.spec, view.plane_offset, view.plane_strides)


def run(queue, token: int) -> None:
    assert token > 0, f"operation rejected with oid {token}"
    queue.wait(token)
