"""GPU: the asynchronous upload / download queue operations equal the synchronous
copy_from_host / copy_to_host of the contract, byte for byte, also when two queues
work on alternate planes."""
import numpy as np
import pytest
import torch

from iom_b200.tensor import DataType
from gpu_support import download, gpu, run, upload  # noqa: F401
from support import HostTensor, random_payload

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [DataType.BF16, DataType.F32])
def test_upload_download_equal_the_synchronous_transfers(gpu, dtype):
    device, queue = gpu
    rng = np.random.default_rng(9)
    shape = (4, 33, 70)
    payload = random_payload(rng, shape, dtype, "normal")
    host = HostTensor(shape, dtype).poison()
    host.view().copy_from_host(payload)
    tensor = device.create_tensor(host.spec)
    tensor.storage().copy_(torch.from_numpy(np.full(tensor.storage_nbytes, 0xA5, dtype=np.uint8)))
    plane_bytes = 33 * 70 * (2 if dtype == DataType.BF16 else 4)
    second = device.create_ops()
    lanes = [(queue, device.create_workspace(plane_bytes + 64)),
             (second, device.create_workspace(plane_bytes + 64))]
    pinned = torch.from_numpy(np.ascontiguousarray(payload).view(np.uint8).reshape(4, plane_bytes).copy()).pin_memory()
    tokens = []
    for plane in range(4):
        q, staging = lanes[plane % 2]
        tokens.append((q, q.upload(tensor.view().select(0, plane), pinned[plane].numpy(), staging.view())))
    for q, token in tokens:
        run(q, token)
    assert np.array_equal(download(tensor), host.storage)      # same physical bytes as the oracle's layout
    back = torch.zeros((4, plane_bytes), dtype=torch.uint8).pin_memory()
    tokens = []
    for plane in range(4):
        q, staging = lanes[plane % 2]
        tokens.append((q, q.download(tensor.view().select(0, plane), back[plane].numpy(), staging.view())))
    for q, token in tokens:
        run(q, token)
    assert torch.equal(back, pinned)
    # rejections: wrong size, missing workspace
    assert queue.upload(tensor.view().select(0, 0), pinned[0].numpy()[:-2], lanes[0][1].view()) == -1
    assert queue.download(tensor.view().select(0, 0), back[0].numpy(), None) == -1
    second.close()
