"""GPU: failures injected on the HOST side of the submission path (an error code from
the launch wrapper, a completion event that cannot be recorded, a completion reported
failed) follow the contract's OID model: negative oid for a synchronous error,
retained failure rethrown by every wait for a post-acceptance one, and a queue that
keeps working afterwards. No device fault is provoked anywhere."""
import numpy as np
import pytest

from iom_b200.device import DeviceError, OID_DEVICE_ERROR
from iom_b200.tensor import DataType
from gpu_support import download, gpu, run, upload  # noqa: F401
from support import HostTensor, abi, oracle, random_payload

pytestmark = pytest.mark.gpu


def operands(device, rng):
    tensors = []
    for _ in range(3):
        t = HostTensor((33, 40), DataType.F32).poison()
        t.view().copy_from_host(random_payload(rng, (33, 40), DataType.F32))
        tensors.append(t)
    return tensors, [upload(device, t) for t in tensors]


def test_launch_failure_is_a_synchronous_device_error(gpu):
    device, queue = gpu
    (a, b, c), (da, db, dc) = operands(device, np.random.default_rng(1))
    queue.faults.arm("launch")
    assert queue.add(da.view(), db.view(), dc.view()) == OID_DEVICE_ERROR
    assert np.array_equal(download(dc), c.storage)            # nothing ran
    run(queue, queue.add(da.view(), db.view(), dc.view()))     # the queue keeps working
    assert oracle().iomo_binary(0, abi(a.view()), abi(b.view()), abi(c.view()), 0) == 0
    assert np.array_equal(download(dc), c.storage)
    # the third passage from now fails, the two before it do not
    queue.faults.arm("launch", skip=2)
    tokens = [queue.mul(da.view(), db.view(), dc.view()) for _ in range(4)]
    assert [t > 0 for t in tokens] == [True, True, False, True]
    queue.wait(tokens[3])


def test_unrecordable_event_falls_back_to_a_stream_drain(gpu):
    device, queue = gpu
    (a, b, c), (da, db, dc) = operands(device, np.random.default_rng(2))
    queue.faults.arm("record")
    token = queue.add(da.view(), db.view(), dc.view())
    assert token > 0
    queue.wait(token)                                          # proven by draining the stream
    assert oracle().iomo_binary(0, abi(a.view()), abi(b.view()), abi(c.view()), 0) == 0
    assert np.array_equal(download(dc), c.storage)


def test_failed_completion_is_retained_and_rethrown(gpu):
    device, queue = gpu
    (a, b, c), (da, db, dc) = operands(device, np.random.default_rng(3))
    queue.faults.arm("complete")
    failed = queue.add(da.view(), db.view(), dc.view())
    later = queue.mul(da.view(), db.view(), dc.view())
    assert failed > 0 and later > 0
    for _ in range(3):                                         # every wait rethrows it
        with pytest.raises(DeviceError):
            queue.wait(failed)
    queue.wait(later)                                          # later work is unaffected
    assert oracle().iomo_binary(1, abi(a.view()), abi(b.view()), abi(c.view()), 0) == 0
    assert np.array_equal(download(dc), c.storage)
