"""GPU: a decode-shaped run of operations recorded into one CUDA graph and replayed
must produce exactly what the same operations produce when issued one by one, for
every replay, with inputs that change between replays."""
import numpy as np
import pytest
import torch

from iom_b200.device import OID_CAPTURED
from iom_b200.tensor import DataType
from gpu_support import download, gpu, run, upload  # noqa: F401
from support import HostTensor, random_payload

pytestmark = pytest.mark.gpu


def device_tensor(device, shape, dtype, rng, kind="normal"):
    host = HostTensor(shape, dtype).poison()
    host.view().copy_from_host(random_payload(rng, shape, dtype, kind))
    return upload(device, host)


def decode_step(queue, t, workspace, positions, status):
    """embedding -> rmsnorm -> K append at per-sequence positions -> gate -> residual add + norm."""
    tokens = [
        queue.embedding(t["table"].view(), t["ids"].view(), t["hidden"].view(), workspace.view()),
        queue.rmsnorm(t["hidden"].view(), t["w"].view(), t["normed"].view(), 1e-5),
        queue.cache_append_batched(t["k"].view(), t["cache"].view(), positions.data_ptr(),
                                   status.data_ptr()),
        queue.silu_mul(t["gate"].view(), t["up"].view(), t["prod"].view()),
        queue.add_rmsnorm(t["hidden"].view(), t["normed"].view(), t["w"].view(), t["sum"].view(),
                          t["out"].view(), 1e-5),
    ]
    return tokens


def make_state(device, rng):
    batch, hidden, inter = 8, 256, 704
    t = {
        "table": device_tensor(device, (500, hidden), DataType.BF16, rng),
        "hidden": device_tensor(device, (batch, hidden), DataType.BF16, rng),
        "normed": device_tensor(device, (batch, hidden), DataType.BF16, rng),
        "sum": device_tensor(device, (batch, hidden), DataType.BF16, rng),
        "out": device_tensor(device, (batch, hidden), DataType.BF16, rng),
        "w": device_tensor(device, (1, hidden), DataType.BF16, rng),
        "gate": device_tensor(device, (batch, inter), DataType.BF16, rng),
        "up": device_tensor(device, (batch, inter), DataType.BF16, rng),
        "prod": device_tensor(device, (batch, inter), DataType.BF16, rng),
        "k": device_tensor(device, (batch, 4, 1, 64), DataType.BF16, rng),
        "cache": device_tensor(device, (batch, 4, 128, 64), DataType.BF16, rng),
    }
    ids = HostTensor((1, batch), DataType.U32).poison(0)
    ids.view().copy_from_host(rng.integers(0, 500, size=(1, batch)).astype(np.uint32))
    t["ids"] = upload(device, ids)
    return t, batch


def snapshot(t):
    return {name: download(t[name]).copy() for name in ("hidden", "normed", "sum", "out", "prod", "cache")}


def test_captured_decode_step_equals_eager(gpu):
    device, queue = gpu
    rng = np.random.default_rng(77)
    eager, batch = make_state(device, np.random.default_rng(5))
    graph, _ = make_state(device, np.random.default_rng(5))
    workspace_e, workspace_g = device.create_workspace(32), device.create_workspace(32)
    positions = torch.zeros(batch, dtype=torch.int32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")

    # one eager run first (one-time set-up such as the SiLU table), on the eager state
    for token in decode_step(queue, eager, workspace_e, positions, status):
        run(queue, token)
    with queue.capture() as step:
        tokens = decode_step(queue, graph, workspace_g, positions, status)
    assert tokens == [OID_CAPTURED] * 5 and step.operations == 5
    with pytest.raises(ValueError):
        queue.wait(OID_CAPTURED)
    # capture itself ran nothing: the recorded state still holds its initial bytes
    fresh, _ = make_state(device, np.random.default_rng(5))
    assert np.array_equal(download(graph["out"]), download(fresh["out"]))
    run(queue, step.replay())               # replay 0 catches up with the eager warm-up run
    for name, value in snapshot(eager).items():
        assert np.array_equal(value, snapshot(graph)[name]), name

    for replay in range(3):
        new_ids = rng.integers(0, 500, size=(1, batch)).astype(np.uint32)
        new_gate = random_payload(rng, (batch, 704), DataType.BF16, "normal")
        host_ids = HostTensor((1, batch), DataType.U32).poison(0)
        host_ids.view().copy_from_host(new_ids)
        host_gate = HostTensor((batch, 704), DataType.BF16).poison()
        host_gate.view().copy_from_host(new_gate)
        for state in (eager, graph):
            state["ids"].storage().copy_(torch.from_numpy(host_ids.storage.copy()))
            state["gate"].storage().copy_(torch.from_numpy(host_gate.storage.copy()))
        positions.copy_(torch.from_numpy(rng.integers(0, 127, size=batch).astype(np.int32)))
        torch.cuda.synchronize()
        for token in decode_step(queue, eager, workspace_e, positions, status):
            run(queue, token)
        run(queue, step.replay())
        want, got = snapshot(eager), snapshot(graph)
        for name in want:
            assert np.array_equal(want[name], got[name]), (replay, name)


def test_captured_failure_surfaces_at_the_replay(gpu):
    """An out-of-range id inside a replayed sequence is reported by the replay's token,
    as the eager embedding reports it."""
    device, queue = gpu
    rng = np.random.default_rng(3)
    table = device_tensor(device, (50, 64), DataType.BF16, rng)
    out = device_tensor(device, (4, 64), DataType.BF16, rng)
    ids = HostTensor((1, 4), DataType.U32).poison(0)
    ids.view().copy_from_host(np.array([[1, 2, 3, 4]], dtype=np.uint32))
    dids = upload(device, ids)
    workspace = device.create_workspace(32)
    run(queue, queue.embedding(table.view(), dids.view(), out.view(), workspace.view()))
    with queue.capture() as step:
        assert queue.embedding(table.view(), dids.view(), out.view(), workspace.view()) == OID_CAPTURED
    run(queue, step.replay())
    ids.view().copy_from_host(np.array([[1, 2, 50, 4]], dtype=np.uint32))
    dids.storage().copy_(torch.from_numpy(ids.storage.copy()))
    torch.cuda.synchronize()
    token = step.replay()
    assert token > 0
    with pytest.raises(ValueError):
        queue.wait(token)
    # a rejected operation inside the block fails the capture as a whole
    with pytest.raises(ValueError):
        with queue.capture():
            assert queue.add(table.view(), out.view(), out.view()) == -1
