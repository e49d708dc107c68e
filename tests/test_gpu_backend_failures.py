"""Failure model, lifetimes and recording of the C++ B200 backend, through the shim.

Failures are injected on the host only (the backend's SubmissionFault table mirrors
src/cuda/copy.hpp:41-60): an error code substituted at a launch wrapper, an event record,
a stream drain, a status copy, a registration. No device is ever faulted. The lifetime
cases follow test/cuda/test_cuda_conformance.cpp:2198-2300 (operands destroyed before the
token is waited for) and test/backend/backend_conformance_memory.hpp:23-135 (queue cap,
mandatory staging workspace).
"""
import ctypes

import numpy as np
import pytest

from iom_b200.tensor import DataType
from support import REF_LIBS, Reference, random_payload

pytestmark = pytest.mark.gpu

NONE, LAUNCH, STATUS_COPY, EVENT_RECORD, STREAM_SYNC, REGISTRATION, OUTCOME = range(7)


@pytest.fixture()
def gpu():
    if not REF_LIBS["b200"].exists():
        pytest.skip("libiomref_b200.so is not built (make -C oracle b200)")
    ref = Reference("b200", accelerator=True, arena_bytes=3 << 30)
    yield ref
    ref.lib.iomref_inject_fault_b200(NONE)
    ref.close()


def filled(ref, shape, dtype, rng):
    payload = random_payload(rng, shape, dtype)
    tensor = ref.tensor(shape, dtype)
    tensor.view().from_host(payload)
    return tensor, payload


def add(ref, a, b, out):
    return ref.lib.iomref_binary(ref.queue, 0, a.view().handle, b.view().handle, out.view().handle)


def expect_sum(a_payload, b_payload, out):
    got = out.view().to_host().view(np.int32)
    assert np.array_equal(got, (a_payload.astype(np.int64) + b_payload).astype(np.int32).reshape(-1))


def test_launch_fault_is_a_retained_failure_and_leaves_the_queue_usable(gpu):
    rng = np.random.default_rng(1)
    a, pa = filled(gpu, (33, 70), DataType.I32, rng)
    b, pb = filled(gpu, (33, 70), DataType.I32, rng)
    out = gpu.tensor((33, 70), DataType.I32)
    before = out.read()
    gpu.lib.iomref_inject_fault_b200(LAUNCH)
    token = add(gpu, a, b, out)
    assert token > 0                                     # accepted: the failure is retained
    assert gpu.lib.iomref_wait(gpu.queue, token) == 5
    assert gpu.lib.iomref_wait(gpu.queue, token) == 5    # rethrown on every wait
    assert np.array_equal(out.read(), before)            # nothing was launched
    assert gpu.lib.iomref_quarantined_events_b200(gpu.queue) == 0
    token = add(gpu, a, b, out)
    assert token > 0 and gpu.run(token) == 0
    expect_sum(pa, pb, out)
    # nothing of the failed submission is still registered: the operands can go
    a.close()
    b.close()


def test_unproven_completion_fails_the_token_and_quarantines_the_event(gpu):
    rng = np.random.default_rng(2)
    a, pa = filled(gpu, (33, 70), DataType.I32, rng)
    b, pb = filled(gpu, (33, 70), DataType.I32, rng)
    out = gpu.tensor((33, 70), DataType.I32)
    assert gpu.lib.iomref_quarantined_events_b200(gpu.queue) == 0
    gpu.lib.iomref_inject_fault_b200(EVENT_RECORD)       # record x2 and the drain fail
    token = add(gpu, a, b, out)
    assert token > 0                                     # accepted: the kernel was launched
    assert gpu.lib.iomref_wait(gpu.queue, token) == 5    # retained failure
    assert gpu.lib.iomref_wait(gpu.queue, token) == 5    # rethrown on every wait
    assert gpu.lib.iomref_quarantined_events_b200(gpu.queue) == 1
    # later work is unaffected
    out2 = gpu.tensor((33, 70), DataType.I32)
    token = add(gpu, a, b, out2)
    assert token > 0 and gpu.run(token) == 0
    expect_sum(pa, pb, out2)
    # an owner of the unproven operation is parked, not recycled: a new tensor of the
    # same size never receives its address
    first = gpu.lib.iomref_tensor_storage(out.handle)
    out.close()
    again = gpu.tensor((33, 70), DataType.I32)
    assert gpu.lib.iomref_tensor_storage(again.handle) != first


def test_event_record_failure_alone_is_proven_by_a_drain(gpu):
    """One failing record is retried; with both records failing but the drain working the
    operation still completes successfully (the second proof)."""
    rng = np.random.default_rng(3)
    a, pa = filled(gpu, (16, 16), DataType.I32, rng)
    b, pb = filled(gpu, (16, 16), DataType.I32, rng)
    out = gpu.tensor((16, 16), DataType.I32)
    gpu.lib.iomref_inject_fault_b200(EVENT_RECORD)
    # consume the drain failure with a host transfer, which reports it and does no harm
    with pytest.raises(AssertionError):
        a.view().from_host(pa)
    token = add(gpu, a, b, out)
    assert token > 0 and gpu.run(token) == 0
    assert gpu.lib.iomref_quarantined_events_b200(gpu.queue) == 0
    expect_sum(pa, pb, out)


def test_stream_synchronize_fault_fails_the_host_transfer_only(gpu):
    rng = np.random.default_rng(4)
    a, pa = filled(gpu, (20, 35), DataType.I32, rng)
    gpu.lib.iomref_inject_fault_b200(STREAM_SYNC)
    data = np.ascontiguousarray(pa).view(np.uint8).reshape(-1)
    assert gpu.lib.iomref_view_from_host(a.view().handle, data.ctypes.data, data.size) == 5
    assert gpu.lib.iomref_view_from_host(a.view().handle, data.ctypes.data, data.size) == 0
    assert np.array_equal(a.view().to_host(), data)


@pytest.mark.parametrize("fault", [REGISTRATION, OUTCOME])
def test_registration_faults_refuse_before_acceptance(gpu, fault):
    rng = np.random.default_rng(5)
    a, pa = filled(gpu, (16, 16), DataType.I32, rng)
    b, pb = filled(gpu, (16, 16), DataType.I32, rng)
    out = gpu.tensor((16, 16), DataType.I32)
    gpu.lib.iomref_inject_fault_b200(fault)
    assert add(gpu, a, b, out) == -4                     # ResourceExhausted
    gpu.lib.iomref_inject_fault_b200(fault)
    x, _ = filled(gpu, (16, 64), DataType.BF16, rng)
    w, _ = filled(gpu, (1, 64), DataType.BF16, rng)
    s = gpu.tensor((16, 64), DataType.BF16)
    n = gpu.tensor((16, 64), DataType.BF16)
    assert gpu.lib.iomref_add_rmsnorm(gpu.queue, x.view().handle, x.view().handle, w.view().handle,
                                      s.view().handle, n.view().handle, ctypes.c_float(1e-5)) == -4
    token = add(gpu, a, b, out)
    assert token > 0 and gpu.run(token) == 0
    expect_sum(pa, pb, out)


def test_embedding_status_copy_fault(gpu):
    rng = np.random.default_rng(6)
    table, _ = filled(gpu, (50, 40), DataType.BF16, rng)
    ids = gpu.tensor((1, 19), DataType.U32)
    ids.view().from_host(rng.integers(0, 50, size=(1, 19)).astype(np.uint32))
    out = gpu.tensor((19, 40), DataType.BF16)
    gpu.lib.iomref_inject_fault_b200(STATUS_COPY)
    token = gpu.lib.iomref_embedding(gpu.queue, table.view().handle, ids.view().handle,
                                     out.view().handle)
    assert token > 0 and gpu.lib.iomref_wait(gpu.queue, token) == 5      # retained
    token = gpu.lib.iomref_embedding(gpu.queue, table.view().handle, ids.view().handle,
                                     out.view().handle)
    assert token > 0 and gpu.run(token) == 0


def test_operands_destroyed_before_wait(gpu):
    """128 MiB operands (F32 [8192,4096]) are destroyed right after submission: the result
    is complete and correct, and storage is not handed out again while it is in use."""
    rng = np.random.default_rng(7)
    shape = (8192, 4096)
    payload_a = rng.integers(-1000, 1000, size=shape, dtype=np.int32)
    payload_b = rng.integers(-1000, 1000, size=shape, dtype=np.int32)
    a = gpu.tensor(shape, DataType.I32)
    b = gpu.tensor(shape, DataType.I32)
    a.view().from_host(payload_a)
    b.view().from_host(payload_b)
    out = gpu.tensor(shape, DataType.I32)
    token = add(gpu, a, b, out)
    assert token > 0
    a.close()
    b.close()
    # allocations made while the operation may still run must not disturb it
    scribble = gpu.tensor(shape, DataType.I32)
    scribble.view().from_host(np.full(shape, 0x5A5A5A5A, dtype=np.uint32))
    assert gpu.run(token) == 0
    expect_sum(payload_a, payload_b, out)


def test_extension_operands_are_registered_until_completion(gpu):
    """The fused ADD + RMSNorm entry registers its five owners like a facade operation:
    x and the residual can be destroyed before the wait."""
    rng = np.random.default_rng(8)
    shape = (4096, 2048)
    x, px = filled(gpu, shape, DataType.BF16, rng)
    r, pr = filled(gpu, shape, DataType.BF16, rng)
    w, _ = filled(gpu, (1, 2048), DataType.BF16, rng)
    s = gpu.tensor(shape, DataType.BF16)
    n = gpu.tensor(shape, DataType.BF16)
    token = gpu.lib.iomref_add_rmsnorm(gpu.queue, x.view().handle, r.view().handle, w.view().handle,
                                       s.view().handle, n.view().handle, ctypes.c_float(1e-5))
    assert token > 0
    x.close()
    r.close()
    scribble = gpu.tensor(shape, DataType.BF16)
    scribble.view().from_host(np.full(shape, 0x7FC0, dtype=np.uint16))
    assert gpu.run(token) == 0
    # the stored sum against a second, undisturbed evaluation
    x2 = gpu.tensor(shape, DataType.BF16)
    r2 = gpu.tensor(shape, DataType.BF16)
    x2.view().from_host(px)
    r2.view().from_host(pr)
    s2 = gpu.tensor(shape, DataType.BF16)
    n2 = gpu.tensor(shape, DataType.BF16)
    token = gpu.lib.iomref_add_rmsnorm(gpu.queue, x2.view().handle, r2.view().handle, w.view().handle,
                                       s2.view().handle, n2.view().handle, ctypes.c_float(1e-5))
    assert token > 0 and gpu.run(token) == 0
    assert np.array_equal(s.read(), s2.read())
    assert np.array_equal(n.read(), n2.read())


def test_queue_cap_and_staging_workspace(gpu):
    queues = [gpu.lib.iomref_queue_create(gpu.device) for _ in range(3)]
    assert all(queues)                                   # four live queues with the fixture's
    assert not gpu.lib.iomref_queue_create(gpu.device)   # the fifth is refused
    for queue in queues:
        gpu.lib.iomref_queue_destroy(queue)
    again = gpu.lib.iomref_queue_create(gpu.device)
    assert again
    gpu.lib.iomref_queue_destroy(again)


def test_recorded_sequence_replays_with_new_inputs(gpu):
    """A decode-shaped sequence (embedding, norm, residual add + norm, gate, add) recorded
    once and replayed: the results equal the same operations issued one by one, for ids and
    activations that change between replays; an invalid id fails the replay's token."""
    rng = np.random.default_rng(9)
    hidden, batch, vocab = 256, 32, 100
    table, _ = filled(gpu, (vocab, hidden), DataType.BF16, rng)
    ids = gpu.tensor((1, batch), DataType.U32)
    w, _ = filled(gpu, (1, hidden), DataType.BF16, rng)
    attn, _ = filled(gpu, (batch, hidden), DataType.BF16, rng)
    h = gpu.tensor((batch, hidden), DataType.BF16)
    normed = gpu.tensor((batch, hidden), DataType.BF16)
    total = gpu.tensor((batch, hidden), DataType.BF16)
    gated = gpu.tensor((batch, hidden), DataType.BF16)
    final = gpu.tensor((batch, hidden), DataType.BF16)
    eps = ctypes.c_float(1e-5)

    def sequence():
        tokens = [
            gpu.lib.iomref_embedding(gpu.queue, table.view().handle, ids.view().handle, h.view().handle),
            gpu.lib.iomref_rmsnorm(gpu.queue, h.view().handle, w.view().handle, normed.view().handle, eps),
            gpu.lib.iomref_add_rmsnorm(gpu.queue, h.view().handle, attn.view().handle, w.view().handle,
                                       total.view().handle, normed.view().handle, eps),
            gpu.lib.iomref_silu_mul(gpu.queue, normed.view().handle, attn.view().handle, None,
                                    gated.view().handle),
            gpu.lib.iomref_binary(gpu.queue, 0, total.view().handle, gated.view().handle,
                                  final.view().handle),
        ]
        assert all(token > 0 for token in tokens), tokens
        return tokens[-1]

    def set_ids(values):
        ids.view().from_host(np.asarray(values, dtype=np.uint32).reshape(1, batch))

    set_ids(rng.integers(0, vocab, size=batch))
    assert gpu.run(sequence()) == 0                      # once eagerly (one-time set-up)
    assert gpu.lib.iomref_capture_begin_b200(gpu.queue) == 0
    sequence()
    recording = gpu.lib.iomref_capture_end_b200(gpu.queue)
    assert recording, gpu.error()
    for _ in range(3):
        set_ids(rng.integers(0, vocab, size=batch))
        attn.view().from_host(random_payload(rng, (batch, hidden), DataType.BF16))
        token = gpu.lib.iomref_replay_b200(gpu.queue, recording)
        assert token > 0 and gpu.run(token) == 0
        replayed = [t.read() for t in (h, normed, total, gated, final)]
        assert gpu.run(sequence()) == 0
        for got, tensor in zip(replayed, (h, normed, total, gated, final)):
            assert np.array_equal(got, tensor.read())
    bad = rng.integers(0, vocab, size=batch)
    bad[5] = vocab
    set_ids(bad)
    token = gpu.lib.iomref_replay_b200(gpu.queue, recording)
    assert token > 0 and gpu.lib.iomref_wait(gpu.queue, token) == 1     # invalid_argument
    gpu.lib.iomref_recording_destroy_b200(recording)
