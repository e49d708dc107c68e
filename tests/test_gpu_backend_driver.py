"""The C driver interface of the C++ backend (include/iom_b200_backend_c.h) and its program
runner, through iom_b200/backend_driver.py: what bench.py measures with.

A program of facade operations issued from C++ must give the oracle's bytes in every mode
(eager, waited one by one, recorded once and replayed); the runner must stay within the
queue's credits; host transfers in the two directions may run from two host threads at once.
"""
import threading

import numpy as np
import pytest
import torch

from iom_b200 import backend_driver as bd
from iom_b200.tensor import DataType
from support import HostTensor, abi, oracle, random_payload

pytestmark = pytest.mark.gpu


@pytest.fixture()
def backend():
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    if not bd.available():
        pytest.skip("libiom_b200_backend.so is not built (python -m iom_b200.build --backend=<checkout>)")
    instance = bd.Backend(0, 1 << 30, max_in_flight=4)
    yield instance
    instance.close()


def pinned_bytes(array: np.ndarray) -> torch.Tensor:
    host = torch.empty(array.nbytes, dtype=torch.uint8, pin_memory=True)
    host.copy_(torch.from_numpy(array.view(np.uint8).reshape(-1).copy()))
    return host


def oracle_step(shape, x, r, w, eps):
    hx, hr, hs, ho = (HostTensor(shape, DataType.BF16) for _ in range(4))
    hw = HostTensor((1, shape[-1]), DataType.BF16)
    hx.view().copy_from_host(x)
    hr.view().copy_from_host(r)
    hw.view().copy_from_host(w)
    assert oracle().iomo_binary(0, abi(hx.view()), abi(hr.view()), abi(hs.view()), 0) == 0
    assert oracle().iomo_rmsnorm(abi(hs.view()), abi(hw.view()), abi(ho.view()), eps, 0) == 0
    return (hs.view().copy_to_host().view(np.uint16).reshape(shape),
            ho.view().copy_to_host().view(np.uint16).reshape(shape))


@pytest.mark.parametrize("shape", [(48, 2048), (40, 8192), (3, 20, 2064)])
@pytest.mark.parametrize("mode", [bd.EAGER, bd.WAIT_EACH, bd.RECORDED])
def test_a_program_gives_the_oracles_bytes_in_every_mode(backend, shape, mode):
    rng = np.random.default_rng(hash((shape, mode)) & 0xFFFF)
    eps = 1e-6
    x = random_payload(rng, shape, DataType.BF16, "normal")
    r = random_payload(rng, shape, DataType.BF16, "normal")
    w = random_payload(rng, (1, shape[-1]), DataType.BF16, "normal")
    want_sum, want_out = oracle_step(shape, x, r, w, eps)
    tx, tr, ts, to = (backend.tensor(shape, DataType.BF16) for _ in range(4))
    tw = backend.tensor((1, shape[-1]), DataType.BF16)
    vx, vr, vs, vo, vw = (backend.view(t) for t in (tx, tr, ts, to, tw))
    nbytes = x.nbytes
    staging = backend.workspace(nbytes + 64)
    hx, hr, hw = pinned_bytes(x), pinned_bytes(r), pinned_bytes(w)
    got_sum = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    got_out = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    op = bd.Backend.op
    upload = [op(bd.FROM_HOST, [vx], workspace=staging, host=hx.data_ptr(), host_bytes=nbytes),
              op(bd.FROM_HOST, [vr], workspace=staging, host=hr.data_ptr(), host_bytes=nbytes),
              op(bd.FROM_HOST, [vw], workspace=staging, host=hw.data_ptr(), host_bytes=w.nbytes)]
    compute = [op(bd.ADD, [vx, vr, vs]), op(bd.RMSNORM, [vs, vw, vo], eps=eps)]
    download = [op(bd.TO_HOST, [vs], workspace=staging, host=got_sum.data_ptr(), host_bytes=nbytes),
                op(bd.TO_HOST, [vo], workspace=staging, host=got_out.data_ptr(), host_bytes=nbytes)]
    backend.run(upload)
    timing = backend.run(compute if mode == bd.RECORDED else compute + [op(bd.WAIT)], passes=3, mode=mode)
    assert timing.operations == (3 if mode == bd.RECORDED else 6)
    backend.run(download)
    assert np.array_equal(got_sum.numpy().view(np.uint16).reshape(shape), want_sum)
    assert np.array_equal(got_out.numpy().view(np.uint16).reshape(shape), want_out)
    # the fused extension gives the same bytes
    ts2, to2 = backend.tensor(shape, DataType.BF16), backend.tensor(shape, DataType.BF16)
    vs2, vo2 = backend.view(ts2), backend.view(to2)
    backend.run([op(bd.ADD_RMSNORM, [vx, vr, vw, vs2, vo2], eps=eps), op(bd.WAIT)], mode=bd.EAGER)
    assert torch.equal(backend.storage(ts2), backend.storage(ts))
    assert torch.equal(backend.storage(to2), backend.storage(to))


def test_the_runner_stays_within_the_queues_credits(backend):
    """200 submissions on a queue of four credits: none is parked past the closing event, so
    the device time covers every launch (each reads the previous result: out = out * 2)."""
    shape = (16, 2048)
    ta, tb = backend.tensor(shape, DataType.F32), backend.tensor((1, 1), DataType.F32)
    backend.storage(ta).view(torch.float32).fill_(1.0)
    backend.storage(tb).view(torch.float32).fill_(2.0)       # [1,1]: slot 0 holds the value
    torch.cuda.synchronize()
    va, vb = backend.view(ta), backend.view(tb)
    timing = backend.run([bd.Backend.op(bd.MUL, [va, vb, va])], passes=100)
    assert timing.operations == 100
    assert float(backend.storage(ta).view(torch.float32)[0]) == float(2.0 ** 100)
    assert timing.device_ms > 0.0


def test_uploads_and_downloads_from_two_threads(backend):
    """Device-to-host transfers have a stream and a lock of their own: a thread that reads one
    tensor back while another uploads a different tensor sees exactly what was stored."""
    shape = (2048, 2048)
    rng = np.random.default_rng(5)
    first = random_payload(rng, shape, DataType.BF16, "normal")
    second = random_payload(rng, shape, DataType.BF16, "normal")
    t_up, t_down = backend.tensor(shape, DataType.BF16), backend.tensor(shape, DataType.BF16)
    v_up, v_down = backend.view(t_up), backend.view(t_down)
    nbytes = first.nbytes
    stage_up, stage_down = backend.workspace(nbytes + 64), backend.workspace(nbytes + 64)
    h_first, h_second = pinned_bytes(first), pinned_bytes(second)
    back = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    op = bd.Backend.op
    backend.run([op(bd.FROM_HOST, [v_down], workspace=stage_down, host=h_first.data_ptr(), host_bytes=nbytes)])
    failures = []

    def uploader():
        try:
            for _ in range(8):
                backend.run([op(bd.FROM_HOST, [v_up], workspace=stage_up, host=h_second.data_ptr(),
                                host_bytes=nbytes)])
        except Exception as error:      # noqa: BLE001
            failures.append(error)

    def downloader():
        try:
            for _ in range(8):
                back.zero_()
                backend.run([op(bd.TO_HOST, [v_down], workspace=stage_down, host=back.data_ptr(),
                                host_bytes=nbytes)])
                if not np.array_equal(back.numpy().view(np.uint16).reshape(shape), first):
                    failures.append(AssertionError("a download returned other bytes"))
        except Exception as error:      # noqa: BLE001
            failures.append(error)

    threads = [threading.Thread(target=uploader), threading.Thread(target=downloader)]
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()
    assert not failures, failures[0]
    backend.run([op(bd.TO_HOST, [v_up], workspace=stage_up, host=back.data_ptr(), host_bytes=nbytes)])
    assert np.array_equal(back.numpy().view(np.uint16).reshape(shape), second)
