"""Failure detection of the device-side collective without faulting anything: a peer that has joined the communicator
but never launches its half of an all-reduce. The launching rank's bounded poll (2 s) runs out, the kernel records
`MUI_DEV_TIMEOUT_PEER` with the late rank in the device status word and returns; the host reads it, and the context
keeps working. Both ranks are processes on GPU 0 (only one of them ever launches a kernel that waits)."""
import os
import time

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, key, q, done):
    try:
        torch.cuda.set_device(0)
        from muillm_b200 import capi, ops
        from muillm_b200.comm import MuiCommunicator

        comm = MuiCommunicator(rank=rank, world_size=2, key=key, capacity_elems=1 << 18, timeout_s=60.0)
        if rank == 0:
            x = torch.ones(8, device="cuda", dtype=torch.float32)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            comm.all_reduce_sum(x)
            torch.cuda.synchronize()
            waited = time.perf_counter() - t0
            status = capi.device_status(clear=True)
            # a large count (several elements per thread, 296 CTAs): the first wait that runs out makes every later
            # one give up at once, so the whole kernel still ends after about one wait limit
            big = torch.ones(200000, device="cuda", dtype=torch.float32)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            comm.all_reduce_sum(big)
            torch.cuda.synchronize()
            waited_big = time.perf_counter() - t0
            status_big = capi.device_status(clear=True)
            # the context is intact: another kernel of the library runs and is correct
            y = ops.muillm_rmsnorm_forward(torch.ones(16, device="cuda", dtype=torch.float16),
                                           torch.full((2, 16), 3.0, device="cuda", dtype=torch.float16), 0.0)
            torch.cuda.synchronize()
            q.put(("ok", status, waited, capi.device_status(), y.float().mean().item(), waited_big, status_big))
        done.wait(90)  # rank 1 keeps its segment mapped until rank 0 has finished
        comm.close()
    except Exception as e:  # pragma: no cover
        q.put(("error", repr(e)))


def test_all_reduce_reports_a_peer_that_never_arrives():
    ctx = mp.get_context("spawn")
    q, done = ctx.Queue(), ctx.Event()
    key = f"tmo{os.getpid()}"
    procs = [ctx.Process(target=_worker, args=(r, key, q, done)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        res = q.get(timeout=120)
    finally:
        done.set()
        for p in procs:
            p.join(timeout=60)
    assert res[0] == "ok", res
    _, status, waited, status_after, mean, waited_big, status_big = res
    assert status >> 24 == 3, f"expected MUI_DEV_TIMEOUT_PEER, got {status:#x}"
    assert status & 0xFFFFFF == 1, "the late rank is rank 1"
    assert 1.5 < waited < 10.0, f"the bounded wait took {waited:.2f} s"
    assert status_big >> 24 == 3 and 1.5 < waited_big < 10.0, f"large count: {waited_big:.2f} s, status {status_big:#x}"
    assert status_after == 0 and abs(mean - 1.0) < 1e-2
