"""Bounded device waits, tested the permitted way: a wait on a flag that nothing ever sets runs out after its limit,
the kernel raises the error flag and returns, tensor memory is released, the context stays usable, and the host-side
check raises.  One GPU, one process; no kernel faults, traps or spins without a limit."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture
def short_waits():
    from miles_b200.ops import cuda as K

    err = K.C.error_flag(torch.empty(0, device="cuda"))
    err.zero_()
    K.C.fabric_configure(err, 200_000_000)        # 0.2 s
    yield err
    err.zero_()
    K.C.fabric_configure(err, 2_000_000_000)
    torch.cuda.synchronize()


def test_barrier_wait_runs_out_and_context_survives(short_waits):
    from miles_b200.ops import cuda as K

    err = short_waits
    # a two-rank flag table whose second row is local memory that no peer will ever write
    mine = torch.zeros(16 * 8, dtype=torch.int32, device="cuda")
    nobody = torch.zeros(16 * 8, dtype=torch.int32, device="cuda")
    ptrs = torch.tensor([mine.data_ptr(), nobody.data_ptr()], dtype=torch.int64)
    epochs = torch.zeros(16, dtype=torch.int32, device="cuda")
    channel = 3
    t0 = time.perf_counter()
    K.C.barrier(ptrs, 0, 2, channel, epochs, err)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert 0.15 < dt < 1.5, dt
    assert int(err.item()) == 100 + channel
    assert int(nobody[channel * 8 + 0].item()) == 1            # our epoch was published to the "peer"
    # the context is alive: an ordinary kernel still runs
    a = torch.randn(256, 256, device="cuda").bfloat16()
    assert torch.isfinite(K.gemm_nt(a, a).float()).all()
    # a poisoned process does not wait again (no second time-out), and dependent peer kernels return at once
    t0 = time.perf_counter()
    K.C.barrier(ptrs, 0, 2, channel, epochs, err)
    out = torch.full((64,), 7.0, device="cuda").bfloat16()
    K.C.sum_rows(torch.tensor([mine.data_ptr(), nobody.data_ptr()], dtype=torch.int64), 2, out)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.1
    assert torch.all(out.float() == 7.0)                        # skipped: nothing consumed, nothing written
    from miles_b200.parallel.fabric import Fabric

    fab = Fabric.__new__(Fabric)
    fab.err = err
    with pytest.raises(RuntimeError, match="error flag 103"):
        fab.check()


def test_ag_gemm_owner_flag_never_set(short_waits):
    from miles_b200.ops import cuda as K

    err = short_waits
    n, Kd, N = 128, 256, 256
    xg0 = torch.randn(2 * n, Kd, device="cuda").bfloat16()      # "rank 0" buffer (ours)
    xg1 = torch.randn(2 * n, Kd, device="cuda").bfloat16()      # stands in for a peer that never signals
    w = torch.randn(N, Kd, device="cuda").bfloat16()
    y = torch.zeros(2 * n, N, device="cuda").bfloat16()
    flags0 = torch.zeros(16 * 8, dtype=torch.int32, device="cuda")
    flags1 = torch.zeros(16 * 8, dtype=torch.int32, device="cuda")
    counters = torch.zeros(1024, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    K.C.ag_gemm(torch.tensor([xg0.data_ptr(), xg1.data_ptr()], dtype=torch.int64), w, y, counters, n, 0, 2,
                torch.tensor([flags0.data_ptr(), flags1.data_ptr()], dtype=torch.int64), 8, 1, err)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert dt < 6.0, dt
    assert int(err.item()) in (11, 17), int(err.item())
    # the rows this rank owns were still computed from local memory before the wait for the peer's block gave up
    want = xg0[:n].float() @ w.float().t()
    assert ((y[:n].float() - want).norm() / want.norm()).item() < 1e-2
    # tensor memory was released on the way out: a following tcgen05 GEMM gets its allocation and is correct
    err.zero_()
    a = torch.randn(512, 512, device="cuda").bfloat16()
    c = K.gemm_nt(a, a)
    torch.cuda.synchronize()
    ref = a.float() @ a.float().t()
    assert ((c.float() - ref).norm() / ref.norm()).item() < 1e-2
    assert int(err.item()) == 0
