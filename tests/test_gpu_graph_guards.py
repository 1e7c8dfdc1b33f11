"""Misuse of a recorded step is reported as an error code, never as a launch into freed memory or a hang:
  * a call made after the recording that makes the context reallocate one of its own buffers invalidates the
    recording (dgc_graph_launch returns DGC_ERR_INVALID, nothing is launched, a new recording works);
  * the gradient exchange is refused inside a recording when the context has a communicator."""
import numpy as np
import pytest
import torch

import dgen_b200

pytestmark = pytest.mark.gpu


def test_replay_after_a_context_buffer_grew_is_refused():
    ctx = dgen_b200.Context(0)
    stream = torch.cuda.Stream()
    x = torch.randn(4, 8192, device="cuda")
    y = torch.empty_like(x)
    big = torch.randn(64, 1 << 16, device="cuda")
    torch.cuda.synchronize()
    with ctx.on_stream(stream), torch.cuda.stream(stream):
        ctx.onepole_fwd(x, 0.9, out=y)                  # first run: the chunk-carry scratch is allocated here
        with ctx.record() as rec:
            ctx.onepole_fwd(x, 0.9, out=y)
        graph = rec.graph
        graph.launch()
        stream.synchronize()
        want = y.clone()
        before = ctx.launch_count()
        ctx.onepole_fwd(big, 0.9)                       # needs more scratch: the context reallocates it
        stream.synchronize()
        mid = ctx.launch_count()
        assert mid > before
        with pytest.raises(dgen_b200.DgenCudaError, match="record the step again"):
            graph.launch()
        assert ctx.launch_count() == mid                # nothing was launched by the refused replay
        graph.close()
        with ctx.record() as rec2:                      # the new recording sees the new buffer and replays fine
            ctx.onepole_fwd(x, 0.9, out=y)
        y.zero_()
        rec2.graph.launch()
        stream.synchronize()
        assert torch.equal(y, want)
        rec2.graph.close()
    ctx.close()


def test_gradient_exchange_is_refused_inside_a_recording():
    """One rank, a communicator of world size one: outside a recording the all-reduce runs (and is the identity);
    between dgc_graph_begin and dgc_graph_end it returns DGC_ERR_INVALID and the recording still ends cleanly."""
    ctx = dgen_b200.Context(0)
    try:
        uid = dgen_b200.comm_unique_id()
    except dgen_b200.DgenCudaError:
        ctx.close()
        pytest.skip("NCCL library not found")
    ctx.comm_init(1, 0, uid)
    stream = torch.cuda.Stream()
    g = torch.arange(1000, device="cuda", dtype=torch.float32)
    x = torch.randn(2, 4096, device="cuda")
    y = torch.empty_like(x)
    torch.cuda.synchronize()
    with ctx.on_stream(stream), torch.cuda.stream(stream):
        ctx.allreduce_sum_(g)
        ctx.onepole_fwd(x, 0.5, out=y)
        stream.synchronize()
        assert torch.equal(g, torch.arange(1000, device="cuda", dtype=torch.float32))
        with ctx.record() as rec:
            ctx.onepole_fwd(x, 0.5, out=y)
            with pytest.raises(dgen_b200.DgenCudaError, match="cannot be recorded"):
                ctx.allreduce_sum_(g)
        rec.graph.launch()
        stream.synchronize()
        rec.graph.close()
    ctx.lib.dgc_comm_destroy(ctx.h)
    ctx.close()


def test_expired_device_wait_and_sync_timeout_are_reported_and_the_context_survives():
    """The failure branches of the bounded waits, exercised without a fault and without an unbounded wait.
    (1) A kernel waits on a barrier that nothing arrives on, with the library's bounded wait cut down to 2000 polls:
    it gives up, writes the status word and returns; dgc_sync reports DGC_ERR_DEVICE (-5) once, then the word is
    clear.  (2) The stream is kept busy for 120 ms and dgc_sync is given 10 ms: DGC_ERR_TIMEOUT (-4); nothing
    is cancelled, the stream drains by itself and the next sync succeeds.  After both, ordinary work runs."""
    import time
    ctx = dgen_b200.Context(0)
    lib, h = ctx.lib, ctx.h
    assert lib.dgc_selftest_expired_wait(h, 0) == -1                 # argument range is checked
    assert lib.dgc_selftest_expired_wait(h, 2000) == 0
    rc = lib.dgc_sync(h, 2000)
    assert rc == -5 and b"status word = 201" in lib.dgc_last_error(h)
    assert lib.dgc_sync(h, 2000) == 0                                # reported once, then clear
    assert lib.dgc_selftest_busy(h, 120) == 0
    t0 = time.perf_counter()
    rc = lib.dgc_sync(h, 10)
    waited = time.perf_counter() - t0
    assert rc == -4 and b"still busy" in lib.dgc_last_error(h)
    assert waited < 0.1                                              # the call came back at its own limit
    assert lib.dgc_sync(h, 2000) == 0                                # the busy kernel ends by itself
    x = torch.randn(2, 4096, device="cuda")
    y = ctx.onepole_fwd(x, 0.5)
    ctx.sync()
    assert bool(torch.isfinite(y).all())
    ctx.close()
