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
