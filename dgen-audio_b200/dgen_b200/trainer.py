"""One training step of the batched harmonic+noise model, HarmonicE2E style
(Examples/HarmonicE2E/Trainer.swift:247-487: forward -> multi-scale spectral loss -> backward ->
optimizer.step), with every tensor resident in HBM and every operation a libdgen_cuda kernel.

Graph (rows of all [F*B, *] matrices are ordered [control frame][voice], the layout of the control tables):
    h = tanh(tanh(tanh(X W1 + b1) W2 + b2) W3 + b3);  z = h Wh + bh                     (Model.swift:96-101)
    amps = softplus(z[:, :K]) / (sum + 1e-6)                                             (Model.swift:102-106)
    bands = sigmoid(z[:, K:])   (this configuration's own band head; the reference decoder has gain, noise-gain and
                                 tap heads instead, Model.swift:107-113)
    taps = bands Wfs^T;  dry = harmonic(f0, amps, gain, uv) + fir(noise, taps, noise_gain)  (Synth.swift:47-102)
    out  = dry + partitioned_convolve(dry, ir)                                           (learnable 1 s IR)
    loss = multi-scale spectral L1 (lin + log) of out against the target                 (Trainer.swift:538-588)
Parameters and Adam state live in ONE flat device buffer; with several ranks the flat gradient is
summed over ranks (NCCL all-reduce over NVLink) before the Adam step, and each rank's loss gradient is
pre-scaled by local_voices / global_voices so that the sum is the gradient of the global-batch mean.
"""
import ctypes as C

import numpy as np

from . import (Context, HnTrainConfig, HnTrainLayout, PLAN_ADAM, PLAN_ALLREDUCE, PLAN_MSS_LOSS_BWD, PHASE_SCAN, Plan,
               PlanStep, mss_params, sharding)


class HarmonicModel:
    """The training step as ONE block plan in the library (dgc_hn_train_plan / dgc_plan_run): this class owns the
    arena (one device buffer that holds parameters, Adam state, inputs, activations and outputs at the offsets the
    library chose), exposes views into it, and decides when the plan's three parts run -- forward + backward, the
    gradient exchange, the update.  No kernel is launched from Python."""

    INPUTS = ("x", "f0", "uv", "gain", "noise_gain", "noise", "w_fs", "target")

    def __init__(self, ctx: Context, B, T, K=100, F=1000, sr=16000.0, nbands=65, taps=257, hidden=512, in_features=2,
                 ir_len=16000, conv_n=2048, conv_hop=1024, sizes=(2048, 1024, 512, 256, 128, 64), seed=0,
                 phase_mode=PHASE_SCAN, global_voices=None, counted_adam=False, n_trunk=3, lr=1e-3):
        import torch
        self.torch, self.ctx = torch, ctx
        self.B, self.T, self.K, self.F, self.sr = B, T, K, F, sr
        self.nbands, self.taps, self.hidden, self.in_features = nbands, taps, hidden, in_features
        self.ir_len, self.conv_n, self.conv_hop, self.sizes = ir_len, conv_n, conv_hop, tuple(sizes)
        self.phase_mode = phase_mode
        self.global_voices = global_voices or B
        self.M = F * B
        cfg = HnTrainConfig(B, T, K, F, sr, nbands, taps, in_features, hidden, n_trunk, ir_len, conv_n, conv_hop,
                            mss_params(B, T, self.sizes), phase_mode, self.global_voices, lr, 0.9, 0.999, 1e-8)
        lay = HnTrainLayout()
        ctx.check(ctx.lib.dgc_hn_train_plan(C.byref(cfg), C.byref(lay), None, 0))
        self.steps = (PlanStep * lay.n_steps)()
        ctx.check(ctx.lib.dgc_hn_train_plan(C.byref(cfg), C.byref(lay), self.steps, lay.n_steps))
        self.lay, self.cfg = lay, cfg
        self.plan = Plan(self.steps, lay.n_steps, None, None, 0)
        ops = [self.steps[i].op for i in range(lay.n_steps)]
        self.i_backward = ops.index(PLAN_MSS_LOSS_BWD)            # [0, i_backward) is the forward
        self.i_exchange, self.i_update = ops.index(PLAN_ALLREDUCE), ops.index(PLAN_ADAM)
        assert self.i_exchange == lay.n_forward_backward and self.i_update == self.i_exchange + 1
        dev = "cuda:%d" % ctx.device
        self.arena_t = torch.zeros(int(lay.total_floats), dtype=torch.float32, device=dev)
        h = C.c_void_p()
        ctx.check(ctx.lib.dgc_arena_wrap(ctx.h, self.arena_t.data_ptr(), int(lay.total_floats), C.byref(h)))
        self.arena = h
        dims = [(in_features, hidden)] + [(hidden, hidden)] * (n_trunk - 1) + [(hidden, K + nbands)]
        self.layout, off = [], 0
        for i, (a, b) in enumerate(dims):
            self.layout.append(("W%d" % i, off, (a, b)))
            off += a * b
            self.layout.append(("b%d" % i, off, (b,)))
            off += b
        self.layout.append(("ir", off, (ir_len,)))
        off += ir_len
        assert off == lay.n_params
        self.n_params = off
        view = lambda o, n: self.arena_t[int(o):int(o) + int(n)]
        self.params, self.grads = view(lay.params, off), view(lay.grads, off)
        self.m, self.v = view(lay.adam_m, off), view(lay.adam_v, off)
        self.t_dev = view(lay.adam_t, 1).view(torch.int32)
        self.corr = view(lay.adam_corr, 2)
        self.loss = view(lay.loss, 2).view(torch.float64)
        self.out = view(lay.audio, B * T).view(B, T)
        shapes = dict(x=(self.M, in_features), f0=(F, B), uv=(F, B), gain=(F, B), noise_gain=(F, B), noise=(B, T),
                      w_fs=(taps, nbands), target=(B, T))
        self.inputs = {k: view(getattr(lay, k), int(np.prod(shapes[k]))).view(*shapes[k]) for k in self.INPUTS}
        rng = np.random.default_rng(seed)
        flat = np.zeros(off, np.float32)
        for name, o, shape in self.layout:
            n = int(np.prod(shape))
            if name.startswith("W"):
                flat[o:o + n] = (rng.standard_normal(n) / np.sqrt(shape[0])).astype(np.float32)
            elif name == "ir":
                t = np.arange(ir_len) / sr
                flat[o:o + n] = (0.05 * rng.standard_normal(n) * np.exp(-6.91 * t / 0.4)).astype(np.float32)
        self.params.copy_(torch.from_numpy(flat).to(dev))
        self.step_index = 0
        # step index in device memory: a recorded step advances it on every replay
        self.counted_adam = counted_adam
        self.graph, self.graph_stream = None, None   # list of recordings (see capture)
        self.static_args = None
        self.exchange_events = None   # a list: replay() appends a CUDA event pair around every gradient exchange
        # the per-(F, T) clock tables are built on first use by a kernel on the then-current stream: build them
        # now, so that the two concurrent branches of the first step both find them complete
        ctx.check(ctx.lib.dgc_ctx_prepare_tables(ctx.h, F, T))

    def close(self):
        for g in self.graph or []:
            g.close()
        self.graph = None
        if self.arena:
            self.ctx.lib.dgc_arena_destroy(self.arena)
            self.arena = None

    def view(self, name, buf=None):
        buf = self.params if buf is None else buf
        for n, o, shape in self.layout:
            if n == name:
                return buf[o:o + int(np.prod(shape))].view(*shape)
        raise KeyError(name)

    def input_views(self):
        """The step's input buffers inside the arena, in the order step() takes them: fill them in place."""
        return [self.inputs[k] for k in self.INPUTS]

    # ------------------------------------------------------------------------------------------
    def _load(self, args):
        """Inputs given as other tensors are copied into their arena slots (device to device)."""
        for k, a in zip(self.INPUTS, args):
            v = self.inputs[k]
            if a.data_ptr() != v.data_ptr():
                v.copy_(a.reshape(v.shape))

    def _run(self, first, count):
        self.ctx.check(self.ctx.lib.dgc_plan_run(self.ctx.h, self.arena, C.byref(self.plan), first, count))

    def forward(self, X, f0, uv, gain, noise_gain, noise, w_fs, target):
        self._load((X, f0, uv, gain, noise_gain, noise, w_fs, target))
        self._run(0, self.i_backward)
        return self.loss

    def backward(self, X, f0, uv, gain, noise_gain, noise, w_fs, target):
        self._run(self.i_backward, self.i_exchange - self.i_backward)
        return self.grads

    def snapshots(self):
        """Named parameter tensors for runfiles.write_model_state: the reference's checkpoint container and its names
        for the trunk and the harmonic head (Examples/HarmonicE2E/Model.swift:122-137); the band head and the impulse
        response are this model's own (W_bands / b_bands, ir)."""
        from . import runfiles
        return runfiles.snapshots_from_flat(self.layout, self.params.cpu().numpy(), self.K)

    def load_snapshots(self, named):
        """Inverse: `named` as runfiles.read_model_state returns it.  Adam moments and the step index are reset."""
        from . import runfiles
        flat = runfiles.flat_from_snapshots(self.layout, named, self.K)
        self.params.copy_(self.torch.from_numpy(flat).to(self.params.device))
        self.m.zero_()
        self.v.zero_()
        self.step_index = 0
        self.t_dev.zero_()

    def _exchange(self):
        if getattr(self, "use_ctx_comm", False):
            self._run(self.i_exchange, 1)         # NCCL communicator owned by the context (the plan's ALLREDUCE step)
        else:
            sharding.allreduce_sum_(self.grads)   # torch.distributed process group

    def _exchanges(self):
        """True when the gradient sum really crosses ranks."""
        if getattr(self, "use_ctx_comm", False):
            return True
        return sharding.world_size() > 1

    def _update(self, lr):
        if self.counted_adam:
            self.steps[self.i_update].f[0] = lr
            self._run(self.i_update, 1)
        else:
            self.ctx.adam_step(self.params, self.grads, self.m, self.v, self.step_index, lr=lr)

    def step(self, X, f0, uv, gain, noise_gain, noise, w_fs, target, lr=1e-3):
        """forward + backward + gradient all-reduce + Adam; returns the device loss tensor (local mean)."""
        self.forward(X, f0, uv, gain, noise_gain, noise, w_fs, target)
        self.backward(X, f0, uv, gain, noise_gain, noise, w_fs, target)
        self._exchange()
        self.step_index += 1
        self._update(lr)
        return self.loss

    def capture(self, X, f0, uv, gain, noise_gain, noise, w_fs, target, lr=1e-3):
        """Record one whole training step (both streams, Adam).  The step's inputs live in the arena
        (input_views()); tensors given here that are not those views are remembered and copied into them at the
        start of every replay().  Where the reference rebuilds and recompiles its graph every step
        (Sources/DGenLazy/Backward.swift:225), this keeps one recording per model.  Needs counted_adam=True and one
        eager step() before it (so that nothing allocates inside).

        With one rank the step is ONE recording.  With several the gradient exchange stays outside: forward +
        backward is one recording, the all-reduce is enqueued call by call between, the update is a second one
        (the library refuses a collective inside a recording)."""
        torch = self.torch
        if not self.counted_adam:
            raise ValueError("capture() needs a model built with counted_adam=True")
        if self.step_index == 0:
            raise ValueError("run one eager step() before capture(): first-use allocations cannot be recorded")
        if self.graph_stream is None:
            self.graph_stream = torch.cuda.Stream(device="cuda:%d" % self.ctx.device)
        s = self.graph_stream
        s.wait_stream(torch.cuda.current_stream())
        args = (X, f0, uv, gain, noise_gain, noise, w_fs, target)
        self.static_args = args
        self._load(args)
        self.steps[self.i_update].f[0] = lr
        split = self._exchanges()
        with self.ctx.on_stream(s), torch.cuda.stream(s):
            with self.ctx.record() as rec:
                self._run(0, self.i_exchange)
                if not split:
                    self._run(self.i_update, 1)
            graphs = [rec.graph]
            if split:
                with self.ctx.record() as rec2:
                    self._run(self.i_update, 1)
                graphs.append(rec2.graph)
        for g in self.graph or []:
            g.close()
        self.graph = graphs
        return graphs

    def replay(self):
        """One recorded step; returns the device loss tensor."""
        torch = self.torch
        cur, s = torch.cuda.current_stream(), self.graph_stream
        s.wait_stream(cur)            # the caller refilled the inputs on its own stream
        with self.ctx.on_stream(s), torch.cuda.stream(s):
            if self.static_args is not None:
                self._load(self.static_args)
            self.graph[0].launch()
            if len(self.graph) > 1:
                if self.exchange_events is not None:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    self._exchange()
                    e1.record()
                    self.exchange_events.append((e0, e1))
                else:
                    self._exchange()
                self.graph[1].launch()
        cur.wait_stream(s)
        self.step_index += 1
        return self.loss


def features_from_controls(f0, gain, f0_min=40.0, f0_max=2000.0):
    """Per-control-frame conditioning [F*B, 2]: normalised log-f0 and loudness
    (Examples/HarmonicE2E/Trainer.swift:590-625 builds the same kind of rows)."""
    lf = (np.log(np.maximum(f0, 1.0)) - np.log(f0_min)) / (np.log(f0_max) - np.log(f0_min))
    return np.stack([lf.reshape(-1), gain.reshape(-1)], axis=1).astype(np.float32)
