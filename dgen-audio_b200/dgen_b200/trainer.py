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

from . import Context, FirParams, HarmonicParams, PHASE_SCAN, mss_params, sharding


class HarmonicModel:
    def __init__(self, ctx: Context, B, T, K=100, F=1000, sr=16000.0, nbands=65, taps=257, hidden=512, in_features=2,
                 ir_len=16000, conv_n=2048, conv_hop=1024, sizes=(2048, 1024, 512, 256, 128, 64), seed=0,
                 phase_mode=PHASE_SCAN, global_voices=None, counted_adam=False):
        import torch
        self.torch, self.ctx = torch, ctx
        self.B, self.T, self.K, self.F, self.sr = B, T, K, F, sr
        self.nbands, self.taps, self.hidden, self.in_features = nbands, taps, hidden, in_features
        self.ir_len, self.conv_n, self.conv_hop, self.sizes = ir_len, conv_n, conv_hop, tuple(sizes)
        self.phase_mode = phase_mode
        self.global_voices = global_voices or B
        self.M = F * B
        dims = [(in_features, hidden), (hidden, hidden), (hidden, hidden), (hidden, K + nbands)]
        self.layout, off = [], 0
        for i, (a, b) in enumerate(dims):
            self.layout.append(("W%d" % i, off, (a, b)))
            off += a * b
            self.layout.append(("b%d" % i, off, (b,)))
            off += b
        self.layout.append(("ir", off, (ir_len,)))
        off += ir_len
        self.n_params = off
        rng = np.random.default_rng(seed)
        flat = np.zeros(off, np.float32)
        for name, o, shape in self.layout:
            n = int(np.prod(shape))
            if name.startswith("W"):
                flat[o:o + n] = (rng.standard_normal(n) / np.sqrt(shape[0])).astype(np.float32)
            elif name == "ir":
                t = np.arange(ir_len) / sr
                flat[o:o + n] = (0.05 * rng.standard_normal(n) * np.exp(-6.91 * t / 0.4)).astype(np.float32)
        dev = "cuda:%d" % ctx.device
        self.params = torch.from_numpy(flat).to(dev)
        self.grads = torch.zeros_like(self.params)
        self.m = torch.zeros_like(self.params)
        self.v = torch.zeros_like(self.params)
        self.step_index = 0
        # step index in device memory: a recorded step advances it on every replay
        self.counted_adam = counted_adam
        self.t_dev = torch.zeros(1, dtype=torch.int32, device=dev)
        self.corr = torch.zeros(2, dtype=torch.float32, device=dev)
        self.graph, self.graph_stream = None, None   # list of recordings (see capture)
        self.exchange_events = None   # a list: replay() appends a CUDA event pair around every gradient exchange
        f = lambda *s: torch.empty(*s, dtype=torch.float32, device=dev)
        M, H = self.M, hidden
        self.act = [f(M, H), f(M, H), f(M, H), f(M, K + nbands)]
        self.act_t = [f(H, M), f(H, M), f(H, M)]         # transposed copies of the trunk activations
        hp0 = HarmonicParams(B, T, K, F, sr, 1.0, phase_mode, 0)
        self.h_scratch = f(int(ctx.lib.dgc_harmonic_bwd_scratch_floats(C.byref(hp0))) + 64)
        self.h_prepared = None
        self.side = torch.cuda.Stream(device=dev)        # second stream for the noise branch
        self.noise_out = f(B, T)
        # the per-(F, T) clock tables are built on first use by a kernel on the then-current stream: build them
        # now, so that the two concurrent branches of the first step both find them complete
        ctx.check(ctx.lib.dgc_ctx_prepare_tables(ctx.h, F, T))
        self.dact = [f(M, H), f(M, H), f(M, H)]          # gradient w.r.t. a layer's input
        self.dz = [f(M, H), f(M, H), f(M, H), f(M, K + nbands)]
        self.head_dz = f(M, K + nbands)
        self.amps, self.bands = f(F, B, K), f(F, B, nbands)
        self.taps_tab, self.g_taps = f(F, B, taps), f(F, B, taps)
        self.g_amps, self.g_bands = f(F, B, K), f(F, B, nbands)
        self.dry, self.out, self.g_out = f(B, T), f(B, T), f(B, T)
        self.loss = torch.zeros(1, dtype=torch.float64, device=dev)
        self.mss = mss_params(B, T, self.sizes)

    def view(self, name, buf=None):
        buf = self.params if buf is None else buf
        for n, o, shape in self.layout:
            if n == name:
                return buf[o:o + int(np.prod(shape))].view(*shape)
        raise KeyError(name)

    # ------------------------------------------------------------------------------------------
    def forward(self, X, f0, uv, gain, noise_gain, noise, w_fs, target):
        c = self.ctx
        lib, h = c.lib, c.h
        a = X
        for i in range(4):
            W, b = self.view("W%d" % i), self.view("b%d" % i)
            # trunk activations are also kept transposed: the next layer's weight gradient reads them along m
            c.check(lib.dgc_linear_fwd(h, a.data_ptr(), W.data_ptr(), b.data_ptr(), self.M, W.shape[0], W.shape[1],
                                       1 if i < 3 else 0, self.act[i].data_ptr(),
                                       self.act_t[i].data_ptr() if i < 3 else None))
            a = self.act[i]
        c.check(lib.dgc_hn_heads_fwd(h, self.act[3].data_ptr(), self.M, self.K, self.nbands, self.amps.data_ptr(),
                                     self.bands.data_ptr()))
        # the noise branch (band -> tap map, FIR) shares nothing with the harmonic branch until the two are
        # summed: it runs on a side stream beside it
        cur = self.torch.cuda.current_stream()
        self.side.wait_stream(cur)
        with c.on_stream(self.side):
            c.check(lib.dgc_bands_to_taps(h, self.bands.data_ptr(), w_fs.data_ptr(), self.M, self.nbands, self.taps,
                                          self.taps_tab.data_ptr()))
            fp = FirParams(self.B, self.T, self.F, self.taps, 0.12, 0)
            c.check(lib.dgc_fir_noise(h, C.byref(fp), noise.data_ptr(), self.taps_tab.data_ptr(),
                                      noise_gain.data_ptr(), self.noise_out.data_ptr()))
        hp = HarmonicParams(self.B, self.T, self.K, self.F, self.sr, 1.0, self.phase_mode, 0)
        # the render's per-sample tracks and phase anchors stay in this scratch for the backward pass
        c.check(lib.dgc_harmonic_render(h, C.byref(hp), f0.data_ptr(), uv.data_ptr(), self.amps.data_ptr(),
                                        gain.data_ptr(), self.h_scratch.data_ptr(), self.dry.data_ptr()))
        self.h_prepared = (f0.data_ptr(), uv.data_ptr(), gain.data_ptr())
        cur.wait_stream(self.side)
        self.torch.add(self.dry, self.noise_out, out=self.dry)
        self.out.copy_(self.dry)
        ir = self.view("ir")
        c.check(lib.dgc_partconv(h, self.dry.data_ptr(), self.B, self.T, ir.data_ptr(), self.ir_len, self.conv_n,
                                 self.conv_hop, 1.0, None, 1, self.out.data_ptr()))
        c.check(lib.dgc_mss_loss_fwd(h, C.byref(self.mss), self.out.data_ptr(), target.data_ptr(), None,
                                     self.loss.data_ptr()))
        return self.loss

    def backward(self, X, f0, uv, gain, noise_gain, noise, w_fs, target):
        c = self.ctx
        lib, h = c.lib, c.h
        upstream = float(self.B) / float(self.global_voices)   # local share of the global-batch mean
        c.check(lib.dgc_mss_loss_bwd(h, C.byref(self.mss), self.out.data_ptr(), target.data_ptr(), upstream,
                                     self.g_out.data_ptr()))
        ir, g_ir = self.view("ir"), self.view("ir", self.grads)
        # g_dry = g_out + A(ir)^T g_out, accumulated in place; g_ir
        c.check(lib.dgc_partconv_bwd(h, self.dry.data_ptr(), self.B, self.T, ir.data_ptr(), self.ir_len, self.conv_n,
                                     self.conv_hop, 1.0, self.g_out.data_ptr(), None, 1, self.g_out.data_ptr(),
                                     g_ir.data_ptr()))
        hp = HarmonicParams(self.B, self.T, self.K, self.F, self.sr, 1.0, self.phase_mode, 0)
        bwd = lib.dgc_harmonic_render_bwd_prepared \
            if getattr(self, "h_prepared", None) == (f0.data_ptr(), uv.data_ptr(), gain.data_ptr()) \
            else lib.dgc_harmonic_render_bwd
        # the two synthesis branches again side by side: noise-branch gradients on the side stream (the context
        # scratch they use is not touched by the harmonic backward, which works in the model's own scratch)
        cur = self.torch.cuda.current_stream()
        self.side.wait_stream(cur)
        with c.on_stream(self.side):
            fp = FirParams(self.B, self.T, self.F, self.taps, 0.12, 0)
            c.check(lib.dgc_fir_noise_bwd(h, C.byref(fp), noise.data_ptr(), noise_gain.data_ptr(),
                                          self.g_out.data_ptr(), self.g_taps.data_ptr()))
            # g_bands = g_taps Wfs   ([M, taps] x [taps, nbands])
            c.check(lib.dgc_linear_fwd(h, self.g_taps.data_ptr(), w_fs.data_ptr(), None, self.M, self.taps,
                                       self.nbands, 0, self.g_bands.data_ptr(), None))
        c.check(bwd(h, C.byref(hp), f0.data_ptr(), uv.data_ptr(), self.amps.data_ptr(), gain.data_ptr(),
                    self.g_out.data_ptr(), self.h_scratch.data_ptr(), self.g_amps.data_ptr()))
        self.h_prepared = None
        cur.wait_stream(self.side)
        c.check(lib.dgc_hn_heads_bwd(h, self.act[3].data_ptr(), self.g_amps.data_ptr(), self.g_bands.data_ptr(),
                                     self.M, self.K, self.nbands, self.dz[3].data_ptr()))
        # head layer: dz[3] is the gradient w.r.t. z (no activation); trunk layers: dact[i] is the gradient
        # w.r.t. act[i] and the kernel applies tanh' to it
        for i in (3, 2, 1, 0):
            W = self.view("W%d" % i)
            inp = X if i == 0 else self.act[i - 1]
            gW, gb = self.view("W%d" % i, self.grads), self.view("b%d" % i, self.grads)
            dc = self.dz[3] if i == 3 else self.dact[i]
            dz_out = self.head_dz if i == 3 else self.dz[i]
            da = self.dact[i - 1].data_ptr() if i > 0 else None
            c.check(lib.dgc_linear_bwd(h, inp.data_ptr(), W.data_ptr(), self.act[i].data_ptr(), dc.data_ptr(), self.M,
                                       W.shape[0], W.shape[1], 1 if i < 3 else 0, dz_out.data_ptr(), da,
                                       gW.data_ptr(), gb.data_ptr(), self.act_t[i - 1].data_ptr() if i > 0 else None))
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
            self.ctx.allreduce_sum_(self.grads)   # NCCL communicator owned by the context (C ABI)
        else:
            sharding.allreduce_sum_(self.grads)   # torch.distributed process group

    def _exchanges(self):
        """True when the gradient sum really crosses ranks."""
        if getattr(self, "use_ctx_comm", False):
            return True
        return sharding.world_size() > 1

    def _update(self, lr):
        if self.counted_adam:
            self.ctx.adam_step_counted(self.params, self.grads, self.m, self.v, self.t_dev, self.corr, lr=lr)
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
        """Record one whole training step (both streams, Adam) on the given tensors, which become the step's static
        input buffers: refill them in place and call replay().  Where the reference rebuilds and recompiles its
        graph every step (Sources/DGenLazy/Backward.swift:225), this keeps one recording per model.  Needs
        counted_adam=True and one eager step() before it (so that nothing allocates inside).

        With one rank the step is ONE recording.  With several the gradient exchange stays outside: forward +
        backward is one recording, the all-reduce is enqueued call by call between, the update is a second one
        (a collective inside a recording makes every rank's replay depend on the others' through the library's
        own host threads; the call-by-call exchange is the path the multi-GPU runs have verified)."""
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
        split = self._exchanges()
        with self.ctx.on_stream(s), torch.cuda.stream(s):
            with self.ctx.record() as rec:
                self.forward(*args)
                self.backward(*args)
                if not split:
                    self._update(lr)
            graphs = [rec.graph]
            if split:
                with self.ctx.record() as rec2:
                    self._update(lr)
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
