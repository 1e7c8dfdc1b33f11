#!/usr/bin/env python
"""Benchmark of the frame-parallel render path: batched harmonic+noise synthesis forward +
multi-scale spectral loss (B=16 voices per GPU, 64000 frames, 100 harmonics, 65 noise bands as
257-tap FIR, FFT sizes 2048..64, 75 % overlap), on synthetic seeded inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one pass of the path over one batch.  `value` is synthesized samples per second
(voices x frames, all GPUs) with inputs resident in HBM; `e2e` is the same metric through the
host-buffer C-ABI call (host->device copies of every input and the device->host loss read inside
the timed region).  Multi-GPU: one process per GPU (torchrun), voices sharded, no data-path
collective (forward-only render): weak scaling.

The same JSON line carries, beside the headline:
  stages       per-stage time with the roofline that bounds that stage (SFU for the oscillator bank, FP32 for the
               FIR and the loss transforms, HBM for the band -> tap map), and the HBM figure beside it;
  sustained    the step replayed for >= 2 s over rotating input sets (working set > L2) with the SM clock sampled;
  target_b256  (one GPU only) the same step at 256 voices on this one GPU: the configuration the path's
               throughput target is stated on;
  train        the full training step (32 voices per GPU, gradient all-reduce between two recordings), at every N;
  other_configs (one GPU only) oscillator -> filter -> FFT, biquad bank forward / BPTT, partitioned convolution.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "dgen-audio_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np  # noqa: E402

METRIC = "synthesized samples/sec (batch x frames) fwd+loss"
UNIT = "samples/s"
CFG = dict(B=16, T=64000, K=100, F=1000, sr=16000.0, nbands=65, taps=257)
SIZES = (2048, 1024, 512, 256, 128, 64)
SEED = 20260001
PHASE = {"mode": "fundamental"}
FP32_LANES_PER_SM, SFU_LANES_PER_SM = 128, 16
STEP_MODE = {"mode": "replay"}


def config_json(n_gpus):
    return {"workload": "harmonic+noise synthesis fwd + multi-scale spectral loss (BASELINE.json configs[1])",
            "voices_per_gpu": CFG["B"], "frames": CFG["T"], "harmonics": CFG["K"], "control_frames": CFG["F"],
            "sample_rate": CFG["sr"], "noise_bands": CFG["nbands"], "fir_taps": CFG["taps"],
            "fft_sizes": list(SIZES), "overlap": 0.75, "global_voices": CFG["B"] * n_gpus,
            "phase_mode": PHASE["mode"], "sharding": "voices across GPUs, no collective in the forward + loss step "
                                                     "(the train block has the gradient all-reduce)",
            "step_mode": STEP_MODE["mode"],
            "l2": "L2 flushed (512 MiB write) between timed steps"}


# --------------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------------
# CPU arm (oracle restatement of the reference C backend), used for cpu_baseline and --impl reference
# --------------------------------------------------------------------------------------------------
def cpu_arm(voices, threads, seed=SEED, min_seconds=0.0):
    """Times render + loss of `voices` voices of the workload on the host with `threads` threads, repeating the pass
    over the same voices until `min_seconds` of timed work have accumulated.
    Returns (samples_per_s, seconds, passes)."""
    import tempfile
    from concurrent.futures import ThreadPoolExecutor
    from dgen_b200 import workloads as wl
    from oracle import oracle as orc
    out_dir = os.path.join(tempfile.gettempdir(), "dgen_oracle_native")
    so = os.path.join(out_dir, "libdgen_oracle_fast.so")
    try:
        orc.build(out_dir=out_dir, march="-march=native")  # built on the machine that runs it
        L = orc.lib(path=so)
    except Exception:
        L = orc.lib(fast=True)
    d = wl.harmonic_noise_inputs(seed, B=voices, **{k: CFG[k] for k in ("T", "K", "F", "sr", "nbands", "taps")})
    t = wl.harmonic_noise_inputs(seed + 1, B=voices, **{k: CFG[k] for k in ("T", "K", "F", "sr", "nbands", "taps")})
    taps = wl.taps_from_bands(d)
    rng = np.random.default_rng(0)
    target = rng.standard_normal((voices, CFG["T"])).astype(np.float32) * 0.1
    del t

    def one(b):
        sl = slice(b, b + 1)
        a = orc.harmonic_noise_render(d["f0"][:, sl], d["uv"][:, sl], d["amps"][:, sl], d["gain"][:, sl],
                                      d["noise_gain"][:, sl], taps[:, sl], d["noise"][sl], CFG["T"], CFG["sr"], L=L)
        return orc.mss_loss(a, target[sl], sizes=SIZES, L=L)

    one(0)  # warm-up (page in, build twiddles)
    dt, passes = 0.0, 0
    with ThreadPoolExecutor(max_workers=threads) as ex:
        while passes == 0 or dt < min_seconds:
            t0 = time.perf_counter()
            list(ex.map(one, range(voices)))
            dt += time.perf_counter() - t0
            passes += 1
    return passes * voices * CFG["T"] / dt, dt, passes


def run_reference(args, rank, world):
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    threads = max(1, min(cores, 64))
    voices = threads * 2 if threads > 1 else 4
    vals, secs = [], []
    for _ in range(min(1, args.warmup)):
        cpu_arm(threads, threads)  # one untimed pass (page-in, native build of the oracle)
    for _ in range(args.steps):
        v, s, _ = cpu_arm(voices, threads)
        vals.append(v)
        secs.append(s)
    value = float(np.mean(vals))
    ms = float(np.mean(secs)) * 1e3
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_json(args.gpus),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": "%d voices x %d frames per step, render + 6-scale loss, one voice per thread; "
                                       "CPU restatement of the reference C backend (the Swift compiler that emits "
                                       "the reference's C is not available)" % (voices, CFG["T"])},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


def audible_fraction(f0):
    """Share of the (control row, voice, partial) triples whose partial lies below Nyquist: fl(k f0) < sr / 2, the
    reference's mask.  The render evaluates a sine only for those; the rest contribute an exact zero."""
    K, nyq = CFG["K"], np.float32(CFG["sr"] * 0.5)
    k = np.arange(1, K + 1, dtype=np.float32)
    return float((np.asarray(f0, np.float32)[..., None] * k < nyq).mean())


def stage_rooflines(B, T, stage_ms, sm_mhz, sm_count, hbm_peak, audible=1.0):
    """Per stage: the bound that applies to it and the fraction reached, the HBM figure beside it.
    Algorithmic work per launch (fp32 = 4 bytes; B voices, T frames, K partials, F control rows):
      harmonic_render  one sine per (voice, frame, partial BELOW NYQUIST) on the special-function lanes (`audible` =
                       that share of the B T K partial-frames; the reference evaluates all K and multiplies the
                       others by a zero mask); bytes 4 (B F (K+2) + B T)
      fir_noise        2 x taps multiply-adds per sample for the two control rows a sample is interpolated between
                       (4 taps flops per sample); bytes 4 (B T + B F nbands + B T): noise in, band magnitudes in, out
      mss_loss_fwd     one complex transform of N points per window carries both signals: 5 N log2 N flops per
                       window, H = ceil(T / hop) windows per voice and scale; bytes 2 x 4 B T per scale
      bands_to_taps    bytes 4 B F (nbands + taps): a memory-bound map (26 flops per byte moved)"""
    K, F, taps, nbands = CFG["K"], CFG["F"], CFG["taps"], CFG["nbands"]
    clk = sm_mhz * 1e6
    fp32_peak = sm_count * FP32_LANES_PER_SM * 2 * clk / 1e12          # TFLOP/s, one FMA per lane and clock
    sfu_peak = sm_count * SFU_LANES_PER_SM * clk / 1e9                 # G results / s
    alg_bytes = {"harmonic_render": 4 * (B * F * (K + 2) + B * T),
                 "fir_noise": 4 * (B * T + B * F * nbands + B * T),
                 "bands_to_taps": 4 * (B * F * nbands + B * F * taps),
                 "mss_loss_fwd": 2 * 4 * B * T * len(SIZES)}
    fft_flops = 0.0
    for n in SIZES:
        if n > T:
            continue
        hop = max(1, n // 4)
        fft_flops += 5.0 * n * np.log2(n) * ((T + hop - 1) // hop) * B
    work = {"harmonic_render": ("sfu", B * T * K * audible / 1e9, sfu_peak, "G sin/s"),
            "fir_noise": ("fp32", 4.0 * taps * B * T / 1e12, fp32_peak, "TFLOP/s"),
            "mss_loss_fwd": ("fp32", fft_flops / 1e12, fp32_peak, "TFLOP/s"),
            "bands_to_taps": ("hbm", alg_bytes["bands_to_taps"] / 1e9, hbm_peak, "GB/s")}
    out, bound_time_ms = {}, 0.0
    for name, ms in stage_ms.items():
        kind, amount, peak, unit = work[name]
        ach = amount / (ms * 1e-3)
        gbs = alg_bytes[name] / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "bound": kind, "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
                     "hbm": {"algorithmic_bytes": alg_bytes[name], "achieved_gbs": gbs, "frac": gbs / hbm_peak}}
        bound_time_ms += amount / peak * 1e3
    out["harmonic_render"]["audible_share_of_partials"] = audible
    out["harmonic_render"]["masked_form_sines_per_s"] = B * T * K / (stage_ms["harmonic_render"] * 1e-3) / 1e9
    return out, alg_bytes, bound_time_ms


def ncu_traffic(stage, B):
    """DRAM bytes (read + write) of the stage's kernels per launch, from the committed ncu summary
    profiles/fwd_loss_dram_traffic.md, which states per kernel the bytes per voice and the hash of the kernel
    sources it was captured from.  None when the summary is absent or was captured from other sources."""
    import hashlib
    import re
    path = os.path.join(ROOT, "profiles", "fwd_loss_dram_traffic.md")
    try:
        text = open(path).read()
    except Exception:
        return None, "no ncu traffic summary committed"
    h = hashlib.sha256()
    csrc = os.path.join(ROOT, "dgen-audio_b200", "csrc")
    for f in sorted(os.listdir(csrc)):
        h.update(open(os.path.join(csrc, f), "rb").read())
    m = re.search(r"sources_sha16:\s*([0-9a-f]{16})", text)
    if not m or m.group(1) != h.hexdigest()[:16]:
        return None, "the committed ncu summary was captured from other kernel sources"
    m = re.search(r"^traffic_bytes_per_voice\s+%s\s+([0-9.eE+]+)" % re.escape(stage), text, re.M)
    if not m:
        return None, "stage not in the ncu summary"
    return float(m.group(1)) * B, "profiles/fwd_loss_dram_traffic.md"


class FwdLoss:
    """The harmonic+noise forward + multi-scale loss step on one GPU for B voices: device buffers, the staged
    single-stream sequence (per-stage times, cross-check) and the composite call (the timed step)."""

    def __init__(self, ctx, B, seed, nsets=1):
        import ctypes as C
        import torch
        import dgen_b200
        from dgen_b200 import workloads as wl
        self.ctx, self.B, self.torch, self.C, self.dg = ctx, B, torch, C, dgen_b200
        cfg = dict(CFG, B=B)
        T, K, F, sr = cfg["T"], cfg["K"], cfg["F"], cfg["sr"]
        self.cfg = cfg
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        self.host = wl.harmonic_noise_inputs(seed, **cfg)
        tg = wl.harmonic_noise_inputs(seed + 1, **cfg)
        self.sets = [{k: dev(v) for k, v in self.host.items() if isinstance(v, np.ndarray)}]
        for _ in range(1, nsets):
            self.sets.append({k: v.clone() for k, v in self.sets[0].items()})
        self.D = self.sets[0]
        G = {k: dev(v) for k, v in tg.items() if isinstance(v, np.ndarray)}
        self.audio = torch.empty(B, T, device="cuda")
        self.loss = torch.zeros(1, dtype=torch.float64, device="cuda")
        self.mss = dgen_b200.mss_params(B, T, SIZES)
        mode = {"scan": dgen_b200.PHASE_SCAN, "sequential": dgen_b200.PHASE_SEQUENTIAL,
                "fundamental": dgen_b200.PHASE_FUNDAMENTAL}[PHASE["mode"]]
        self.hp = dgen_b200.HarmonicParams(B, T, K, F, sr, 1.0, mode, 0)
        self.fp = dgen_b200.FirParams(B, T, F, cfg["taps"], 0.12, 1)
        self.taps_buf = torch.empty(F, B, cfg["taps"], device="cuda")
        self.st = dgen_b200.HnStep()
        self.st.harm, self.st.fir, self.st.mss, self.st.nbands = self.hp, self.fp, self.mss, cfg["nbands"]
        nwork = int(ctx.lib.dgc_hn_forward_loss_work_floats(C.byref(self.st)))
        self.works = [torch.empty(nwork, device="cuda") for _ in range(nsets)]
        # target audio: rendered once from seed+1 (setup, untimed)
        self.target = torch.empty(B, T, device="cuda")
        self.stage_taps(G); self.stage_harm(G, self.target); self.stage_fir(G, self.target)
        self.targets = [self.target] + [self.target.clone() for _ in range(1, nsets)]
        torch.cuda.synchronize()

    def stage_taps(self, X):
        c, cfg = self.ctx, self.cfg
        c.check(c.lib.dgc_bands_to_taps(c.h, X["bands"].data_ptr(), X["W"].data_ptr(), cfg["F"] * self.B,
                                        cfg["nbands"], cfg["taps"], self.taps_buf.data_ptr()))

    def stage_harm(self, X, out):
        c = self.ctx
        c.check(c.lib.dgc_harmonic_render(c.h, self.C.byref(self.hp), X["f0"].data_ptr(), X["uv"].data_ptr(),
                                          X["amps"].data_ptr(), X["gain"].data_ptr(), None, out.data_ptr()))

    def stage_fir(self, X, out):
        c = self.ctx
        c.check(c.lib.dgc_fir_noise(c.h, self.C.byref(self.fp), X["noise"].data_ptr(), self.taps_buf.data_ptr(),
                                    X["noise_gain"].data_ptr(), out.data_ptr()))

    def stage_loss(self, pred, target):
        c = self.ctx
        c.check(c.lib.dgc_mss_loss_fwd(c.h, self.C.byref(self.mss), pred.data_ptr(), target.data_ptr(), None,
                                       self.loss.data_ptr()))

    def step_staged(self):
        D = self.D
        self.stage_taps(D); self.stage_harm(D, self.audio); self.stage_fir(D, self.audio)
        self.stage_loss(self.audio, self.target)

    def step(self, i=0):
        """ONE call of the device-resident composite (harmonic and noise branch on two streams, joined at the loss)."""
        c, D = self.ctx, self.sets[i]
        c.check(c.lib.dgc_hn_forward_loss(c.h, self.C.byref(self.st), D["f0"].data_ptr(), D["uv"].data_ptr(),
                                          D["amps"].data_ptr(), D["gain"].data_ptr(), D["noise_gain"].data_ptr(),
                                          D["bands"].data_ptr(), D["W"].data_ptr(), D["noise"].data_ptr(),
                                          self.targets[i].data_ptr(), self.works[i].data_ptr(), self.loss.data_ptr(),
                                          None))

    def check_composite(self):
        self.step_staged()
        a = float(self.loss.cpu()[0])
        self.step()
        b = float(self.loss.cpu()[0])
        if not abs(b - a) <= 1e-9 * abs(a):
            raise SystemExit("composite step and staged step disagree: %r vs %r" % (b, a))
        return b

    def record(self, stream, i=0):
        """Record the composite step on `stream` (its two streams and their join included); returns the graph."""
        torch = self.torch
        stream.wait_stream(torch.cuda.current_stream())
        with self.ctx.on_stream(stream), torch.cuda.stream(stream):
            with self.ctx.record() as rec:
                self.step(i)
            for _ in range(2):
                rec.graph.launch()
        torch.cuda.synchronize()
        return rec.graph

    def stage_times(self, flush, reps):
        torch, D = self.torch, self.D
        stages = {"bands_to_taps": lambda: self.stage_taps(D), "harmonic_render": lambda: self.stage_harm(D, self.audio),
                  "fir_noise": lambda: self.stage_fir(D, self.audio),
                  "mss_loss_fwd": lambda: self.stage_loss(self.audio, self.target)}
        out = {}
        for name, fn in stages.items():
            fn()
            acc = 0.0
            for r in range(reps):
                flush.fill_(float(r))
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); fn(); b.record()
                torch.cuda.synchronize()
                acc += a.elapsed_time(b)
            out[name] = acc / reps
        return out


def timed_replay(ctx, fl, graphs, run_stream, flush, steps, barrier):
    """`steps` launches of the recorded step(s), each bracketed by CUDA events on the launching stream, L2 flushed
    before every step.  Returns the summed device time in ms."""
    torch = fl.torch
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    barrier()
    with ctx.on_stream(run_stream), torch.cuda.stream(run_stream):
        for s in range(steps):
            flush.fill_(float(s))
            evs[s][0].record()
            graphs[s % len(graphs)].launch()
            evs[s][1].record()
    barrier()
    return sum(a.elapsed_time(b) for a, b in evs)


def sustained_run(ctx, fl, graphs, run_stream, local_rank, seconds=2.5):
    """The recorded step replayed back to back for at least `seconds`, rotating over input sets whose total exceeds
    L2, with the SM clock sampled every 100 ms: a clock or throttle problem shows here, not in a 6 ms region."""
    torch = fl.torch
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.25)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n, t0 = 0, time.perf_counter()
    with ctx.on_stream(run_stream), torch.cuda.stream(run_stream):
        a.record()
        while True:
            for _ in range(256):
                graphs[n % len(graphs)].launch()
                n += 1
            run_stream.synchronize()
            if time.perf_counter() - t0 >= seconds:
                break
        b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b)
    clocks = sampler.stop()
    return {"seconds": ms * 1e-3, "steps": n, "ms_per_step": ms / n, "value": fl.B * fl.cfg["T"] * n / (ms * 1e-3),
            "unit": UNIT, "clocks": clocks, "input_sets": len(graphs),
            "l2": "%d input sets in rotation (%.0f MB per set): the working set exceeds L2, no flush kernels between steps"
                  % (len(graphs), sum(v.numel() for v in fl.D.values()) * 4 / 1e6)}


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import dgen_b200
    from dgen_b200 import sharding

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = dgen_b200.Context(local_rank)
    sm_count = torch.cuda.get_device_properties(local_rank).multi_processor_count
    B, T, K, F = CFG["B"], CFG["T"], CFG["K"], CFG["F"]
    NSETS = 4
    fl = FwdLoss(ctx, B, SEED + 100 * rank, nsets=NSETS)
    loss_fused = fl.check_composite()
    flush = torch.empty(512 * 1024 * 1024 // 4, device="cuda")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        fl.step()
    barrier()
    # --step-mode replay (the default): the composite step is recorded once (its two streams and their join
    # included) and the timed step is one launch of that recording; eager: the call itself is timed.  Same kernels,
    # same inputs, same loss; the recording only removes the host's launch gaps between the kernels.
    replay = args.step_mode != "eager"
    run_stream = torch.cuda.Stream() if replay else torch.cuda.current_stream()
    graphs = []
    if replay:
        graphs = [fl.record(run_stream, i) for i in range(NSETS)]
        loss_replayed = float(fl.loss.cpu()[0])
        if loss_replayed != loss_fused:
            raise SystemExit("replayed step and direct call disagree: %r vs %r" % (loss_replayed, loss_fused))
    launches0 = ctx.launch_count()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if replay:
        total_ms = timed_replay(ctx, fl, graphs[:1], run_stream, flush, args.steps, barrier)
    else:
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        barrier()
        for s in range(args.steps):
            flush.fill_(float(s))
            evs[s][0].record()
            fl.step()
            evs[s][1].record()
        barrier()
        total_ms = sum(a.elapsed_time(b) for a, b in evs)
    launches = ctx.launch_count() - launches0
    loss_val = float(fl.loss.cpu()[0])
    stage_ms = fl.stage_times(flush, max(3, min(args.steps, 10)))
    audible = audible_fraction(fl.host["f0"])

    # end to end through the host-buffer entry point: pinned host inputs, H2D + D2H inside the timed region
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    P = {k: pin(v) for k, v in fl.host.items() if isinstance(v, np.ndarray)}
    target_host = pin(fl.target.cpu().numpy())
    st = fl.st

    def e2e_step():
        return ctx.hn_forward_loss_host(st, P["f0"], P["uv"], P["amps"], P["gain"], P["noise_gain"], P["bands"],
                                        P["W"], P["noise"], target_host)

    for _ in range(max(3, args.warmup)):
        e2e_loss = e2e_step()
    barrier()
    e2e_ms = 0.0
    for s in range(args.steps):
        flush.fill_(float(s))
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        e2e_loss = e2e_step()
        b.record()
        torch.cuda.synchronize()
        e2e_ms += a.elapsed_time(b)
    barrier()
    # the same steps with TWO in flight (submit / wait over two staging slots): every step still uploads its inputs
    # from pinned host memory and returns its loss to the host inside the timed region, but the upload of step i+1
    # crosses PCIe while step i computes.  Timed as one region over all steps (the steps overlap by design).
    hargs = (st, P["f0"], P["uv"], P["amps"], P["gain"], P["noise_gain"], P["bands"], P["W"], P["noise"], target_host)
    for i in range(4):
        ctx.hn_forward_loss_host_submit(*hargs, i % 2)
        ctx.hn_forward_loss_host_wait(i % 2)
    barrier()
    flush.fill_(1.0)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    ctx.hn_forward_loss_host_submit(*hargs, 0)
    for s in range(1, args.steps):
        ctx.hn_forward_loss_host_submit(*hargs, s % 2)
        piped_loss = ctx.hn_forward_loss_host_wait((s - 1) % 2)
    piped_loss = ctx.hn_forward_loss_host_wait((args.steps - 1) % 2)
    b.record()
    torch.cuda.synchronize()
    piped_ms = a.elapsed_time(b)
    barrier()
    # the lean form of the same API: the noise is generated on the device from a seed (the reference generates its
    # noise inside the graph too) and the target clip stays resident in HBM (the reference loads it once per run);
    # what crosses PCIe every step is the control-rate inputs and the loss.
    st_lean = type(st).from_buffer_copy(st)
    st_lean.noise_seed, st_lean.noise_mode, st_lean.noise_sigma = SEED + 17, dgen_b200.NOISE_GAUSSIAN, 1.0
    st_lean.target_dev = fl.target.data_ptr()
    largs = (st_lean, P["f0"], P["uv"], P["amps"], P["gain"], P["noise_gain"], P["bands"], P["W"], None, None)
    for i in range(4):
        ctx.hn_forward_loss_host_submit(*largs, i % 2)
        ctx.hn_forward_loss_host_wait(i % 2)
    barrier()
    flush.fill_(2.0)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    ctx.hn_forward_loss_host_submit(*largs, 0)
    for s in range(1, args.steps):
        ctx.hn_forward_loss_host_submit(*largs, s % 2)
        lean_loss = ctx.hn_forward_loss_host_wait((s - 1) % 2)
    lean_loss = ctx.hn_forward_loss_host_wait((args.steps - 1) % 2)
    b.record()
    torch.cuda.synchronize()
    lean_ms = a.elapsed_time(b)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    h2d_lean = 4 * sum(int(P[k].numel()) for k in ("f0", "uv", "amps", "gain", "noise_gain", "bands", "W"))
    h2d = 4 * sum(int(P[k].numel()) for k in ("f0", "uv", "amps", "gain", "noise_gain", "bands", "W", "noise")) \
        + 4 * int(target_host.numel())
    total_ms, e2e_ms, piped_ms, lean_ms = sharding.max_over_ranks([total_ms, e2e_ms, piped_ms, lean_ms], device="cuda")

    # sustained run (every rank runs it; rank 0 reports its own)
    sustained = sustained_run(ctx, fl, graphs, run_stream, local_rank) if replay else None
    barrier()
    for g in graphs:
        g.close()
    del P, target_host

    # the throughput target's own configuration: 256 voices on ONE GPU (device resident, replayed, per stage)
    target_b256 = None
    if world == 1 and B != 256 and not args.no_target:
        target_b256 = run_target(ctx, args, flush, sm_count, local_rank)

    # the training step, at every N: 32 voices per GPU, gradient all-reduce between the two recordings
    train = None
    if not args.no_train:
        del fl
        torch.cuda.empty_cache()
        train = train_measure(ctx, args, rank, world, local_rank, steps=max(5, min(args.steps, 20)))

    other = None
    if world == 1 and not args.no_other:
        torch.cuda.empty_cache()
        other = filters_measure(ctx, args, quick=True)

    if rank == 0:
        samples_per_step = B * T * world
        value = samples_per_step * args.steps / (total_ms * 1e-3)
        e2e_value = samples_per_step * args.steps / (e2e_ms * 1e-3)
        peaks = measured_peaks()
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        sm_mhz = float((clocks or {}).get("sm_mhz") or (sustained or {}).get("clocks", {}).get("sm_mhz") or 1965.0)
        stages, alg, bound_ms = stage_rooflines(B, T, stage_ms, sm_mhz, sm_count, hbm_peak, audible)
        dom = max(stage_ms, key=stage_ms.get)
        traffic, traffic_src = ncu_traffic(dom, B)
        rl = dict(stages[dom])
        rl.pop("ms")
        step_ms = total_ms / args.steps
        step_bytes = sum(alg.values())
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": config_json(world), "clocks": clocks,
                # throughput through the host-buffer API with two steps in flight (dgc_hn_forward_loss_host_submit /
                # _wait); "blocking" is the one-call-at-a-time form of the same API (dgc_hn_forward_loss_host)
                "e2e": {"value": samples_per_step * args.steps / (lean_ms * 1e-3), "unit": UNIT,
                        "h2d_bytes_per_step": h2d_lean, "d2h_bytes_per_step": 8, "ms_per_step": lean_ms / args.steps,
                        "mode": "two steps in flight: step i+1 uploads while step i computes; every step's control-rate "
                                "inputs (f0, voicing, harmonic amplitudes, gains, band magnitudes, band->tap matrix) come "
                                "from pinned host memory and its loss returns to the host inside the timed region; the "
                                "noise is generated on the device from a seed each step (as the reference generates it "
                                "inside its graph) and the target clip is resident in HBM (uploaded once, as the "
                                "reference loads it once per run)",
                        "loss": lean_loss,
                        "full_upload": {"value": samples_per_step * args.steps / (piped_ms * 1e-3),
                                        "ms_per_step": piped_ms / args.steps, "h2d_bytes_per_step": h2d,
                                        "what": "the same two-in-flight calls with the noise and the target uploaded "
                                                "from pinned host memory every step as well", "loss": piped_loss},
                        "blocking": {"value": e2e_value, "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": h2d,
                                     "l2": "flushed between steps",
                                     "what": "one call at a time, everything uploaded every step"}},
                "gpu_launches": int(launches),
                # the stage with the largest measured share, against the bound that applies to it
                "roofline": dict(rl, kernel=dom, traffic=traffic, traffic_source=traffic_src,
                                 peak_source=("measured" if peaks else "fallback") if rl["bound"] == "hbm" else
                                 "%d SMs x lanes x sampled SM clock %.0f MHz" % (sm_count, sm_mhz)),
                "stage_ms": stage_ms, "stages": stages,
                "whole_step": {"algorithmic_bytes": step_bytes,
                               "hbm": {"achieved_gbs": step_bytes / (step_ms * 1e-3) / 1e9,
                                       "frac": step_bytes / (step_ms * 1e-3) / 1e9 / hbm_peak,
                                       "peak": hbm_peak, "peak_source": "measured" if peaks else "fallback"},
                               "bound_ms": bound_ms, "frac_of_bound": bound_ms / step_ms,
                               "what": "bound_ms = sum over the stages of (stage work / the peak that bounds it): "
                                       "special-function lanes for the oscillator bank, FP32 lanes for the FIR "
                                       "and the loss transforms, measured copy bandwidth for the band -> tap map"},
                "loss": loss_val, "e2e_loss": e2e_loss}
        if sustained:
            line["sustained"] = sustained
        if target_b256:
            line["target_b256"] = target_b256
        if train:
            line["train"] = train
        if other:
            line["other_configs"] = other
        if not args.no_cpu and world == 1:
            v, secs, passes = cpu_arm(16, 1, min_seconds=12.0)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": 1, "kind": "port",
                                    "sample": "%d passes over 16 voices x %d frames (the workload's batch), render + "
                                              "6-scale loss, single thread (%.1f s); CPU restatement of the "
                                              "reference's single-threaded C backend" % (passes, T, secs)}
        print(json.dumps(line))
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def run_target(ctx, args, flush, sm_count, local_rank):
    """256 voices on this one GPU: replayed device-resident step, per-stage times and rooflines."""
    import torch
    Bt = 256
    fl = FwdLoss(ctx, Bt, SEED + 7, nsets=1)
    fl.check_composite()
    for _ in range(3):
        fl.step()
    stream = torch.cuda.Stream()
    graph = fl.record(stream)
    steps = max(5, min(args.steps, 20))
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed_replay(ctx, fl, [graph], stream, flush, steps, torch.cuda.synchronize) / steps
    # a second, longer region for the clock record: >= 1.5 s of back-to-back replays (inputs of 0.5 GB exceed L2)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n, t0 = 0, time.perf_counter()
    with ctx.on_stream(stream), torch.cuda.stream(stream):
        a.record()
        while time.perf_counter() - t0 < 1.5:
            for _ in range(32):
                graph.launch()
                n += 1
            stream.synchronize()
        b.record()
    torch.cuda.synchronize()
    sus_ms = a.elapsed_time(b) / n
    clocks = sampler.stop()
    stage_ms = fl.stage_times(flush, 5)
    graph.close()
    peaks = measured_peaks()
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    sm_mhz = float(clocks.get("sm_mhz") or 1965.0)
    stages, alg, bound_ms = stage_rooflines(Bt, fl.cfg["T"], stage_ms, sm_mhz, sm_count, hbm_peak,
                                            audible_fraction(fl.host["f0"]))
    step_bytes = sum(alg.values())
    out = {"voices": Bt, "n_gpus": 1, "ms_per_step": ms, "value": Bt * fl.cfg["T"] / (ms * 1e-3), "unit": UNIT,
           "steps": steps, "l2": "L2 flushed between timed steps; inputs (0.5 GB) exceed L2 anyway",
           "sustained": {"ms_per_step": sus_ms, "value": Bt * fl.cfg["T"] / (sus_ms * 1e-3), "steps": n,
                         "seconds": sus_ms * n * 1e-3}, "clocks": clocks,
           "stages": stages,
           "whole_step": {"algorithmic_bytes": step_bytes,
                          "hbm": {"achieved_gbs": step_bytes / (ms * 1e-3) / 1e9,
                                  "frac": step_bytes / (ms * 1e-3) / 1e9 / hbm_peak, "peak": hbm_peak},
                          "bound_ms": bound_ms, "frac_of_bound": bound_ms / ms}}
    del fl
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------------------------------
# training-step workload (BASELINE.json configs[4]): 32 voices per GPU, controller MLP 2-512-512-512-165,
# harmonic+noise synthesis, 1 s learnable IR reverb, multi-scale spectral loss, backward, gradient
# all-reduce (NCCL) and one Adam step
# --------------------------------------------------------------------------------------------------
def train_measure(ctx, args, rank, world, local_rank, steps, voices=32, want_e2e=True):
    """Times the training step on an initialised context (and, for world > 1, process group).  Returns the
    measurement as a dict on rank 0 (None elsewhere)."""
    import torch
    import torch.distributed as dist
    import dgen_b200
    from dgen_b200 import sharding, trainer as tr, workloads as wl

    B = voices
    T, K, F, sr, NB, NT = CFG["T"], CFG["K"], CFG["F"], CFG["sr"], CFG["nbands"], CFG["taps"]
    d = wl.harmonic_noise_inputs(SEED + 100 * rank, B=B, T=T, K=K, F=F, sr=sr, nbands=NB, taps=NT)
    tg = wl.harmonic_noise_inputs(SEED + 100 * rank + 1, B=B, T=T, K=K, F=F, sr=sr, nbands=NB, taps=NT)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    mode = {"scan": dgen_b200.PHASE_SCAN, "sequential": dgen_b200.PHASE_SEQUENTIAL,
            "fundamental": dgen_b200.PHASE_FUNDAMENTAL}[PHASE["mode"]]
    model = tr.HarmonicModel(ctx, B, T, K=K, F=F, sr=sr, nbands=NB, taps=NT, hidden=512, ir_len=16000, conv_n=2048,
                             conv_hop=1024, sizes=SIZES, seed=7, global_voices=B * world, counted_adam=True,
                             phase_mode=mode)
    # gradient exchange: the context's own NCCL communicator (dgc_allreduce_sum through the C ABI) unless
    # --allreduce torch asks for the torch.distributed call
    model.use_ctx_comm = args.allreduce == "dgc" and sharding.init_ctx_comm(ctx)
    # target: rendered from seed+1 controls (setup, untimed)
    G = {k: dev(v) for k, v in tg.items() if isinstance(v, np.ndarray)}
    target = ctx.harmonic_render(G["f0"], G["uv"], G["amps"], G["gain"], T, sr)
    ctx.fir_noise(G["noise"], ctx.bands_to_taps(G["bands"], G["W"]), G["noise_gain"], out=target, accumulate=True)
    host = dict(X=tr.features_from_controls(d["f0"], d["gain"]), f0=d["f0"], uv=d["uv"], gain=d["gain"],
                noise_gain=d["noise_gain"], noise=d["noise"], W=d["W"], target=target.cpu().numpy())
    order = ("X", "f0", "uv", "gain", "noise_gain", "noise", "W", "target")
    P = {k: pin(host[k]) for k in order}
    # the step's inputs live in the model's arena: fill them in place (no per-step device-to-device copies)
    D = dict(zip(order, model.input_views()))
    for k in order:
        D[k].copy_(torch.from_numpy(np.ascontiguousarray(host[k])).reshape(D[k].shape))
    dargs = [D[k] for k in order]
    del G

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        model.step(*dargs)
    # step mode: "replay" records the step once (both streams, Adam; with several ranks the gradient exchange stays
    # between two recordings) and launches the recording per step; "eager" enqueues it call by call.
    mode_s = args.step_mode if args.step_mode != "auto" else "replay"
    if mode_s == "replay":
        model.capture(*dargs)
        step_fn = model.replay
        for _ in range(2):
            step_fn()
    else:
        step_fn = lambda: model.step(*dargs)
    barrier()
    l0 = ctx.launch_count()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    model.exchange_events = [] if (mode_s == "replay" and world > 1) else None
    barrier()
    for s in range(steps):
        evs[s][0].record()
        loss = step_fn()
        evs[s][1].record()
    barrier()
    launches = ctx.launch_count() - l0
    total_ms = sum(a.elapsed_time(b) for a, b in evs)
    exch_ms = 0.0
    if model.exchange_events:
        exch_ms = sum(a.elapsed_time(b) for a, b in model.exchange_events) / len(model.exchange_events)
    model.exchange_events = None
    e2e_ms = piped_ms = 0.0
    loss_host = float(loss.cpu()[0])
    if want_e2e:
        # end to end: the step's inputs come from pinned host memory, the loss goes back to the host
        for s in range(steps):
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for k in order:
                D[k].copy_(P[k], non_blocking=True)
            loss = step_fn()
            loss_host = float(loss.cpu()[0])
            b.record()
            torch.cuda.synchronize()
            e2e_ms += a.elapsed_time(b)
        barrier()
        # the same with the NEXT step's inputs crossing PCIe (copy stream, device staging) while this step runs; at
        # the start of a step the staged inputs move into the step's static buffers device to device.  Every step
        # still takes its inputs from pinned host memory and returns its loss to the host inside the timed region.
        cur, cs = torch.cuda.current_stream(), torch.cuda.Stream()
        S = {k: torch.empty_like(D[k]) for k in order}

        def prefetch():
            with torch.cuda.stream(cs):
                for k in order:
                    S[k].copy_(P[k], non_blocking=True)

        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        cs.wait_stream(cur)
        prefetch()
        for s in range(steps):
            cur.wait_stream(cs)
            for k in order:
                D[k].copy_(S[k], non_blocking=True)
            cs.wait_stream(cur)
            if s + 1 < steps:
                prefetch()
            loss = step_fn()
            loss_host = float(loss.cpu()[0])
        b.record()
        torch.cuda.synchronize()
        piped_ms = a.elapsed_time(b)
        barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms, e2e_ms, piped_ms, exch_ms = sharding.max_over_ranks([total_ms, e2e_ms, piped_ms, exch_ms], device="cuda")
    glob_loss = sharding.global_mean_loss(loss_host, B, device="cuda")
    n_params = model.n_params
    used_ctx_comm = bool(model.use_ctx_comm)
    model.close()
    if used_ctx_comm:
        ctx.lib.dgc_comm_destroy(ctx.h)
    del model, D, P
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    ms = total_ms / steps
    h2d = 4 * sum(int(np.asarray(host[k]).size) for k in order)
    out = {"metric": "ms/train step", "ms_per_step": ms, "unit": "ms", "n_gpus": world, "steps": steps,
           "voices_per_gpu": B, "global_voices": B * world, "samples_per_s": B * world * T / (ms * 1e-3),
           "scaling": "weak", "step_mode": mode_s,
           "allreduce": {"floats": n_params, "bytes": 4 * n_params, "ms": exch_ms, "share_of_step": exch_ms / ms,
                         "via": "dgc_allreduce_sum" if used_ctx_comm else
                                ("torch.distributed" if world > 1 else "none (one rank)"),
                         "what": "CUDA events around the NCCL all-reduce between the two recordings, max over ranks"},
           "config": {"workload": "full training step (BASELINE.json configs[4])", "frames": T, "harmonics": K,
                      "control_frames": F, "controller": "MLP 2-512-512-512-165 fp32", "ir_taps": 16000,
                      "fft_sizes": list(SIZES), "optimizer": "Adam lr 1e-3", "phase_mode": PHASE["mode"],
                      "l2": "working set (>1 GB per step) exceeds L2"},
           "clocks": clocks, "gpu_launches": int(launches), "loss": glob_loss}
    if want_e2e:
        out["e2e"] = {"value": piped_ms / steps, "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8,
                      "mode": "the next step's inputs upload on a copy stream while this step runs",
                      "blocking": {"value": e2e_ms / steps, "unit": "ms"}}
    return out


def run_train(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import dgen_b200
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = dgen_b200.Context(local_rank)
    t = train_measure(ctx, args, rank, world, local_rank, args.steps, voices=args.voices if args.voices > 0 else 32)
    if rank == 0:
        line = {"metric": "ms/train step", "value": t["ms_per_step"], "unit": "ms", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": t["ms_per_step"], "higher_is_better": False, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic"}
        line.update({k: v for k, v in t.items() if k not in line})
        line["config"] = dict(t["config"], voices_per_gpu=t["voices_per_gpu"], global_voices=t["global_voices"],
                              step_mode=t["step_mode"],
                              parallelism="dp%d, NCCL all-reduce of %d gradients (%s)"
                              % (world, t["allreduce"]["floats"], t["allreduce"]["via"]))
        print(json.dumps(line))
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------------------
# the other configurations of the path (BASELINE.json configs[2], configs[3]) and the streaming kernels: one JSON
# line per kernel family with its own roofline (algorithmic bytes / CUDA-event time against the measured copy
# bandwidth).  Single GPU; these are replicas-only workloads (no exchange between voices).
# --------------------------------------------------------------------------------------------------
def measured_hbm_peak():
    """(GB/s, "measured" | "fallback"): the driver-written copy bandwidth of this pool's B200s, else 6650."""
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def run_filters(args, local_rank):
    import torch
    import dgen_b200
    torch.cuda.set_device(local_rank)
    ctx = dgen_b200.Context(local_rank)
    for line in filters_measure(ctx, args, quick=False):
        print(json.dumps(line))
    ctx.close()


def filters_measure(ctx, args, quick):
    """One dict per kernel family (the JSON lines of --workload filters).  quick: the configurations BASELINE.json
    names only (oscillator -> filter -> FFT, biquad bank forward / BPTT, partitioned convolution), fewer steps."""
    import ctypes as C
    import torch
    import dgen_b200
    from dgen_b200 import workloads as wl

    lines = []
    steps = max(3, min(args.steps, 10)) if quick else args.steps
    peak, peak_kind = measured_hbm_peak()
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()

    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    def emit(metric, workload, ms, bytes_, extra=None, l2="inputs + outputs larger than L2"):
        gbs = bytes_ / ms / 1e6
        line = {"metric": metric, "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": steps,
                "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "dtype": "f32",
                "data": "synthetic", "config": {"workload": workload, "l2": l2},
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                             "peak_kind": peak_kind, "algorithmic_bytes": bytes_}}
        if extra:
            line.update(extra)
        lines.append(line)

    scale = args.voices if args.voices > 0 else 0
    # the reference's own small case (BASELINE.json configs[0]): 64 partials -> one-pole -> buffer(1024, hop 256) -> FFT
    # magnitudes, 65536 frames.  Three launches' worth of work: launch latency, not a roofline, bounds it.
    c1 = wl.osc_filter_fft_inputs()
    fq, am = dev(c1["freq"]), dev(c1["amp"])

    def c1_chain():
        osc = ctx.osc_bank_const(fq, am, c1["T"], c1["sr"], dgen_b200.PHASE_DETERMINISTIC)
        return ctx.stft_mag(ctx.onepole_fwd(osc.view(1, -1), c1["pole"]), c1["N"], c1["hop"])

    ms = timed(c1_chain)
    emit("oscillator bank -> one-pole -> FFT", "64 partials, 65536 frames at 44.1 kHz, FFT 1024 hop 256 (BASELINE.json configs[0])",
         ms, 4.0 * (2 * 64 + c1["T"] + 256 * 513),
         {"samples_per_s": c1["T"] / (ms * 1e-3), "partial_samples_per_s": 64 * c1["T"] / (ms * 1e-3),
          "roofline_note": "launch bound at this size: three small launches and their allocations"},
         l2="working set (0.8 MB) is L2 resident: a latency figure, not a bandwidth one")
    # biquad bank: 256 lanes x 32 voices x 262144 frames (8.6 GB of lane signals)
    d = wl.biquad_bank_inputs(20260002)
    B, L, T = (scale or d["B"]), d["L"], d["T"]
    x, cut, q = dev(d["x"][:B]), dev(d["cutoff"]), dev(d["q"])
    y = ctx.biquad_fwd(x, cut, q)
    p = dgen_b200.BiquadParams(B, T, L, 1.0, 0.0)
    ms = timed(lambda: ctx.check(ctx.lib.dgc_biquad_fwd(ctx.h, C.byref(p), x.data_ptr(), cut.data_ptr(), q.data_ptr(),
                                                        None, y.data_ptr())))
    emit("biquad bank forward", "biquad bank %d lanes x %d voices x %d frames (BASELINE.json configs[2])" % (L, B, T),
         ms, 4.0 * T * (B + B * L), {"lane_samples_per_s": B * L * T / (ms * 1e-3)})
    target = ctx.biquad_fwd(x, cut * 1.05, q)
    gc, gq = torch.empty(L, device="cuda"), torch.empty(L, device="cuda")
    loss = torch.zeros(1, dtype=torch.float64, device="cuda")
    ms = timed(lambda: ctx.check(ctx.lib.dgc_biquad_mse_bwd(ctx.h, C.byref(p), x.data_ptr(), cut.data_ptr(), q.data_ptr(),
                                                            y.data_ptr(), target.data_ptr(), 1.0 / (B * T), None,
                                                            gc.data_ptr(), gq.data_ptr(), loss.data_ptr())))
    emit("biquad bank BPTT", "biquad bank %d lanes x %d voices x %d frames, MSE loss, gradients of cutoff and Q" % (L, B, T),
         ms, 4.0 * T * (2 * B * L + B), {"lane_samples_per_s": B * L * T / (ms * 1e-3)})
    del y, target, x
    torch.cuda.empty_cache()
    if not quick:
        filters_streams(ctx, args, scale, timed, emit)
    # partitioned convolution: 16 voices x 480000 frames, 96000-tap IR
    dd = wl.partconv_inputs(20260003)
    V = min(scale, dd["V"]) if scale else dd["V"]
    px, ir = dev(dd["x"][:V]), dev(dd["ir"])
    po = torch.empty_like(px)
    ms = timed(lambda: ctx.partconv(px, ir, dd["N"], dd["hop"], out=po))
    K, H, N = (dd["ir"].size + dd["hop"] - 1) // dd["hop"], (px.shape[1] + dd["hop"] - 1) // dd["hop"], dd["N"]
    emit("partitioned convolution", "partitioned convolution %d voices x %d frames, %d-tap IR (BASELINE.json configs[3])"
         % (V, px.shape[1], dd["ir"].size), ms, 4.0 * 2 * px.numel() + 8.0 * K * N,
         {"mac_gflops": 8.0 * K * N * H * V / (ms * 1e6),
          "roofline_fp32": {"bound": "fp32", "achieved": 8.0 * K * N * H * V / (ms * 1e9), "unit": "TFLOP/s",
                            "peak": 148 * FP32_LANES_PER_SM * 2 * 1.965e-3,
                            "frac": 8.0 * K * N * H * V / (ms * 1e9) / (148 * FP32_LANES_PER_SM * 2 * 1.965e-3),
                            "what": "complex multiply-accumulates of the partitions alone against 148 SMs x 128 "
                                    "lanes x 2 flops at the maximum SM clock"},
          "roofline_note": "compute bound: the partitioned multiply-accumulate does 8 K N flops per hop and voice"})
    del px, ir, po
    torch.cuda.empty_cache()
    return lines


def filters_streams(ctx, args, scale, timed, emit):
    """The streaming kernels and the ring / hold ops on long signals (not BASELINE.json configurations)."""
    import ctypes as C
    import torch
    import dgen_b200
    # one-pole and the output sanitiser on long streams
    n = 1 << 28 if not scale else 1 << 26
    xx = torch.randn(64, n // 64, device="cuda")
    yy = torch.empty_like(xx)
    ms = timed(lambda: ctx.check(ctx.lib.dgc_onepole_fwd(ctx.h, xx.data_ptr(), 64, n // 64, C.c_float(0.9), yy.data_ptr())))
    emit("one-pole scan", "one-pole y = x + 0.9 y1, 64 voices x %d frames" % (n // 64), ms, 8.0 * n,
         {"traffic_note": "x is read in both passes: 12 bytes per sample of traffic"})
    ms = timed(lambda: ctx.sanitize(xx, yy))
    emit("output sanitiser", "non-finite -> 0 over %d samples" % n, ms, 8.0 * n)
    del xx, yy
    # ring / hold ops on long tensor streams: [frames][lanes] in, the same out
    fr, ln = (1 << 20, 256) if not scale else (1 << 18, 256)
    sig = torch.randn(fr, ln, device="cuda")
    dly = (torch.rand(fr, device="cuda") * 3000.0)
    out = torch.empty_like(sig)
    ms = timed(lambda: ctx.check(ctx.lib.dgc_delay_line(ctx.h, sig.data_ptr(), dly.data_ptr(), 1, fr, ln, 4096, None, None,
                                                        out.data_ptr())))
    emit("tensor delay line", "interpolated delay lines, %d frames x %d lanes, per-frame delay time up to 3000 samples"
         % (fr, ln), ms, 8.0 * fr * ln + 4.0 * fr,
         {"traffic_note": "both taps of a lane are neighbouring rows: the second read hits L2"})
    trig = (torch.rand(fr, device="cuda") < 0.004).float()
    ms = timed(lambda: ctx.check(ctx.lib.dgc_latch(ctx.h, sig.data_ptr(), trig.data_ptr(), 1, fr, ln, None, None,
                                                   out.data_ptr())))
    emit("latch", "sample and hold, %d frames x %d lanes, shared trigger" % (fr, ln), ms, 8.0 * fr * ln + 4.0 * fr)
    del sig, dly, out, trig
    cb, ct = (64, 1 << 20) if not scale else (64, 1 << 18)
    cx = torch.randn(cb, ct, device="cuda") * 0.3
    cy = torch.empty_like(cx)
    cp = dgen_b200.CompressorParams(cb, ct, 4.0, -20.0, 6.0, 0.005, 0.05, 44100.0)
    ms = timed(lambda: ctx.check(ctx.lib.dgc_compressor(ctx.h, C.byref(cp), cx.data_ptr(), None, None, cy.data_ptr())))
    emit("compressor", "compressor, %d voices x %d frames" % (cb, ct), ms, 8.0 * cb * ct,
         {"samples_per_s": cb * ct / (ms * 1e-3),
          "roofline_note": "latency bound: the attack / release smoother is a data-dependent recurrence, one warp per voice"})
    del cx, cy


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--step-mode", default="auto", choices=["auto", "eager", "replay"],
                    help="enqueue the timed step call by call, or replay one recording of it (auto = replay)")
    ap.add_argument("--workload", default="fwd_loss", choices=["fwd_loss", "train", "filters"],
                    help="fwd_loss: synthesis forward + loss (the headline metric); train: full training step; "
                         "filters: biquad bank forward / BPTT, one-pole, sanitiser, partitioned convolution at "
                         "their full sizes, one JSON line each")
    ap.add_argument("--allreduce", default="dgc", choices=["dgc", "torch"],
                    help="training workload: gradient all-reduce through the library's communicator or torch's")
    ap.add_argument("--voices", type=int, default=0,
                    help="voices per GPU (default: the configuration's 16); other values are for profiling "
                         "captures and scaling studies, not for the headline number")
    ap.add_argument("--phase", default="fundamental", choices=["scan", "sequential", "fundamental"],
                    help="phase-anchor mode of the oscillator bank (all three are inside the 1e-4 sample tolerance "
                         "against the step-by-step recurrence; tests/test_gpu_harmonic.py)")
    ap.add_argument("--no-target", action="store_true", help="skip the 256-voice single-GPU block")
    ap.add_argument("--no-train", action="store_true", help="skip the training-step block")
    ap.add_argument("--no-other", action="store_true", help="skip the other configurations (single GPU)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.voices > 0:
        CFG["B"] = args.voices
    PHASE["mode"] = args.phase
    STEP_MODE["mode"] = "eager" if args.step_mode == "eager" else "replay"
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "train":
        run_train(args, rank, world, local_rank)
    elif args.workload == "filters":
        if rank == 0:
            run_filters(args, local_rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
