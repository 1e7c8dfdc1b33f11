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
            "phase_mode": PHASE["mode"], "sharding": "voices across GPUs, no collective",
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
def cpu_arm(voices, threads, seed=SEED):
    """Times render + loss of `voices` voices of the workload on the host with `threads` threads.
    Returns (samples_per_s, seconds)."""
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
    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as ex:
        list(ex.map(one, range(voices)))
    dt = time.perf_counter() - t0
    return voices * CFG["T"] / dt, dt


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
        v, s = cpu_arm(voices, threads)
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
def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import dgen_b200
    from dgen_b200 import workloads as wl

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = dgen_b200.Context(local_rank)
    B, T, K, F, sr = CFG["B"], CFG["T"], CFG["K"], CFG["F"], CFG["sr"]
    d = wl.harmonic_noise_inputs(SEED + 100 * rank, **CFG)
    tg = wl.harmonic_noise_inputs(SEED + 100 * rank + 1, **CFG)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    D = {k: dev(v) for k, v in d.items() if isinstance(v, np.ndarray)}
    G = {k: dev(v) for k, v in tg.items() if isinstance(v, np.ndarray)}
    audio = torch.empty(B, T, device="cuda")
    loss = torch.zeros(1, dtype=torch.float64, device="cuda")
    mss = dgen_b200.mss_params(B, T, SIZES)
    import ctypes as C
    hp = dgen_b200.HarmonicParams(B, T, K, F, sr, 1.0,
                                  {"scan": dgen_b200.PHASE_SCAN, "sequential": dgen_b200.PHASE_SEQUENTIAL,
                                   "fundamental": dgen_b200.PHASE_FUNDAMENTAL}[PHASE["mode"]], 0)
    fp = dgen_b200.FirParams(B, T, F, CFG["taps"], 0.12, 1)
    lib, h = ctx.lib, ctx.h
    taps_buf = torch.empty(F, B, CFG["taps"], device="cuda")

    def stage_taps(X):
        ctx.check(lib.dgc_bands_to_taps(h, X["bands"].data_ptr(), X["W"].data_ptr(), F * B, CFG["nbands"], CFG["taps"],
                                        taps_buf.data_ptr()))

    def stage_harm(X, out):
        ctx.check(lib.dgc_harmonic_render(h, C.byref(hp), X["f0"].data_ptr(), X["uv"].data_ptr(),
                                          X["amps"].data_ptr(), X["gain"].data_ptr(), None, out.data_ptr()))

    def stage_fir(X, out):
        ctx.check(lib.dgc_fir_noise(h, C.byref(fp), X["noise"].data_ptr(), taps_buf.data_ptr(),
                                    X["noise_gain"].data_ptr(), out.data_ptr()))

    def stage_loss(pred, target):
        ctx.check(lib.dgc_mss_loss_fwd(h, C.byref(mss), pred.data_ptr(), target.data_ptr(), None, loss.data_ptr()))

    # target audio: rendered once from seed+1 (setup, untimed)
    target = torch.empty(B, T, device="cuda")
    stage_taps(G); stage_harm(G, target); stage_fir(G, target)
    torch.cuda.synchronize()

    def step_staged():
        stage_taps(D); stage_harm(D, audio); stage_fir(D, audio); stage_loss(audio, target)

    # the timed step: ONE call of the device-resident composite (harmonic and noise branch on two streams,
    # joined at the loss); the staged sequence above is kept for the per-stage times and as a cross-check
    st_dev = dgen_b200.HnStep()
    st_dev.harm, st_dev.fir, st_dev.mss, st_dev.nbands = hp, fp, mss, CFG["nbands"]
    work = torch.empty(int(lib.dgc_hn_forward_loss_work_floats(C.byref(st_dev))), device="cuda")

    def step():
        ctx.check(lib.dgc_hn_forward_loss(h, C.byref(st_dev), D["f0"].data_ptr(), D["uv"].data_ptr(),
                                          D["amps"].data_ptr(), D["gain"].data_ptr(), D["noise_gain"].data_ptr(),
                                          D["bands"].data_ptr(), D["W"].data_ptr(), D["noise"].data_ptr(),
                                          target.data_ptr(), work.data_ptr(), loss.data_ptr(), None))

    step_staged()
    loss_staged = float(loss.cpu()[0])
    step()
    loss_fused = float(loss.cpu()[0])
    if not abs(loss_fused - loss_staged) <= 1e-9 * abs(loss_staged):
        raise SystemExit("composite step and staged step disagree: %r vs %r" % (loss_fused, loss_staged))

    flush = torch.empty(512 * 1024 * 1024 // 4, device="cuda")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    # --step-mode replay (the default): the composite step is recorded once (its two streams and their join
    # included) and the timed step is one launch of that recording; eager: the call itself is timed.  Same kernels,
    # same inputs, same loss; the recording only removes the host's launch gaps between the nine kernels.
    replay = args.step_mode != "eager"
    graph, run_stream = None, torch.cuda.current_stream()
    if replay:
        run_stream = torch.cuda.Stream()
        run_stream.wait_stream(torch.cuda.current_stream())
        with ctx.on_stream(run_stream), torch.cuda.stream(run_stream):
            with ctx.record() as rec:
                step()
            graph = rec.graph
            for _ in range(3):
                graph.launch()
        torch.cuda.synchronize()
        loss_replayed = float(loss.cpu()[0])
        if loss_replayed != loss_fused:
            raise SystemExit("replayed step and direct call disagree: %r vs %r" % (loss_replayed, loss_fused))
    launches0 = ctx.launch_count()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    with ctx.on_stream(run_stream), torch.cuda.stream(run_stream):
        for s in range(args.steps):
            flush.fill_(float(s))
            evs[s][0].record()
            if replay:
                graph.launch()
            else:
                step()
            evs[s][1].record()
    barrier()
    launches = ctx.launch_count() - launches0
    total_ms = sum(a.elapsed_time(b) for a, b in evs)
    loss_val = float(loss.cpu()[0])
    if graph is not None:
        graph.close()

    # per-stage times (device events, same L2-flush discipline) for the roofline of the dominant kernel
    stages = {"bands_to_taps": lambda: stage_taps(D), "harmonic_render": lambda: stage_harm(D, audio),
              "fir_noise": lambda: stage_fir(D, audio), "mss_loss_fwd": lambda: stage_loss(audio, target)}
    stage_ms = {}
    reps = max(3, min(args.steps, 10))
    for name, fn in stages.items():
        acc = 0.0
        for r in range(reps):
            flush.fill_(float(r))
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            acc += a.elapsed_time(b)
        stage_ms[name] = acc / reps

    # end to end through the host-buffer entry point: pinned host inputs, H2D + D2H inside the timed region
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    P = {k: pin(v) for k, v in d.items() if isinstance(v, np.ndarray)}
    target_host = pin(target.cpu().numpy())
    st = dgen_b200.HnStep()
    st.harm, st.fir, st.mss, st.nbands = hp, dgen_b200.FirParams(B, T, F, CFG["taps"], 0.12, 1), mss, CFG["nbands"]

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
    clocks = sampler.stop() if rank == 0 else None
    h2d = 4 * sum(int(P[k].numel()) for k in ("f0", "uv", "amps", "gain", "noise_gain", "bands", "W", "noise")) \
        + 4 * int(target_host.numel())

    from dgen_b200 import sharding
    total_ms, e2e_ms, piped_ms = sharding.max_over_ranks([total_ms, e2e_ms, piped_ms], device="cuda")
    if rank == 0:
        samples_per_step = B * T * world
        value = samples_per_step * args.steps / (total_ms * 1e-3)
        e2e_value = samples_per_step * args.steps / (e2e_ms * 1e-3)
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        # algorithmic bytes per launch of each stage (fp32 = 4 bytes)
        alg = {"harmonic_render": 4 * (B * F * (K + 2) + B * T),
               "fir_noise": 4 * (B * T + B * F * CFG["taps"] + 2 * B * T),
               "bands_to_taps": 4 * (B * F * CFG["nbands"] + B * F * CFG["taps"]),
               "mss_loss_fwd": 2 * 4 * B * T * len(SIZES)}
        # DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per voice of each stage's kernels, from the
        # ncu --set full capture of this workload at 16 voices summarised in
        # profiles/fwd_loss_c2_kernels_full_set.md; traffic grows in proportion to the voices per launch.
        ncu_traffic_per_voice = {"harmonic_render": (21.55e6 + 4.12e6) / 16, "fir_noise": 25.02e6 / 16,
                                 "mss_loss_fwd": 8.34e6 / 16, "bands_to_taps": 4.26e6 / 16}
        dom = max(stage_ms, key=stage_ms.get)
        achieved = alg[dom] / (stage_ms[dom] * 1e-3) / 1e9
        traffic = ncu_traffic_per_voice.get(dom)
        traffic = traffic * B if traffic is not None else None
        step_bytes = sum(alg.values())
        sm_mhz = float((clocks or {}).get("sm_mhz") or 1965.0)
        sfu_peak = 148 * 16 * sm_mhz / 1e3                                    # G sin/s
        sfu_ach = B * T * K / (stage_ms["harmonic_render"] * 1e-3) / 1e9
        sfu = {"unit": "G sin/s", "achieved": sfu_ach, "peak": sfu_peak, "frac": sfu_ach / sfu_peak,
               "what": "render stage (4 kernels), one sine per voice x frame x harmonic"}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": config_json(world), "clocks": clocks,
                # throughput through the host-buffer API with two steps in flight (dgc_hn_forward_loss_host_submit /
                # _wait); "blocking" is the one-call-at-a-time form of the same API (dgc_hn_forward_loss_host)
                "e2e": {"value": samples_per_step * args.steps / (piped_ms * 1e-3), "unit": UNIT,
                        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8, "ms_per_step": piped_ms / args.steps,
                        "mode": "two steps in flight: step i+1 uploads while step i computes; every step's inputs "
                                "come from pinned host memory and its loss returns to the host inside the timed region",
                        "blocking": {"value": e2e_value, "ms_per_step": e2e_ms / args.steps,
                                     "l2": "flushed between steps"},
                        "loss": piped_loss},
                "gpu_launches": int(launches),
                "roofline": {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s",
                             "frac": achieved / peak, "traffic": traffic,
                             "peak_source": "measured" if peaks else "fallback",
                             "note": "the stage is FP32/SFU-issue bound, not HBM bound; see roofline.sfu",
                             # the bound that does apply to the oscillator bank: one sine per (voice, frame,
                             # harmonic) on the 16 SFU lanes of each SM at the sampled SM clock
                             "sfu": sfu},
                "stage_ms": stage_ms,
                "whole_step": {"algorithmic_bytes": step_bytes,
                               "achieved_gbs": step_bytes / (total_ms / args.steps * 1e-3) / 1e9},
                "loss": loss_val, "e2e_loss": e2e_loss}
        if not args.no_cpu and world == 1:
            v, secs = cpu_arm(4, 1)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": 1, "kind": "port",
                                    "sample": "4 voices x %d frames, render + 6-scale loss, single thread (%.1f s); "
                                              "CPU restatement of the reference's single-threaded C backend"
                                              % (T, secs)}
        print(json.dumps(line))
    ctx.close()
    if world > 1:
        dist.destroy_process_group()



# --------------------------------------------------------------------------------------------------
# training-step workload (BASELINE.json configs[4]): 32 voices per GPU, controller MLP 2-512-512-512-165,
# harmonic+noise synthesis, 1 s learnable IR reverb, multi-scale spectral loss, backward, gradient
# all-reduce (NCCL) and one Adam step
# --------------------------------------------------------------------------------------------------
def run_train(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import dgen_b200
    from dgen_b200 import sharding, trainer as tr, workloads as wl

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = dgen_b200.Context(local_rank)
    B = args.voices if args.voices > 0 else 32
    T, K, F, sr, NB, NT = CFG["T"], CFG["K"], CFG["F"], CFG["sr"], CFG["nbands"], CFG["taps"]
    d = wl.harmonic_noise_inputs(SEED + 100 * rank, B=B, T=T, K=K, F=F, sr=sr, nbands=NB, taps=NT)
    tg = wl.harmonic_noise_inputs(SEED + 100 * rank + 1, B=B, T=T, K=K, F=F, sr=sr, nbands=NB, taps=NT)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    model = tr.HarmonicModel(ctx, B, T, K=K, F=F, sr=sr, nbands=NB, taps=NT, hidden=512, ir_len=16000, conv_n=2048,
                             conv_hop=1024, sizes=SIZES, seed=7, global_voices=B * world, counted_adam=True)
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
    D = {k: dev(host[k]) for k in order}
    dargs = [D[k] for k in order]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        model.step(*dargs)
    # step mode: "replay" records the step once (both streams, Adam; with several ranks the gradient exchange stays
    # between two recordings) and launches the recording per step; "eager" enqueues it call by call.
    mode = args.step_mode if args.step_mode != "auto" else "replay"
    if mode == "replay":
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
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    for s in range(args.steps):
        evs[s][0].record()
        loss = step_fn()
        evs[s][1].record()
    barrier()
    launches = ctx.launch_count() - l0
    total_ms = sum(a.elapsed_time(b) for a, b in evs)
    # end to end: the step's inputs come from pinned host memory, the loss goes back to the host
    e2e_ms = 0.0
    for s in range(args.steps):
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
    # the same with the NEXT step's inputs crossing PCIe (copy stream, device staging) while this step runs; at the
    # start of a step the staged inputs move into the step's static buffers device to device.  Every step still
    # takes its inputs from pinned host memory and returns its loss to the host inside the timed region.
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
    for s in range(args.steps):
        cur.wait_stream(cs)
        for k in order:
            D[k].copy_(S[k], non_blocking=True)
        cs.wait_stream(cur)
        if s + 1 < args.steps:
            prefetch()
        loss = step_fn()
        loss_host = float(loss.cpu()[0])
    b.record()
    torch.cuda.synchronize()
    piped_ms = a.elapsed_time(b)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms, e2e_ms, piped_ms = sharding.max_over_ranks([total_ms, e2e_ms, piped_ms], device="cuda")
    glob_loss = sharding.global_mean_loss(loss_host, B, device="cuda")
    if rank == 0:
        ms = total_ms / args.steps
        h2d = 4 * sum(int(P[k].numel()) for k in order)
        line = {"metric": "ms/train step", "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "full training step (BASELINE.json configs[4])", "voices_per_gpu": B,
                           "global_voices": B * world, "frames": T, "harmonics": K, "control_frames": F,
                           "controller": "MLP 2-512-512-512-165 fp32", "ir_taps": 16000, "fft_sizes": list(SIZES),
                           "optimizer": "Adam lr 1e-3", "step_mode": mode, "parallelism": "dp%d, NCCL all-reduce of %d gradients (%s)"
                           % (world, model.n_params,
                              "dgc_allreduce_sum" if model.use_ctx_comm else "torch.distributed"), "l2": "working set (>1 GB per step) exceeds L2"},
                "samples_per_s": B * world * T / (ms * 1e-3), "clocks": clocks,
                "e2e": {"value": piped_ms / args.steps, "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8,
                        "mode": "the next step's inputs upload on a copy stream while this step runs",
                        "blocking": {"value": e2e_ms / args.steps, "unit": "ms"}},
                "gpu_launches": int(launches), "loss": glob_loss}
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
    import ctypes as C
    import torch
    import dgen_b200
    from dgen_b200 import workloads as wl

    torch.cuda.set_device(local_rank)
    ctx = dgen_b200.Context(local_rank)
    peak, peak_kind = measured_hbm_peak()
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()

    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.steps

    def emit(metric, workload, ms, bytes_, extra=None, l2="inputs + outputs larger than L2"):
        gbs = bytes_ / ms / 1e6
        line = {"metric": metric, "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "dtype": "f32",
                "data": "synthetic", "config": {"workload": workload, "l2": l2},
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                             "peak_kind": peak_kind, "algorithmic_bytes": bytes_}}
        if extra:
            line.update(extra)
        print(json.dumps(line))

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
    del y, target
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
          "roofline_note": "compute bound: the partitioned multiply-accumulate does 8 K N flops per hop and voice"})
    ctx.close()


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
    ap.add_argument("--phase", default="scan", choices=["scan", "sequential", "fundamental"],
                    help="phase-anchor mode of the oscillator bank")
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
