"""Two ranks x one voice produce the gradient of one rank x two voices.

The training step shards by voice: every rank differentiates the loss of its own voices with the upstream gradient
scaled by local_voices / global_voices, and ONE all-reduce (sum) of the flat gradient makes every rank hold the
gradient of the global-batch mean (the reference applies 1/B before reducing,
Sources/DGen/Emit+SpectralLoss.swift:960-961; what is exchanged is what readGradients collects,
Sources/DGenLazy/Backward.swift:132-165).  Here the two ranks run as child processes on two GPUs (NVLS off, the
exchange through dgc_allreduce_sum), and the reduced gradient and the updated parameters are compared with a
single-process run over both voices.  Needs two GPUs.
"""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

import dgen_b200
from dgen_b200 import trainer as tr, workloads as wl

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = dict(T=8192, K=24, F=40, sr=16000.0, nbands=9, taps=33)
MODEL = dict(hidden=48, ir_len=1500, conv_n=512, conv_hop=256, sizes=(512, 128, 64), seed=3)

RANK_SCRIPT = r"""
import os, sys, time
sys.path.insert(0, os.path.join(%(root)r, "dgen-audio_b200"))
sys.path.insert(0, os.path.join(%(root)r, "tests"))
import numpy as np, torch
import dgen_b200
from test_gpu_train_two_ranks import build_inputs, make_model
rank, world, path = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
torch.cuda.set_device(rank)
ctx = dgen_b200.Context(rank)
if rank == 0:
    uid = dgen_b200.comm_unique_id()
    with open(path + ".tmp", "wb") as f:
        f.write(uid)
    os.rename(path + ".tmp", path)
else:
    for _ in range(600):                      # bounded wait for rank 0 (60 s)
        if os.path.exists(path):
            break
        time.sleep(0.1)
    uid = open(path, "rb").read()
ctx.comm_init(world, rank, uid)
args = build_inputs(slice(rank, rank + 1), "cuda:%%d" %% rank)
model = make_model(ctx, 1, world)
model.use_ctx_comm = True
loss = model.step(*args)
ctx.sync()
np.savez(path + ".rank%%d.npz" %% rank, grads=model.grads.cpu().numpy(), params=model.params.cpu().numpy(),
         loss=float(loss.cpu()[0]))
ctx.close()
print("rank %%d ok" %% rank)
"""


def build_inputs(voices, device):
    """The step's inputs for the given slice of a fixed two-voice batch."""
    d = wl.harmonic_noise_inputs(31, B=2, **CFG)
    rng = np.random.default_rng(5)
    target = (rng.standard_normal((2, CFG["T"])) * 0.1).astype(np.float32)
    sl = lambda a: np.ascontiguousarray(a[:, voices])
    f0, gain = sl(d["f0"]), sl(d["gain"])
    host = [tr.features_from_controls(f0, gain), f0, sl(d["uv"]), gain, sl(d["noise_gain"]),
            np.ascontiguousarray(d["noise"][voices]), d["W"], np.ascontiguousarray(target[voices])]
    return [torch.from_numpy(np.ascontiguousarray(a)).to(device) for a in host]


def make_model(ctx, local_voices, world):
    return tr.HarmonicModel(ctx, local_voices, CFG["T"], K=CFG["K"], F=CFG["F"], sr=CFG["sr"], nbands=CFG["nbands"],
                            taps=CFG["taps"], global_voices=local_voices * world, **MODEL)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_one_voice_each_equal_one_rank_two_voices():
    ctx = dgen_b200.Context(0)
    model = make_model(ctx, 2, 1)
    loss = model.step(*build_inputs(slice(0, 2), "cuda:0"))
    ctx.sync()
    want_g, want_p, want_loss = model.grads.cpu().numpy(), model.params.cpu().numpy(), float(loss.cpu()[0])
    ctx.close()
    world = 2
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "uid")
        script = os.path.join(d, "rank.py")
        with open(script, "w") as f:
            f.write(RANK_SCRIPT % {"root": ROOT})
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        procs = [subprocess.Popen([sys.executable, script, str(r), str(world), path], env=env, stdout=subprocess.PIPE,
                                  stderr=subprocess.STDOUT, text=True) for r in range(world)]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=300)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
            outs.append(out)
        for r, (p, out) in enumerate(zip(procs, outs)):
            assert p.returncode == 0 and "rank %d ok" % r in out, out[-3000:]
        got = [np.load(path + ".rank%d.npz" % r) for r in range(world)]
    # both ranks hold the same reduced gradient and the same updated parameters
    assert np.array_equal(got[0]["grads"], got[1]["grads"])
    assert np.array_equal(got[0]["params"], got[1]["params"])
    scale = np.abs(want_g).max()
    assert np.abs(got[0]["grads"] - want_g).max() <= 1e-6 * scale + 1e-9
    # Adam's first update is -lr g / (|g| + eps): where the gradient is well above eps the updated parameters agree
    big = np.abs(want_g) > 1e-3 * scale
    assert big.sum() > 100 and np.abs(got[0]["params"] - want_p)[big].max() <= 1e-5
    # the global-batch loss is the mean of the two ranks' local means
    assert abs(0.5 * (float(got[0]["loss"]) + float(got[1]["loss"])) - want_loss) <= 1e-6 * abs(want_loss)
