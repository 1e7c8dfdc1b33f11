"""Gradient exchange through the C ABI (dgc_comm_init / dgc_allreduce_sum): one process per GPU, the id travels
through a file.  Needs two GPUs; on a single-GPU box only the world-of-one behaviour is checked."""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

import dgen_b200

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

RANK_SCRIPT = r"""
import os, sys, time
sys.path.insert(0, os.path.join(%(root)r, "dgen-audio_b200"))
import torch
import dgen_b200
rank, world, path = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
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
assert len(uid) == 128
ctx.comm_init(world, rank, uid)
n = 627493                                    # the flat gradient of the training configuration
buf = torch.full((n,), float(rank + 1), device="cuda:%%d" %% rank)
buf[rank] += 0.5
for _ in range(3):
    ctx.allreduce_sum_(buf)
ctx.sync()
# three sums in a row: x_r -> S = sum_r x_r -> W * S -> W^2 * S
tot = torch.full((n,), float(world * (world + 1) // 2), device=buf.device)
for r in range(world):
    tot[r] += 0.5
assert torch.equal(buf, tot * world * world), (buf[:4], tot[:4])
ctx.close()
print("rank %%d ok" %% rank)
"""


def test_world_of_one_is_the_identity():
    ctx = dgen_b200.Context(0)
    g = torch.arange(1000, device="cuda", dtype=torch.float32)
    ctx.allreduce_sum_(g)
    ctx.sync()
    assert torch.equal(g, torch.arange(1000, device="cuda", dtype=torch.float32))
    ctx.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_allreduce_sum_over_two_ranks():
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
                out, _ = p.communicate(timeout=240)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
            outs.append(out)
        for r, (p, out) in enumerate(zip(procs, outs)):
            assert p.returncode == 0 and "rank %d ok" % r in out, out[-2000:]
