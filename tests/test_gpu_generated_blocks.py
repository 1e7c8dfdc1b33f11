"""Generated elementwise blocks through the C ABI: CUDA C as a renderer would emit it for a block that no
primitive covers is compiled in process (dgc_module_compile), launched over device memory (dgc_launch) and
checked against numpy; the image path (dgc_module_load) takes the committed PTX of the same kind of block."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import dgen_b200

pytestmark = pytest.mark.gpu
f32 = np.float32
HERE = os.path.dirname(os.path.abspath(__file__))

# what the C renderer writes as a frame loop over arena cells (Sources/DGen/Renderer/CRenderer.swift:479-1307),
# with the loop replaced by the thread index: out = tanh(a * gain + b), then the output sanitiser
BLOCK_SRC = r"""
extern "C" __global__ void dgen_block_7(float *memory, int a_off, int b_off, int out_off, float gain, int frameCount) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= frameCount) return;
  float t1 = memory[a_off + i], t2 = memory[b_off + i];
  float t3 = tanhf(t1 * gain + t2);
  unsigned bits = __float_as_uint(t3);
  memory[out_off + i] = ((bits & 0x7f800000u) == 0x7f800000u) ? 0.0f : t3;
}
extern "C" __global__ void dgen_block_8(const float *x, float *y, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = x[i] * x[i];
}
"""


@pytest.fixture(scope="module")
def ctx():
    c = dgen_b200.Context(0)
    yield c
    c.close()


def test_compiled_block_runs_over_an_arena(ctx):
    n = 100003
    rng = np.random.default_rng(1)
    a, b = rng.standard_normal(n).astype(f32), rng.standard_normal(n).astype(f32)
    a[5] = np.inf
    b[5] = -np.inf          # inf - inf -> NaN -> sanitised to 0
    mem = torch.zeros(3 * n, device="cuda")
    mem[:n] = torch.from_numpy(a).cuda()
    mem[n:2 * n] = torch.from_numpy(b).cuda()
    m = ctx.compile_module(BLOCK_SRC)
    m.launch("dgen_block_7", (n + 255) // 256, 256, [mem, C.c_int(0), C.c_int(n), C.c_int(2 * n), C.c_float(0.5), C.c_int(n)])
    ctx.sync()
    got = mem[2 * n:].cpu().numpy()
    with np.errstate(invalid="ignore"):
        want = np.tanh((a * f32(0.5) + b).astype(np.float64))
    want[~np.isfinite(want)] = 0.0
    assert np.abs(got - want).max() < 2e-6
    assert got[5] == 0.0
    # a second kernel of the same module, torch tensors as plain pointers
    x = torch.arange(1000, device="cuda", dtype=torch.float32)
    y = torch.empty_like(x)
    m.launch("dgen_block_8", 4, 256, [x, y, C.c_int(1000)])
    ctx.sync()
    assert torch.equal(y, x * x)
    m.close()


def test_errors_are_reported_not_thrown_across_the_abi(ctx):
    with pytest.raises(dgen_b200.DgenCudaError, match="does not compile"):
        ctx.compile_module("extern \"C\" __global__ void k(float *x) { x[0] = undefined_symbol; }")
    m = ctx.compile_module(BLOCK_SRC)
    with pytest.raises(dgen_b200.DgenCudaError, match="no kernel"):
        m.launch("not_there", 1, 32, [C.c_int(0)])
    m.close()
    with pytest.raises(dgen_b200.DgenCudaError, match="dgc_module_load"):
        ctx.load_module(b"this is not device code\0")
    # the context is still usable after the refused calls
    t = torch.ones(8, device="cuda")
    ctx.sanitize(t)
    ctx.sync()


def test_ptx_image_path(ctx):
    """dgc_module_load on PTX text (tests/golden/scale_block_sm100a.ptx, made from scale_block.cu by
    tests/golden/make_ptx.sh)."""
    ptx = open(os.path.join(HERE, "golden", "scale_block_sm100a.ptx")).read()
    m = ctx.load_module(ptx)
    x = torch.linspace(-1, 1, 4097, device="cuda")
    y = torch.empty_like(x)
    m.launch("dgen_scale_block", (4097 + 127) // 128, 128, [x, y, C.c_float(3.0), C.c_int(4097)])
    ctx.sync()
    assert torch.equal(y, x * 3.0)
    m.close()
