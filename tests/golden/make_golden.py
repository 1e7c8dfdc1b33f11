"""Regenerates tests/golden/ref_artefacts.npz from the reference's own generated C artefacts.

Run in a container that has the reference tree:
    sh oracle/build_ref.sh <reference checkout> && python tests/golden/make_golden.py
It executes oracle/_ref/*.so (the reference's toolchain/generated/hermetic/*.c, compiled as they
lie) with the memory initialisation, process context (48 kHz) and input signal of the reference's
harness (toolchain/harness/toolchain_harness.c:153-181, 270-278) and stores the outputs, so the
oracle can be checked against the reference's emitted code on machines without the reference.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402

BLOCKS, FRAMES, SR = 128, 64, 48000.0


def harness_input(n):
    """toolchain_harness.c:270-278: 0.25*sinf(2*pi*330*frame/48000) + 0.5 at frame 0 (Float math)."""
    f = np.arange(n, dtype=np.float32)
    arg = (np.float32(2.0) * np.float32(3.14159265358979323846) * np.float32(330.0)) * f / np.float32(48000.0)
    x = (np.float32(0.25) * np.sin(arg.astype(np.float32), dtype=np.float32)).astype(np.float32)
    x[0] += np.float32(0.5)
    return x


HANN16 = np.array([0.0, 0.038060218, 0.14644659, 0.3086583, 0.49999997, 0.69134164, 0.8535534, 0.96193975,
                   1.0, 0.9619398, 0.85355353, 0.69134176, 0.5, 0.30865842, 0.14644668, 0.038060308], np.float32)


# toolchain/harness/toolchain_harness.c:106-112 (kWavetable), copied to memory[0..31] as it stands; the generated
# code reads the two waves as memory[16 * wave + sample]
WAVETABLE = np.array([0.0, 0.0, 0.38268343, 0.125, 0.70710677, 0.25, 0.9238795, 0.375, 1.0, 0.5, 0.9238795, 0.625,
                      0.70710677, 0.75, 0.38268343, 0.875, 0.0, -1.0, -0.38268343, -0.875, -0.70710677, -0.75,
                      -0.9238795, -0.625, -1.0, -0.5, -0.9238795, -0.375, -0.70710677, -0.25, -0.38268343, -0.125],
                     np.float32)


def memory_for(kind):
    if kind == "scalar-synth":
        m = np.zeros(1024, np.float32)
        m[:3] = [220.0, 1.75, 0.2]
    elif kind == "feedback-delay-effect":
        m = np.zeros(88005, np.float32)
        m[:3] = [37.0, 0.35, 0.4]
    elif kind == "wavetable-instrument":
        m = np.zeros(1024, np.float32)
        m[:32] = WAVETABLE
        m[32:35] = [110.0, 0.35, 0.2]
    elif kind == "spectral-effect":
        m = np.zeros(3700, np.float32)
        m[0], m[8], m[16], m[24] = 1.0, 0.35, 0.15, 0.05
        m[32:48] = HANN16
        m[48:64], m[64:80], m[80:96], m[96:112] = 1.0, 0.35, 0.15, 0.05
    else:
        raise ValueError(kind)
    return m


def main():
    n = BLOCKS * FRAMES
    x = harness_input(n)
    out = {"input": x}
    m = memory_for("scalar-synth")
    out["scalar_synth"] = orc.ref_run("scalar-synth", m, None, BLOCKS, FRAMES, SR)
    out["scalar_synth_final_phase"] = m[3:4].copy()
    m = memory_for("feedback-delay-effect")
    out["feedback_delay"] = orc.ref_run("feedback-delay-effect", m, x, BLOCKS, FRAMES, SR)
    m = memory_for("spectral-effect")
    out["spectral_effect"] = orc.ref_run("spectral-effect", m, x, BLOCKS, FRAMES, SR)
    m = memory_for("wavetable-instrument")
    out["wavetable_instrument"] = orc.ref_run("wavetable-instrument", m, None, BLOCKS, FRAMES, SR)
    out["wavetable_memory"] = memory_for("wavetable-instrument")[:36].copy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_artefacts.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
