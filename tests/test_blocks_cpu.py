"""The block emitter is a pure host function: its CUDA C follows the scalar expressions of the reference's C
renderer (Sources/DGen/Renderer/CRenderer.swift:484-1040)."""
import pytest

import dgen_b200


def body(ops):
    src = dgen_b200.block_source(ops, "k")
    assert src.startswith("// generated block")
    assert 'extern "C" __global__ void k(float *memory, int count)' in src
    return [l.strip() for l in src.splitlines()[4:-1]]


def test_constant_specialisations_match_the_reference_renderer():
    lines = body([("LOAD", 16), ("CONST", 0, 0, 0, 1.0), ("MOD", 0, 1), ("CONST", 0, 0, 0, 0.25), ("MOD", 0, 3),
                  ("DIV", 0, 3), ("CONST", 0, 0, 0, 3.0), ("POW", 0, 6), ("POW", 6, 0), ("SIGN", 0), ("XOR", 0, 1)])
    assert lines[0] == "float t0 = memory[16 + i];"
    assert lines[2] == "float t2 = (t0 - floorf(t0));"                        # mod 1: a - floor(a)
    assert lines[4] == "float t4 = (t0 - floorf(t0 / 0.25f) * 0.25f);"        # mod c: a - floor(a / c) * c
    assert lines[5] == "float t5 = (t0 / 0.25f);"
    assert lines[7] == "float t7 = (t0 * t0 * t0);"                           # pow 3
    assert lines[8] == "float t8 = expf((t0) * logf(3.0f));"                  # constant base
    assert lines[9] == "float t9 = (t0 == 0.0f) ? 0.0f : copysignf(1.0f, t0);"
    assert lines[10] == "float t10 = ((((t0 != 0.0f) ^ (t1 != 0.0f))) ? 1.0f : 0.0f);"


def test_output_sanitises_and_store_does_not():
    lines = body([("LOAD_SCALAR", 3), ("STORE", 100, 0), ("OUTPUT", 200, 0)])
    assert lines[0] == "float t0 = memory[3];"
    assert lines[1] == "memory[100 + i] = t0;"
    assert "0x7f800000u" in lines[3] and lines[4] == "memory[200 + i] = t2;"


def test_operands_must_precede_their_use():
    with pytest.raises(dgen_b200.DgenCudaError):
        dgen_b200.block_source([("ADD", 0, 1)])
    with pytest.raises(dgen_b200.DgenCudaError):
        dgen_b200.block_source([("CONST", 0, 0, 0, 1.0), ("SIN", 1)])
    with pytest.raises(dgen_b200.DgenCudaError):
        dgen_b200.block_source([(999, 0, 0, 0, 0.0)])


def test_sequential_form_keeps_state_cells_in_registers_across_the_frame_loop():
    """History feedback (Sources/DGen/Emit+State.swift:150-224): y = x * gain[lane] + 0.9 * y1 per lane."""
    ops = [("LOAD", 0), ("LOAD_LANE", 1000), ("MUL", 0, 1), ("HISTORY_READ", 2000), ("CONST", 0, 0, 0, 0.9),
           ("MUL", 3, 4), ("ADD", 2, 5), ("HISTORY_WRITE", 2000, 6), ("STORE_FRAME_LANE", 3000, 7)]
    src = dgen_b200.block_source(ops, "k", sequential=True)
    lines = [l.strip() for l in src.splitlines()]
    assert 'extern "C" __global__ void k(float *memory, int frames, int lanes) {' in lines
    assert lines.index("float s2000 = memory[2000 + e];") < lines.index("for (int i = 0; i < frames; ++i) {")
    assert "float t3 = s2000;" in lines and "s2000 = t6;" in lines
    assert "memory[3000 + (size_t)i * lanes + e] = t7;" in lines
    assert lines.index("memory[2000 + e] = s2000;") > lines.index("memory[3000 + (size_t)i * lanes + e] = t7;")


def test_phasor_and_latch_render_the_reference_state_updates():
    ops = [("LOAD_LANE", 10), ("CONST", 0, 0, 0, 0.0), ("PHASOR", 500, 0, 1, 44100.0), ("LATCH", 600, 2, 0)]
    lines = [l.strip() for l in dgen_b200.block_source(ops, "k", sequential=True).splitlines()]
    assert "float t2 = s500;" in lines                                  # output = phase before the update
    assert "float n2 = s500 + t0 / 44100.0f;" in lines
    assert "n2 = n2 - floorf(n2);" in lines and "if (n2 >= 1.0f) n2 -= 1.0f;" in lines
    assert "s500 = t1 > 0.0f ? 0.0f : n2;" in lines
    assert "if (t0 > 0.0f) s600 = t2;" in lines and "float t3 = s600;" in lines


def test_state_ops_need_the_sequential_form():
    with pytest.raises(dgen_b200.DgenCudaError):
        dgen_b200.block_source([("HISTORY_READ", 5)])
    with pytest.raises(dgen_b200.DgenCudaError):
        dgen_b200.block_source([("LOAD_LANE", 5)])


def test_accum_and_noise_render_the_reference_state_updates():
    ops = [("CONST", 0, 0, 0, 0.25), ("CONST", 0, 0, 0, 0.0), ("ACCUM", 100, 0, 1, 3.0), ("NOISE", 200)]
    lines = [l.strip() for l in dgen_b200.block_source(ops, "k", sequential=True).splitlines()]
    assert "float t2 = s100;" in lines and "n2 = n2 - floorf(n2 / 3.0f) * 3.0f;" in lines
    assert "if (n2 >= 3.0f) n2 -= 3.0f;" in lines
    assert "x3 ^= x3 << 13; x3 ^= x3 >> 17; x3 ^= x3 << 5;" in lines and "if (x3 == 0u) x3 = 1u;" in lines
    assert "float t3 = (float)x3 / 4294967296.0f;" in lines and "memory[200 + e] = s200;" in lines
