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
