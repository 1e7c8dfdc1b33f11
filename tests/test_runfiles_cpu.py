"""Run-directory formats (WAV, checkpoints, training log) against the layouts the reference writes and parses
(Sources/DGenLazy/AudioFile.swift, Examples/HarmonicE2E/Checkpoint.swift, Examples/HarmonicE2E/Trainer.swift)."""
import json
import os
import struct

import numpy as np
import pytest

from dgen_b200 import runfiles as rf

f32 = np.float32


def test_wav_save_layout_and_round_trip(tmp_path):
    x = np.random.default_rng(0).standard_normal(1001).astype(f32)
    p = str(tmp_path / "a.wav")
    rf.wav_save(p, x, 16000)
    raw = open(p, "rb").read()
    assert len(raw) == 44 + 4 * 1001
    assert raw[:4] == b"RIFF" and struct.unpack_from("<I", raw, 4)[0] == 36 + 4 * 1001 and raw[8:16] == b"WAVEfmt "
    assert struct.unpack_from("<IHHIIHH", raw, 16) == (16, 3, 1, 16000, 64000, 4, 32)   # IEEE float, mono, 32 bit
    assert raw[36:40] == b"data" and struct.unpack_from("<I", raw, 40)[0] == 4 * 1001
    y, sr = rf.wav_load(p)
    assert sr == 16000.0 and np.array_equal(y.view(np.uint32), x.view(np.uint32))


def pcm_file(fmt, channels, bits, payload, extra=b"", declared=None):
    fmtc = struct.pack("<HHIIHH", fmt, channels, 44100, 44100 * channels * bits // 8, channels * bits // 8, bits)
    body = b"WAVE" + b"LIST" + struct.pack("<I", 3) + b"abc\0" + b"fmt " + struct.pack("<I", 16) + fmtc + extra \
        + b"data" + struct.pack("<I", len(payload) if declared is None else declared) + payload
    return b"RIFF" + struct.pack("<I", len(body)) + body


def test_wav_parse_pcm16_stereo_after_an_odd_sized_chunk():
    frames = np.array([[1000, -1000], [32767, -32768], [0, 2]], dtype="<i2")
    x, sr = rf.wav_parse(pcm_file(1, 2, 16, frames.tobytes()), mono=True)
    want = (frames.astype(f32) / f32(32768.0)).sum(1, dtype=f32) * f32(0.5)
    assert sr == 44100.0 and np.array_equal(x, want)
    xi, _ = rf.wav_parse(pcm_file(1, 2, 16, frames.tobytes()), mono=False)
    assert np.array_equal(xi, (frames.astype(f32) / f32(32768.0)).reshape(-1))


def test_wav_parse_pcm24_and_clamped_sizes():
    vals = [0x000001, 0x7FFFFF, 0x800000, 0xFFFFFF]
    payload = b"".join(struct.pack("<I", v)[:3] for v in vals)
    x, _ = rf.wav_parse(pcm_file(1, 1, 24, payload))
    assert np.array_equal(x, np.array([1, 8388607, -8388608, -1], f32) / f32(8388608.0))
    # a streaming encoder's placeholder size and a trailing incomplete frame
    y, _ = rf.wav_parse(pcm_file(3, 1, 32, np.array([0.5, -0.25], "<f4").tobytes() + b"\x01\x02", declared=0xFFFFFFFF))
    assert np.array_equal(y, np.array([0.5, -0.25], f32))


@pytest.mark.parametrize("blob,msg", [(b"RIFF" + b"\0" * 10, "too small"), (b"JUNK" + b"\0" * 60, "RIFF/WAVE"),
                                      (pcm_file(2, 1, 16, b"\0" * 8), "audioFormat 2"),
                                      (pcm_file(1, 1, 8, b"\0" * 8), "PCM 8-bit"), (pcm_file(3, 1, 32, b"\0\0"), "no complete")])
def test_wav_errors(blob, msg):
    with pytest.raises(rf.WavError, match=msg):
        rf.wav_parse(blob)


def test_checkpoint_files_and_parameter_names(tmp_path):
    run = rf.RunDirectories(str(tmp_path / "run"))
    assert all(os.path.isdir(d) for d in (run.checkpoints, run.renders, run.logs))
    K, H, NB = 5, 4, 3
    layout, off = [], 0
    for i, (a, b) in enumerate([(2, H), (H, H), (H, K + NB)]):
        layout += [("W%d" % i, off, (a, b)), ("b%d" % i, off + a * b, (b,))]
        off += a * b + b
    layout.append(("ir", off, (7,)))
    off += 7
    flat = np.arange(off, dtype=f32) / f32(8)
    snaps = rf.snapshots_from_flat(layout, flat, K)
    assert [n for n, _, _ in snaps] == ["W1", "b1", "W2", "b2", "W_harm", "b_harm", "W_bands", "b_bands", "ir"]
    p = rf.write_model_state(run.checkpoints, 12, snaps)
    assert os.path.basename(p) == "model_step_00000012.json"
    doc = json.load(open(p))
    assert list(doc.keys()) == ["createdAtUTC", "params", "step"] and doc["step"] == 12     # sorted keys
    assert list(doc["params"][0].keys()) == ["data", "name", "shape"] and doc["params"][4]["shape"] == [H, K]
    assert open(p).read().startswith("{\n")                                                # pretty printed
    step, named = rf.read_model_state(p)
    assert step == 12 and np.array_equal(rf.flat_from_snapshots(layout, named, K), flat)
    assert os.path.basename(rf.write_best_model_state(run.checkpoints, 3, snaps)) == "model_best.json"
    # a checkpoint with the REFERENCE decoder's heads (W_gain, W_noise [hidden, 1], W_noiseFilter) is refused by name,
    # a tensor of the wrong shape is refused too -- never concatenated into the wrong head
    import pytest
    ref_like = dict(named)
    ref_like.pop("W_bands"); ref_like.pop("b_bands")
    ref_like.update(W_gain=np.zeros((H, 1), f32), b_gain=np.zeros((1, 1), f32), W_noise=np.zeros((H, 1), f32),
                    b_noise=np.zeros((1, 1), f32), W_noiseFilter=np.zeros((H, NB), f32), b_noiseFilter=np.zeros((1, NB), f32))
    with pytest.raises(ValueError, match="W_bands"):
        rf.flat_from_snapshots(layout, ref_like, K)
    bad = dict(named)
    bad["W_harm"] = np.zeros((K, H), f32)                 # transposed: same size, wrong shape
    with pytest.raises(ValueError, match="shape"):
        rf.flat_from_snapshots(layout, bad, K)


def test_train_log_files(tmp_path):
    log = rf.TrainLog()
    for s, l in enumerate([3.0, 2.5, 2.75]):
        log.append(s, l, "c%d" % s)
    log.write(str(tmp_path), batch_size=32)
    lines = open(tmp_path / "train_log.csv").read().split("\n")
    assert lines[0] == "step,loss,chunk_ids" and lines[2] == "1,2.5,c1" and len(lines) == 4
    summ = json.load(open(tmp_path / "train_summary.json"))
    assert summ == {"steps": "3", "minStep": "1", "minLoss": "2.5", "firstLoss": "3.0", "finalLoss": "2.75",
                    "batchSize": "32"}
