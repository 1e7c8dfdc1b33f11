"""On-disk formats of a HarmonicE2E-style run, so that a run made with this library and one made with the
reference's example trainer are interchangeable: WAV files, model checkpoints, the training log.

* WAV (Sources/DGenLazy/AudioFile.swift:56-98 save, :101-262 parse): save writes 32-bit IEEE-float mono with a
  16-byte fmt chunk; load walks the chunks (word-aligned), accepts PCM 16 / 24 bit and float 32 bit, clamps the
  declared data size to what the file holds, drops an incomplete last frame and mixes to mono as
  (sum over channels) * (1 / channels) in single precision.
* Checkpoints (Examples/HarmonicE2E/Checkpoint.swift:3-44): `model_step_%08d.json` / `model_best.json`,
  pretty-printed JSON with sorted keys: {"createdAtUTC", "params": [{"data", "name", "shape"}], "step"}.
* Run directory (Examples/HarmonicE2E/Trainer.swift:5-24): <root>/checkpoints, <root>/renders, <root>/logs;
  `logs/train_log.csv` with header `step,loss,chunk_ids`, `logs/train_summary.json` with string values.
"""
import datetime
import json
import os
import struct

import numpy as np


class WavError(ValueError):
    pass


def wav_save(path, samples, sample_rate):
    """32-bit float mono WAV, byte for byte the reference's header layout."""
    x = np.ascontiguousarray(samples, dtype="<f4").reshape(-1)
    sr = int(sample_rate)
    data_bytes = x.size * 4
    hdr = b"RIFF" + struct.pack("<I", 36 + data_bytes) + b"WAVE" + b"fmt " + struct.pack(
        "<IHHIIHH", 16, 3, 1, sr, sr * 4, 4, 32) + b"data" + struct.pack("<I", data_bytes)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(hdr)
        f.write(x.tobytes())
    os.replace(tmp, path)   # the reference writes atomically


def wav_parse(data, mono=True):
    """bytes -> (float32 samples, sample rate).  Multi-channel data stays interleaved when mono is False."""
    if len(data) < 44:
        raise WavError("File too small for WAV header")
    if data[0:4] != b"RIFF" or data[8:12] != b"WAVE":
        raise WavError("Missing RIFF/WAVE header")
    fmt = None
    data_off = data_size = None
    off = 12
    while off + 8 <= len(data):
        cid = data[off:off + 4]
        size = struct.unpack_from("<I", data, off + 4)[0]
        start = off + 8
        if cid == b"fmt ":
            if size < 16 or start + 16 > len(data):
                raise WavError("fmt chunk truncated")
            audio_format, channels, rate = struct.unpack_from("<HHI", data, start)
            bits = struct.unpack_from("<H", data, start + 14)[0]
            fmt = (audio_format, channels, rate, bits)
        elif cid == b"data":
            data_off, data_size = start, size
        off = start + size + (size & 1)
        if fmt is not None and data_off is not None:
            break
    if fmt is None:
        raise WavError("No fmt chunk found")
    if data_off is None:
        raise WavError("No data chunk found")
    audio_format, channels, rate, bits = fmt
    if channels < 1:
        raise WavError("Invalid channel count")
    if data_off >= len(data):
        raise WavError("data chunk offset past end of file")
    data_size = min(data_size, len(data) - data_off)   # placeholder sizes of streaming encoders, truncated files

    def usable(bytes_per_sample):
        frame = channels * bytes_per_sample
        n = (data_size // frame) * frame
        if n <= 0:
            raise WavError("data chunk has no complete frames")
        return n

    if audio_format == 1:
        if bits == 16:
            n = usable(2)
            x = np.frombuffer(data, dtype="<i2", count=n // 2, offset=data_off).astype(np.float32) / np.float32(32768.0)
        elif bits == 24:
            n = usable(3)
            b = np.frombuffer(data, dtype=np.uint8, count=n, offset=data_off).reshape(-1, 3).astype(np.int32)
            raw = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
            raw = np.where(raw & 0x800000, raw - (1 << 24), raw)
            x = raw.astype(np.float32) / np.float32(8388608.0)
        else:
            raise WavError("PCM %d-bit (only 16-bit and 24-bit supported)" % bits)
    elif audio_format == 3:
        if bits != 32:
            raise WavError("Float %d-bit (only 32-bit supported)" % bits)
        n = usable(4)
        x = np.frombuffer(data, dtype="<f4", count=n // 4, offset=data_off).astype(np.float32)
    else:
        raise WavError("audioFormat %d (only PCM int16 and float32 supported)" % audio_format)
    if mono and channels > 1:
        fr = x.reshape(-1, channels)
        acc = np.zeros(fr.shape[0], np.float32)
        for ch in range(channels):          # channel order, single precision, as the reference sums
            acc = acc + fr[:, ch]
        x = acc * np.float32(1.0 / channels)
    return np.ascontiguousarray(x), float(rate)


def wav_load(path, mono=True):
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    with open(path, "rb") as f:
        return wav_parse(f.read(), mono)


# ---- run directory ------------------------------------------------------------------------------------------
class RunDirectories:
    def __init__(self, root):
        self.root = root
        self.checkpoints = os.path.join(root, "checkpoints")
        self.renders = os.path.join(root, "renders")
        self.logs = os.path.join(root, "logs")
        for d in (self.checkpoints, self.renders, self.logs):
            os.makedirs(d, exist_ok=True)


def _checkpoint_json(step, params):
    doc = {"step": int(step),
           "createdAtUTC": datetime.datetime.now(datetime.timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ"),
           "params": [{"name": str(n), "shape": [int(s) for s in shape],
                       "data": [float(v) for v in np.asarray(data, np.float32).reshape(-1)]}
                      for n, shape, data in params]}
    return json.dumps(doc, indent=2, sort_keys=True)


def write_model_state(checkpoints_dir, step, params):
    """params: list of (name, shape, data).  Returns the path written."""
    path = os.path.join(checkpoints_dir, "model_step_%08d.json" % step)
    with open(path, "w") as f:
        f.write(_checkpoint_json(step, params))
    return path


def write_best_model_state(checkpoints_dir, step, params):
    path = os.path.join(checkpoints_dir, "model_best.json")
    with open(path, "w") as f:
        f.write(_checkpoint_json(step, params))
    return path


def read_model_state(path):
    """-> (step, {name: float32 array of the stored shape})."""
    with open(path) as f:
        doc = json.load(f)
    out = {}
    for p in doc["params"]:
        a = np.asarray(p["data"], np.float32)
        if int(np.prod(p["shape"])) != a.size:
            raise ValueError("checkpoint tensor %s: %d values for shape %s" % (p["name"], a.size, p["shape"]))
        out[p["name"]] = a.reshape(p["shape"])
    return int(doc["step"]), out


class TrainLog:
    """logs/train_log.csv (header step,loss,chunk_ids) and logs/train_summary.json."""

    def __init__(self):
        self.lines = ["step,loss,chunk_ids"]
        self.losses = []

    def append(self, step, loss, chunk_ids=""):
        self.lines.append("%d,%s,%s" % (step, repr(float(loss)), chunk_ids))
        self.losses.append((int(step), float(loss)))

    def write(self, logs_dir, batch_size=None):
        with open(os.path.join(logs_dir, "train_log.csv"), "w") as f:
            f.write("\n".join(self.lines))
        if self.losses:
            min_step, min_loss = min(self.losses, key=lambda t: t[1])
            summary = {"steps": str(len(self.losses)), "minStep": str(min_step), "minLoss": str(min_loss),
                       "firstLoss": str(self.losses[0][1]), "finalLoss": str(self.losses[-1][1])}
            if batch_size is not None:
                summary["batchSize"] = str(batch_size)
            with open(os.path.join(logs_dir, "train_summary.json"), "w") as f:
                f.write(json.dumps(summary, indent=2, sort_keys=True))


# ---- flat parameter vector <-> named snapshots ----------------------------------------------------------------
def snapshots_from_flat(layout, flat, K):
    """layout: [(name, offset, shape)] of the flat parameter vector with W0.. / b0.. trunk + head and "ir".
    Only the CONTAINER follows the reference (the JSON layout and file names of Examples/HarmonicE2E/Checkpoint.swift,
    trunk layers named W1/b1 .. 1-based, the harmonic head W_harm / b_harm as in Examples/HarmonicE2E/Model.swift:122-137);
    the parameter SET is this model's own.  The reference decoder has four heads -- W_harm, W_gain, W_noise (a
    [hidden, 1] noise-gain head) and W_noiseFilter (FIR taps through tanh and an L1 normalisation) -- while the
    benchmark configuration's controller maps to harmonic amplitudes and 65 noise-band magnitudes only.  The band
    head is therefore stored as W_bands / b_bands (the rest of the head's columns) so that it cannot be mistaken
    for the reference's W_noise, and the learnable impulse response as "ir".  A checkpoint written by the
    reference trainer does not load into this model, and the loader says so by name."""
    flat = np.asarray(flat, np.float32)
    t = {n: flat[o:o + int(np.prod(s))].reshape(s) for n, o, s in layout}
    n_lin = sum(1 for n in t if n.startswith("W"))
    out = []
    for i in range(n_lin - 1):
        out.append(("W%d" % (i + 1), t["W%d" % i].shape, t["W%d" % i]))
        out.append(("b%d" % (i + 1), t["b%d" % i].shape, t["b%d" % i]))
    Wh, bh = t["W%d" % (n_lin - 1)], t["b%d" % (n_lin - 1)]
    out += [("W_harm", Wh[:, :K].shape, Wh[:, :K]), ("b_harm", (K,), bh[:K]),
            ("W_bands", Wh[:, K:].shape, Wh[:, K:]), ("b_bands", (bh.size - K,), bh[K:])]
    if "ir" in t:
        out.append(("ir", t["ir"].shape, t["ir"]))
    return out


def flat_from_snapshots(layout, named, K):
    """Inverse of snapshots_from_flat: named = {name: array} as read_model_state returns.  Raises ValueError on a
    missing tensor, on a tensor the model does not have, and on any shape that differs from the model's."""
    expect = {n: tuple(int(v) for v in s) for n, s, _ in
              snapshots_from_flat(layout, np.zeros(max(o + int(np.prod(s)) for _, o, s in layout), np.float32), K)}
    missing = sorted(set(expect) - set(named))
    extra = sorted(set(named) - set(expect))
    if missing or extra:
        raise ValueError("checkpoint does not hold this model's parameter set: missing %s, unexpected %s"
                         % (missing or "none", extra or "none"))
    for n, shp in expect.items():
        got = tuple(int(v) for v in np.asarray(named[n]).shape)
        if got != shp and not (len(shp) == 1 and got == (1,) + shp):   # biases may be stored as [1, n]
            raise ValueError("checkpoint tensor %s has shape %s, the model needs %s" % (n, got, shp))
    total = max(o + int(np.prod(s)) for _, o, s in layout)
    flat = np.zeros(total, np.float32)
    n_lin = sum(1 for n, _, _ in layout if n.startswith("W"))
    for n, o, s in layout:
        cnt = int(np.prod(s))
        if n == "ir":
            src = named["ir"]
        elif n[0] in "Wb" and int(n[1:]) < n_lin - 1:
            src = named["%s%d" % (n[0], int(n[1:]) + 1)]
        elif n[0] == "W":
            src = np.concatenate([named["W_harm"], named["W_bands"]], axis=1)
        else:
            src = np.concatenate([np.ravel(named["b_harm"]), np.ravel(named["b_bands"])])
        src = np.asarray(src, np.float32)
        if src.size != cnt:
            raise ValueError("checkpoint tensor for %s has %d values, the model needs %d" % (n, src.size, cnt))
        flat[o:o + cnt] = src.reshape(-1)
    return flat
