"""Audio inputs for speech recognition: WAV decoding, resampling, the log-mel front end, the
feature-count contract and the encoder whose outputs overlay the audio placeholder rows.

Contracts follow the reference's crates/orinfer-model-sdk/src/audio.rs (mel is
``[128, ceil(frames / 100) * 100]``; at most 120 000 frames = 1 200 s; features per recording
``(frames // 100) * 13 + ceil((frames % 100) / 8)``, i.e. three stride-2 stages over
100-frame chunks; optional 104-feature attention windows) and
crates/orinfer-api/src/server/audio.rs (decode -> mono -> 16 kHz -> log-mel on the CPU).
Only RIFF/WAVE PCM and float containers are decoded here: no FLAC / MP3 / AAC / Ogg decoder
library is a dependency of this package, and those uploads are refused with a clear error.
"""

from __future__ import annotations

import hashlib
import io
import math
import struct
import wave
from dataclasses import dataclass
from typing import Tuple

import numpy as np
import torch

SAMPLE_RATE = 16000
N_FFT = 400
HOP = 160
N_MELS = 128
CHUNK_FRAMES = 100
MAX_FRAMES = 120000
WINDOW_FEATURES = 104


class AudioError(ValueError):
    pass


def decode_wav(data: bytes) -> Tuple[np.ndarray, int]:
    """RIFF/WAVE bytes -> (float32 mono samples in [-1, 1], sample rate).  PCM 8/16/24/32-bit
    and IEEE float 32-bit are accepted; channels are averaged."""
    if len(data) < 12 or data[:4] != b"RIFF" or data[8:12] != b"WAVE":
        kind = {b"fLaC": "FLAC", b"OggS": "Ogg", b"ID3": "MP3"}.get(data[:4]) or \
            {b"ID3": "MP3"}.get(data[:3]) or "unknown"
        raise AudioError(f"unsupported audio container ({kind}); this build decodes WAV only")
    fmt = struct.unpack_from("<H", data, 20)[0] if len(data) > 22 else 1
    if fmt == 3 or (fmt == 0xFFFE and len(data) > 46 and data[44:46] == b"\x03\x00"):
        return _decode_float_wav(data)
    try:
        with wave.open(io.BytesIO(data)) as w:
            ch, width, rate, n = w.getnchannels(), w.getsampwidth(), w.getframerate(), w.getnframes()
            raw = w.readframes(n)
    except (wave.Error, EOFError) as e:
        raise AudioError(f"cannot decode WAV: {e}") from None
    if width == 1:
        x = (np.frombuffer(raw, np.uint8).astype(np.float32) - 128.0) / 128.0
    elif width == 2:
        x = np.frombuffer(raw, "<i2").astype(np.float32) / 32768.0
    elif width == 3:
        b = np.frombuffer(raw, np.uint8).reshape(-1, 3).astype(np.int32)
        v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
        x = np.where(v >= 1 << 23, v - (1 << 24), v).astype(np.float32) / float(1 << 23)
    elif width == 4:
        x = np.frombuffer(raw, "<i4").astype(np.float32) / float(1 << 31)
    else:
        raise AudioError("unsupported WAV sample width")
    if ch > 1:
        x = x[: len(x) // ch * ch].reshape(-1, ch).mean(axis=1)
    return x.astype(np.float32), rate


def _decode_float_wav(data: bytes) -> Tuple[np.ndarray, int]:
    pos, ch, rate, body = 12, 1, SAMPLE_RATE, None
    while pos + 8 <= len(data):
        tag, size = data[pos:pos + 4], struct.unpack_from("<I", data, pos + 4)[0]
        if tag == b"fmt ":
            ch, rate = struct.unpack_from("<HI", data, pos + 10)
        elif tag == b"data":
            body = data[pos + 8:pos + 8 + size]
        pos += 8 + size + (size & 1)
    if body is None or ch == 0:
        raise AudioError("cannot decode WAV: no data chunk")
    x = np.frombuffer(body[: len(body) // 4 * 4], "<f4")
    if ch > 1:
        x = x[: len(x) // ch * ch].reshape(-1, ch).mean(axis=1)
    return np.nan_to_num(x).astype(np.float32), rate


def resample(x: np.ndarray, rate: int, target: int = SAMPLE_RATE) -> np.ndarray:
    """Polyphase (windowed-sinc) rate conversion."""
    if rate == target:
        return x.astype(np.float32)
    if rate <= 0:
        raise AudioError("invalid sample rate")
    from scipy.signal import resample_poly
    g = math.gcd(rate, target)
    return resample_poly(x.astype(np.float64), target // g, rate // g).astype(np.float32)


def mel_filterbank(n_mels: int = N_MELS, n_fft: int = N_FFT, rate: int = SAMPLE_RATE) -> np.ndarray:
    """Slaney-style triangular filters [n_mels, n_fft / 2 + 1], area-normalised."""
    def hz_to_mel(f):
        f = np.asarray(f, dtype=np.float64)
        lin = f / (200.0 / 3)
        log = 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (np.log(6.4) / 27.0)
        return np.where(f >= 1000.0, log, lin)

    def mel_to_hz(m):
        m = np.asarray(m, dtype=np.float64)
        return np.where(m >= 15.0, 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0)),
                        m * (200.0 / 3))

    freqs = np.linspace(0, rate / 2, n_fft // 2 + 1)
    edges = mel_to_hz(np.linspace(hz_to_mel(0.0), hz_to_mel(rate / 2.0), n_mels + 2))
    lower = (freqs[None, :] - edges[:-2, None]) / np.diff(edges)[:-1, None]
    upper = (edges[2:, None] - freqs[None, :]) / np.diff(edges)[1:, None]
    fb = np.maximum(0.0, np.minimum(lower, upper))
    return (fb * (2.0 / (edges[2:] - edges[:-2]))[:, None]).astype(np.float32)


_FILTERS = None


def log_mel(samples: np.ndarray) -> Tuple[np.ndarray, int]:
    """(mel float32 [128, ceil(frames / 100) * 100] right-padded with the floor value, frames).
    25 ms Hann window, 10 ms hop, reflect padding, power spectrum, log10 clamped to 8 decades
    below the maximum, then (x + 4) / 4."""
    global _FILTERS
    if _FILTERS is None:
        _FILTERS = mel_filterbank()
    x = np.asarray(samples, dtype=np.float32)
    frames = len(x) // HOP
    if frames == 0:
        raise AudioError("audio is shorter than one frame")
    if frames > MAX_FRAMES:
        raise AudioError("audio is longer than 1200 s")
    pad = N_FFT // 2
    x = np.pad(x, (pad, pad), mode="reflect" if len(x) > pad else "constant")
    idx = np.arange(N_FFT)[None, :] + HOP * np.arange(frames)[:, None]
    window = np.hanning(N_FFT + 1)[:-1].astype(np.float32)
    power = np.abs(np.fft.rfft(x[idx] * window, axis=1)) ** 2          # [frames, 201]
    mel = np.log10(np.maximum(_FILTERS @ power.T.astype(np.float32), 1e-10))
    mel = np.maximum(mel, mel.max() - 8.0)
    mel = ((mel + 4.0) / 4.0).astype(np.float32)
    padded = -(-frames // CHUNK_FRAMES) * CHUNK_FRAMES
    out = np.full((N_MELS, padded), mel.min(), dtype=np.float32)
    out[:, :frames] = mel
    return out, frames


def feature_count(frames: int) -> int:
    if frames <= 0 or frames > MAX_FRAMES:
        raise AudioError("invalid mel geometry")
    return (frames // CHUNK_FRAMES) * 13 + -(-(frames % CHUNK_FRAMES) // 8)


@dataclass
class AudioInput:
    frames: int
    mel: np.ndarray                       # [128, ceil(frames / 100) * 100]

    @property
    def features(self) -> int:
        want = (N_MELS, -(-self.frames // CHUNK_FRAMES) * CHUNK_FRAMES)
        if tuple(self.mel.shape) != want or not np.isfinite(self.mel).all():
            raise AudioError("invalid mel geometry or values")
        return feature_count(self.frames)

    def digest(self) -> int:
        h = hashlib.sha256(f"{self.frames}:".encode())
        h.update(np.ascontiguousarray(self.mel).tobytes())
        return int.from_bytes(h.digest()[:8], "little")


def load_audio(data: bytes) -> AudioInput:
    samples, rate = decode_wav(data)
    mel, frames = log_mel(resample(samples, rate))
    return AudioInput(frames, mel)


class AudioEncoder(torch.nn.Module):
    """Stem of three stride-2 convolutions over each 100-frame chunk (100 -> 13 features),
    sinusoidal positions, self-attention blocks restricted to windows of 104 features, and a
    projection to the decoder width.  Random-init from a seed; the layout is the one a
    converted checkpoint would fill."""

    def __init__(self, hidden: int, width: int = 128, depth: int = 2, heads: int = 4,
                 seed: int = 0):
        super().__init__()
        torch.manual_seed(seed)
        self.width, self.heads = width, heads
        self.stem = torch.nn.ModuleList(
            [torch.nn.Conv1d(N_MELS if i == 0 else width, width, 3, stride=2, padding=1)
             for i in range(3)])
        self.blocks = torch.nn.ModuleList(
            [torch.nn.TransformerEncoderLayer(width, heads, 4 * width, dropout=0.0,
                                              activation="gelu", batch_first=True,
                                              norm_first=True) for _ in range(depth)])
        self.norm = torch.nn.LayerNorm(width)
        self.proj = torch.nn.Linear(width, hidden)
        self.requires_grad_(False)
        self.eval()

    @torch.no_grad()
    def forward(self, mel: torch.Tensor, frames: int) -> torch.Tensor:
        """mel [128, chunks * 100] -> features [feature_count(frames), hidden]."""
        dt = self.proj.weight.dtype
        chunks = mel.shape[1] // CHUNK_FRAMES
        x = mel.to(dt).view(N_MELS, chunks, CHUNK_FRAMES).permute(1, 0, 2)   # [chunks, 128, 100]
        for conv in self.stem:
            x = torch.nn.functional.gelu(conv(x))
        x = x.permute(0, 2, 1)                                               # [chunks, 13, width]
        keep = []
        for c in range(chunks):
            valid = min(CHUNK_FRAMES, frames - c * CHUNK_FRAMES)
            keep.append(x[c, : (13 if valid == CHUNK_FRAMES else -(-valid // 8))])
        x = torch.cat(keep)                                                  # [features, width]
        n = x.shape[0]
        pos = torch.arange(n, device=x.device, dtype=torch.float32)[:, None]
        inv = torch.exp(-math.log(10000.0) * torch.arange(0, self.width, 2, device=x.device,
                                                          dtype=torch.float32) / self.width)
        x = x + torch.cat([(pos * inv).sin(), (pos * inv).cos()], dim=1).to(dt)
        win = torch.arange(n, device=x.device) // WINDOW_FEATURES
        mask = win[:, None] != win[None, :]                                  # True = blocked
        x = x[None]
        for b in self.blocks:
            x = b(x, src_mask=mask)
        return self.proj(self.norm(x[0]))

    def encode(self, audio: AudioInput) -> torch.Tensor:
        dev = self.proj.weight.device
        out = self(torch.from_numpy(np.array(audio.mel, copy=True)).to(dev), audio.frames)
        if out.shape[0] != audio.features:
            raise AudioError("encoder produced a feature count that breaks the contract")
        return out
