"""Audio front end, feature contract, encoder and the transcription route."""
import io
import struct
import wave

import numpy as np
import pytest
import torch

from orinfer_b200.models import audio as A


def wav_bytes(samples, rate=16000, width=2, channels=1):
    buf = io.BytesIO()
    with wave.open(buf, "wb") as w:
        w.setnchannels(channels)
        w.setsampwidth(width)
        w.setframerate(rate)
        x = np.clip(samples, -1, 1)
        if width == 2:
            raw = (x * 32767).astype("<i2").tobytes()
        elif width == 1:
            raw = (x * 127 + 128).astype(np.uint8).tobytes()
        else:
            raw = b"".join(struct.pack("<i", int(v * (2 ** 23 - 1)))[:3] for v in x)
        w.writeframes(raw)
    return buf.getvalue()


def tone(freq, seconds, rate=16000):
    t = np.arange(int(seconds * rate)) / rate
    return (0.5 * np.sin(2 * np.pi * freq * t)).astype(np.float32)


def test_wav_decoding_widths_channels_and_refusals():
    x = tone(440, 0.1)
    for width, tol in ((2, 1e-4), (1, 2e-2), (3, 1e-6)):
        got, rate = A.decode_wav(wav_bytes(x, width=width))
        assert rate == 16000 and got.shape == x.shape and np.abs(got - x).max() < tol
    stereo = np.stack([x, -x], axis=1).reshape(-1)
    got, _ = A.decode_wav(wav_bytes(stereo, channels=2))
    assert np.abs(got).max() < 1e-4                                  # channels averaged
    body = x.astype("<f4").tobytes()
    flt = (b"RIFF" + struct.pack("<I", 36 + len(body)) + b"WAVEfmt " +
           struct.pack("<IHHIIHH", 16, 3, 1, 16000, 64000, 4, 32) + b"data" +
           struct.pack("<I", len(body)) + body)
    got, rate = A.decode_wav(flt)
    assert rate == 16000 and np.array_equal(got, x)
    with pytest.raises(A.AudioError, match="FLAC"):
        A.decode_wav(b"fLaC" + b"\0" * 40)
    with pytest.raises(A.AudioError, match="WAV only"):
        A.decode_wav(b"\xff\xfb" + b"\0" * 40)


def test_resample_keeps_the_tone():
    y = A.resample(tone(1000, 0.5, 44100), 44100)
    assert abs(len(y) - 8000) <= 1
    spec = np.abs(np.fft.rfft(y))
    assert abs(np.argmax(spec) * 16000 / len(y) - 1000) < 4
    assert A.resample(tone(100, 0.1), 16000).dtype == np.float32


def test_log_mel_geometry_and_content():
    fb = A.mel_filterbank()
    assert fb.shape == (128, 201) and (fb >= 0).all() and (fb.sum(axis=1) > 0).all()
    centres = (fb * np.arange(201)).sum(axis=1) / fb.sum(axis=1)
    assert np.all(np.diff(centres) >= 0)      # low filters are narrower than a bin
    mel, frames = A.log_mel(tone(2000, 1.234))
    assert frames == 123 and mel.shape == (128, 200) and np.isfinite(mel).all()
    band = mel[:, :frames].mean(axis=1)
    peak_hz = centres[np.argmax(band)] * 16000 / 400
    assert abs(peak_hz - 2000) < 150
    assert np.all(mel[:, frames:] == mel.min())                      # right padding at the floor
    assert mel.max() - mel.min() <= 2.0 + 1e-6                       # 8 decades / 4
    with pytest.raises(A.AudioError, match="shorter"):
        A.log_mel(np.zeros(100, np.float32))
    with pytest.raises(A.AudioError, match="1200"):
        A.log_mel(np.zeros(16000 * 1201, np.float32))


def test_feature_count_contract_and_encoder():
    assert [A.feature_count(f) for f in (1, 8, 9, 100, 101, 123, 120000)] == \
        [1, 1, 2, 13, 14, 16, 15600]
    with pytest.raises(A.AudioError):
        A.feature_count(120001)
    audio = A.load_audio(wav_bytes(tone(300, 1.234, 8000), rate=8000))
    assert audio.frames == 123 and audio.features == 16
    enc = A.AudioEncoder(hidden=256, width=64, depth=1, heads=2, seed=3)
    f = enc.encode(audio)
    assert f.shape == (16, 256) and torch.isfinite(f).all()
    assert torch.equal(f, A.AudioEncoder(hidden=256, width=64, depth=1, heads=2, seed=3).encode(audio))
    # attention is confined to 104-feature windows: changing audio beyond the first window
    # leaves the first window's features as they were
    long_a = tone(300, 10.0)
    long_b = long_a.copy()
    long_b[16000 * 9:] = tone(900, 1.0)
    fa = enc.encode(A.AudioInput(*reversed(A.log_mel(long_a))))
    fb = enc.encode(A.AudioInput(*reversed(A.log_mel(long_b))))
    assert fa.shape == (130, 256)
    assert not torch.allclose(fa[104:], fb[104:])
    with pytest.raises(A.AudioError):
        A.AudioInput(50, np.zeros((128, 50), np.float32)).features


@pytest.fixture(scope="module")
def client():
    from fastapi.testclient import TestClient
    from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec
    from orinfer_b200.api.server import Service, create_app
    from orinfer_b200.config import PRESETS, SchedulerOptions
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.models.weights import random_model
    weights = random_model(PRESETS["tiny"], seed=0)
    codec = ChatCodec(ByteTokenizer(1024), context=512, model_name="tiny-asr")
    svc = Service(lambda: Engine(weights, sched=SchedulerOptions(max_active=4, prefill_chunk=64),
                                 kv_pages=24, max_context=512), codec, "tiny-asr")
    svc.start()
    with TestClient(create_app(svc)) as c:
        yield c
    svc.stop(1000)


def test_transcription_route(client):
    data = wav_bytes(tone(500, 2.0))
    r = client.post("/v1/audio/transcriptions", files={"file": ("a.wav", data, "audio/wav")},
                    data={"max_tokens": "5", "language": "en", "prompt": "Names: Ada."})
    assert r.status_code == 200, r.text
    body = r.json()
    assert isinstance(body["text"], str) and body["usage"]["output_tokens"] <= 5
    # 200 frames -> 26 features, plus the fixed prompt tokens
    assert body["usage"]["input_tokens"] > 26
    again = client.post("/v1/audio/transcriptions", files={"file": ("a.wav", data, "audio/wav")},
                        data={"max_tokens": "5", "language": "en", "prompt": "Names: Ada.",
                              "response_format": "text"})
    assert again.status_code == 200 and again.text == body["text"]
    assert again.headers["content-type"].startswith("text/plain")
    bad = client.post("/v1/audio/transcriptions", files={"file": ("a.flac", b"fLaC" + b"\0" * 64)})
    assert bad.status_code == 400 and bad.json()["error"]["param"] == "file"
    assert client.post("/v1/audio/transcriptions", data={"language": "en"}).status_code == 400
    fmt = client.post("/v1/audio/transcriptions", files={"file": ("a.wav", data)},
                      data={"response_format": "srt"})
    assert fmt.status_code == 400
    long = client.post("/v1/audio/transcriptions",
                       files={"file": ("l.wav", wav_bytes(tone(500, 40.0)))})
    assert long.status_code == 400 and long.json()["error"]["code"] == "context_length_exceeded"
    assert "orinfer_audio_inputs_total" in client.get("/metrics").text
