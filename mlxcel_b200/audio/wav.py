"""WAV decoding / encoding and resampling.

RIFF/WAVE with PCM 8 / 16 / 24 / 32-bit integers or 32 / 64-bit floats (format tags 1, 3 and the
extensible tag 0xFFFE), any channel count (mixed down to mono). Compressed containers (mp3, flac,
ogg) are not decoded in this build: the reference links decoders for them
(src/audio/preprocessing_container.rs); here the caller gets an error that says so.
"""
from __future__ import annotations

import io
import struct

import numpy as np


def read_wav(data: bytes) -> tuple[np.ndarray, int]:
    """bytes of a WAV file → (mono float32 samples in [-1, 1], sample rate)."""
    if len(data) < 12 or data[:4] != b"RIFF" or data[8:12] != b"WAVE":
        kind = "mp3" if data[:3] == b"ID3" or data[:2] in (b"\xff\xfb", b"\xff\xf3") else \
            "flac" if data[:4] == b"fLaC" else "ogg" if data[:4] == b"OggS" else "unknown"
        raise ValueError(f"unsupported audio container ({kind}); send 16 kHz mono WAV (PCM or float)")
    pos, fmt, pcm = 12, None, None
    while pos + 8 <= len(data):
        cid, size = data[pos:pos + 4], struct.unpack("<I", data[pos + 4:pos + 8])[0]
        body = data[pos + 8:pos + 8 + size]
        if cid == b"fmt ":
            tag, ch, rate, _, _, bits = struct.unpack("<HHIIHH", body[:16])
            if tag == 0xFFFE and len(body) >= 26:
                tag = struct.unpack("<H", body[24:26])[0]
            fmt = (tag, ch, rate, bits)
        elif cid == b"data":
            pcm = body
        pos += 8 + size + (size & 1)
    if fmt is None or pcm is None:
        raise ValueError("WAV file without fmt or data chunk")
    tag, ch, rate, bits = fmt
    if tag == 1:
        if bits == 8:
            x = (np.frombuffer(pcm, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
        elif bits == 16:
            x = np.frombuffer(pcm[: len(pcm) // 2 * 2], dtype="<i2").astype(np.float32) / 32768.0
        elif bits == 24:
            b = np.frombuffer(pcm[: len(pcm) // 3 * 3], dtype=np.uint8).reshape(-1, 3).astype(np.int32)
            v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
            x = (v - ((v & 0x800000) << 1)).astype(np.float32) / 8388608.0
        elif bits == 32:
            x = np.frombuffer(pcm[: len(pcm) // 4 * 4], dtype="<i4").astype(np.float32) / 2147483648.0
        else:
            raise ValueError(f"unsupported PCM width {bits}")
    elif tag == 3:
        x = np.frombuffer(pcm, dtype="<f4" if bits == 32 else "<f8").astype(np.float32)
    else:
        raise ValueError(f"unsupported WAV format tag {tag}")
    if ch > 1:
        x = x[: len(x) // ch * ch].reshape(-1, ch).mean(axis=1)
    return np.ascontiguousarray(x, dtype=np.float32), int(rate)


def write_wav(samples: np.ndarray, rate: int) -> bytes:
    """Mono float samples → 16-bit PCM WAV bytes."""
    pcm = (np.clip(np.asarray(samples, dtype=np.float32), -1.0, 1.0) * 32767.0).astype("<i2").tobytes()
    out = io.BytesIO()
    out.write(b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVE")
    out.write(b"fmt " + struct.pack("<IHHIIHH", 16, 1, 1, rate, rate * 2, 2, 16))
    out.write(b"data" + struct.pack("<I", len(pcm)) + pcm)
    return out.getvalue()


def resample(x: np.ndarray, src: int, dst: int) -> np.ndarray:
    """Polyphase resampling with an anti-aliasing filter."""
    if src == dst:
        return x
    from math import gcd

    from scipy.signal import resample_poly
    g = gcd(src, dst)
    return resample_poly(x, dst // g, src // g).astype(np.float32)


def decode_audio(data: bytes, rate: int = 16000) -> np.ndarray:
    x, sr = read_wav(data)
    return resample(x, sr, rate)
