"""Log-mel spectrogram features (Whisper layout).

25 ms Hann window (n_fft 400), 10 ms hop (160), power spectrum → slaney-scale mel filters with area
normalisation → log10, clamped to 8 dB (in log10 units) below the maximum, then ``(x + 4) / 4``.
Audio is padded or cut to 30 s, giving [n_mels, 3000] (reference: src/audio/whisper_mel.rs; the
same definition as the feature extractor Whisper checkpoints ship with).
"""
from __future__ import annotations

import numpy as np
import torch


def _hz_to_mel(f):
    f = np.asarray(f, dtype=np.float64)
    mel = 3.0 * f / 200.0
    log_region = f >= 1000.0
    return np.where(log_region, 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) * (27.0 / np.log(6.4)), mel)


def _mel_to_hz(m):
    m = np.asarray(m, dtype=np.float64)
    f = 200.0 * m / 3.0
    log_region = m >= 15.0
    return np.where(log_region, 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0)), f)


def mel_filter_bank(n_freqs: int, n_mels: int, sr: int, fmin: float = 0.0, fmax: float | None = None) -> np.ndarray:
    """[n_freqs, n_mels] triangular filters on the slaney mel scale, each normalised to unit area."""
    fmax = fmax if fmax is not None else sr / 2
    fft_freqs = np.linspace(0, sr / 2, n_freqs)
    pts = _mel_to_hz(np.linspace(_hz_to_mel(fmin), _hz_to_mel(fmax), n_mels + 2))
    diff = np.diff(pts)
    slopes = pts[None, :] - fft_freqs[:, None]
    down = -slopes[:, :-2] / diff[:-1]
    up = slopes[:, 2:] / diff[1:]
    fb = np.maximum(0.0, np.minimum(down, up))
    fb *= (2.0 / (pts[2:n_mels + 2] - pts[:n_mels]))[None, :]
    return fb.astype(np.float32)


class LogMel:
    def __init__(self, n_mels: int = 80, sr: int = 16000, n_fft: int = 400, hop: int = 160, chunk_seconds: int = 30):
        self.n_mels, self.sr, self.n_fft, self.hop = n_mels, sr, n_fft, hop
        self.n_samples = chunk_seconds * sr
        self.filters = torch.from_numpy(mel_filter_bank(n_fft // 2 + 1, n_mels, sr)).t().contiguous()    # [n_mels, n_freqs]
        self.window = torch.hann_window(n_fft, periodic=True)

    def __call__(self, samples, pad: bool = True) -> torch.Tensor:
        """float samples at ``sr`` → [n_mels, frames] (3000 frames when padded to the 30 s chunk)."""
        x = torch.as_tensor(np.asarray(samples, dtype=np.float32))
        if pad:
            x = torch.nn.functional.pad(x[: self.n_samples], (0, max(0, self.n_samples - x.numel())))
        st = torch.stft(x, self.n_fft, self.hop, window=self.window, center=True, pad_mode="reflect", return_complex=True)
        power = st[:, :-1].abs().pow(2)                      # the last frame is dropped
        mel = self.filters @ power
        log = torch.clamp(mel, min=1e-10).log10()
        log = torch.maximum(log, log.max() - 8.0)
        return (log + 4.0) / 4.0
