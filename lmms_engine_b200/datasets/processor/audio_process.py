"""Log-mel features for the audio encoders, Whisper convention (16 kHz, 25 ms window, 10 ms hop,
Slaney-normalised mel filters, ``log10`` clamped to 8 dB below the maximum, scaled to about [-1, 1]).
The reference obtains them from the ``transformers`` WhisperFeatureExtractor inside its processors
(src/lmms_engine/datasets/processor/qwen2_audio_processor.py, aero_processor.py)."""
from __future__ import annotations

from functools import lru_cache

import numpy as np
import torch

SAMPLE_RATE, N_FFT, HOP = 16000, 400, 160


def _hz_to_mel(f):
    f = np.asarray(f, dtype=np.float64)
    mel = 3.0 * f / 200.0
    log_region = f >= 1000.0
    return np.where(log_region, 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (np.log(6.4) / 27.0), mel)


def _mel_to_hz(m):
    m = np.asarray(m, dtype=np.float64)
    f = 200.0 * m / 3.0
    log_region = m >= 15.0
    return np.where(log_region, 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0)), f)


@lru_cache(maxsize=4)
def mel_filters(n_mels: int = 128, n_fft: int = N_FFT, sr: int = SAMPLE_RATE) -> torch.Tensor:
    """``[n_mels, n_fft // 2 + 1]`` triangular filters on the Slaney mel scale, area-normalised."""
    freqs = np.linspace(0, sr / 2, n_fft // 2 + 1)
    pts = _mel_to_hz(np.linspace(_hz_to_mel(0.0), _hz_to_mel(sr / 2.0), n_mels + 2))
    diff = np.diff(pts)
    ramps = pts[:, None] - freqs[None, :]
    lower, upper = -ramps[:-2] / diff[:-1, None], ramps[2:] / diff[1:, None]
    w = np.maximum(0.0, np.minimum(lower, upper))
    w *= (2.0 / (pts[2:] - pts[:-2]))[:, None]
    return torch.from_numpy(w.astype(np.float32))


def log_mel_spectrogram(wave, n_mels: int = 128, n_frames: int = 3000):
    """``wave`` (1-D float, 16 kHz) -> ``(features [n_mels, n_frames], mask [n_frames], valid_frames)``;
    audio is zero-padded / cut to ``n_frames`` hops (30 s)."""
    x = torch.as_tensor(np.asarray(wave), dtype=torch.float32).flatten()
    valid = min(int(x.numel()) // HOP, n_frames)
    total = n_frames * HOP
    x = x[:total] if x.numel() >= total else torch.cat([x, x.new_zeros(total - x.numel())])
    spec = torch.stft(x, N_FFT, HOP, window=torch.hann_window(N_FFT), return_complex=True)
    mag = spec[..., :-1].abs() ** 2
    mel = mel_filters(n_mels) @ mag
    log = torch.clamp(mel, min=1e-10).log10()
    log = torch.maximum(log, log.max() - 8.0)
    feats = (log + 4.0) / 4.0
    mask = torch.zeros(n_frames, dtype=torch.long)
    mask[:max(valid, 1)] = 1
    return feats, mask, max(valid, 1)
