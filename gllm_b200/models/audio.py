"""Audio front end and Conformer encoder: log-mel spectrogram, convolutional subsampling, Conformer blocks
(half-step FFN, self-attention, depthwise-conv module, half-step FFN), projector into the LLM's hidden size.

Reference parity: USM Conformer graph with ``DepthwiseConv1D`` (CLAUDE.md:996-1007; src/compat/audio_forward.rs and
audio_fragments/), mel spectrogram in plain code (src/compat/multimodal.rs).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F


@dataclass
class AudioConfig:
    sample_rate: int = 16000
    n_fft: int = 400
    hop: int = 160
    n_mels: int = 80
    hidden: int = 256
    layers: int = 4
    heads: int = 4
    ffn_mult: int = 4
    conv_kernel: int = 15
    subsample: int = 4
    out_hidden: int = 0
    eps: float = 1e-5


def mel_filterbank(n_mels: int, n_fft: int, sr: int, fmin: float = 0.0, fmax: Optional[float] = None) -> torch.Tensor:
    """Triangular filters on the HTK mel scale: [n_mels, n_fft//2 + 1]."""
    fmax = fmax or sr / 2
    mel = lambda f: 2595.0 * math.log10(1.0 + f / 700.0)
    inv = lambda m: 700.0 * (10 ** (m / 2595.0) - 1.0)
    pts = torch.linspace(mel(fmin), mel(fmax), n_mels + 2).apply_(inv)
    bins = torch.linspace(0, sr / 2, n_fft // 2 + 1)
    fb = torch.zeros(n_mels, n_fft // 2 + 1)
    for i in range(n_mels):
        lo, c, hi = pts[i], pts[i + 1], pts[i + 2]
        up, down = (bins - lo) / (c - lo), (hi - bins) / (hi - c)
        fb[i] = torch.clamp(torch.minimum(up, down), min=0)
    return fb


def log_mel_spectrogram(wave: torch.Tensor, cfg: AudioConfig) -> torch.Tensor:
    """wave [B, samples] -> [B, frames, n_mels] (log10, clamped, scaled to roughly [-1, 1])."""
    win = torch.hann_window(cfg.n_fft, device=wave.device)
    spec = torch.stft(wave.float(), cfg.n_fft, cfg.hop, window=win, return_complex=True).abs() ** 2     # [B, F, T]
    mel = mel_filterbank(cfg.n_mels, cfg.n_fft, cfg.sample_rate).to(wave.device) @ spec
    lm = torch.log10(mel.clamp_min(1e-10))
    lm = torch.maximum(lm, lm.amax((1, 2), keepdim=True) - 8.0)
    return ((lm + 4.0) / 4.0).transpose(1, 2)


class AudioWeights:
    def __init__(self, cfg: AudioConfig, device="cpu", dtype=torch.float32, seed=0):
        g = torch.Generator().manual_seed(seed)
        mk = lambda *s, std=0.05: (torch.randn(*s, generator=g) * std).to(device, dtype)
        H, Fm = cfg.hidden, cfg.hidden * cfg.ffn_mult
        self.sub_w = mk(H, cfg.n_mels * cfg.subsample)
        self.layers = []
        for _ in range(cfg.layers):
            self.layers.append({
                "ff1_ln": torch.ones(H, device=device), "ff1_a": mk(Fm, H), "ff1_b": mk(H, Fm),
                "att_ln": torch.ones(H, device=device), "qkv": mk(3 * H, H), "o": mk(H, H),
                "conv_ln": torch.ones(H, device=device), "pw1": mk(2 * H, H), "dw": mk(H, 1, cfg.conv_kernel, std=0.2),
                "bn_w": torch.ones(H, device=device), "pw2": mk(H, H),
                "ff2_ln": torch.ones(H, device=device), "ff2_a": mk(Fm, H), "ff2_b": mk(H, Fm),
                "out_ln": torch.ones(H, device=device),
            })
        self.proj = mk(cfg.out_hidden, H) if cfg.out_hidden else None


def depthwise_conv1d(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [B, T, C], w [C, 1, K] -> same-length depthwise convolution over time."""
    k = w.shape[-1]
    return F.conv1d(x.transpose(1, 2), w, padding=k // 2, groups=w.shape[0]).transpose(1, 2)


class ConformerEncoder:
    def __init__(self, cfg: AudioConfig, weights: AudioWeights):
        self.cfg, self.w = cfg, weights

    def _ln(self, x, w):
        return F.layer_norm(x, (x.shape[-1],), w, None, self.cfg.eps)

    def forward_features(self, mel: torch.Tensor) -> torch.Tensor:
        """mel [B, frames, n_mels] -> [B, frames / subsample, out_hidden or hidden]."""
        c, w = self.cfg, self.w
        B, T, M = mel.shape
        T4 = T // c.subsample * c.subsample
        x = mel[:, :T4].reshape(B, T4 // c.subsample, c.subsample * M).to(w.sub_w.dtype) @ w.sub_w.t()
        H, hd = c.hidden, c.hidden // c.heads
        for lw in w.layers:
            h = self._ln(x, lw["ff1_ln"])
            x = x + 0.5 * (F.silu(h @ lw["ff1_a"].t()) @ lw["ff1_b"].t())
            h = self._ln(x, lw["att_ln"])
            qkv = (h @ lw["qkv"].t()).reshape(B, -1, 3, c.heads, hd).permute(2, 0, 3, 1, 4)
            a = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2]).transpose(1, 2).reshape(B, -1, H)
            x = x + a @ lw["o"].t()
            h = self._ln(x, lw["conv_ln"])
            h = F.glu(h @ lw["pw1"].t(), dim=-1)
            h = depthwise_conv1d(h, lw["dw"])
            h = F.silu(self._ln(h, lw["bn_w"]))
            x = x + h @ lw["pw2"].t()
            h = self._ln(x, lw["ff2_ln"])
            x = x + 0.5 * (F.silu(h @ lw["ff2_a"].t()) @ lw["ff2_b"].t())
            x = self._ln(x, lw["out_ln"])
        if w.proj is not None:
            x = x @ w.proj.t()
        return x

    def forward(self, wave: torch.Tensor) -> torch.Tensor:
        return self.forward_features(log_mel_spectrogram(wave, self.cfg))
