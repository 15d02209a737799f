"""LTX-2 vocoder (BigVGAN-style, mel-spectrogram -> waveform) with the bandwidth-extension wrapper.

Reference: src/maxdiffusion/models/ltx2/vocoder_ltx2.py — Kaiser-sinc filters (:32-72), `DownSample1d` / `UpSample1d`
(kaiser and hann windows, :75-205), `SnakeBeta` x + sin^2(alpha x) / beta in log scale (:207-250), anti-aliased
activation (:253-270), `ResBlock` (:272-365), `LTX2Vocoder` (transposed-conv up-sampling stack, resnet outputs
averaged, :367-530), `CausalSTFT` / `MelSTFT` (:532-590) and `LTX2VocoderWithBWE` (16 kHz vocoder -> mel of its output
-> residual generator at 48 kHz + hann-sinc resampled skip, :591-723).
Tensors are [B, C, T]. On CUDA the anti-aliased activation is ONE fused kernel (`ops.kernels.snake_aa`); the
separable three-op path below is the reference used on CPU and in the numerics test.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import kernels as K


def kaiser_sinc_filter1d(cutoff: float, half_width: float, kernel_size: int) -> torch.Tensor:
  delta_f = 4 * half_width
  half = kernel_size // 2
  amp = 2.285 * (half - 1) * math.pi * delta_f + 7.95
  beta = 0.1102 * (amp - 8.7) if amp > 50.0 else (0.5842 * (amp - 21) ** 0.4 + 0.07886 * (amp - 21.0) if amp >= 21.0 else 0.0)
  window = torch.kaiser_window(kernel_size, periodic=False, beta=beta, dtype=torch.float64)
  t = (torch.arange(-half, half, dtype=torch.float64) + 0.5) if kernel_size % 2 == 0 else (torch.arange(kernel_size, dtype=torch.float64) - half)
  if cutoff == 0.0:
    return torch.zeros_like(t).float()
  t = 2 * cutoff * t
  filt = 2 * cutoff * window * torch.sinc(t)
  return (filt / filt.sum()).float()


class DownSample1d(nn.Module):

  def __init__(self, ratio: int = 2, kernel_size: Optional[int] = None):
    super().__init__()
    self.ratio = ratio
    self.kernel_size = kernel_size or int(6 * ratio // 2) * 2
    self.pad_left = self.kernel_size // 2 + (self.kernel_size % 2) - 1
    self.pad_right = self.kernel_size // 2
    self.register_buffer("filter", kaiser_sinc_filter1d(0.5 / ratio, 0.6 / ratio, self.kernel_size), persistent=False)

  def forward(self, x):
    C = x.shape[1]
    x = F.pad(x, (self.pad_left, self.pad_right), mode="replicate")
    return F.conv1d(x, self.filter.to(x.dtype)[None, None].expand(C, 1, -1), stride=self.ratio, groups=C)


class UpSample1d(nn.Module):

  def __init__(self, ratio: int = 2, kernel_size: Optional[int] = None, window_type: str = "kaiser"):
    super().__init__()
    self.ratio = ratio
    if window_type == "hann":
      rolloff, width_f = 0.99, 6
      width = math.ceil(width_f / rolloff)
      self.kernel_size = 2 * width * ratio + 1
      self.pad, self.pad_left, self.pad_right = width, 2 * width * ratio, self.kernel_size - ratio
      t = (torch.arange(self.kernel_size, dtype=torch.float64) / ratio - width) * rolloff
      window = torch.cos(t.clamp(-width_f, width_f) * math.pi / width_f / 2) ** 2
      filt = (torch.sinc(t) * window * rolloff / ratio).float()
    else:
      self.kernel_size = int(6 * ratio // 2) * 2 if kernel_size is None else kernel_size
      self.pad = self.kernel_size // ratio - 1
      self.pad_left = self.pad * ratio + (self.kernel_size - ratio) // 2
      self.pad_right = self.pad * ratio + (self.kernel_size - ratio + 1) // 2
      filt = kaiser_sinc_filter1d(0.5 / ratio, 0.6 / ratio, self.kernel_size)
    self.register_buffer("filter", filt, persistent=False)

  def forward(self, x):
    C = x.shape[1]
    x = F.pad(x, (self.pad, self.pad), mode="replicate")
    y = self.ratio * F.conv_transpose1d(x, self.filter.to(x.dtype)[None, None].expand(C, 1, -1), stride=self.ratio, groups=C)
    return y[..., self.pad_left:-self.pad_right]


class SnakeBeta(nn.Module):

  def __init__(self, channels: int, alpha: float = 1.0, eps: float = 1e-9, logscale: bool = True, use_beta: bool = True):
    super().__init__()
    self.eps, self.logscale, self.use_beta = eps, logscale, use_beta
    init = torch.zeros(channels) if logscale else torch.ones(channels) * alpha
    self.alpha = nn.Parameter(init.clone())
    self.beta = nn.Parameter(init.clone()) if use_beta else None

  def params(self):
    a = self.alpha.float().exp() if self.logscale else self.alpha.float()
    b = a if self.beta is None else (self.beta.float().exp() if self.logscale else self.beta.float())
    return a, 1.0 / (b + self.eps)

  def forward(self, x):
    a, ib = self.params()
    return (x.float() + ib[None, :, None] * torch.sin(x.float() * a[None, :, None]) ** 2).to(x.dtype)


class AntiAliasAct1d(nn.Module):

  def __init__(self, act: nn.Module, ratio: int = 2, kernel_size: int = 12):
    super().__init__()
    self.upsample, self.act, self.downsample = UpSample1d(ratio, kernel_size), act, DownSample1d(ratio, kernel_size)
    self.fusable = ratio == 2 and kernel_size == 12

  def forward(self, x):
    if self.fusable and x.is_cuda and x.dtype in (torch.float32, torch.bfloat16):
      x = x if x.is_contiguous() else x.contiguous()
      up, dn = self.upsample.filter.tolist(), self.downsample.filter.tolist()
      if isinstance(self.act, SnakeBeta):
        a, ib = self.act.params()
        return K.snake_aa(x, a.contiguous(), ib.contiguous(), up, dn)
      if isinstance(self.act, nn.LeakyReLU):
        return K.snake_aa(x, None, None, up, dn, leaky_slope=self.act.negative_slope)
    return self.downsample(self.act(self.upsample(x)))


def _act(act_fn: str, channels: int, slope: float, antialias: bool, ratio: int, k: int):
  if act_fn == "snakebeta":
    act = SnakeBeta(channels, use_beta=True)
  elif act_fn == "snake":
    act = SnakeBeta(channels, use_beta=False)
  else:
    act = nn.LeakyReLU(slope)
  return AntiAliasAct1d(act, ratio, k) if antialias else act


class ResBlock(nn.Module):

  def __init__(self, channels, kernel_size=3, dilations=(1, 3, 5), act_fn="leaky_relu", slope=0.1, antialias=False,
               ratio=2, aa_kernel=12):
    super().__init__()
    same = lambda d: (kernel_size - 1) * d // 2
    self.convs1 = nn.ModuleList([nn.Conv1d(channels, channels, kernel_size, dilation=d, padding=same(d)) for d in dilations])
    self.convs2 = nn.ModuleList([nn.Conv1d(channels, channels, kernel_size, padding=same(1)) for _ in dilations])
    self.acts1 = nn.ModuleList([_act(act_fn, channels, slope, antialias, ratio, aa_kernel) for _ in dilations])
    self.acts2 = nn.ModuleList([_act(act_fn, channels, slope, antialias, ratio, aa_kernel) for _ in dilations])

  def forward(self, x):
    for a1, c1, a2, c2 in zip(self.acts1, self.convs1, self.acts2, self.convs2):
      x = x + c2(a2(c1(a1(x))))
    return x


class LTX2Vocoder(nn.Module):

  def __init__(self, in_channels=128, hidden_channels=1024, out_channels=2, upsample_kernel_sizes=(16, 15, 8, 4, 4),
               upsample_factors=(6, 5, 2, 2, 2), resnet_kernel_sizes=(3, 7, 11), resnet_dilations=((1, 3, 5),) * 3,
               act_fn="leaky_relu", leaky_relu_negative_slope=0.1, antialias=False, antialias_ratio=2,
               antialias_kernel_size=12, final_act_fn: Optional[str] = "tanh", final_bias=True, output_sampling_rate=24000):
    super().__init__()
    if len(upsample_kernel_sizes) != len(upsample_factors):
      raise ValueError("`upsample_kernel_sizes` and `upsample_factors` should be lists of the same length")
    if len(resnet_kernel_sizes) != len(resnet_dilations):
      raise ValueError("`resnet_kernel_sizes` and `resnet_dilations` should be lists of the same length")
    self.n_up, self.per_up = len(upsample_factors), len(resnet_kernel_sizes)
    self.act_fn, self.slope, self.final_act_fn = act_fn, leaky_relu_negative_slope, final_act_fn
    self.total_upsample_factor = math.prod(upsample_factors)
    self.output_sampling_rate = output_sampling_rate
    self.conv_in = nn.Conv1d(in_channels, hidden_channels, 7, padding=3)
    ups, res, ch = [], [], hidden_channels
    for stride, k in zip(upsample_factors, upsample_kernel_sizes):
      # "SAME" transposed convolution: output length = input length * stride
      pad = (k - stride) // 2
      ups.append(nn.ConvTranspose1d(ch, ch // 2, k, stride=stride, padding=pad, output_padding=(k - stride) % 2))
      ch //= 2
      for rk, dil in zip(resnet_kernel_sizes, resnet_dilations):
        res.append(ResBlock(ch, rk, dil, act_fn, leaky_relu_negative_slope, antialias, antialias_ratio, antialias_kernel_size))
    self.upsamplers, self.resnets = nn.ModuleList(ups), nn.ModuleList(res)
    if act_fn in ("snakebeta", "snake"):
      self.act_out = AntiAliasAct1d(SnakeBeta(ch, use_beta=act_fn == "snakebeta"), antialias_ratio, antialias_kernel_size)
    else:
      self.act_out = nn.LeakyReLU(0.01)
    self.conv_out = nn.Conv1d(ch, out_channels, 7, padding=3, bias=final_bias)

  def forward(self, mel, time_last: bool = False):
    """mel [B, C, T, F] (or [B, C, F, T] with `time_last`) -> waveform [B, out_channels, T * total_upsample_factor]."""
    if not time_last:
      mel = mel.transpose(2, 3)
    B, C, Fq, T = mel.shape
    h = self.conv_in(mel.reshape(B, C * Fq, T))
    for i in range(self.n_up):
      if self.act_fn == "leaky_relu":
        h = F.leaky_relu(h, self.slope)
      h = self.upsamplers[i](h)
      h = sum(self.resnets[j](h) for j in range(i * self.per_up, (i + 1) * self.per_up)) / self.per_up
    h = self.conv_out(self.act_out(h))
    if self.final_act_fn == "tanh":
      h = torch.tanh(h)
    elif self.final_act_fn == "clamp":
      h = h.clamp(-1, 1)
    return h


class CausalSTFT(nn.Module):

  def __init__(self, filter_length=512, hop_length=80, window_length=512):
    super().__init__()
    self.hop_length, self.window_length = hop_length, window_length
    n = filter_length // 2 + 1
    self.forward_basis = nn.Parameter(torch.zeros(n * 2, 1, filter_length), requires_grad=False)
    self.inverse_basis = nn.Parameter(torch.zeros(n * 2, 1, filter_length), requires_grad=False)

  def forward(self, wav):
    """wav [N, 1, L] -> (magnitude, phase) [N, frames, n_freqs]."""
    wav = F.pad(wav, (max(0, self.window_length - self.hop_length), 0))
    spec = F.conv1d(wav.to(self.forward_basis.dtype), self.forward_basis, stride=self.hop_length).transpose(1, 2)
    n = spec.shape[-1] // 2
    real, imag = spec[..., :n], spec[..., n:]
    return torch.sqrt(real ** 2 + imag ** 2), torch.atan2(imag, real)


class MelSTFT(nn.Module):

  def __init__(self, filter_length=512, hop_length=80, window_length=512, num_mel_channels=64):
    super().__init__()
    self.stft_fn = CausalSTFT(filter_length, hop_length, window_length)
    self.mel_basis = nn.Parameter(torch.zeros(num_mel_channels, filter_length // 2 + 1), requires_grad=False)

  def forward(self, wav):
    mag, phase = self.stft_fn(wav)
    mel = mag @ self.mel_basis.t().to(mag.dtype)
    return torch.log(mel.clamp(min=1e-5)), mag, phase, torch.linalg.norm(mag, dim=-1)


class LTX2VocoderWithBWE(nn.Module):

  def __init__(self, vocoder_kwargs: Optional[dict] = None, bwe_kwargs: Optional[dict] = None, filter_length=512,
               hop_length=80, window_length=512, num_mel_channels=64, input_sampling_rate=16000, output_sampling_rate=48000):
    super().__init__()
    vk = dict(in_channels=128, hidden_channels=1536, out_channels=2, upsample_kernel_sizes=(11, 4, 4, 4, 4, 4),
              upsample_factors=(5, 2, 2, 2, 2, 2), act_fn="snakebeta", antialias=True, final_act_fn=None, final_bias=False,
              output_sampling_rate=input_sampling_rate)
    bk = dict(in_channels=128, hidden_channels=512, out_channels=2, upsample_kernel_sizes=(12, 11, 4, 4, 4),
              upsample_factors=(6, 5, 2, 2, 2), act_fn="snakebeta", antialias=True, final_act_fn=None, final_bias=False,
              output_sampling_rate=output_sampling_rate)
    vk.update(vocoder_kwargs or {})
    bk.update(bwe_kwargs or {})
    self.hop_length, self.input_sampling_rate, self.output_sampling_rate = hop_length, input_sampling_rate, output_sampling_rate
    self.vocoder, self.bwe_generator = LTX2Vocoder(**vk), LTX2Vocoder(**bk)
    self.mel_stft = MelSTFT(filter_length, hop_length, window_length, num_mel_channels)
    self.resampler = UpSample1d(output_sampling_rate // input_sampling_rate, window_type="hann")

  def forward(self, mel):
    x = self.vocoder(mel)                                        # [B, ch, N] at the input rate
    B, ch, n = x.shape
    rem = n % self.hop_length
    if rem:
      x = F.pad(x, (0, self.hop_length - rem))
    log_mel = self.mel_stft(x.reshape(B * ch, 1, -1))[0]          # [B*ch, frames, mel]
    residual = self.bwe_generator(log_mel.reshape(B, ch, -1, log_mel.shape[-1]))
    skip = self.resampler(x)
    if residual.shape[-1] < skip.shape[-1]:
      residual = F.pad(residual, (0, skip.shape[-1] - residual.shape[-1]), mode="replicate")
    residual = residual[..., :skip.shape[-1]]
    out = (residual + skip).clamp(-1, 1)
    return out[..., :n * self.output_sampling_rate // self.input_sampling_rate]
