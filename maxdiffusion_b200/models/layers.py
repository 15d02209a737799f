"""Small building blocks shared by the model families."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import functional as OF


class Linear(nn.Module):
  """y = x @ Wᵀ + b with W stored [out, in] (the diffusers / PyTorch checkpoint orientation).

  CUDA bf16 inputs run on the tcgen05 GEMM through `ops.functional.linear`.
  """

  def __init__(self, in_features: int, out_features: int, bias: bool = True):
    super().__init__()
    self.in_features, self.out_features = in_features, out_features
    self.weight = nn.Parameter(torch.empty(out_features, in_features))
    self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
    nn.init.normal_(self.weight, std=1.0 / math.sqrt(in_features))

  def forward(self, x, activation: str | None = None, residual=None):
    return OF.linear(x, self.weight, self.bias, activation, residual)

  def extra_repr(self) -> str:
    return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


def project_gated_residual(proj: nn.Module, x, residual, gate):
  """residual + gate * proj(x). A plain `Linear` takes the fused GEMM-epilogue path; any other projection (e.g. a
  quantised one) runs as a module followed by the fused gated-residual kernel."""
  if type(proj) is Linear:
    return OF.linear_gated_residual(x, proj.weight, proj.bias, residual, gate)
  return OF.gated_residual(residual, proj(x), gate)


def sinusoidal_embedding(timesteps: torch.Tensor, dim: int, flip_sin_to_cos: bool = True, freq_shift: float = 0.0,
                         max_period: float = 10000.0, scale: float = 1.0) -> torch.Tensor:
  """Sinusoidal timestep features [N, dim] in fp32 (reference: src/maxdiffusion/models/embeddings_flax.py:28-62)."""
  half = dim // 2
  exponent = -math.log(max_period) * torch.arange(half, dtype=torch.float32, device=timesteps.device) / (half - freq_shift)
  emb = scale * timesteps.float()[:, None] * torch.exp(exponent)[None, :]
  emb = torch.cat([emb.cos(), emb.sin()], dim=-1) if flip_sin_to_cos else torch.cat([emb.sin(), emb.cos()], dim=-1)
  if dim % 2 == 1:
    emb = torch.nn.functional.pad(emb, (0, 1))
  return emb


class RMSNorm(nn.Module):

  def __init__(self, dim: int, eps: float = 1e-6, elementwise_affine: bool = True):
    super().__init__()
    self.eps = eps
    self.weight = nn.Parameter(torch.ones(dim)) if elementwise_affine else None

  def forward(self, x):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
    if self.weight is not None:
      y = y * self.weight.float()
    return y.to(x.dtype)


class Conv2d(nn.Conv2d):
  """3x3 / 1x1 convolution with the parameter names of `torch.nn.Conv2d` (checkpoints load directly).

  CUDA bf16 inputs run on this repository's implicit-GEMM kernels (`ops.functional.conv2d`: forward, input gradient
  and weight gradient) and come back in channels-last memory, which the GroupNorm and the attention blocks of the
  UNet / VAE consume as they are. `padding="far"` pads after the image only (the VAE's stride-2 down-sampling);
  `forward(x, upsample=True)` applies the convolution to the nearest-2x up-sampled input without building it.
  reference: the `nn.Conv` layers of src/maxdiffusion/models/resnet_flax.py:37-186 and vae_flax.py."""

  def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, bias=True):
    self.pad_mode = padding
    super().__init__(in_channels, out_channels, kernel_size, stride=stride, padding=0 if padding == "far" else padding, bias=bias)

  def forward(self, x, upsample: bool = False):
    return OF.conv2d(x, self.weight, self.bias, stride=self.stride[0], padding=self.pad_mode, upsample=upsample)


class GroupNorm(nn.GroupNorm):
  """GroupNorm with an optional fused SiLU (`act=True`); parameter names are those of `torch.nn.GroupNorm`.

  reference: the GroupNorm -> swish pairs of src/maxdiffusion/models/resnet_flax.py:150-176."""

  def forward(self, x, act: bool = False):
    return OF.group_norm(x, self.num_groups, self.weight, self.bias, self.eps, act)


class LayerNorm(nn.LayerNorm):
  """`nn.LayerNorm` (same parameters and checkpoint keys) whose [B, S, C] CUDA bf16 inputs run on this repository's row
  kernels, forward and backward (`ops.functional.layer_norm_mod`); statistics in fp32."""

  def forward(self, x):
    if x.dim() == 3 and self.elementwise_affine and len(self.normalized_shape) == 1:
      return OF.layer_norm_mod(x, self.weight, self.bias, eps=self.eps)
    return super().forward(x)


class FP32LayerNorm(nn.Module):
  """LayerNorm with statistics in fp32 (reference: src/maxdiffusion/models/normalization_flax.py:160-180)."""

  def __init__(self, dim: int, eps: float = 1e-6, elementwise_affine: bool = True):
    super().__init__()
    self.eps = eps
    self.weight = nn.Parameter(torch.ones(dim)) if elementwise_affine else None
    self.bias = nn.Parameter(torch.zeros(dim)) if elementwise_affine else None

  def forward(self, x):
    return OF.layer_norm_mod(x, gamma=self.weight, beta=self.bias, eps=self.eps)
