"""Wan-Animate transformer: the Wan DiT with pose conditioning and a face-motion adapter.

Reference: src/maxdiffusion/models/wan/transformers/transformer_wan_animate.py
  * motion encoder (:52-450): a StyleGAN2-style discriminator trunk (equalised-LR convs, blur + stride-2
    down-sampling, fused leaky ReLU * sqrt 2) from a 512x512 face crop to a 512-d style vector, 5 equalised
    linears to a 20-d motion code, projected onto the orthonormal basis Q of `motion_synthesis_weight` (QR);
  * face encoder (:453-578): causal 1-D convs over time (replicate-left padding), two stride-2 stages (4x
    temporal compression to the latent frame rate), 4 heads + one learned padding token per frame;
  * face adapter (:581-745): every `inject_face_latents_blocks`-th block adds a cross-attention from the video
    tokens of latent frame t to the 5 face tokens of frame t (LayerNorm without affine on both sides, per-head
    RMSNorm on q and k);
  * pose latents are patch-embedded by their own projection and added to all frames but the first (:1096-1112).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import functional as OF
from ..layers import Linear, RMSNorm
from .transformer_wan import WAN_PRESETS, WanConfig, WanModel

MOTION_ENCODER_CHANNELS = {"4": 512, "8": 512, "16": 512, "32": 512, "64": 256, "128": 128, "256": 64, "512": 32,
                           "1024": 16}


@dataclass
class WanAnimateConfig(WanConfig):
  in_channels: int = 36
  latent_channels: int = 16
  image_dim: Optional[int] = 1280
  motion_encoder_size: int = 512
  motion_style_dim: int = 512
  motion_dim: int = 20
  motion_encoder_dim: int = 512
  face_encoder_hidden_dim: int = 1024
  face_encoder_num_heads: int = 4
  inject_face_latents_blocks: int = 5
  motion_encoder_batch_size: int = 8
  motion_encoder_channel_sizes: Optional[Dict[str, int]] = None


WAN_ANIMATE_PRESETS = {
    "wan2.2-animate-14b": dict(WAN_PRESETS["wan2.1-t2v-14b"], in_channels=36, image_dim=1280),
    "tiny": dict(num_attention_heads=2, attention_head_dim=32, ffn_dim=64, num_layers=2, text_dim=32, freq_dim=32,
                 in_channels=36, image_dim=24, motion_encoder_size=16, motion_style_dim=16, motion_dim=6,
                 motion_encoder_dim=16, face_encoder_hidden_dim=16, face_encoder_num_heads=2,
                 inject_face_latents_blocks=1, motion_encoder_batch_size=4,
                 motion_encoder_channel_sizes={"4": 16, "8": 16, "16": 8}),
}


class FusedLeakyReLU(nn.Module):

  def __init__(self, channels: Optional[int], negative_slope: float = 0.2, scale: float = 2 ** 0.5):
    super().__init__()
    self.negative_slope, self.scale = negative_slope, scale
    self.bias = nn.Parameter(torch.zeros(channels)) if channels is not None else None

  def forward(self, x, channel_dim: int = 1):
    if self.bias is not None:
      shape = [1] * x.dim()
      shape[channel_dim] = -1
      x = x + self.bias.reshape(shape).to(x.dtype)
    return F.leaky_relu(x, self.negative_slope) * self.scale


class MotionConv2d(nn.Module):
  """Equalised-LR conv (weight * 1/sqrt(fan_in)), optional depthwise blur before a strided conv."""

  def __init__(self, cin, cout, k, stride=1, padding=0, bias=True, blur_kernel: Optional[Sequence[int]] = None,
               use_activation=True):
    super().__init__()
    self.stride, self.padding, self.cin = stride, padding, cin
    self.weight = nn.Parameter(torch.randn(cout, cin, k, k))
    self.scale = 1.0 / math.sqrt(cin * k * k)
    self.bias = nn.Parameter(torch.zeros(cout)) if (bias and not use_activation) else None
    self.act_fn = FusedLeakyReLU(cout) if use_activation else None
    self.blur_padding = None
    if blur_kernel is not None:
      p = (len(blur_kernel) - stride) + (k - 1)
      self.blur_padding = ((p + 1) // 2, p // 2)
      kern = torch.tensor(blur_kernel, dtype=torch.float32)
      kern = kern[None, :] * kern[:, None]
      self.register_buffer("blur_kernel", kern / kern.sum(), persistent=False)

  def forward(self, x):
    if self.blur_padding is not None:
      k = self.blur_kernel.to(x.dtype)[None, None].expand(self.cin, 1, -1, -1)
      ph, pw = self.blur_padding
      # the reference pads (ph, ph) on the rows and (pw, pw) on the columns
      x = F.conv2d(F.pad(x, (pw, pw, ph, ph)), k, groups=self.cin)
    x = F.conv2d(x, self.weight.to(x.dtype) * self.scale, self.bias.to(x.dtype) if self.bias is not None else None,
                 stride=self.stride, padding=self.padding)
    return self.act_fn(x) if self.act_fn is not None else x


class MotionLinear(nn.Module):

  def __init__(self, din, dout, bias=True, use_activation=False):
    super().__init__()
    self.weight = nn.Parameter(torch.randn(dout, din))
    self.scale = 1.0 / math.sqrt(din)
    self.bias = nn.Parameter(torch.zeros(dout)) if (bias and not use_activation) else None
    self.act_fn = FusedLeakyReLU(dout) if use_activation else None

  def forward(self, x):
    y = F.linear(x, self.weight.to(x.dtype) * self.scale, self.bias.to(x.dtype) if self.bias is not None else None)
    return self.act_fn(y, channel_dim=-1) if self.act_fn is not None else y


class MotionEncoderResBlock(nn.Module):

  def __init__(self, cin, cout, blur_kernel=(1, 3, 3, 1)):
    super().__init__()
    self.conv1 = MotionConv2d(cin, cin, 3, stride=1, padding=1)
    self.conv2 = MotionConv2d(cin, cout, 3, stride=2, padding=0, blur_kernel=blur_kernel)
    self.conv_skip = MotionConv2d(cin, cout, 1, stride=2, padding=0, bias=False, blur_kernel=blur_kernel, use_activation=False)

  def forward(self, x):
    return (self.conv2(self.conv1(x)) + self.conv_skip(x)) / math.sqrt(2.0)


class WanAnimateMotionEncoder(nn.Module):

  def __init__(self, size=512, style_dim=512, motion_dim=20, out_dim=512, motion_blocks=5, channels=None):
    super().__init__()
    channels = channels or MOTION_ENCODER_CHANNELS
    self.size = size
    self.conv_in = MotionConv2d(3, channels[str(size)], 1)
    blocks, cin = [], channels[str(size)]
    for i in range(int(math.log2(size)), 2, -1):
      cout = channels[str(2 ** (i - 1))]
      blocks.append(MotionEncoderResBlock(cin, cout))
      cin = cout
    self.res_blocks = nn.ModuleList(blocks)
    self.conv_out = MotionConv2d(cin, style_dim, 4, padding=0, bias=False, use_activation=False)
    self.motion_network = nn.ModuleList([MotionLinear(style_dim, style_dim) for _ in range(motion_blocks - 1)] +
                                        [MotionLinear(style_dim, motion_dim)])
    self.motion_synthesis_weight = nn.Parameter(torch.randn(out_dim, motion_dim))

  def forward(self, face_image):
    if face_image.shape[-2] != self.size or face_image.shape[-1] != self.size:
      raise ValueError(f"Expected {self.size} got {face_image.shape[-1]}")
    x = self.conv_in(face_image)
    for blk in self.res_blocks:
      x = blk(x)
    feat = self.conv_out(x).squeeze(-1).squeeze(-1)
    for lin in self.motion_network:
      feat = lin(feat)
    q, _ = torch.linalg.qr(self.motion_synthesis_weight.float() + 1e-8)
    return (feat.float() @ q.t()).to(feat.dtype)


class WanAnimateFaceEncoder(nn.Module):

  def __init__(self, in_dim, out_dim, hidden_dim=1024, num_heads=4, kernel_size=3, eps=1e-6):
    super().__init__()
    self.num_heads, self.k, self.eps, self.out_dim = num_heads, kernel_size, eps, out_dim
    self.conv1_local = nn.Conv1d(in_dim, hidden_dim * num_heads, kernel_size)
    self.conv2 = nn.Conv1d(hidden_dim, hidden_dim, kernel_size, stride=2)
    self.conv3 = nn.Conv1d(hidden_dim, hidden_dim, kernel_size, stride=2)
    self.out_proj = nn.Linear(hidden_dim, out_dim)
    self.padding_tokens = nn.Parameter(torch.zeros(1, 1, 1, out_dim))

  def _stage(self, x, conv):
    """x: [N, T, C] -> causal conv over T (replicate padding on the left) -> LayerNorm (no affine) -> SiLU."""
    x = F.pad(x.transpose(1, 2), (self.k - 1, 0), mode="replicate")
    x = conv(x).transpose(1, 2)
    return F.silu(F.layer_norm(x, x.shape[-1:], eps=self.eps))

  def forward(self, x):
    """x: [B, T, in_dim] motion codes -> [B, T/4 (ceil), num_heads + 1, out_dim]."""
    B = x.shape[0]
    x = F.pad(x.transpose(1, 2), (self.k - 1, 0), mode="replicate")
    x = self.conv1_local(x).transpose(1, 2)                                      # [B, T, H*hidden]
    x = x.reshape(B, x.shape[1], self.num_heads, -1).permute(0, 2, 1, 3).reshape(B * self.num_heads, x.shape[1], -1)
    x = F.silu(F.layer_norm(x, x.shape[-1:], eps=self.eps))
    x = self._stage(x, self.conv2)
    x = self._stage(x, self.conv3)
    x = self.out_proj(x)
    x = x.reshape(B, self.num_heads, x.shape[1], x.shape[2]).permute(0, 2, 1, 3)
    pad = self.padding_tokens.to(x.dtype).expand(B, x.shape[1], 1, self.out_dim)
    return torch.cat([x, pad], dim=2)


class WanAnimateFaceBlockCrossAttention(nn.Module):

  def __init__(self, dim, heads, eps=1e-6):
    super().__init__()
    self.heads, self.eps = heads, eps
    d = dim // heads
    self.to_q, self.to_k, self.to_v = Linear(dim, dim), Linear(dim, dim), Linear(dim, dim)
    self.to_out = Linear(dim, dim)
    self.norm_q, self.norm_k = RMSNorm(d, eps), RMSNorm(d, eps)

  def forward(self, x, face, frames: int):
    """x: [B, S, dim] video tokens (S = frames * tokens_per_frame); face: [B, frames, n_kv, dim]."""
    B, S, dim = x.shape
    T, n_kv = face.shape[1], face.shape[2]
    if T != frames:
      raise ValueError(f"face latents cover {T} frames, the video tokens {frames}")
    d = dim // self.heads
    q = self.to_q(OF.layer_norm_mod(x, eps=self.eps))
    f = F.layer_norm(face.float(), (dim,), eps=self.eps).to(x.dtype)
    k, v = self.to_k(f), self.to_v(f)
    q = self.norm_q(q.reshape(B * T, S // T, self.heads, d))
    k = self.norm_k(k.reshape(B * T, n_kv, self.heads, d))
    o = OF.attention(q, k, v.reshape(B * T, n_kv, self.heads, d))
    return self.to_out(o.reshape(B, S, dim))


class WanAnimateModel(WanModel):
  """`forward(latents, t, text, encoder_hidden_states_image, pose_hidden_states, face_pixel_values | face_motion_vec)`."""

  def __init__(self, cfg: WanAnimateConfig, remat_policy: str = "NONE"):
    super().__init__(cfg, remat_policy)
    pt, ph, pw = cfg.patch_size
    self.pose_patch_embedding = Linear(cfg.latent_channels * pt * ph * pw, cfg.dim)
    self.motion_encoder = WanAnimateMotionEncoder(cfg.motion_encoder_size, cfg.motion_style_dim, cfg.motion_dim,
                                                  cfg.motion_encoder_dim, channels=cfg.motion_encoder_channel_sizes)
    self.face_encoder = WanAnimateFaceEncoder(cfg.motion_encoder_dim, cfg.dim, cfg.face_encoder_hidden_dim,
                                              cfg.face_encoder_num_heads)
    n = (cfg.num_layers + cfg.inject_face_latents_blocks - 1) // cfg.inject_face_latents_blocks
    self.face_adapter = nn.ModuleList([WanAnimateFaceBlockCrossAttention(cfg.dim, cfg.num_attention_heads, cfg.eps)
                                       for _ in range(n)])

  @torch.no_grad()
  def encode_face_motion(self, face_pixel_values: torch.Tensor, batch_size: int, chunk: Optional[int] = None):
    """[B, 3, T, H, W] face crops -> face latents [B, 1 + T/4, heads + 1, dim] (leading zero frame). Call once per
    segment and pass the result as `face_motion_vec` (reference :1018-1066)."""
    B, C, T, H, W = face_pixel_values.shape
    frames = face_pixel_values.permute(0, 2, 1, 3, 4).reshape(-1, C, H, W)
    chunk = chunk or self.cfg.motion_encoder_batch_size
    mdtype = self.motion_encoder.motion_synthesis_weight.dtype
    codes = torch.cat([self.motion_encoder(frames[i:i + chunk].to(mdtype)) for i in range(0, frames.shape[0], chunk)])
    face = self.face_encoder(codes.reshape(batch_size, T, -1).to(self.face_encoder.out_proj.weight.dtype))
    return torch.cat([torch.zeros_like(face[:, :1]), face], dim=1)

  def forward(self, hidden_states, timestep, encoder_hidden_states, encoder_hidden_states_image=None,
              pose_hidden_states=None, face_pixel_values=None, face_motion_vec=None, pctx=None, **kw):
    cfg = self.cfg
    if pctx is not None:
      raise NotImplementedError("the face adapter attends per frame; run Wan-Animate without context parallelism")
    B, _, Fr, H, W = hidden_states.shape
    if pose_hidden_states is not None and pose_hidden_states.shape[2] + 1 != Fr:
      raise ValueError(f"Pose frames + 1 ({pose_hidden_states.shape[2]} + 1) must equal hidden_states frames ({Fr})")
    dtype = self.patch_embedding.weight.dtype
    motion = face_motion_vec
    if motion is None and face_pixel_values is not None:
      motion = self.encode_face_motion(face_pixel_values, B)
    pose_tokens = None
    if pose_hidden_states is not None:
      tok, _ = self.patchify(pose_hidden_states.to(dtype))
      pose = self.pose_patch_embedding(tok)                                       # frames 1..F-1
      per_frame = pose.shape[1] // pose_hidden_states.shape[2]
      pose_tokens = torch.cat([pose.new_zeros((B, per_frame, pose.shape[2])), pose], dim=1)

    frames = Fr // cfg.patch_size[0]

    def post(i, x):
      if motion is not None and i % cfg.inject_face_latents_blocks == 0:
        x = x + self.face_adapter[i // cfg.inject_face_latents_blocks](x, motion.to(x.dtype), frames)
      return x

    return super().forward(hidden_states, timestep, encoder_hidden_states, encoder_hidden_states_image,
                           block_post=post, token_bias=pose_tokens, **kw)
