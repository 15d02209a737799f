"""LTX-2 joint audio + video diffusion transformer.

Reference: src/maxdiffusion/models/ltx2/transformer_ltx2.py — `LTX2AdaLayerNormSingle` (:78-137),
`LTX2VideoTransformerBlock` (:140-763), `LTX2VideoTransformer3DModel` (:766-1765).

One block (both streams advance together):
  video self-attn, audio self-attn (AdaLN: RMSNorm without affine * (1 + scale) + shift; gated residual);
  video x text and audio x text cross-attention (with `cross_attn_mod`: modulated query, modulated text K/V
    through `prompt_scale_shift_table`, gated output);
  audio -> video and video -> audio cross-attention with their own 5-row tables (4 scale/shift rows + 1 gate) added
    to cross-attention time embeddings; `modality_mask` zeroes both for the "isolated" guidance branch;
  video FFN, audio FFN (Linear -> GELU -> Linear, gated residual).
Spatio-temporal guidance: blocks listed in `spatio_temporal_guidance_blocks` get `perturbation_mask` ([B,1,1],
0 = perturbed sample) in their self-attentions.
`compute_kv_cache` projects the text K/V of every block once per prompt; `precompute_time_embeds` evaluates the six
timestep embedders for all sampling steps up front; both are what the sampling loop reuses.
Parameter names follow the diffusers `LTX2VideoTransformer3DModel` checkpoint.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import functional as OF
from ..embeddings import PixArtAlphaTextProjection, TimestepEmbedding, Timesteps
from ..layers import Linear, RMSNorm
from .attention_ltx2 import LTX2Attention, LTX2RotaryPosEmbed


@dataclass
class LTX2Config:
  in_channels: int = 128
  out_channels: int = 128
  patch_size: int = 1
  patch_size_t: int = 1
  num_attention_heads: int = 32
  attention_head_dim: int = 128
  cross_attention_dim: int = 4096
  vae_scale_factors: Sequence[int] = (8, 32, 32)
  pos_embed_max_pos: int = 20
  base_height: int = 2048
  base_width: int = 2048
  audio_in_channels: int = 128
  audio_out_channels: int = 128
  audio_patch_size: int = 1
  audio_patch_size_t: int = 1
  audio_num_attention_heads: int = 32
  audio_attention_head_dim: int = 64
  audio_cross_attention_dim: int = 2048
  audio_scale_factor: int = 4
  audio_pos_embed_max_pos: int = 20
  audio_sampling_rate: int = 16000
  audio_hop_length: int = 160
  num_layers: int = 48
  activation_fn: str = "gelu-approximate"
  norm_eps: float = 1e-6
  caption_channels: int = 3840
  attention_bias: bool = True
  attention_out_bias: bool = True
  rope_theta: float = 10000.0
  causal_offset: int = 1
  timestep_scale_multiplier: int = 1000
  cross_attn_timestep_scale_multiplier: int = 1000
  rope_type: str = "interleaved"
  gated_attn: bool = False
  cross_attn_mod: bool = False
  use_prompt_embeddings: bool = True
  perturbed_attn: bool = False
  spatio_temporal_guidance_blocks: Sequence[int] = ()

  @property
  def inner_dim(self):
    return self.num_attention_heads * self.attention_head_dim

  @property
  def audio_inner_dim(self):
    return self.audio_num_attention_heads * self.audio_attention_head_dim

  @classmethod
  def from_dict(cls, d):
    return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

  def to_dict(self):
    return {k: (list(v) if isinstance(v, tuple) else v) for k, v in self.__dict__.items()}


LTX2_PRESETS = {
    "ltx2-19b": dict(),
    "ltx2.3": dict(gated_attn=True, cross_attn_mod=True, perturbed_attn=True, rope_type="split",
                   spatio_temporal_guidance_blocks=(29,)),
    "tiny": dict(in_channels=16, out_channels=16, num_attention_heads=2, attention_head_dim=32, cross_attention_dim=64,
                 audio_in_channels=8, audio_out_channels=8, audio_num_attention_heads=2, audio_attention_head_dim=16,
                 audio_cross_attention_dim=32, num_layers=2, caption_channels=24),
}


class LTX2AdaLayerNormSingle(nn.Module):
  """timestep -> (num_mod_params * dim modulation, embedded timestep)."""

  def __init__(self, embedding_dim: int, num_mod_params: int = 6):
    super().__init__()
    self.time_proj = Timesteps(256, flip_sin_to_cos=True, freq_shift=0.0)
    self.emb = nn.ModuleDict({"timestep_embedder": TimestepEmbedding(256, embedding_dim)})
    self.linear = Linear(embedding_dim, num_mod_params * embedding_dim)

  def forward(self, timestep, dtype):
    e = self.emb["timestep_embedder"](self.time_proj(timestep).to(dtype))
    return self.linear(F.silu(e)), e


class FeedForward(nn.Module):

  def __init__(self, dim: int, activation_fn: str = "gelu-approximate", mult: int = 4):
    super().__init__()
    self.net = nn.ModuleList([nn.ModuleDict({"proj": Linear(dim, dim * mult)}), nn.Identity(), Linear(dim * mult, dim)])
    self.tanh = activation_fn in ("gelu-approximate", "gelu_tanh")

  def forward(self, x):
    proj = self.net[0]["proj"]
    h = proj(x, activation="gelu_tanh") if self.tanh else F.gelu(proj(x))
    return self.net[2](h)


def _ada(table: torch.Tensor, temb: torch.Tensor, n: int):
  """table [n, dim] + temb [B, T, n*dim] -> n tensors [B, T, dim] in fp32 (T = 1, or the token count)."""
  B, T = temb.shape[:2]
  v = table.float()[None, None] + temb.float().reshape(B, T, n, -1)
  return v.unbind(dim=2)


def _mod(x_norm, scale, shift):
  return (x_norm.float() * (1.0 + scale) + shift).to(x_norm.dtype)


def _gated_add(x, y, gate):
  """x + y * gate; per-sample gates (T == 1) take the fused kernel."""
  if gate.shape[1] == 1:
    return OF.gated_residual(x, y, gate[:, 0].contiguous())
  return (x.float() + y.float() * gate).to(x.dtype)


class LTX2VideoTransformerBlock(nn.Module):

  def __init__(self, cfg: LTX2Config):
    super().__init__()
    d, ad, eps = cfg.inner_dim, cfg.audio_inner_dim, cfg.norm_eps
    kw = dict(bias=cfg.attention_bias, out_bias=cfg.attention_out_bias, eps=eps, rope_type=cfg.rope_type, gated_attn=cfg.gated_attn)
    H, D, AH, AD = cfg.num_attention_heads, cfg.attention_head_dim, cfg.audio_num_attention_heads, cfg.audio_attention_head_dim
    norm = lambda n: RMSNorm(n, eps, elementwise_affine=False)
    self.norm1, self.attn1 = norm(d), LTX2Attention(d, H, D, **kw)
    self.audio_norm1, self.audio_attn1 = norm(ad), LTX2Attention(ad, AH, AD, **kw)
    self.norm2, self.attn2 = norm(d), LTX2Attention(d, H, D, context_dim=d, **kw)
    self.audio_norm2, self.audio_attn2 = norm(ad), LTX2Attention(ad, AH, AD, context_dim=ad, **kw)
    self.audio_to_video_norm, self.audio_to_video_attn = norm(d), LTX2Attention(d, AH, AD, context_dim=ad, **kw)
    self.video_to_audio_norm, self.video_to_audio_attn = norm(ad), LTX2Attention(ad, AH, AD, context_dim=d, **kw)
    self.norm3, self.ff = norm(d), FeedForward(d, cfg.activation_fn)
    self.audio_norm3, self.audio_ff = norm(ad), FeedForward(ad, cfg.activation_fn)
    self.cross_attn_mod = cfg.cross_attn_mod
    n = 9 if cfg.cross_attn_mod else 6
    self.scale_shift_table = nn.Parameter(torch.randn(n, d) / d ** 0.5)
    self.audio_scale_shift_table = nn.Parameter(torch.randn(n, ad) / ad ** 0.5)
    self.video_a2v_cross_attn_scale_shift_table = nn.Parameter(torch.randn(5, d) / d ** 0.5)
    self.audio_a2v_cross_attn_scale_shift_table = nn.Parameter(torch.randn(5, ad) / ad ** 0.5)
    if cfg.cross_attn_mod:
      self.prompt_scale_shift_table = nn.Parameter(torch.randn(2, d) / d ** 0.5)
      self.audio_prompt_scale_shift_table = nn.Parameter(torch.randn(2, ad) / ad ** 0.5)

  def compute_kv(self, text, audio_text):
    return {"attn2": self.attn2.compute_kv(text), "audio_attn2": self.audio_attn2.compute_kv(audio_text)}

  def forward(self, x, a, s: dict, perturbation_mask=None, layer_kv: Optional[dict] = None):
    """x: video tokens [B,S,d]; a: audio tokens [B,Sa,ad]; `s`: the step-constant context built by the model."""
    n = 9 if self.cross_attn_mod else 6
    v_ada = _ada(self.scale_shift_table, s["temb"], n)
    a_ada = _ada(self.audio_scale_shift_table, s["temb_audio"], n)
    text, audio_text = s["encoder_hidden_states"], s["audio_encoder_hidden_states"]

    # self-attention
    x = _gated_add(x, self.attn1(_mod(self.norm1(x), v_ada[1], v_ada[0]), rotary_emb=s["video_rotary_emb"],
                                 perturbation_mask=perturbation_mask), v_ada[2])
    a = _gated_add(a, self.audio_attn1(_mod(self.audio_norm1(a), a_ada[1], a_ada[0]), rotary_emb=s["audio_rotary_emb"],
                                       perturbation_mask=perturbation_mask), a_ada[2])

    # text cross-attention
    def text_cross(h, norm, attn, ada, table, temb_prompt, ctx, mask, kv):
      q = norm(h)
      if self.cross_attn_mod:
        q = _mod(q, ada[7], ada[6])
        if temb_prompt is not None and kv is None:
          p = _ada(table, temb_prompt, 2)
          ctx = _mod(ctx, p[1], p[0])
      o = attn(q, encoder_hidden_states=ctx, attention_mask=mask, cached_kv=kv)
      if self.cross_attn_mod:
        return _gated_add(h, o, ada[8])
      return h + o

    x = text_cross(x, self.norm2, self.attn2, v_ada, getattr(self, "prompt_scale_shift_table", None), s.get("temb_prompt"),
                   text, s.get("encoder_attention_mask"), layer_kv.get("attn2") if layer_kv else None)
    a = text_cross(a, self.audio_norm2, self.audio_attn2, a_ada, getattr(self, "audio_prompt_scale_shift_table", None),
                   s.get("temb_prompt_audio"), audio_text, s.get("audio_encoder_attention_mask"),
                   layer_kv.get("audio_attn2") if layer_kv else None)

    # audio <-> video cross-attention
    nx, na = self.audio_to_video_norm(x), self.video_to_audio_norm(a)
    v_ca = _ada(self.video_a2v_cross_attn_scale_shift_table[:4], s["temb_ca_scale_shift"], 4)
    a_ca = _ada(self.audio_a2v_cross_attn_scale_shift_table[:4], s["temb_ca_audio_scale_shift"], 4)
    a2v_gate = _ada(self.video_a2v_cross_attn_scale_shift_table[4:], s["temb_ca_gate"], 1)[0]
    v2a_gate = _ada(self.audio_a2v_cross_attn_scale_shift_table[4:], s["temb_ca_audio_gate"], 1)[0]
    mm = s.get("modality_mask")
    a2v = self.audio_to_video_attn(_mod(nx, v_ca[0], v_ca[1]), encoder_hidden_states=_mod(na, a_ca[0], a_ca[1]),
                                   rotary_emb=s["ca_video_rotary_emb"], k_rotary_emb=s["ca_audio_rotary_emb"],
                                   attention_mask=s.get("a2v_cross_attention_mask"))
    v2a = self.video_to_audio_attn(_mod(na, a_ca[2], a_ca[3]), encoder_hidden_states=_mod(nx, v_ca[2], v_ca[3]),
                                   rotary_emb=s["ca_audio_rotary_emb"], k_rotary_emb=s["ca_video_rotary_emb"],
                                   attention_mask=s.get("v2a_cross_attention_mask"))
    if mm is not None:
      a2v, v2a = a2v * mm.to(a2v.dtype), v2a * mm.to(v2a.dtype)
    x = _gated_add(x, a2v, a2v_gate)
    a = _gated_add(a, v2a, v2a_gate)

    # feed-forward
    x = _gated_add(x, self.ff(_mod(self.norm3(x), v_ada[4], v_ada[3])), v_ada[5])
    a = _gated_add(a, self.audio_ff(_mod(self.audio_norm3(a), a_ada[4], a_ada[3])), a_ada[5])
    return x, a


class LTX2VideoTransformer3DModel(nn.Module):

  def __init__(self, cfg: LTX2Config):
    super().__init__()
    self.cfg = cfg
    d, ad = cfg.inner_dim, cfg.audio_inner_dim
    self.proj_in, self.audio_proj_in = Linear(cfg.in_channels, d), Linear(cfg.audio_in_channels, ad)
    if cfg.use_prompt_embeddings:
      self.caption_projection = PixArtAlphaTextProjection(cfg.caption_channels, d)
      self.audio_caption_projection = PixArtAlphaTextProjection(cfg.caption_channels, ad)
    else:
      self.caption_projection = self.audio_caption_projection = None
    n = 9 if cfg.cross_attn_mod else 6
    if cfg.cross_attn_mod:
      self.prompt_adaln, self.audio_prompt_adaln = LTX2AdaLayerNormSingle(d, 2), LTX2AdaLayerNormSingle(ad, 2)
    self.time_embed, self.audio_time_embed = LTX2AdaLayerNormSingle(d, n), LTX2AdaLayerNormSingle(ad, n)
    self.av_cross_attn_video_scale_shift = LTX2AdaLayerNormSingle(d, 4)
    self.av_cross_attn_audio_scale_shift = LTX2AdaLayerNormSingle(ad, 4)
    self.av_cross_attn_video_a2v_gate = LTX2AdaLayerNormSingle(d, 1)
    self.av_cross_attn_audio_v2a_gate = LTX2AdaLayerNormSingle(ad, 1)
    self.scale_shift_table = nn.Parameter(torch.randn(2, d) / d ** 0.5)
    self.audio_scale_shift_table = nn.Parameter(torch.randn(2, ad) / ad ** 0.5)
    rk = dict(theta=cfg.rope_theta, causal_offset=cfg.causal_offset, rope_type=cfg.rope_type)
    vk = dict(patch_size=cfg.patch_size, patch_size_t=cfg.patch_size_t, base_height=cfg.base_height, base_width=cfg.base_width)
    ak = dict(patch_size=cfg.audio_patch_size, patch_size_t=cfg.audio_patch_size_t, sampling_rate=cfg.audio_sampling_rate,
              hop_length=cfg.audio_hop_length)
    self.rope = LTX2RotaryPosEmbed(d, base_num_frames=cfg.pos_embed_max_pos, scale_factors=cfg.vae_scale_factors,
                                   modality="video", num_attention_heads=cfg.num_attention_heads, **vk, **rk)
    self.audio_rope = LTX2RotaryPosEmbed(ad, base_num_frames=cfg.audio_pos_embed_max_pos, scale_factors=[cfg.audio_scale_factor],
                                         modality="audio", num_attention_heads=cfg.audio_num_attention_heads, **ak, **rk)
    ca_max = max(cfg.pos_embed_max_pos, cfg.audio_pos_embed_max_pos)
    self.cross_attn_rope = LTX2RotaryPosEmbed(cfg.audio_cross_attention_dim, base_num_frames=ca_max, modality="video",
                                              num_attention_heads=cfg.num_attention_heads, **vk, **rk)
    self.cross_attn_audio_rope = LTX2RotaryPosEmbed(cfg.audio_cross_attention_dim, base_num_frames=ca_max, modality="audio",
                                                    num_attention_heads=cfg.audio_num_attention_heads, **ak, **rk)
    self.transformer_blocks = nn.ModuleList([LTX2VideoTransformerBlock(cfg) for _ in range(cfg.num_layers)])
    self.proj_out, self.audio_proj_out = Linear(d, cfg.out_channels or cfg.in_channels), Linear(ad, cfg.audio_out_channels or cfg.audio_in_channels)

  # ---- per-prompt / per-schedule caches ------------------------------------------------------
  def project_captions(self, text, audio_text):
    dtype = self.proj_in.weight.dtype
    if self.caption_projection is None:
      return text.to(dtype), audio_text.to(dtype)
    return self.caption_projection(text.to(dtype)), self.audio_caption_projection(audio_text.to(dtype))

  @torch.no_grad()
  def compute_kv_cache(self, encoder_hidden_states, audio_encoder_hidden_states):
    """Text K/V of every block (list of {"attn2": (k, v), "audio_attn2": (k, v)}), reference :1244-1311. Only valid
    without prompt modulation (`cross_attn_mod` changes the text per step)."""
    text, audio_text = self.project_captions(encoder_hidden_states, audio_encoder_hidden_states)
    if self.cfg.cross_attn_mod:
      # the prompt is modulated by the timestep (LTX-2.3), so its keys and values change every step and caching them
      # would bypass the modulation (the reference refuses the call: ltx2 `compute_kv_cache`); what does not depend on
      # the step -- the caption projections -- is still handed back, and `forward` recomputes K / V from it
      return None, (text, audio_text)
    return [blk.compute_kv(text, audio_text) for blk in self.transformer_blocks], (text, audio_text)

  def rope_tables(self, batch, num_frames, height, width, audio_num_frames, fps=24.0, device=None, video_coords=None,
                  audio_coords=None) -> dict:
    vc = video_coords if video_coords is not None else self.rope.prepare_video_coords(batch, num_frames, height, width, fps, device)
    ac = audio_coords if audio_coords is not None else self.audio_rope.prepare_audio_coords(batch, audio_num_frames, device=device)
    return {"video_rotary_emb": self.rope(vc), "audio_rotary_emb": self.audio_rope(ac),
            "ca_video_rotary_emb": self.cross_attn_rope(vc[:, 0:1]), "ca_audio_rotary_emb": self.cross_attn_audio_rope(ac[:, 0:1])}

  def time_embeds(self, timestep, audio_timestep=None, sigma=None, audio_sigma=None, use_cross_timestep=False) -> dict:
    """All timestep-dependent modulation inputs of one step; `timestep` [B] or per token [B, S] (already multiplied
    by `timestep_scale_multiplier` by the caller)."""
    cfg = self.cfg
    dtype = self.proj_in.weight.dtype
    B = timestep.shape[0]
    audio_timestep = audio_timestep if audio_timestep is not None else timestep
    shape = lambda t: t.reshape(B, -1, t.shape[-1])
    out = {}
    t, e = self.time_embed(timestep.flatten(), dtype)
    ta, ea = self.audio_time_embed(audio_timestep.flatten(), dtype)
    out.update(temb=shape(t), embedded_timestep=shape(e), temb_audio=shape(ta), audio_embedded_timestep=shape(ea))
    if cfg.cross_attn_mod and sigma is not None:
      audio_sigma = audio_sigma if audio_sigma is not None else sigma
      out["temb_prompt"] = shape(self.prompt_adaln(sigma.flatten(), dtype)[0])
      out["temb_prompt_audio"] = shape(self.audio_prompt_adaln(audio_sigma.flatten(), dtype)[0])
    if use_cross_timestep:
      if sigma is None or audio_sigma is None:
        raise ValueError("sigma and audio_sigma must be provided when use_cross_timestep is True")
      v_t, a_t = audio_sigma.flatten(), sigma.flatten()
    else:
      v_t, a_t = timestep.flatten(), audio_timestep.flatten()
    f = cfg.cross_attn_timestep_scale_multiplier / cfg.timestep_scale_multiplier
    out["temb_ca_scale_shift"] = shape(self.av_cross_attn_video_scale_shift(v_t, dtype)[0])
    out["temb_ca_gate"] = shape(self.av_cross_attn_video_a2v_gate(v_t * f, dtype)[0])
    out["temb_ca_audio_scale_shift"] = shape(self.av_cross_attn_audio_scale_shift(a_t, dtype)[0])
    out["temb_ca_audio_gate"] = shape(self.av_cross_attn_audio_v2a_gate(a_t * f, dtype)[0])
    return out

  @torch.no_grad()
  def precompute_time_embeds(self, timesteps: torch.Tensor, sigmas: Optional[torch.Tensor] = None) -> list:
    """Embeddings of every sampling step for batch 1 (reference :1313-1373); entries are expanded over the batch."""
    return [self.time_embeds(timesteps[i:i + 1], sigma=None if sigmas is None else sigmas[i:i + 1],
                             audio_sigma=None if sigmas is None else sigmas[i:i + 1]) for i in range(timesteps.shape[0])]

  # ---- forward -------------------------------------------------------------------------------
  def forward(self, hidden_states, audio_hidden_states, encoder_hidden_states, audio_encoder_hidden_states, timestep,
              audio_timestep=None, sigma=None, audio_sigma=None, encoder_attention_mask=None,
              audio_encoder_attention_mask=None, num_frames=None, height=None, width=None, fps: float = 24.0,
              audio_num_frames=None, video_coords=None, audio_coords=None, attention_kwargs: Optional[dict] = None,
              use_cross_timestep: bool = False, modality_mask=None, perturbation_mask=None, cached_kv=None,
              rope_cache: Optional[dict] = None, time_embed_cache: Optional[dict] = None):
    """hidden_states [B,S,in]; audio_hidden_states [B,Sa,audio_in]; text [B,T,caption] (or already projected when
    `cached_kv` comes with it). Returns (video prediction [B,S,out], audio prediction [B,Sa,audio_out])."""
    cfg = self.cfg
    dtype = self.proj_in.weight.dtype
    B = hidden_states.shape[0]
    for name, m in (("encoder_attention_mask", encoder_attention_mask), ("audio_encoder_attention_mask", audio_encoder_attention_mask)):
      if m is not None and (m.dim() != 2 or m.shape[0] != B or m.dtype != torch.bool):
        raise ValueError(f"{name} must be a boolean mask of shape [batch, kv_length], got {tuple(m.shape)} {m.dtype}")
    s = dict(rope_cache) if rope_cache is not None else self.rope_tables(
        B, num_frames, height, width, audio_num_frames, fps, hidden_states.device, video_coords, audio_coords)
    if time_embed_cache is not None:
      te = {k: v.expand(B, *v.shape[1:]) for k, v in time_embed_cache.items()}
    else:
      te = self.time_embeds(timestep, audio_timestep, sigma, audio_sigma, use_cross_timestep)
    s.update(te)
    x = self.proj_in(hidden_states.to(dtype))
    a = self.audio_proj_in(audio_hidden_states.to(dtype))
    if cached_kv is not None:
      layers_kv, (text, audio_text) = cached_kv
    else:
      layers_kv = None
      text, audio_text = self.project_captions(encoder_hidden_states, audio_encoder_hidden_states)
    ak = attention_kwargs or {}
    s.update(encoder_hidden_states=text, audio_encoder_hidden_states=audio_text, modality_mask=modality_mask,
             encoder_attention_mask=encoder_attention_mask, audio_encoder_attention_mask=audio_encoder_attention_mask,
             a2v_cross_attention_mask=ak.get("a2v_cross_attention_mask"), v2a_cross_attention_mask=ak.get("v2a_cross_attention_mask"))
    stg = set(int(i) for i in cfg.spatio_temporal_guidance_blocks)
    use_kv = layers_kv is not None and not (cfg.cross_attn_mod and s.get("temb_prompt") is not None)
    for i, blk in enumerate(self.transformer_blocks):
      pm = perturbation_mask if (perturbation_mask is not None and i in stg) else None
      x, a = blk(x, a, s, pm, layers_kv[i] if use_kv else None)
    sh = self.scale_shift_table.float()[None, None, 0] + s["embedded_timestep"].float()
    sc = self.scale_shift_table.float()[None, None, 1] + s["embedded_timestep"].float()
    out = self.proj_out(_mod(F.layer_norm(x.float(), (x.shape[-1],), eps=1e-6).to(x.dtype), sc, sh))
    ash = self.audio_scale_shift_table.float()[None, None, 0] + s["audio_embedded_timestep"].float()
    asc = self.audio_scale_shift_table.float()[None, None, 1] + s["audio_embedded_timestep"].float()
    audio_out = self.audio_proj_out(_mod(F.layer_norm(a.float(), (a.shape[-1],), eps=1e-6).to(a.dtype), asc, ash))
    return out, audio_out
