"""CLIP-based content filter of the Stable Diffusion pipelines.

An image is flagged when the cosine similarity between its projected CLIP image embedding and any of 17 concept
embeddings exceeds that concept's threshold; a match with one of 3 "special care" embeddings lowers all thresholds
by 0.01 first. Scores are rounded to 3 decimals before the comparison
(reference: src/maxdiffusion/pipelines/stable_diffusion/safety_checker_flax.py:32-72).
Parameter names match the `safety_checker` folder of the SD 1.x checkpoints, so it loads by name.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn


def cosine_distance(a: torch.Tensor, b: torch.Tensor, eps: float = 1e-12) -> torch.Tensor:
  a = a / a.norm(dim=1, keepdim=True).clamp_min(eps)
  b = b / b.norm(dim=1, keepdim=True).clamp_min(eps)
  return a @ b.T


class StableDiffusionSafetyChecker(nn.Module):

  def __init__(self, vision_model: nn.Module, hidden_size: int, projection_dim: int = 768):
    super().__init__()
    self.vision_model = vision_model  # returns (last_hidden_state, pooled_output) or an object with `.pooler_output`
    self.visual_projection = nn.Linear(hidden_size, projection_dim, bias=False)
    self.concept_embeds = nn.Parameter(torch.ones(17, projection_dim), requires_grad=False)
    self.special_care_embeds = nn.Parameter(torch.ones(3, projection_dim), requires_grad=False)
    self.concept_embeds_weights = nn.Parameter(torch.ones(17), requires_grad=False)
    self.special_care_embeds_weights = nn.Parameter(torch.ones(3), requires_grad=False)

  @classmethod
  def from_pretrained(cls, folder: str, device=None):
    """`safety_checker/` folder of a diffusers SD checkpoint (a `CLIPConfig` + weights)."""
    from transformers import CLIPConfig, CLIPVisionModel

    from ...models.modeling_utils import read_state_dict

    cfg = CLIPConfig.from_pretrained(folder)
    m = cls(CLIPVisionModel(cfg.vision_config).vision_model, cfg.vision_config.hidden_size, cfg.projection_dim)
    sd = {k.replace("vision_model.vision_model.", "vision_model."): v for k, v in read_state_dict(folder).items()}
    m.load_state_dict(sd, strict=False)
    return m.to(device) if device is not None else m

  @torch.no_grad()
  def forward(self, clip_input: torch.Tensor, adjustment: float = 0.0) -> torch.Tensor:
    out = self.vision_model(clip_input)
    pooled = out.pooler_output if hasattr(out, "pooler_output") else out[1]
    emb = self.visual_projection(pooled).float()
    special = torch.round((cosine_distance(emb, self.special_care_embeds.float()) - self.special_care_embeds_weights.float()[None]
                           + adjustment) * 1000) / 1000
    special_adjust = (special > 0).any(dim=1, keepdim=True).float() * 0.01
    scores = torch.round((cosine_distance(emb, self.concept_embeds.float()) - self.concept_embeds_weights.float()[None]
                          + special_adjust) * 1000) / 1000
    return (scores > 0).any(dim=1)


def run_safety_checker(checker: Optional[StableDiffusionSafetyChecker], images_uint8: torch.Tensor, feature_extractor=None):
  """images [B,H,W,3] uint8 -> (images with flagged ones blacked out, flags)."""
  if checker is None:
    return images_uint8, torch.zeros(images_uint8.shape[0], dtype=torch.bool)
  p = next(checker.parameters())
  if feature_extractor is not None:
    clip_in = torch.as_tensor(feature_extractor(list(images_uint8.cpu().numpy()), return_tensors="pt").pixel_values)
  else:
    x = images_uint8.permute(0, 3, 1, 2).float() / 255.0
    x = torch.nn.functional.interpolate(x, size=(224, 224), mode="bicubic", align_corners=False).clamp(0, 1)
    mean = torch.tensor([0.48145466, 0.4578275, 0.40821073]).view(1, 3, 1, 1)
    std = torch.tensor([0.26862954, 0.26130258, 0.27577711]).view(1, 3, 1, 1)
    clip_in = (x - mean.to(x.device)) / std.to(x.device)
  flags = checker(clip_in.to(p.device, p.dtype)).cpu()
  out = images_uint8.clone()
  out[flags.to(out.device)] = 0
  return out, flags
