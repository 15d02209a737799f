"""Synthetic batches with the shapes of the real data, for benchmarking without a dataset.

Reference: src/maxdiffusion/input_pipeline/synthetic_data_iterator.py:192-452 (Wan: `latents`
[B,16,(F-1)/4+1,H/8,W/8] and `encoder_hidden_states` [B,512,4096] in fp32, dims derived from the config or
the `synthetic_override_*` keys; Flux: packed latents, T5 / CLIP embeddings, ids).
Batches are produced in pinned host memory so that the trainer's host-to-device copy is asynchronous.
"""
from __future__ import annotations

from typing import Iterator, Optional

import torch


def _pin(t: torch.Tensor) -> torch.Tensor:
  return t.pin_memory() if torch.cuda.is_available() else t


class SyntheticWanIterator:

  def __init__(self, config, batch_size: int, seed: int = 0, num_samples: Optional[int] = None,
               with_timesteps: bool = False):
    g = config.get
    self.height = int(g("synthetic_override_height", 0) or g("height", 480))
    self.width = int(g("synthetic_override_width", 0) or g("width", 832))
    self.frames = int(g("synthetic_override_num_frames", 0) or g("num_frames", 81))
    self.text_len = int(g("synthetic_override_text_len", 0) or g("max_sequence_length", 512))
    self.text_dim = int(g("synthetic_override_text_dim", 0) or 4096)
    self.channels = int(g("synthetic_override_latent_channels", 0) or 16)
    self.batch_size = batch_size
    self.num_samples = num_samples
    self.with_timesteps = with_timesteps
    self.gen = torch.Generator().manual_seed(seed)
    self.produced = 0

  @property
  def latent_shape(self):
    return (self.batch_size, self.channels, (self.frames - 1) // 4 + 1, self.height // 8, self.width // 8)

  def __iter__(self) -> Iterator[dict]:
    return self

  def __next__(self) -> dict:
    if self.num_samples is not None and self.produced >= self.num_samples:
      raise StopIteration
    self.produced += self.batch_size
    batch = {
        "latents": _pin(torch.randn(self.latent_shape, generator=self.gen, dtype=torch.float32)),
        "encoder_hidden_states": _pin(torch.randn((self.batch_size, self.text_len, self.text_dim), generator=self.gen,
                                                  dtype=torch.float32)),
    }
    if self.with_timesteps:
      batch["timesteps"] = torch.randint(0, 1000, (self.batch_size,), generator=self.gen, dtype=torch.int32)
    return batch


class SyntheticFluxIterator:
  """Packed latents [B, (H/16)*(W/16), 64], T5 embeddings [B,512,4096], CLIP pooled [B,768], position ids."""

  def __init__(self, config, batch_size: int, seed: int = 0, num_samples: Optional[int] = None, text_dim: int = 4096,
               pooled_dim: int = 768, latent_dim: int = 64):
    g = config.get
    self.res = int(g("resolution", 1024))
    self.text_len = int(g("max_sequence_length", 512))
    self.text_dim, self.pooled_dim, self.latent_dim = text_dim, pooled_dim, latent_dim
    self.batch_size, self.num_samples, self.produced = batch_size, num_samples, 0
    self.gen = torch.Generator().manual_seed(seed)

  def __iter__(self):
    return self

  def __next__(self) -> dict:
    if self.num_samples is not None and self.produced >= self.num_samples:
      raise StopIteration
    self.produced += self.batch_size
    h = w = self.res // 16
    B = self.batch_size
    ids = torch.zeros(h, w, 3)
    ids[..., 1] = torch.arange(h)[:, None]
    ids[..., 2] = torch.arange(w)[None, :]
    return {
        "pixel_values": _pin(torch.randn((B, h * w, self.latent_dim), generator=self.gen)),
        "text_embeds": _pin(torch.randn((B, self.text_len, self.text_dim), generator=self.gen)),
        "prompt_embeds": _pin(torch.randn((B, self.pooled_dim), generator=self.gen)),
        "img_ids": ids.reshape(1, h * w, 3).expand(B, -1, -1).contiguous(),
        "txt_ids": (txt := torch.zeros((B, self.text_len, 3))),
        "input_ids": txt,  # the reference's name for the text position ids (the same tensor)
    }


def make_synthetic_iterator(config, batch_size: int, seed: int = 0, is_training: bool = True, **kw):
  """Random batches of the model family's shapes. `is_training=False` builds evaluation batches: Wan batches then carry
  the `timesteps` the loss is evaluated at (reference: src/maxdiffusion/input_pipeline/synthetic_data_iterator.py)."""
  name = str(config.get("model_name", "wan2.1"))
  if name.startswith("flux"):
    return SyntheticFluxIterator(config, batch_size, seed, **kw)
  if not is_training:
    kw.setdefault("with_timesteps", True)
  return SyntheticWanIterator(config, batch_size, seed, **kw)
