"""Prompt enhancement for LTX-Video: a language model rewrites a short user prompt into a detailed cinematic one; for
image-to-video the first conditioning frame is captioned by an image-caption model first and the caption is given
to the language model with the prompt (reference: src/maxdiffusion/models/ltx_video/utils/prompt_enhance_utils.py:80-205).
Both models are Hugging Face `generate` models passed in by the caller; nothing here is specific to a checkpoint.
"""
from __future__ import annotations

from typing import List, Optional, Union

import torch

from ....utils import logging

logger = logging.get_logger(__name__)

T2V_CINEMATIC_PROMPT = (
    "You are an expert cinematic director with many award winning movies. When writing prompts based on the user input, "
    "focus on detailed, chronological descriptions of actions and scenes. Include specific movements, appearances, camera "
    "angles, and environmental details - all in a single flowing paragraph. Start directly with the action, and keep "
    "descriptions literal and precise. Think like a cinematographer describing a shot list. Do not change the user input "
    "intent, just enhance it. Keep within 150 words. For best results, build your prompts using this structure: start with "
    "main action in a single sentence; add specific details about movements and gestures; describe character/object "
    "appearances precisely; include background and environment details; specify camera angles and movements; describe "
    "lighting and colors; note any changes or sudden events. Do not exceed the 150 word limit! Output the enhanced prompt only.")
I2V_CINEMATIC_PROMPT = (
    "You are an expert cinematic director with many award winning movies. When writing prompts based on the user input and "
    "the image caption, focus on detailed, chronological descriptions of actions and scenes that continue from the image. "
    "Include specific movements, appearances, camera angles, and environmental details - all in a single flowing paragraph. "
    "Start directly with the action, and keep descriptions literal and precise. Do not change the user input intent, just "
    "enhance it, and stay consistent with the image caption. Keep within 150 words. Output the enhanced prompt only.")


def tensor_to_pil(t: torch.Tensor):
  """[3,H,W] in [-1,1] -> PIL image."""
  from PIL import Image

  a = ((t.detach().float().cpu().clamp(-1, 1) + 1) / 2 * 255).round().to(torch.uint8).permute(1, 2, 0).numpy()
  return Image.fromarray(a)


def first_frames_of(conditioning_item) -> list:
  m = conditioning_item.media_item  # [B,3,F,H,W]
  return [tensor_to_pil(m[i, :, 0]) for i in range(m.shape[0])]


def _chat(tokenizer, system: str, user: str) -> str:
  return tokenizer.apply_chat_template([{"role": "system", "content": system}, {"role": "user", "content": user}],
                                       tokenize=False, add_generation_prompt=True)


def _generate(model, tokenizer, texts: List[str], max_new_tokens: int) -> List[str]:
  inputs = tokenizer(texts, return_tensors="pt", padding=len(texts) > 1)
  inputs = inputs.to(model.device) if hasattr(inputs, "to") else inputs
  with torch.inference_mode():
    out = model.generate(**inputs, max_new_tokens=max_new_tokens)
  new = [o[len(i):] for i, o in zip(inputs["input_ids"], out)]
  return tokenizer.batch_decode(new, skip_special_tokens=True)


def caption_images(caption_model, caption_processor, images: list, task: str = "<DETAILED_CAPTION>") -> List[str]:
  inputs = caption_processor([task] * len(images), images, return_tensors="pt")
  inputs = inputs.to(caption_model.device) if hasattr(inputs, "to") else inputs
  with torch.inference_mode():
    ids = caption_model.generate(input_ids=inputs["input_ids"], pixel_values=inputs["pixel_values"], max_new_tokens=1024,
                                 do_sample=False, num_beams=3)
  return caption_processor.batch_decode(ids, skip_special_tokens=True)


def generate_cinematic_prompt(image_caption_model, image_caption_processor, prompt_enhancer_model, prompt_enhancer_tokenizer,
                              prompt: Union[str, List[str]], conditioning_items: Optional[list] = None,
                              max_new_tokens: int = 256) -> List[str]:
  prompts = [prompt] if isinstance(prompt, str) else list(prompt)
  if not conditioning_items:
    texts = [_chat(prompt_enhancer_tokenizer, T2V_CINEMATIC_PROMPT, f"user_prompt: {p}") for p in prompts]
    return _generate(prompt_enhancer_model, prompt_enhancer_tokenizer, texts, max_new_tokens)
  if len(conditioning_items) > 1 or conditioning_items[0].media_frame_number != 0:
    logger.warning("prompt enhancement supports no conditioning or one item at frame 0 only: returning the original prompts")
    return prompts
  frames = first_frames_of(conditioning_items[0])
  if len(frames) != len(prompts):
    raise ValueError(f"{len(frames)} conditioning frames for {len(prompts)} prompts")
  caps = caption_images(image_caption_model, image_caption_processor, frames)
  texts = [_chat(prompt_enhancer_tokenizer, I2V_CINEMATIC_PROMPT, f"user_prompt: {p}\nimage_caption: {c}") for p, c in zip(prompts, caps)]
  return _generate(prompt_enhancer_model, prompt_enhancer_tokenizer, texts, max_new_tokens)
