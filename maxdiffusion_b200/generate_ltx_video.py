"""python -m maxdiffusion_b200.generate_ltx_video <config.yml> key=value ...   (reference: src/maxdiffusion/generate_ltx_video.py)

`pipeline_type: multi-scale` runs the two-pass pipeline (first pass at `downscale_factor`, latent up-sampler, second
pass); anything else runs a single pass with the first-pass schedule. `num_frames` is rounded to 8k + 1 and the
resolution to multiples of 32, as the reference pads its inputs (generate_ltx_video.py:60-110)."""
import json
import os
import sys
import time

import torch

from . import max_logging, pyconfig
from .models.ltx2.autoencoder_kl_ltx2 import LTX2VAEConfig, LTX2VideoAutoencoderKL
from .models.ltx2.latent_upsampler_ltx2 import LTX2LatentUpsamplerModel
from .models.ltx_video.transformer3d import LTXV_PRESETS, LTXVideoConfig, Transformer3DModel
from .parallel.mesh import init_distributed
from .pipelines.ltx_video.ltx_video_pipeline import STG_MODES, LTXMultiScalePipeline, LTXVideoPipeline
from .utils.export_utils import export_to_video


def load_pipeline(config):
  device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
  dtype = config.weights_dtype if device.type == "cuda" else torch.float32
  root = str(config.pretrained_model_name_or_path)
  over = config.get("ltxv_component_overrides", {}) or {}
  tcfg = dict(LTXV_PRESETS[str(config.get("ltxv_preset", "ltxv-13b"))])
  tcfg.update(config.get("ltxv_config_overrides", {}) or {})
  text_encoder = tokenizer = None
  if not config.get("random_init", False) and os.path.isdir(os.path.join(root, "transformer")):
    from safetensors.torch import load_file

    def read(folder):
      out = {}
      for n in sorted(os.listdir(folder)):
        if n.endswith(".safetensors"):
          out.update(load_file(os.path.join(folder, n)))
      return out

    with open(os.path.join(root, "transformer", "config.json")) as f:
      transformer = Transformer3DModel(LTXVideoConfig.from_dict(json.load(f))).to(dtype)
    transformer.load_state_dict({k: v.to(dtype) for k, v in read(os.path.join(root, "transformer")).items()}, strict=False)
    with open(os.path.join(root, "vae", "config.json")) as f:
      vae = LTX2VideoAutoencoderKL(LTX2VAEConfig.from_dict(json.load(f)))
    vae.load_state_dict(read(os.path.join(root, "vae")), strict=False)
    if os.path.isdir(os.path.join(root, "text_encoder")):
      from transformers import T5EncoderModel, T5TokenizerFast

      text_encoder = T5EncoderModel.from_pretrained(os.path.join(root, "text_encoder"), torch_dtype=dtype).to(device).eval()
      tokenizer = T5TokenizerFast.from_pretrained(os.path.join(root, "tokenizer"))
  else:
    transformer = Transformer3DModel(LTXVideoConfig(**tcfg)).to(dtype)
    vae = LTX2VideoAutoencoderKL(LTX2VAEConfig(**({"timestep_conditioning": True, "decoder_causal": True} | over.get("vae", {}))))
  pipe = LTXVideoPipeline(transformer.to(device).eval(), vae.to(device).eval(), text_encoder, tokenizer, device=device)
  upsampler = None
  if str(config.get("pipeline_type", "")) == "multi-scale":
    upsampler = LTX2LatentUpsamplerModel(**({"in_channels": transformer.cfg.in_channels, "rational_spatial_scale": None, "dims": 3}
                                            | over.get("latent_upsampler", {}))).to(device).eval()
    path = str(config.get("spatial_upscaler_model_path", ""))
    if os.path.isfile(path) and not config.get("random_init", False):
      from safetensors.torch import load_file

      upsampler.load_state_dict(load_file(path), strict=False)
  return pipe, upsampler


def run(config):
  pipe, upsampler = load_pipeline(config)
  H = (int(config.height) + 31) // 32 * 32
  W = (int(config.width) + 31) // 32 * 32
  Fr = (int(config.num_frames) - 2) // 8 * 8 + 9 if (int(config.num_frames) - 1) % 8 else int(config.num_frames)
  common = dict(frame_rate=float(config.frame_rate), seed=int(config.seed), decode_timestep=float(config.decode_timestep),
                decode_noise_scale=float(config.decode_noise_scale), max_sequence_length=int(config.max_sequence_length),
                skip_layer_strategy=STG_MODES[str(config.get("stg_mode", "attention_values")).lower()])
  if pipe.text_encoder is None:
    g = torch.Generator().manual_seed(int(config.seed))
    T, D = int(config.max_sequence_length), pipe.transformer.cfg.caption_channels
    common.update(prompt_embeds=torch.randn((1, T, D), generator=g), negative_prompt_embeds=torch.randn((1, T, D), generator=g),
                  prompt_attention_mask=torch.ones((1, T), dtype=torch.long), negative_prompt_attention_mask=torch.ones((1, T), dtype=torch.long))
  else:
    common.update(prompt=config.prompt, negative_prompt=config.get("negative_prompt", ""))
  t0 = time.perf_counter()
  first, second = dict(config.first_pass), dict(config.second_pass)
  if upsampler is not None:
    video = LTXMultiScalePipeline(pipe, upsampler)(H, W, Fr, first, second, float(config.downscale_factor), **common)
  else:
    video = pipe(height=H, width=W, num_frames=Fr, **{**common, **first})
  max_logging.log(f"generation_time: {time.perf_counter() - t0:.1f}s")
  video = video[:, :int(config.num_frames), :int(config.height), :int(config.width)]
  if int(os.environ.get("RANK", "0")) == 0:
    out_dir = config.get("output_dir", ".") or "."
    os.makedirs(out_dir, exist_ok=True)
    for i in range(video.shape[0]):
      max_logging.log("wrote " + export_to_video(video[i].cpu().numpy(), os.path.join(out_dir, f"ltx_video_{config.seed}_{i}.mp4"),
                                                 fps=int(config.frame_rate)))
  return video


def main(argv=None):
  init_distributed()
  run(pyconfig.initialize(list(sys.argv if argv is None else argv)))


if __name__ == "__main__":
  main()
