"""python -m maxdiffusion_b200.generate_ltx2 <config.yml> key=value ...   (reference: src/maxdiffusion/generate_ltx2.py)

Builds the pipeline (`LTX2Checkpointer`), optionally runs the attention tile search first (`enable_tile_search`),
installs the CUDA-graph / autotune cache keyed by the source revision (`aot_cache_dir`), generates, and writes the
video with its audio track."""
import os
import sys
import time

import torch

from . import max_logging, pyconfig
from .checkpointing.ltx2_checkpointer import LTX2Checkpointer
from .parallel.mesh import init_distributed
from .utils.export_utils import export_to_video, export_to_video_with_audio


def call_pipeline(config, pipe, **extra):
  kw = dict(height=int(config.height), width=int(config.width), num_frames=int(config.num_frames),
            frame_rate=float(config.fps), num_inference_steps=int(config.num_inference_steps),
            guidance_scale=float(config.guidance_scale), guidance_rescale=float(config.guidance_rescale),
            stg_scale=float(config.stg_scale), modality_scale=float(config.modality_scale),
            audio_guidance_scale=float(config.audio_guidance_scale) or None,
            audio_guidance_rescale=float(config.audio_guidance_rescale),
            audio_stg_scale=float(config.audio_stg_scale) if config.get("audio_stg_scale", None) is not None else None,
            audio_modality_scale=float(config.audio_modality_scale), decode_timestep=float(config.decode_timestep),
            decode_noise_scale=float(config.decode_noise_scale), max_sequence_length=int(config.max_sequence_length),
            use_cross_timestep=bool(config.use_cross_timestep), use_kv_cache=bool(config.get("use_kv_cache", False)) or True,
            noise_scale=float(config.noise_scale) if config.get("noise_scale", None) is not None else None,
            generator=torch.Generator().manual_seed(int(config.seed)))
  kw.update(extra)
  if pipe.text_encoder is None:
    g = torch.Generator().manual_seed(int(config.seed))
    factor_dim = pipe.connectors.feature_extractor.linear.in_features if hasattr(pipe.connectors.feature_extractor, "linear") \
        else pipe.connectors.feature_extractor.video_linear.in_features
    layers = int((config.get("ltx2_component_overrides", {}) or {}).get("connectors", {}).get("text_proj_in_factor", 49))
    T = int(config.max_sequence_length)
    mk = lambda: torch.randn((1, T, factor_dim // layers, layers), generator=g)
    kw.update(prompt_embeds=mk(), negative_prompt_embeds=mk(), prompt_attention_mask=torch.ones((1, T), dtype=torch.long),
              negative_prompt_attention_mask=torch.ones((1, T), dtype=torch.long))
  else:
    kw.update(prompt=config.prompt, negative_prompt=config.negative_prompt)
  return pipe(**kw)


def run(config):
  if config.get("aot_cache_dir", ""):
    from . import aot_cache

    aot_cache.install(config.aot_cache_dir, revision=config.get("aot_build_revision", "") or None)
  if config.get("enable_tile_search", False):
    from .utils.ltx2_block_benchmark import run_tile_search

    run_tile_search(config)
  t0 = time.perf_counter()
  pipe = LTX2Checkpointer(config).load_pipeline()
  max_logging.log(f"load_time: {time.perf_counter() - t0:.1f}s")
  lora = config.get("lora_config", None) or {}
  if config.get("enable_lora", False) and lora.get("lora_model_name_or_path"):
    from .loaders.lora_loader import merge_ltx2_loras

    merge_ltx2_loras(pipe, config)
  t0 = time.perf_counter()
  call_pipeline(config, pipe, num_inference_steps=2, output_type="latent")  # warm-up
  max_logging.log(f"warmup_time: {time.perf_counter() - t0:.1f}s")
  t0 = time.perf_counter()
  out = call_pipeline(config, pipe)
  max_logging.log(f"generation_time: {time.perf_counter() - t0:.1f}s  " + "  ".join(f"{k}: {v:.2f}s" for k, v in out.timings.items()))
  if int(os.environ.get("RANK", "0")) == 0:
    out_dir = config.get("output_dir", ".") or "."
    os.makedirs(out_dir, exist_ok=True)
    rate = getattr(pipe.vocoder, "output_sampling_rate", 24000)
    for i in range(out.frames.shape[0]):
      path = os.path.join(out_dir, f"ltx2_{config.seed}_{i}.mp4")
      frames = out.frames[i].cpu().numpy()
      if out.audio is not None:
        max_logging.log("wrote " + export_to_video_with_audio(frames, out.audio[i].cpu().numpy(), path, fps=int(config.fps), sample_rate=rate))
      else:
        max_logging.log("wrote " + export_to_video(frames, path, fps=int(config.fps)))
  return out


def main(argv=None):
  init_distributed()
  run(pyconfig.initialize(list(sys.argv if argv is None else argv)))


if __name__ == "__main__":
  main()
