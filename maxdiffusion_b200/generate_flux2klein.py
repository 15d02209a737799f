"""python -m maxdiffusion_b200.generate_flux2klein <config.yml> key=value ...

reference: src/maxdiffusion/generate_flux2klein.py. `pretrained_model_name_or_path` is a local diffusers folder
(`transformer/`, `vae/`, `text_encoder/`, `tokenizer/`); `random_init: True` builds the architecture without weights.
Several prompts can be given separated by `||`; they are spread over the batch."""
import json
import os
import sys

import torch

from . import max_logging, pyconfig
from .models.flux.transformer_flux2_klein import FLUX2_KLEIN_PRESETS, Flux2KleinConfig, Flux2KleinTransformer2DModel
from .models.vae import VAE_PRESETS, AutoencoderKL, VAEConfig
from .parallel.mesh import init_distributed
from .pipelines.flux.flux2klein_pipeline import Flux2KleinPipeline
from .utils.export_utils import export_to_png


def partition_prompts(prompt: str, batch_size: int):
  parts = [p.strip() for p in prompt.split("||") if p.strip()]
  return [parts[i % len(parts)] for i in range(batch_size)]


def _read_dir(folder):
  from safetensors.torch import load_file

  out = {}
  for n in sorted(os.listdir(folder)):
    if n.endswith(".safetensors"):
      out.update(load_file(os.path.join(folder, n)))
  return out


def load_pipeline(config) -> Flux2KleinPipeline:
  device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
  dtype = config.weights_dtype if device.type == "cuda" else torch.float32
  root = config.pretrained_model_name_or_path
  bn_mean = bn_std = tok = enc = None
  if config.get("random_init", False) or not os.path.isdir(os.path.join(root, "transformer")):
    name = "flux2-klein-9b" if "9b" in str(config.get("flux_name", "")).lower() else "flux2-klein-4b"
    over = dict(FLUX2_KLEIN_PRESETS[config.get("flux_preset", "") or name])
    over.update(config.get("flux_config_overrides", {}) or {})
    model = Flux2KleinTransformer2DModel(Flux2KleinConfig(**over)).to(device, dtype)
    vover = dict(VAE_PRESETS["flux"], latent_channels=32)
    vover.update(config.get("vae_config_overrides", {}) or {})
    vae = AutoencoderKL(VAEConfig(**vover)).to(device, dtype)
  else:
    with open(os.path.join(root, "transformer", "config.json")) as f:
      model = Flux2KleinTransformer2DModel(Flux2KleinConfig.from_dict(json.load(f))).to(dtype)
    sd = {k: v.to(dtype) for k, v in _read_dir(os.path.join(root, "transformer")).items()}
    missing, unexpected = model.load_state_dict(sd, strict=False)
    if missing or unexpected:
      raise ValueError(f"Flux.2-Klein weight mapping: missing {missing[:4]}, unexpected {unexpected[:4]}")
    model = model.to(device)
    with open(os.path.join(root, "vae", "config.json")) as f:
      vae = AutoencoderKL(VAEConfig.from_dict(json.load(f)))
    vsd = _read_dir(os.path.join(root, "vae"))
    if "bn.running_mean" in vsd:
      bn_mean = vsd.pop("bn.running_mean").float()
      bn_std = torch.sqrt(vsd.pop("bn.running_var").float() + 1e-4)
    vae.load_state_dict(vsd, strict=False)
    vae = vae.to(device, dtype)
    if os.path.isdir(os.path.join(root, "text_encoder")):
      from transformers import AutoTokenizer

      from .models.qwen3 import Qwen3Model

      tok = AutoTokenizer.from_pretrained(os.path.join(root, "tokenizer"))
      enc = Qwen3Model.from_pretrained(os.path.join(root, "text_encoder"), dtype=dtype, device=device)
  return Flux2KleinPipeline(model.eval(), vae.eval(), enc, tok, vae_bn_mean=bn_mean, vae_bn_std=bn_std, device=device,
                            max_sequence_length=int(config.max_sequence_length))


def _write(config, images, name: str) -> list:
  out_dir = config.get("output_dir", "output/") or "."
  os.makedirs(out_dir, exist_ok=True)
  paths = []
  for i in range(images.shape[0]):
    path = os.path.join(out_dir, name if images.shape[0] == 1 else name.replace(".png", f"_b{i}.png"))
    paths.append(export_to_png(images[i].cpu().numpy(), path))
    max_logging.log("wrote " + paths[-1])
  return paths


def interactive_loop(config, pipe, kw, read=input) -> int:
  """Prompts typed at the console (several separated by `||` fill the batch) are generated one after another as
  `generated_NNN.png` until `exit` / `quit` / end of input; the starting noise is drawn fresh for every request
  (reference: src/maxdiffusion/generate_flux2klein.py:467-509). Returns how many requests were served."""
  B = int(config.get("batch_size", 1))
  max_logging.log(f"interactive mode: batch of {B}; prompts separated by '||'; 'exit' to quit")
  served = 0
  while True:
    try:
      text = read("\nEnter prompt(s): ")
    except (KeyboardInterrupt, EOFError):
      break
    if text.strip().lower() in ("exit", "quit"):
      break
    if not text.strip():
      continue
    served += 1
    images = pipe(**{**kw, "prompt": partition_prompts(text, B), "latents": None, "seed": int(config.seed) + served})
    if int(os.environ.get("RANK", "0")) == 0:
      _write(config, images, f"generated_{served:03d}.png")
  return served


def run(config, read=input):
  pipe = load_pipeline(config)
  B = int(config.get("batch_size", 1))
  kw = dict(height=int(config.resolution), width=int(config.resolution), num_inference_steps=int(config.num_inference_steps),
            batch_size=B, seed=int(config.seed))
  if pipe.text_encoder is None:
    g = torch.Generator().manual_seed(int(config.seed))
    kw["prompt_embeds"] = torch.randn((B, int(config.max_sequence_length), pipe.transformer.cfg.joint_attention_dim), generator=g)
  else:
    if not str(config.get("prompt", "") or "").strip():
      raise ValueError("a prompt must be given in the configuration file or as prompt='...'")
    kw["prompt"] = partition_prompts(str(config.prompt), B)
  pipe(**{**kw, "num_inference_steps": 1, "output_type": "latent"})   # warm-up
  if config.get("interactive", False):
    if pipe.text_encoder is None:
      raise ValueError("interactive mode needs the text encoder (a pretrained folder with text_encoder/ and tokenizer/)")
    kw.pop("prompt_embeds", None)
    return interactive_loop(config, pipe, kw, read)
  if str(config.get("latents_path", "") or ""):
    # custom starting noise: [B, 32, H/8, W/8], or already packed [B, tokens, 128]
    import numpy as np

    max_logging.log(f"loading the starting noise from {config.latents_path}")
    kw["latents"] = torch.from_numpy(np.load(str(config.latents_path))).float()
  reps = max(1, int(config.get("num_reps", 1)))
  traces, images = [], None
  for rep in range(reps):
    images, trace = pipe(**kw, return_trace=True)
    traces.append(trace)
    max_logging.log((f"[rep {rep + 1}/{reps}] " if reps > 1 else "") + "  ".join(f"{k}: {v:.4f}s" for k, v in trace.items()))
    if int(os.environ.get("RANK", "0")) == 0:
      name = str(config.get("output_name", "flux2klein_generated_image.png"))
      _write(config, images, f"rep_{rep + 1}_{name}" if reps > 1 else name)
  if reps > 1:
    max_logging.log("average over the repetitions: " + "  ".join(
        f"{k}: {sum(t.get(k, 0.0) for t in traces) / reps:.4f}s" for k in traces[0]))
  return images


def main(argv=None):
  init_distributed()
  run(pyconfig.initialize(list(sys.argv if argv is None else argv)))


if __name__ == "__main__":
  main()
