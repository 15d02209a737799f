"""python -m maxdiffusion_b200.generate_zimage <config.yml> key=value ...   (reference: src/maxdiffusion/generate_zimage.py)"""
import os
import sys

import torch

from . import max_logging, pyconfig
from .checkpointing.z_image_checkpointer import ZImageCheckpointer
from .parallel.mesh import init_distributed
from .utils.export_utils import export_to_png


def run(config):
  pipe = ZImageCheckpointer(config).load_pipeline()
  batch = max(1, int(float(config.per_device_batch_size)))
  kw = dict(height=int(config.height), width=int(config.width), num_inference_steps=int(config.num_inference_steps),
            seed=int(config.seed), max_sequence_length=int(config.max_sequence_length),
            vae_decode_chunk=int(config.get("vae_decode_chunk", 1)))
  if pipe.text_encoder is None:
    g = torch.Generator().manual_seed(int(config.seed))
    dim = pipe.transformer.cfg.cap_feat_dim
    kw["prompt_embeds"] = [torch.randn((64, dim), generator=g) for _ in range(batch)]
  else:
    kw["prompt"] = [config.prompt] * batch
  pipe(**{**kw, "num_inference_steps": 1, "output_type": "latent"})  # warm-up (allocator, kernel library)
  images, trace = pipe(**kw, return_timings=True)
  total = sum(trace.values())
  max_logging.log("  ".join(f"{k}: {v:.3f}s" for k, v in trace.items()) + f"  total: {total:.3f}s")
  if int(os.environ.get("RANK", "0")) == 0:
    out = config.get("output_file", "") or os.path.join(config.get("output_dir", ".") or ".", "zimage.png")
    os.makedirs(os.path.dirname(out) or ".", exist_ok=True)
    root, ext = os.path.splitext(out)
    for i in range(images.shape[0]):
      max_logging.log("wrote " + export_to_png(images[i].cpu().numpy(), out if i == 0 else f"{root}_{i}{ext}"))
  return images


def main(argv=None):
  init_distributed()
  run(pyconfig.initialize(list(sys.argv if argv is None else argv)))


if __name__ == "__main__":
  main()
