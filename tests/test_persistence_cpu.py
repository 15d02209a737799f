"""`save_model` / `load_model` / pipeline folders: every model family round-trips through the diffusers layout."""
import json
import os

import pytest
import torch

from maxdiffusion_b200.models.modeling_utils import config_to_dict, load_model, read_state_dict, save_model


def _families():
  from maxdiffusion_b200.models.flux.transformer_flux import FLUX_PRESETS, FluxConfig, FluxTransformer2DModel
  from maxdiffusion_b200.models.unet_2d_condition import UNET_PRESETS, UNet2DConditionModel, UNetConfig
  from maxdiffusion_b200.models.vae import AutoencoderKL, VAEConfig
  from maxdiffusion_b200.models.wan.transformer_wan import WAN_PRESETS, WanConfig, WanModel
  from maxdiffusion_b200.models.z_image.transformer_z_image import ZIMAGE_PRESETS, ZImageConfig, ZImageTransformer2DModel

  yield WanModel, WanConfig(**WAN_PRESETS["tiny"])
  yield FluxTransformer2DModel, FluxConfig(**FLUX_PRESETS["tiny"])
  yield UNet2DConditionModel, UNetConfig(**UNET_PRESETS["tiny"])
  yield AutoencoderKL, VAEConfig(block_out_channels=(32, 32), layers_per_block=1, norm_num_groups=8)
  z = ZIMAGE_PRESETS["tiny"]
  yield ZImageTransformer2DModel, z if isinstance(z, ZImageConfig) else ZImageConfig(**z)


@pytest.mark.parametrize("shard", ["10GB", "64KB"])
def test_model_round_trip(tmp_path, shard):
  for cls, cfg in _families():
    torch.manual_seed(0)
    m = cls(cfg)
    folder = str(tmp_path / cls.__name__)
    save_model(m, folder, max_shard_size=shard)
    with open(os.path.join(folder, "config.json")) as f:
      assert json.load(f)["_class_name"] == cls.__name__
    if shard == "64KB":
      assert os.path.exists(os.path.join(folder, "diffusion_pytorch_model.safetensors.index.json")), cls.__name__
    m2 = load_model(cls, folder)
    assert json.dumps(config_to_dict(m2.cfg), sort_keys=True) == json.dumps(config_to_dict(cfg), sort_keys=True)
    a, b = m.state_dict(), m2.state_dict()
    assert a.keys() == b.keys()
    for k in a:
      assert torch.equal(a[k], b[k]), (cls.__name__, k)
      assert not b[k].is_meta
    assert set(read_state_dict(folder)) <= set(a)


def test_pipeline_folder(tmp_path):
  from maxdiffusion_b200.models.vae import AutoencoderKL, VAEConfig
  from maxdiffusion_b200.pipelines.pipeline_utils import load_components, save_pipeline
  from maxdiffusion_b200.schedulers.scheduling_euler_discrete import EulerDiscreteScheduler

  class P:
    pass

  p = P()
  p.vae = AutoencoderKL(VAEConfig(block_out_channels=(32, 32), layers_per_block=1, norm_num_groups=8))
  p.scheduler = EulerDiscreteScheduler(beta_start=0.001, beta_end=0.02)
  index = save_pipeline(p, str(tmp_path / "pipe"))
  assert set(index) == {"_class_name", "vae", "scheduler"}
  comps = load_components(str(tmp_path / "pipe"))
  assert comps["scheduler"].config.beta_end == 0.02
  for (k, a), (_, b) in zip(p.vae.state_dict().items(), comps["vae"].state_dict().items()):
    assert torch.equal(a, b), k
