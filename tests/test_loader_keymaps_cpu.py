"""Weight key maps of the Flux and Stable Diffusion loaders against checkpoint key lists written down from the
published file formats (BFL single-file Flux, diffusers Flux, diffusers UNet / VAE): every checkpoint tensor must land
on exactly one model parameter with the right shape, nothing may be left over on either side, and fused matrices
must be the concatenation of their parts in the documented order.
reference: src/maxdiffusion/models/flux/util.py:57-281 (BFL rename table), src/maxdiffusion/models/modeling_flax_pytorch_utils.py:89-172."""
import torch

from maxdiffusion_b200.loaders import flux_loader
from maxdiffusion_b200.models.flux.transformer_flux import FLUX_PRESETS, FluxConfig, FluxTransformer2DModel


def _flux():
  torch.manual_seed(0)
  cfg = FluxConfig(**FLUX_PRESETS["tiny"])
  return cfg, FluxTransformer2DModel(cfg)


def _bfl_keys(cfg):
  """name -> shape of a BFL `flux1-*.safetensors` for this architecture (hidden = heads * head_dim, mlp = 4 hidden)."""
  h = cfg.num_attention_heads * cfg.attention_head_dim
  d, mlp = cfg.attention_head_dim, 4 * h
  keys = {"img_in.weight": (h, cfg.in_channels), "img_in.bias": (h,), "txt_in.weight": (h, cfg.joint_attention_dim), "txt_in.bias": (h,),
          "time_in.in_layer.weight": (h, 256), "time_in.in_layer.bias": (h,), "time_in.out_layer.weight": (h, h), "time_in.out_layer.bias": (h,),
          "vector_in.in_layer.weight": (h, cfg.pooled_projection_dim), "vector_in.in_layer.bias": (h,),
          "vector_in.out_layer.weight": (h, h), "vector_in.out_layer.bias": (h,),
          "final_layer.linear.weight": (cfg.in_channels, h), "final_layer.linear.bias": (cfg.in_channels,),
          "final_layer.adaLN_modulation.1.weight": (2 * h, h), "final_layer.adaLN_modulation.1.bias": (2 * h,)}
  if cfg.guidance_embeds:
    keys.update({"guidance_in.in_layer.weight": (h, 256), "guidance_in.in_layer.bias": (h,),
                 "guidance_in.out_layer.weight": (h, h), "guidance_in.out_layer.bias": (h,)})
  for i in range(cfg.num_layers):
    p = f"double_blocks.{i}."
    for s in ("img", "txt"):
      keys.update({p + f"{s}_mod.lin.weight": (6 * h, h), p + f"{s}_mod.lin.bias": (6 * h,),
                   p + f"{s}_attn.qkv.weight": (3 * h, h), p + f"{s}_attn.qkv.bias": (3 * h,),
                   p + f"{s}_attn.norm.query_norm.scale": (d,), p + f"{s}_attn.norm.key_norm.scale": (d,),
                   p + f"{s}_attn.proj.weight": (h, h), p + f"{s}_attn.proj.bias": (h,),
                   p + f"{s}_mlp.0.weight": (mlp, h), p + f"{s}_mlp.0.bias": (mlp,),
                   p + f"{s}_mlp.2.weight": (h, mlp), p + f"{s}_mlp.2.bias": (h,)})
  for i in range(cfg.num_single_layers):
    p = f"single_blocks.{i}."
    keys.update({p + "modulation.lin.weight": (3 * h, h), p + "modulation.lin.bias": (3 * h,),
                 p + "linear1.weight": (3 * h + mlp, h), p + "linear1.bias": (3 * h + mlp,),
                 p + "linear2.weight": (h, h + mlp), p + "linear2.bias": (h,),
                 p + "norm.query_norm.scale": (d,), p + "norm.key_norm.scale": (d,)})
  return keys


def _diffusers_keys(cfg):
  """name -> shape of a diffusers `FluxTransformer2DModel` state dict."""
  h = cfg.num_attention_heads * cfg.attention_head_dim
  d, mlp = cfg.attention_head_dim, 4 * h
  keys = {"x_embedder.weight": (h, cfg.in_channels), "x_embedder.bias": (h,),
          "context_embedder.weight": (h, cfg.joint_attention_dim), "context_embedder.bias": (h,),
          "norm_out.linear.weight": (2 * h, h), "norm_out.linear.bias": (2 * h,),
          "proj_out.weight": (cfg.in_channels, h), "proj_out.bias": (cfg.in_channels,)}
  emb = [("timestep_embedder", 256), ("text_embedder", cfg.pooled_projection_dim)] + ([("guidance_embedder", 256)] if cfg.guidance_embeds else [])
  for name, cin in emb:
    keys.update({f"time_text_embed.{name}.linear_1.weight": (h, cin), f"time_text_embed.{name}.linear_1.bias": (h,),
                 f"time_text_embed.{name}.linear_2.weight": (h, h), f"time_text_embed.{name}.linear_2.bias": (h,)})
  for i in range(cfg.num_layers):
    p = f"transformer_blocks.{i}."
    keys.update({p + "norm1.linear.weight": (6 * h, h), p + "norm1.linear.bias": (6 * h,),
                 p + "norm1_context.linear.weight": (6 * h, h), p + "norm1_context.linear.bias": (6 * h,)})
    for proj in ("to_q", "to_k", "to_v", "add_q_proj", "add_k_proj", "add_v_proj"):
      keys.update({p + f"attn.{proj}.weight": (h, h), p + f"attn.{proj}.bias": (h,)})
    for nrm in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
      keys[p + f"attn.{nrm}.weight"] = (d,)
    keys.update({p + "attn.to_out.0.weight": (h, h), p + "attn.to_out.0.bias": (h,),
                 p + "attn.to_add_out.weight": (h, h), p + "attn.to_add_out.bias": (h,)})
    for ff in ("ff", "ff_context"):
      keys.update({p + f"{ff}.net.0.proj.weight": (mlp, h), p + f"{ff}.net.0.proj.bias": (mlp,),
                   p + f"{ff}.net.2.weight": (h, mlp), p + f"{ff}.net.2.bias": (h,)})
  for i in range(cfg.num_single_layers):
    p = f"single_transformer_blocks.{i}."
    keys.update({p + "norm.linear.weight": (3 * h, h), p + "norm.linear.bias": (3 * h,),
                 p + "proj_mlp.weight": (mlp, h), p + "proj_mlp.bias": (mlp,),
                 p + "proj_out.weight": (h, h + mlp), p + "proj_out.bias": (h,),
                 p + "attn.norm_q.weight": (d,), p + "attn.norm_k.weight": (d,)})
    for proj in ("to_q", "to_k", "to_v"):
      keys.update({p + f"attn.{proj}.weight": (h, h), p + f"attn.{proj}.bias": (h,)})
  return keys


def _fill(keys):
  g = torch.Generator().manual_seed(1)
  return {k: torch.randn(s, generator=g) for k, s in keys.items()}


def _check_cover(mapped, model, source):
  want = model.state_dict()
  assert set(mapped) == set(want), sorted(set(mapped) ^ set(want))[:8]
  for k, v in mapped.items():
    assert tuple(v.shape) == tuple(want[k].shape), (k, tuple(v.shape), tuple(want[k].shape))
  assert sum(v.numel() for v in mapped.values()) == sum(v.numel() for v in source.values())
  model.load_state_dict(mapped, strict=True)


def test_bfl_single_file_keys_cover_the_flux_model_exactly_once():
  cfg, model = _flux()
  sd = _fill(_bfl_keys(cfg))
  mapped = flux_loader.bfl_to_ours(sd)
  _check_cover(mapped, model, sd)
  # BFL stores the final modulation as (shift, scale); the model applies (scale, shift)
  h = cfg.num_attention_heads * cfg.attention_head_dim
  assert torch.equal(mapped["norm_out.weight"][:h], sd["final_layer.adaLN_modulation.1.weight"][h:])
  assert torch.equal(mapped["norm_out.weight"][h:], sd["final_layer.adaLN_modulation.1.weight"][:h])
  assert torch.equal(mapped["transformer_blocks.0.to_qkv.weight"], sd["double_blocks.0.img_attn.qkv.weight"])
  assert torch.equal(mapped["single_transformer_blocks.0.qkv_mlp.weight"], sd["single_blocks.0.linear1.weight"])


def test_diffusers_keys_cover_the_flux_model_exactly_once_and_agree_with_the_bfl_route():
  cfg, model = _flux()
  sd = _fill(_diffusers_keys(cfg))
  mapped = flux_loader.diffusers_to_ours(sd)
  _check_cover(mapped, model, sd)
  p = "transformer_blocks.1."
  assert torch.equal(mapped[p + "to_qkv.weight"], torch.cat([sd[p + f"attn.{n}.weight"] for n in ("to_q", "to_k", "to_v")]))
  assert torch.equal(mapped[p + "add_qkv_proj.bias"], torch.cat([sd[p + f"attn.{n}.bias"] for n in ("add_q_proj", "add_k_proj", "add_v_proj")]))
  s = "single_transformer_blocks.0."
  assert torch.equal(mapped[s + "qkv_mlp.weight"],
                     torch.cat([sd[s + "attn.to_q.weight"], sd[s + "attn.to_k.weight"], sd[s + "attn.to_v.weight"], sd[s + "proj_mlp.weight"]]))
  # the same weights written in the BFL layout give the same model: q, k, v and the mlp share one matrix there
  bfl = {}
  h = cfg.num_attention_heads * cfg.attention_head_dim
  bfl["single_blocks.0.linear1.weight"] = mapped[s + "qkv_mlp.weight"]
  assert torch.equal(flux_loader.bfl_to_ours(bfl)[s + "qkv_mlp.weight"], mapped[s + "qkv_mlp.weight"])


def test_sd_loader_accepts_old_vae_attention_names(tmp_path):
  """Old diffusers VAE files call the mid-block attention projections query / key / value / proj_attn and may store
  them as 1x1 convolutions: `load_by_name` renames and reshapes them; a missing tensor is an error."""
  import pytest
  from safetensors.torch import save_file

  from maxdiffusion_b200.loaders.sd_loader import load_by_name
  from maxdiffusion_b200.models.vae import VAE_PRESETS, AutoencoderKL, VAEConfig

  torch.manual_seed(0)
  src = AutoencoderKL(VAEConfig(**VAE_PRESETS["tiny"]))
  sd = {}
  for k, v in src.state_dict().items():
    k2 = k.replace(".to_q.", ".query.").replace(".to_k.", ".key.").replace(".to_v.", ".value.").replace(".to_out.0.", ".proj_attn.")
    if k2 != k and v.dim() == 2:
      v = v[:, :, None, None]  # 1x1 convolution form
    sd[k2] = v.contiguous()
  folder = tmp_path / "vae"
  folder.mkdir()
  save_file(sd, str(folder / "diffusion_pytorch_model.safetensors"))
  dst = load_by_name(AutoencoderKL(VAEConfig(**VAE_PRESETS["tiny"])), str(folder))
  for (k, a), (_, b) in zip(src.state_dict().items(), dst.state_dict().items()):
    assert torch.equal(a, b), k
  del sd["decoder.conv_in.weight"]
  save_file(sd, str(folder / "diffusion_pytorch_model.safetensors"))
  with pytest.raises(ValueError, match="not covered"):
    load_by_name(AutoencoderKL(VAEConfig(**VAE_PRESETS["tiny"])), str(folder))
