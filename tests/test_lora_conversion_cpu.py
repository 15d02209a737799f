"""LoRA files in every published naming resolve onto this repository's modules, and an applied adapter changes the
output exactly like the merged weight W + scale * alpha / rank * up @ down (LoCon: the composed convolution).
reference: src/maxdiffusion/loaders/lora_conversion_utils.py:22-705, models/lora_nnx.py:90-245."""
import pytest
import torch

from maxdiffusion_b200.loaders import lora_conversion_utils as LC
from maxdiffusion_b200.loaders.lora_loader import LoRAConv2d, LoRALinear, add_flux_adapters, add_unet_adapters
from maxdiffusion_b200.models.flux.transformer_flux import FLUX_PRESETS, FluxConfig, FluxTransformer2DModel
from maxdiffusion_b200.models.unet_2d_condition import UNET_PRESETS, UNet2DConditionModel, UNetConfig


def _lora(style, path, cin, cout, rank=4, k=None, g=None):
  down = torch.randn((rank, cin) if k is None else (rank, cin, k, k), generator=g) * 0.2
  up = torch.randn((cout, rank) if k is None else (cout, rank, 1, 1), generator=g) * 0.2
  if style == "peft":
    return {f"unet.{path}.lora_A.weight": down, f"unet.{path}.lora_B.weight": up}, down, up, float(rank)
  flat = "lora_unet_" + path.replace(".", "_")
  return {f"{flat}.lora_down.weight": down, f"{flat}.lora_up.weight": up, f"{flat}.alpha": torch.tensor(2.0)}, down, up, 2.0


def test_sgm_block_numbers_map_to_diffusers_blocks():
  f = LC.sgm_block_to_diffusers
  assert f("input_blocks_0_0") == "conv_in"
  assert f("input_blocks_1_0_in_layers_2") == "down_blocks_0_resnets_0_conv1"
  assert f("input_blocks_3_0_op") == "down_blocks_0_downsamplers_0_conv"
  assert f("input_blocks_4_1_transformer_blocks_0_attn1_to_q") == "down_blocks_1_attentions_0_transformer_blocks_0_attn1_to_q"
  assert f("input_blocks_8_1_proj_in") == "down_blocks_2_attentions_1_proj_in"
  assert f("middle_block_1_transformer_blocks_3_ff_net_2") == "mid_block_attentions_0_transformer_blocks_3_ff_net_2"
  assert f("middle_block_2_out_layers_3") == "mid_block_resnets_1_conv2"
  assert f("output_blocks_2_2_conv") == f("output_blocks_2_1_conv") == "up_blocks_0_upsamplers_0_conv"
  assert f("output_blocks_5_0_skip_connection") == "up_blocks_1_resnets_2_conv_shortcut"
  assert f("output_blocks_8_0_emb_layers_1") == "up_blocks_2_resnets_2_time_emb_proj"


def test_unet_adapters_from_kohya_sgm_and_peft_files_equal_the_merged_weights():
  torch.manual_seed(0)
  g = torch.Generator().manual_seed(1)
  unet = UNet2DConditionModel(UNetConfig(**UNET_PRESETS["tiny_sd"])).eval()
  mods = dict(unet.named_modules())
  q = "down_blocks.1.attentions.0.transformer_blocks.0.attn1.to_q"
  ff = "up_blocks.0.attentions.0.transformer_blocks.0.ff.net.2"
  conv = "down_blocks.0.resnets.0.conv1"
  sd = {}
  wq, wff, wc = mods[q].weight, mods[ff].weight, mods[conv].weight
  a, dq, uq, aq = _lora("kohya", q, wq.shape[1], wq.shape[0], g=g)
  sd.update(a)
  a, dff, uff, aff = _lora("peft", ff, wff.shape[1], wff.shape[0], g=g)
  sd.update(a)
  # LoCon on a resnet convolution, written with SGM block numbers (input block 1 = level 0, resnet 0)
  dc, uc = torch.randn((4, wc.shape[1], 3, 3), generator=g) * 0.1, torch.randn((wc.shape[0], 4, 1, 1), generator=g) * 0.1
  sd.update({"lora_unet_input_blocks_1_0_in_layers_2.lora_down.weight": dc, "lora_unet_input_blocks_1_0_in_layers_2.lora_up.weight": uc,
             "lora_unet_input_blocks_1_0_in_layers_2.alpha": torch.tensor(4.0)})
  sd["lora_te1_text_model_encoder_layers_0_self_attn_q_proj.lora_down.weight"] = torch.zeros(4, 8)
  sd["lora_te1_text_model_encoder_layers_0_self_attn_q_proj.lora_up.weight"] = torch.zeros(8, 4)
  sd["lora_unet_nowhere_to_q.lora_down.weight"] = torch.zeros(4, 8)
  sd["lora_unet_nowhere_to_q.lora_up.weight"] = torch.zeros(8, 4)

  cfg = unet.cfg
  x = torch.randn(2, cfg.in_channels, 16, 16, generator=g)
  t = torch.tensor([10, 500])
  ctx = torch.randn(2, 7, cfg.cross_attention_dim, generator=g)
  with torch.no_grad():
    base = unet(x, t, ctx)
  import copy

  merged = copy.deepcopy(unet)
  mm = dict(merged.named_modules())
  scale = 0.7
  with torch.no_grad():
    mm[q].weight += scale * aq / 4 * (uq @ dq)
    mm[ff].weight += scale * aff / 4 * (uff @ dff)
    mm[conv].weight += scale * 4.0 / 4 * torch.einsum("or,rikl->oikl", uc.flatten(1), dc)
    want = merged(x, t, ctx)
  counts = add_unet_adapters(unet, sd, "style", scale)
  assert counts["unet"] == 3 and counts["text_encoder"] == 0
  assert sorted(counts["unresolved"]) == ["lora_te1_text_model_encoder_layers_0_self_attn_q_proj", "nowhere_to_q"]
  m2 = dict(unet.named_modules())
  assert isinstance(m2[q], LoRALinear) and isinstance(m2[conv], LoRAConv2d)
  with torch.no_grad():
    got = unet(x, t, ctx)
  assert (base - want).abs().max() > 1e-3  # the adapters do something
  assert torch.allclose(got, want, atol=2e-4, rtol=1e-3)


@pytest.mark.parametrize("style", ["bfl", "xlabs", "diffusers"])
def test_flux_adapters_in_three_namings_equal_the_merged_fused_weights(style):
  torch.manual_seed(0)
  g = torch.Generator().manual_seed(2)
  cfg = FluxConfig(**FLUX_PRESETS["tiny"])
  model = FluxTransformer2DModel(cfg).eval()
  h = cfg.num_attention_heads * cfg.attention_head_dim
  r = 4

  def pair(cin, cout):
    return torch.randn(r, cin, generator=g) * 0.2, torch.randn(cout, r, generator=g) * 0.2

  import copy

  merged = copy.deepcopy(model)
  mm = dict(merged.named_modules())
  sd, scale = {}, 0.5
  with torch.no_grad():
    if style == "bfl":
      d, u = pair(h, 3 * h)
      sd.update({"lora_unet_double_blocks_0_img_attn_qkv.lora_down.weight": d, "lora_unet_double_blocks_0_img_attn_qkv.lora_up.weight": u,
                 "lora_unet_double_blocks_0_img_attn_qkv.alpha": torch.tensor(8.0)})
      mm["transformer_blocks.0.to_qkv"].weight += scale * 8.0 / r * (u @ d)
      d2, u2 = pair(mm["single_transformer_blocks.0.proj_out"].weight.shape[1], h)
      sd.update({"lora_unet_single_blocks_0_linear2.lora_down.weight": d2, "lora_unet_single_blocks_0_linear2.lora_up.weight": u2})
      mm["single_transformer_blocks.0.proj_out"].weight += scale * (u2 @ d2)
      expect = 2
    elif style == "xlabs":
      d, u = pair(h, 3 * h)
      sd.update({"double_blocks.1.processor.qkv_lora2.down.weight": d, "double_blocks.1.processor.qkv_lora2.up.weight": u})
      mm["transformer_blocks.1.add_qkv_proj"].weight += scale * (u @ d)
      d2, u2 = pair(h, 3 * h)
      sd.update({"single_blocks.0.processor.qkv_lora.down.weight": d2, "single_blocks.0.processor.qkv_lora.up.weight": u2})
      mm["single_transformer_blocks.0.qkv_mlp"].weight[:3 * h] += scale * (u2 @ d2)
      expect = 2
    else:
      for i, name in enumerate(("to_q", "to_k", "to_v")):
        d, u = pair(h, h)
        sd.update({f"transformer.transformer_blocks.0.attn.{name}.lora_A.weight": d, f"transformer.transformer_blocks.0.attn.{name}.lora_B.weight": u})
        mm["transformer_blocks.0.to_qkv"].weight[i * h:(i + 1) * h] += scale * (u @ d)
      mlp = mm["single_transformer_blocks.1.qkv_mlp"].weight.shape[0] - 3 * h
      d, u = pair(h, mlp)
      sd.update({"transformer.single_transformer_blocks.1.proj_mlp.lora_A.weight": d, "transformer.single_transformer_blocks.1.proj_mlp.lora_B.weight": u})
      mm["single_transformer_blocks.1.qkv_mlp"].weight[3 * h:] += scale * (u @ d)
      expect = 4
  res = add_flux_adapters(model, sd, "a", scale)
  assert res == {"adapters": expect, "unresolved": []}
  B, S, T = 1, 16, 8
  from maxdiffusion_b200.models.flux.transformer_flux import prepare_latent_image_ids

  x = torch.randn(B, S, cfg.in_channels, generator=g)
  txt = torch.randn(B, T, cfg.joint_attention_dim, generator=g)
  pooled = torch.randn(B, cfg.pooled_projection_dim, generator=g)
  tt = torch.tensor([0.3])
  img_ids = prepare_latent_image_ids(4, 4, "cpu")[None]
  txt_ids = torch.zeros(B, T, 3)
  guidance = torch.full((B,), 3.5)
  with torch.no_grad():
    got = model(x, txt, pooled, tt, img_ids, txt_ids, guidance)
    want = merged(x, txt, pooled, tt, img_ids, txt_ids, guidance)
  assert torch.allclose(got, want, atol=2e-4, rtol=1e-3)


def test_ltx2_lora_in_the_original_key_namespace_merges_into_transformer_and_connectors(tmp_path):
  """Keys as LTX-2 LoRA files carry them: `diffusion_model.` + the ORIGINAL module names (`patchify_proj`,
  `adaln_single`, `av_ca_*_adaln_single`, blocks as they are) and `text_embedding_projection.aggregate_embed` for the
  connectors' feature projection. Every delta must land as W + scale * alpha / rank * up @ down."""
  from safetensors.torch import save_file

  from maxdiffusion_b200 import pyconfig
  from maxdiffusion_b200.loaders.lora_loader import merge_lora_into_ltx2, merge_ltx2_loras
  from maxdiffusion_b200.models.ltx2.transformer_ltx2 import LTX2Config, LTX2VideoTransformer3DModel

  torch.manual_seed(0)
  cfg = LTX2Config(in_channels=8, out_channels=8, num_attention_heads=2, attention_head_dim=32, cross_attention_dim=64,
                   audio_in_channels=16, audio_out_channels=16, audio_num_attention_heads=2, audio_attention_head_dim=16,
                   audio_cross_attention_dim=32, num_layers=2, caption_channels=32)
  model = LTX2VideoTransformer3DModel(cfg)
  connectors = torch.nn.Module()
  connectors.feature_extractor = torch.nn.Module()
  connectors.feature_extractor.linear = torch.nn.Linear(24, 16, bias=False)
  before = {n: p.detach().clone() for n, p in model.named_parameters()}
  c_before = connectors.feature_extractor.linear.weight.detach().clone()
  ours_to_file = {"proj_in": "patchify_proj", "audio_proj_in": "audio_patchify_proj", "time_embed.linear": "adaln_single.linear",
                  "audio_time_embed.emb.timestep_embedder.linear_1": "audio_adaln_single.emb.timestep_embedder.linear_1",
                  "av_cross_attn_video_a2v_gate.linear": "av_ca_a2v_gate_adaln_single.linear",
                  "av_cross_attn_audio_scale_shift.linear": "av_ca_audio_scale_shift_adaln_single.linear",
                  "transformer_blocks.1.attn1.to_out.0": "transformer_blocks.1.attn1.to_out.0",
                  "transformer_blocks.0.audio_to_video_attn.to_q": "transformer_blocks.0.audio_to_video_attn.to_q",
                  "transformer_blocks.1.ff.net.0.proj": "transformer_blocks.1.ff.net.0.proj",
                  "transformer_blocks.0.audio_ff.net.2": "transformer_blocks.0.audio_ff.net.2",
                  "caption_projection.linear_2": "caption_projection.linear_2", "proj_out": "proj_out"}
  rank, alpha, scale = 4, 2.0, 0.5
  sd, want = {}, {}
  for ours, theirs in ours_to_file.items():
    w = before[ours + ".weight"]
    down, up = torch.randn(rank, w.shape[1]) * 0.1, torch.randn(w.shape[0], rank) * 0.1
    sd[f"diffusion_model.{theirs}.lora_A.weight"], sd[f"diffusion_model.{theirs}.lora_B.weight"] = down, up
    sd[f"diffusion_model.{theirs}.alpha"] = torch.tensor(alpha)
    want[ours] = w + scale * alpha / rank * up @ down
  cd, cu = torch.randn(rank, 24) * 0.1, torch.randn(16, rank) * 0.1
  sd["text_embedding_projection.aggregate_embed.lora_A.weight"], sd["text_embedding_projection.aggregate_embed.lora_B.weight"] = cd, cu
  sd["diffusion_model.not_a_module.lora_A.weight"], sd["diffusion_model.not_a_module.lora_B.weight"] = cd, cu
  rep = merge_lora_into_ltx2(model, sd, scale, connectors)
  assert rep == {"transformer": len(ours_to_file), "connectors": 1, "unmatched": ["not_a_module"]}
  after = dict(model.named_parameters())
  for ours in ours_to_file:
    assert torch.allclose(after[ours + ".weight"], want[ours], atol=1e-6), ours
  untouched = [n for n in before if n.rsplit(".", 1)[0] not in ours_to_file]
  assert untouched and all(torch.equal(after[n], before[n]) for n in untouched)
  assert torch.allclose(connectors.feature_extractor.linear.weight, c_before + scale * cu @ cd, atol=1e-6)  # alpha = rank

  # through the configuration: a folder + file name, scale from `lora_config`
  save_file({k: v.clone().contiguous() for k, v in sd.items()}, str(tmp_path / "cam.safetensors"))
  config = pyconfig.initialize(
      ["x", "maxdiffusion_b200/configs/ltx2_video.yml", "log_config=false", "enable_lora=True",
       'lora_config={"lora_model_name_or_path": ["%s"], "weight_name": ["cam.safetensors"], "scale": [0.5], "rank": [4], '
       '"adapter_name": ["cam"], "from_pt": []}' % tmp_path], unittest=True)
  pipe = torch.nn.Module()
  pipe.transformer, pipe.connectors = LTX2VideoTransformer3DModel(cfg), connectors
  pipe.transformer.load_state_dict(before)
  merge_ltx2_loras(pipe, config)
  again = dict(pipe.transformer.named_parameters())
  assert all(torch.allclose(again[o + ".weight"], want[o], atol=1e-6) for o in ours_to_file)
  with pytest.raises(ValueError, match="has shape"):
    merge_lora_into_ltx2(model, {"diffusion_model.proj_out.lora_A.weight": torch.zeros(2, 3),
                                 "diffusion_model.proj_out.lora_B.weight": torch.zeros(5, 2)})
