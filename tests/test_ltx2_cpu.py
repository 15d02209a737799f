"""LTX-2 on CPU: rotary embeddings, transformer caches and guidance masks, VAEs, vocoder, connectors, pipeline."""
import math

import pytest
import torch

from maxdiffusion_b200 import aot_cache, pyconfig
from maxdiffusion_b200.models.ltx2.attention_ltx2 import LTX2RotaryPosEmbed, apply_rotary_emb, apply_split_rotary_emb
from maxdiffusion_b200.models.ltx2.autoencoder_kl_ltx2 import LTX2VAEConfig, LTX2VideoAutoencoderKL
from maxdiffusion_b200.models.ltx2.autoencoder_kl_ltx2_audio import AutoencoderKLLTX2Audio, LTX2AudioVAEConfig
from maxdiffusion_b200.models.ltx2.latent_upsampler_ltx2 import (LTX2LatentUpsamplerModel, adain_filter_latent,
                                                                 pixel_shuffle_nd, tone_map_latents)
from maxdiffusion_b200.models.ltx2.text_encoders_ltx2 import Embeddings1DConnector, norm_and_concat_padded_batch
from maxdiffusion_b200.models.ltx2.transformer_ltx2 import LTX2_PRESETS, LTX2Config, LTX2VideoTransformer3DModel
from maxdiffusion_b200.models.ltx2.vocoder_ltx2 import DownSample1d, LTX2Vocoder, LTX2VocoderWithBWE, UpSample1d
from maxdiffusion_b200.pipelines.ltx2.ltx2_pipeline import apply_ltx2_guidance, calculate_shift, rescale_noise_cfg

TINY_VAE = dict(latent_channels=8, block_out_channels=(8, 16, 16, 32), decoder_block_out_channels=(8, 16, 32),
                layers_per_block=(1, 1, 1, 1, 1), decoder_layers_per_block=(1, 1, 1, 1))


def test_rope_layouts_are_rotations():
  for kind in ("interleaved", "split"):
    rope = LTX2RotaryPosEmbed(32, modality="video", rope_type=kind, num_attention_heads=2)
    coords = rope.prepare_video_coords(1, 2, 2, 3)
    assert coords.shape == (1, 3, 12, 2) and float(coords[0, 0, 0, 0]) == 0.0  # causal offset clamps the first frame
    cos, sin = rope(coords)
    x = torch.randn(1, 12, 32)
    y = (apply_split_rotary_emb if kind == "split" else apply_rotary_emb)(x, (cos, sin))
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)  # rotations keep the norm
  a = LTX2RotaryPosEmbed(16, modality="audio", scale_factors=[4], num_attention_heads=2)
  ac = a.prepare_audio_coords(1, 5)
  assert ac.shape == (1, 1, 5, 2) and abs(float(ac[0, 0, 1, 0]) - (4 + 1 - 4) * 160 / 16000) < 1e-9


def test_transformer_caches_and_guidance_masks():
  torch.manual_seed(0)
  extra = dict(gated_attn=True, cross_attn_mod=True, perturbed_attn=True, rope_type="split", spatio_temporal_guidance_blocks=(1,))
  for over in ({}, extra):
    m = LTX2VideoTransformer3DModel(LTX2Config(**{**LTX2_PRESETS["tiny"], **over})).eval()
    B, Fr, H, W, Fa = 2, 2, 4, 4, 6
    x, a, txt = torch.randn(B, Fr * H * W, 16), torch.randn(B, Fa, 8), torch.randn(B, 5, 24)
    t = torch.tensor([500.0, 500.0])
    with torch.no_grad():
      o, ao = m(x, a, txt, txt, t, sigma=t / 1000, num_frames=Fr, height=H, width=W, audio_num_frames=Fa)
      kv, rc = m.compute_kv_cache(txt, txt), m.rope_tables(B, Fr, H, W, Fa)
      te = m.time_embeds(t[:1], sigma=t[:1] / 1000, audio_sigma=t[:1] / 1000)
      o2, ao2 = m(x, a, None, None, t, sigma=t / 1000, cached_kv=kv, rope_cache=rc, time_embed_cache=te)
      pm = torch.tensor([1.0, 0.0]).view(2, 1, 1)
      o3, _ = m(x, a, txt, txt, t, sigma=t / 1000, num_frames=Fr, height=H, width=W, audio_num_frames=Fa,
                perturbation_mask=pm, modality_mask=pm)
    assert torch.allclose(o, o2, atol=1e-5) and torch.allclose(ao, ao2, atol=1e-5)
    assert torch.allclose(o3[0], o[0], atol=1e-5) and (o3[1] - o[1]).abs().max() > 1e-3


def test_guidance_algebra():
  torch.manual_seed(0)
  x, ax = torch.randn(1, 6, 4), torch.randn(1, 3, 4)
  pred, apred = torch.randn(4, 6, 4), torch.randn(4, 3, 4)
  v, _ = apply_ltx2_guidance(pred, apred, x, ax, 0.7, 3.0, 1.0, 2.0, 0.0, do_cfg=True, do_stg=True)
  u, t, p, iso = pred.chunk(4)
  # in velocity space the x0 combination is the same linear combination of the branches
  want = t + 2.0 * (t - u) + 1.0 * (t - p) + 1.0 * (t - iso)
  assert torch.allclose(v, want, atol=1e-5)
  v2, _ = apply_ltx2_guidance(pred[:2], apred[:2], x, ax, 0.7, 3.0, 0.0, 1.0, 0.0, do_cfg=True, do_stg=False)
  assert torch.allclose(v2, pred[0:1] + 3.0 * (pred[1:2] - pred[0:1]), atol=1e-5)
  r = rescale_noise_cfg(v, t, 1.0)
  assert torch.allclose(r.std(unbiased=False), t.std(unbiased=False), atol=1e-4)
  assert abs(calculate_shift(4096, 1024, 4096, 0.95, 2.05) - 2.05) < 1e-9


def test_guidance_and_shift_reproduce_the_values_of_the_reference_tests():
  """src/maxdiffusion/tests/ltx2/test_pipeline_ltx2.py:46-118: the shift at the ends and the middle of the token range,
  two-way CFG on [unconditional, conditional] rows, and the four-way CFG + STG + modality combination."""
  assert abs(calculate_shift(256) - 0.5) < 1e-12 and abs(calculate_shift(4096) - 1.15) < 1e-12
  assert abs(calculate_shift((256 + 4096) / 2) - (0.5 + 1.15) / 2) < 1e-12
  lat, alat = torch.tensor([[10.0]]), torch.tensor([[20.0]])
  v, a = apply_ltx2_guidance(torch.tensor([[1.0], [3.0]]), torch.tensor([[2.0], [4.0]]), lat, alat, 2.0, 2.0, 0.0, 1.0, 0.0,
                             None, None, None, 0.0, True, False)
  assert v.tolist() == [[5.0]] and a.tolist() == [[6.0]]
  four = torch.tensor([[1.0], [3.0], [4.0], [5.0]])
  v, a = apply_ltx2_guidance(four, four, lat, lat, 2.0, 2.0, 1.0, 2.0, 0.0, None, None, None, 0.0, True, True)
  assert torch.allclose(v, torch.tensor([[2.0]])) and torch.allclose(a, torch.tensor([[2.0]]))
  cfg = torch.tensor([[[1.0, 2.0], [3.0, 4.0]]])
  assert torch.equal(rescale_noise_cfg(cfg, torch.ones_like(cfg), 0.0), cfg)


def test_video_vae_shapes_tiling_and_patch_order():
  torch.manual_seed(0)
  v = LTX2VideoAutoencoderKL(LTX2VAEConfig(**TINY_VAE)).eval()
  x = torch.rand(1, 3, 9, 64, 64) * 2 - 1
  mean, logvar = v.encode(x)
  assert mean.shape == (1, 8, 2, 2, 2) and logvar.shape == mean.shape
  assert torch.equal(logvar[:, 0], logvar[:, 3])  # one log-variance channel, replicated
  assert v.decode(mean).shape == (1, 3, 9, 64, 64)
  v.enable_tiling(tile_sample_min_height=96, tile_sample_min_width=96, tile_sample_stride_height=64, tile_sample_stride_width=64)
  m2, _ = v.encode(torch.rand(1, 3, 9, 128, 128) * 2 - 1)
  assert m2.shape == (1, 8, 2, 4, 4) and v.decode(m2).shape == (1, 3, 9, 128, 128)
  a, b = torch.zeros(1, 1, 1, 4, 2), torch.ones(1, 1, 1, 4, 2)
  assert v.blend_v(a, b, 4)[0, 0, 0, :, 0].tolist() == [0.0, 0.25, 0.5, 0.75]
  z = (torch.randn(1, 8, 2, 2, 2) - 0.3) * 2
  assert torch.allclose(v.denormalize_latents(v.normalize_latents(z)), z, atol=1e-6)


def test_audio_vae_is_causal_in_time_and_vocoder_lengths():
  torch.manual_seed(0)
  v = AutoencoderKLLTX2Audio(LTX2AudioVAEConfig(base_channels=8, mel_bins=16, resolution=16, latent_channels=4)).eval()
  x = torch.randn(1, 2, 13, 16)
  m, _ = v.encode(x)
  assert m.shape == (1, 4, 4, 4) and v.decode(m).shape == (1, 2, 13, 16)
  x2 = x.clone()
  x2[:, :, 9:] += 1.0
  m2, _ = v.encode(x2)
  assert torch.allclose(m2[:, :, :2], m[:, :, :2], atol=1e-6) and (m2[:, :, 3] - m[:, :, 3]).abs().max() > 1e-4
  t = v.patchify(m)
  assert t.shape == (1, 4, 16) and torch.equal(v.unpatchify(t, 4, 4), m)
  up, dn = UpSample1d(2, 12), DownSample1d(2, 12)
  sig = torch.sin(torch.arange(200.0) / 20)[None, None]
  assert up(sig).shape[-1] == 400 and (dn(up(sig)) - sig)[..., 20:-20].abs().max() < 1e-3  # low-pass round trip
  voc = LTX2Vocoder(in_channels=8, hidden_channels=32, upsample_kernel_sizes=(4, 3), upsample_factors=(2, 3),
                    act_fn="snakebeta", antialias=True, final_act_fn=None)
  assert voc(torch.randn(1, 2, 7, 4)).shape == (1, 2, 42)
  bwe = LTX2VocoderWithBWE(dict(in_channels=8, hidden_channels=32, upsample_kernel_sizes=(4, 4), upsample_factors=(2, 2)),
                           dict(in_channels=8, hidden_channels=16, upsample_kernel_sizes=(6, 4), upsample_factors=(3, 2)),
                           filter_length=16, hop_length=2, window_length=16, num_mel_channels=4)
  assert bwe(torch.randn(1, 2, 6, 4)).shape == (1, 2, 72)  # 6 * 4 samples at 16 kHz -> x3 at 48 kHz


def test_connectors_and_upsampler():
  torch.manual_seed(0)
  h = torch.randn(2, 8, 4, 3)
  mask = torch.tensor([[0, 0, 0, 1, 1, 1, 1, 1], [1] * 8])
  n = norm_and_concat_padded_batch(h, mask)
  assert n.shape == (2, 8, 12) and float(n[0, :3].abs().max()) == 0.0
  valid = h[0, 3:]
  want = 8 * (valid[..., 0] - valid[..., 0].mean()) / (valid[..., 0].max() - valid[..., 0].min() + 1e-6)
  assert torch.allclose(n[0, 3:].reshape(5, 4, 3)[..., 0], want, atol=1e-5)
  c = Embeddings1DConnector(32, heads=2, head_dim=16, layers=1, num_learnable_registers=4)
  x = torch.arange(8.0).reshape(1, 8, 1).repeat(1, 1, 32)
  o, m = c.replace_padded_with_registers(x, mask[:1])
  assert o[0, :5, 0].tolist() == [3.0, 4.0, 5.0, 6.0, 7.0] and bool(m.all())
  assert torch.equal(o[0, 5:], c.learnable_registers.detach().repeat(2, 1)[5:])
  up = LTX2LatentUpsamplerModel(in_channels=8, mid_channels=32, num_blocks_per_stage=1).eval()
  with torch.no_grad():
    assert up(torch.randn(1, 8, 3, 4, 6)).shape == (1, 8, 3, 8, 12)
    assert LTX2LatentUpsamplerModel(8, 32, 1, rational_spatial_scale=1.5)(torch.randn(1, 8, 2, 4, 4)).shape == (1, 8, 2, 6, 6)
  y = pixel_shuffle_nd(torch.arange(16.0).reshape(1, 4, 2, 2), 2)
  assert y.shape == (1, 1, 4, 4) and y[0, 0, 0, 1] == 4.0  # channel (p1=0, p2=1) of pixel (0, 0)
  lat, ref = torch.randn(1, 4, 2, 3, 3) * 3 + 1, torch.randn(1, 4, 2, 3, 3)
  out = adain_filter_latent(lat, ref, 1.0)
  assert torch.allclose(out.mean(dim=(2, 3, 4)), ref.mean(dim=(2, 3, 4)), atol=1e-3)
  assert torch.equal(tone_map_latents(lat, 0.0), lat) and tone_map_latents(lat, 1.0).abs().max() < lat.abs().max()


def test_generate_ltx2_tiny_and_checkpoint(tmp_path):
  from maxdiffusion_b200 import generate_ltx2 as G
  from maxdiffusion_b200.checkpointing.ltx2_checkpointer import LTX2Checkpointer

  tcfg = ('{"in_channels": 8, "out_channels": 8, "num_attention_heads": 2, "attention_head_dim": 32, "cross_attention_dim": 64, '
          '"audio_in_channels": 16, "audio_out_channels": 16, "audio_num_attention_heads": 2, "audio_attention_head_dim": 16, '
          '"audio_cross_attention_dim": 32, "num_layers": 2, "caption_channels": 32}')
  comps = ('{"vae": {"latent_channels": 8, "block_out_channels": [8, 16, 16, 32], "decoder_block_out_channels": [8, 16, 32], '
           '"layers_per_block": [1, 1, 1, 1, 1], "decoder_layers_per_block": [1, 1, 1, 1]}, '
           '"audio_vae": {"base_channels": 8, "mel_bins": 16, "resolution": 16, "latent_channels": 4}, '
           '"vocoder": {"in_channels": 32, "hidden_channels": 32, "upsample_kernel_sizes": [4, 4], "upsample_factors": [2, 2]}, '
           '"connectors": {"text_proj_in_factor": 3, "video_connector_attention_head_dim": 16, '
           '"video_connector_num_attention_heads": 2, "video_connector_num_learnable_registers": 4, '
           '"audio_connector_attention_head_dim": 16, "audio_connector_num_attention_heads": 2, '
           '"audio_connector_num_learnable_registers": 4}, "latent_upsampler": {"mid_channels": 32, "num_blocks_per_stage": 1}}')
  argv = ["x", "maxdiffusion_b200/configs/ltx2_3_video.yml", "random_init=True", "ltx2_preset=tiny",
          f"ltx2_config_overrides={tcfg}", f"ltx2_component_overrides={comps}", "height=64", "width=64", "num_frames=9",
          "num_inference_steps=2", "max_sequence_length=8", "use_bwe=False", "spatio_temporal_guidance_blocks=[1]",
          "run_latent_upsampler=True", "upsampler_adain_factor=0.5", f"output_dir={tmp_path}/out",
          f"checkpoint_dir={tmp_path}/ckpt", "log_config=false", "pretrained_model_name_or_path=/nonexistent"]
  config = pyconfig.initialize(argv, unittest=True)
  out = G.run(config)
  assert out.frames.shape == (1, 9, 128, 128, 3) and out.audio.shape[:2] == (1, 2)  # the up-sampler doubles H and W
  ck = LTX2Checkpointer(config)
  pipe = ck.load_pipeline(device="cpu")
  ck.save_checkpoint(7, pipe)
  pipe2 = LTX2Checkpointer(config).load_pipeline(device="cpu")
  for (n, p), (_, q) in zip(pipe.transformer.state_dict().items(), pipe2.transformer.state_dict().items()):
    assert torch.equal(p, q), n


def test_pipeline_argument_rules_renoising_and_videos_per_prompt(tmp_path):
  """`check_inputs`, `noise_scale` (start = s * noise + (1 - s) * normalised latents), `num_videos_per_prompt`, custom
  `timesteps` and per-video `decode_timestep` lists of the LTX-2 pipeline."""
  from maxdiffusion_b200.checkpointing.ltx2_checkpointer import LTX2Checkpointer

  tcfg = ('{"in_channels": 8, "out_channels": 8, "num_attention_heads": 2, "attention_head_dim": 32, "cross_attention_dim": 64, '
          '"audio_in_channels": 16, "audio_out_channels": 16, "audio_num_attention_heads": 2, "audio_attention_head_dim": 16, '
          '"audio_cross_attention_dim": 32, "num_layers": 1, "caption_channels": 32}')
  comps = ('{"vae": {"latent_channels": 8, "block_out_channels": [8, 16, 16, 32], "decoder_block_out_channels": [8, 16, 32], '
           '"layers_per_block": [1, 1, 1, 1, 1], "decoder_layers_per_block": [1, 1, 1, 1]}, '
           '"audio_vae": {"base_channels": 8, "mel_bins": 16, "resolution": 16, "latent_channels": 4}, '
           '"vocoder": {"in_channels": 32, "hidden_channels": 32, "upsample_kernel_sizes": [4, 4], "upsample_factors": [2, 2]}, '
           '"connectors": {"text_proj_in_factor": 3, "video_connector_attention_head_dim": 16, '
           '"video_connector_num_attention_heads": 2, "video_connector_num_learnable_registers": 4, '
           '"audio_connector_attention_head_dim": 16, "audio_connector_num_attention_heads": 2, '
           '"audio_connector_num_learnable_registers": 4}}')
  config = pyconfig.initialize(
      ["x", "maxdiffusion_b200/configs/ltx2_video.yml", "random_init=True", "ltx2_preset=tiny", f"ltx2_config_overrides={tcfg}",
       f"ltx2_component_overrides={comps}", "max_sequence_length=8", "use_bwe=False", f"output_dir={tmp_path}/out",
       "log_config=false", "pretrained_model_name_or_path=/nonexistent"], unittest=True)
  pipe = LTX2Checkpointer(config).load_pipeline(device="cpu")
  fe = pipe.connectors.feature_extractor
  dim = (fe.linear if hasattr(fe, "linear") else fe.video_linear).in_features // 3
  g = torch.Generator().manual_seed(0)
  emb = lambda n: torch.randn((n, 8, dim, 3), generator=g)
  ones = lambda n: torch.ones((n, 8), dtype=torch.long)
  kw = dict(height=64, width=64, num_frames=9, num_inference_steps=2, guidance_scale=1.0, stg_scale=0.0, output_type="latent")
  pe = emb(1)

  with pytest.raises(ValueError, match="divisible"):
    pipe(prompt_embeds=pe, prompt_attention_mask=ones(1), **{**kw, "height": 70})
  with pytest.raises(ValueError, match="not both"):
    pipe(prompt="a", prompt_embeds=pe, prompt_attention_mask=ones(1), **kw)
  with pytest.raises(ValueError, match="either"):
    pipe(**kw)
  with pytest.raises(ValueError, match="prompt_attention_mask` is required"):
    pipe(prompt_embeds=pe, **kw)
  with pytest.raises(ValueError, match="same shape"):
    pipe(prompt_embeds=pe, prompt_attention_mask=ones(1), negative_prompt_embeds=emb(2), negative_prompt_attention_mask=ones(2), **kw)
  with pytest.raises(ValueError, match="only one of"):
    pipe(prompt_embeds=pe, prompt_attention_mask=ones(1), timesteps=[1000.0, 500.0], sigmas=[1.0, 0.5], **kw)

  # two videos for one prompt; custom timesteps equal the same values given as sigmas
  two = pipe(prompt_embeds=pe, prompt_attention_mask=ones(1), num_videos_per_prompt=2, generator=torch.Generator().manual_seed(3), **kw)
  assert two.frames.shape[0] == 2 and not torch.equal(two.frames[0], two.frames[1])
  a = pipe(prompt_embeds=pe, prompt_attention_mask=ones(1), timesteps=[1000.0, 400.0], generator=torch.Generator().manual_seed(3), **kw)
  b = pipe(prompt_embeds=pe, prompt_attention_mask=ones(1), sigmas=[1.0, 0.4], generator=torch.Generator().manual_seed(3), **kw)
  assert torch.equal(a.frames, b.frames)

  # re-noising: the start state of a continued pass
  lat = torch.randn((1, 8, 2, 2, 2), generator=g) * 3 + 1
  start0 = pipe.prepare_latents(1, 2, 2, 2, torch.Generator().manual_seed(5), lat, noise_scale=0.0)
  assert torch.allclose(start0, pipe.pack_latents(pipe.vae.normalize_latents(lat), pipe.patch, pipe.patch_t), atol=1e-6)
  start1 = pipe.prepare_latents(1, 2, 2, 2, torch.Generator().manual_seed(5), lat, noise_scale=1.0)
  noise = torch.randn(start0.shape, generator=torch.Generator().manual_seed(5))
  assert torch.allclose(start1, noise)
  half = pipe.prepare_latents(1, 2, 2, 2, torch.Generator().manual_seed(5), lat, noise_scale=0.25)
  assert torch.allclose(half, 0.25 * noise + 0.75 * start0, atol=1e-6)
  assert torch.equal(pipe.prepare_latents(1, 2, 2, 2, None, lat), pipe.pack_latents(lat, pipe.patch, pipe.patch_t))  # as given
  packed_audio = torch.randn((1, 3, 4 * 4), generator=g)
  assert torch.allclose(pipe.prepare_audio_latents(1, 4, 3, 4, None, packed_audio, noise_scale=0.0),
                        pipe.audio_vae.normalize_latents(packed_audio))

  # per-video decode timesteps need one value per video
  dec = dict(kw, output_type="pt")
  if pipe.vae.cfg.timestep_conditioning:
    with pytest.raises(ValueError, match="one value per video"):
      pipe(prompt_embeds=pe, prompt_attention_mask=ones(1), decode_timestep=[0.05, 0.05], **dec)
    out = pipe(prompt_embeds=pe, prompt_attention_mask=ones(1), decode_timestep=[0.05], decode_noise_scale=[0.025], **dec)
    assert out.frames.shape[:2] == (1, 3)


def test_aot_cache_is_a_pass_through_on_cpu_and_fingerprints_revisions(tmp_path):
  calls = []

  @aot_cache.cached_graph
  def f(x, k=2):
    calls.append(1)
    return x * k

  assert torch.equal(f(torch.ones(3)), torch.ones(3) * 2)
  d = aot_cache.install(str(tmp_path), revision="abc")
  assert d != aot_cache.install(str(tmp_path), revision="abd") and aot_cache.is_installed()
  assert torch.equal(f(torch.ones(3), k=3), torch.ones(3) * 3) and len(calls) == 2  # CPU tensors: eager
  aot_cache.uninstall()
  assert aot_cache.source_fingerprint("r1") == aot_cache.source_fingerprint("r1") != aot_cache.source_fingerprint("r2")


def test_single_file_upsampler_and_reference_only_config_keys(tmp_path):
  """`upsampler_filename` (the LTX-2.3 layout: one weights file inside `upsampler_model_path`, its name saying what it
  up-samples) and the keys that only the reference's runtime reads, which must still parse as overrides."""
  from safetensors.torch import save_file

  from maxdiffusion_b200.checkpointing.ltx2_checkpointer import LTX2Checkpointer, upsampler_kind_from_filename
  from maxdiffusion_b200.models.ltx2.latent_upsampler_ltx2 import LTX2LatentUpsamplerModel

  assert upsampler_kind_from_filename("ltx-2.3-spatial-upscaler-x2-1.0.safetensors") == {
      "spatial_upsample": True, "temporal_upsample": False, "rational_spatial_scale": 2.0}
  assert upsampler_kind_from_filename("ltx-2-temporal-upscaler-x2.safetensors")["temporal_upsample"] is True
  assert upsampler_kind_from_filename("spatial-upscaler-x1.5.safetensors")["rational_spatial_scale"] == 1.5
  assert upsampler_kind_from_filename("weights.safetensors") == {}

  torch.manual_seed(0)
  src = LTX2LatentUpsamplerModel(in_channels=8, mid_channels=32, num_blocks_per_stage=1)
  name = "tiny-spatial-upscaler-x2.safetensors"
  save_file({k: v.contiguous() for k, v in src.state_dict().items()}, str(tmp_path / name))
  tcfg = ('{"in_channels": 8, "out_channels": 8, "num_attention_heads": 2, "attention_head_dim": 32, "cross_attention_dim": 64, '
          '"audio_in_channels": 16, "audio_out_channels": 16, "audio_num_attention_heads": 2, "audio_attention_head_dim": 16, '
          '"audio_cross_attention_dim": 32, "num_layers": 1, "caption_channels": 32}')
  comps = ('{"vae": {"latent_channels": 8, "block_out_channels": [8, 16, 16, 32], "decoder_block_out_channels": [8, 16, 32], '
           '"layers_per_block": [1, 1, 1, 1, 1], "decoder_layers_per_block": [1, 1, 1, 1]}, '
           '"audio_vae": {"base_channels": 8, "mel_bins": 16, "resolution": 16, "latent_channels": 4}, '
           '"vocoder": {"in_channels": 32, "hidden_channels": 32, "upsample_kernel_sizes": [4, 4], "upsample_factors": [2, 2]}, '
           '"connectors": {"text_proj_in_factor": 3, "video_connector_attention_head_dim": 16, '
           '"video_connector_num_attention_heads": 2, "video_connector_num_learnable_registers": 4, '
           '"audio_connector_attention_head_dim": 16, "audio_connector_num_attention_heads": 2, '
           '"audio_connector_num_learnable_registers": 4}, "latent_upsampler": {"mid_channels": 32, "num_blocks_per_stage": 1}}')
  config = pyconfig.initialize(
      ["x", "maxdiffusion_b200/configs/ltx2_3_video.yml", "ltx2_preset=tiny", f"ltx2_config_overrides={tcfg}",
       f"ltx2_component_overrides={comps}", "use_bwe=False", "run_latent_upsampler=True", f"upsampler_model_path={tmp_path}",
       f"upsampler_filename={name}", f"output_dir={tmp_path}/out", "log_config=false", "pretrained_model_name_or_path=/nonexistent",
       # keys of the reference's runtime: accepted, some of them ignored
       "run_text_encoder_on_tpu=False", "tile_search_vmem_limit_bytes=67108864", 'sharding={"transformer": "default"}',
       "config_path=", "global_batch_size_to_train_on=1", "enable_dynamic_vae_sharding=True", "upsampler_spatial_patch_size=1",
       "upsampler_temporal_patch_size=1", "use_batched_text_encoder=False", "train_new_unet=False", "tensorboard_dir="],
      unittest=True)
  pipe = LTX2Checkpointer(config).load_pipeline(device="cpu")
  got = pipe.latent_upsampler.state_dict()
  assert all(torch.equal(got[k], v) for k, v in src.state_dict().items())
  assert pipe.latent_upsampler.spatial and not pipe.latent_upsampler.temporal


def test_prompt_modulation_keeps_text_keys_and_values_out_of_the_cache():
  """Caching must not bypass the per-timestep prompt modulation of LTX-2.3 (the reference refuses the call,
  src/maxdiffusion/tests/ltx2/test_transformer_ltx2.py:158): here the cache then holds the caption projections only and
  the forward pass computes the modulated K / V itself, with the same result as without a cache."""
  from maxdiffusion_b200.models.ltx2.transformer_ltx2 import LTX2Config, LTX2VideoTransformer3DModel

  cfg = LTX2Config(**{**LTX2_PRESETS["tiny"], "cross_attn_mod": True})
  model = LTX2VideoTransformer3DModel(cfg).eval()
  txt = torch.randn(1, 5, 24)
  layers_kv, (text, audio_text) = model.compute_kv_cache(txt, txt)
  assert layers_kv is None and text.shape[:2] == (1, 5) and audio_text.shape[:2] == (1, 5)
  plain = LTX2VideoTransformer3DModel(LTX2Config(**LTX2_PRESETS["tiny"])).eval()
  assert len(plain.compute_kv_cache(txt, txt)[0]) == plain.cfg.num_layers
