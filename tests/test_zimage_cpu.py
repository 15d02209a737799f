"""Z-Image DiT, Qwen3 text encoder and the Z-Image pipeline on tiny CPU configurations."""
import torch

from maxdiffusion_b200 import pyconfig
from maxdiffusion_b200.models.qwen3 import QWEN3_PRESETS, Qwen3Model
from maxdiffusion_b200.models.z_image.transformer_z_image import ZIMAGE_PRESETS, ZImageTransformer2DModel
from maxdiffusion_b200.pipelines.z_image.z_image_pipeline import shifted_sigmas

CFG = "maxdiffusion_b200/configs/base_zimage_turbo.yml"
TINY_VAE = '{"block_out_channels":[32,32],"layers_per_block":1,"norm_num_groups":8,"latent_channels":4}'


def test_patchify_round_trip_and_ragged_batch():
  torch.manual_seed(0)
  m = ZImageTransformer2DModel(ZIMAGE_PRESETS["tiny"]).eval()
  img = torch.randn(4, 1, 8, 12)
  tokens, size, grid = m.patchify(img)
  assert tokens.shape == (24, 16) and grid == (1, 4, 6)
  assert torch.equal(m.unpatchify(tokens, size), img)
  x = [torch.randn(4, 1, 8, 8), torch.randn(4, 1, 8, 8)]
  caps = [torch.randn(10, 32), torch.randn(40, 32)]  # padded caption lengths 32 and 64: ragged batch, masked path
  with torch.no_grad():
    both = m(x, torch.tensor([0.3, 0.3]), caps)
    alone = m(x[1:], torch.tensor([0.3]), caps[1:])
  assert both[1].shape == (4, 1, 8, 8)
  assert (both[1] - alone[0]).abs().max() < 1e-4


def test_qwen3_padding_does_not_change_real_tokens():
  torch.manual_seed(0)
  q = Qwen3Model(QWEN3_PRESETS["tiny"]).eval()
  ids = torch.randint(0, 128, (2, 12))
  am = torch.ones(2, 12, dtype=torch.long)
  am[1, 8:] = 0
  h, hidden = q(ids, am)
  assert len(hidden) == 4 and h.shape == (2, 12, 64)
  h2, _ = q(ids[1:, :8], am[1:, :8])
  assert (h[1, :8] - h2[0]).abs().max() < 1e-5


def test_sigmas_and_pipeline_and_checkpoint_round_trip(tmp_path):
  s = shifted_sigmas(9, 3.0)
  assert s[0] == 1.0 and s[-1] == 0.0 and torch.all(s[:-1] > s[1:])
  assert abs(float(s[4]) - 3.0 * (5 / 9) / (1 + 2 * (5 / 9))) < 1e-6
  from maxdiffusion_b200.checkpointing.z_image_checkpointer import ZImageCheckpointer

  argv = ["x", CFG, "random_init=True", "zimage_preset=tiny", f"vae_config_overrides={TINY_VAE}",
          f"output_dir={tmp_path}/out", "pretrained_model_name_or_path=/nonexistent"]
  config = pyconfig.initialize(argv)
  ck = ZImageCheckpointer(config)
  pipe = ck.load_pipeline()
  emb = [torch.randn(20, 32)]
  img = pipe(prompt_embeds=emb, height=64, width=64, num_inference_steps=2, seed=1)
  assert img.shape == (1, 64, 64, 3) and img.dtype == torch.uint8
  ck.save_checkpoint(3, pipe)
  pipe2 = ZImageCheckpointer(config).load_pipeline()
  a = pipe(prompt_embeds=emb, height=64, width=64, num_inference_steps=2, seed=1, output_type="latent")
  b = pipe2(prompt_embeds=emb, height=64, width=64, num_inference_steps=2, seed=1, output_type="latent")
  assert torch.allclose(a, b, atol=1e-5)


def test_qwen3_matches_the_hugging_face_implementation_through_its_own_checkpoint_names():
  """An outside oracle: `transformers`' Qwen3 with the same tiny configuration. Its state dict loads into this
  repository's model unchanged (the parameter names are the checkpoint's), and the last hidden state and every
  intermediate hidden state agree on real tokens, with and without right padding."""
  import pytest

  transformers = pytest.importorskip("transformers")
  cfg = QWEN3_PRESETS["tiny"]
  hf_cfg = transformers.Qwen3Config(
      vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
      num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
      num_key_value_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, rms_norm_eps=cfg.rms_norm_eps,
      rope_theta=cfg.rope_theta, max_position_embeddings=cfg.max_position_embeddings, attention_bias=False,
      tie_word_embeddings=False, use_sliding_window=False)
  torch.manual_seed(0)
  hf = transformers.Qwen3Model(hf_cfg).eval()
  for p in hf.parameters():          # norm weights start at exactly one: move everything so that they matter
    torch.nn.init.normal_(p, mean=0.3 if p.dim() == 1 else 0.0, std=0.2)
  ours = Qwen3Model(cfg).eval()
  missing, unexpected = ours.load_state_dict({"model." + k: v for k, v in hf.state_dict().items()}, strict=True)
  assert not missing and not unexpected
  ids = torch.randint(0, cfg.vocab_size, (2, 12), generator=torch.Generator().manual_seed(1))
  mask = torch.ones(2, 12, dtype=torch.long)
  mask[1, 8:] = 0
  with torch.no_grad():
    want = hf(input_ids=ids, attention_mask=mask, output_hidden_states=True)
    got_last, got_all = ours(ids, mask)
  real = mask.bool()
  assert torch.allclose(got_last[real], want.last_hidden_state[real], atol=2e-5, rtol=1e-4)
  assert len(got_all) == cfg.num_hidden_layers + 1
  for i in range(cfg.num_hidden_layers):    # HF's last entry is after the final norm; the earlier ones are layer outputs
    assert torch.allclose(got_all[i][real], want.hidden_states[i][real], atol=2e-5, rtol=1e-4), i
