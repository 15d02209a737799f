"""Quantisation plumbing on CPU: mode parsing, layer replacement, and the fake-quantised fallback."""
import pytest
import torch

from maxdiffusion_b200 import pyconfig
from maxdiffusion_b200.models.layers import Linear
from maxdiffusion_b200.models.quantizations import Fp8Linear, fake_quantize, get_quantization_mode, quantize_model
from maxdiffusion_b200.models.wan.transformer_wan import WanConfig, WanModel


def test_fake_quantize_error_bound():
  torch.manual_seed(0)
  x = torch.randn(64, 64)
  q = fake_quantize(x)
  assert (q - x).abs().max() <= x.abs().max() / 448.0 * 16 + 1e-6  # e4m3: 3 mantissa bits
  assert torch.equal(fake_quantize(q), q) or (fake_quantize(q) - q).abs().max() < 1e-6


def test_quantize_model_replaces_block_linears_only():
  cfg = WanConfig(num_attention_heads=2, attention_head_dim=32, ffn_dim=64, num_layers=2, text_dim=32, freq_dim=32)
  m = WanModel(cfg)
  n = quantize_model(m, "fp8")
  assert n > 0 and isinstance(m.blocks[0].ffn_in, Fp8Linear) and type(m.proj_out) is Linear
  x, t, e = torch.randn(1, 16, 2, 8, 8), torch.tensor([300.0]), torch.randn(1, 5, 32)
  with torch.no_grad():
    assert m(x, t, e).shape == x.shape


def test_mode_from_config():
  base = ["x", "maxdiffusion_b200/configs/base_wan_14b.yml", "log_config=false"]
  assert get_quantization_mode(pyconfig.initialize(base, unittest=True)) is None
  c = pyconfig.initialize(base + ["use_qwix_quantization=True", "quantization=fp8_full"], unittest=True)
  assert get_quantization_mode(c) == "fp8_full"
  with pytest.raises(ValueError):
    get_quantization_mode(pyconfig.initialize(base + ["use_qwix_quantization=True", "quantization=int4"], unittest=True))


def test_int8_mode_uses_the_integer_layer_and_its_reference_quantiser_rounds_to_127_levels():
  import torch

  from maxdiffusion_b200.models.layers import Linear
  from maxdiffusion_b200.models.quantizations import Int8Linear, fake_quantize_int8, quantize_model

  x = torch.linspace(-2.0, 2.0, 1001)
  q = fake_quantize_int8(x)
  assert (q - x).abs().max() <= 2.0 / 127 / 2 + 1e-6 and len(torch.unique(q)) <= 255
  m = torch.nn.ModuleDict({"blocks": torch.nn.ModuleList([torch.nn.ModuleDict({"a": Linear(32, 32)})]), "head": Linear(32, 32)})
  assert quantize_model(m, "int8") == 1
  layer = m["blocks"][0]["a"]
  assert isinstance(layer, Int8Linear) and type(m["head"]) is Linear
  y = layer(torch.randn(3, 32))  # CPU: the reference quantiser on the weights
  assert y.shape == (3, 32)
