"""FLOP accounting: the analytic Wan training count against the value the reference's test asserts, and the traced
counter against hand counts of dense, convolution and attention layers (the cases of the reference's
src/maxdiffusion/tests/flop_calculations_test.py)."""
import torch

from maxdiffusion_b200.max_utils import calculate_model_tflops
from maxdiffusion_b200.models.wan.transformer_wan import WAN_PRESETS, WanConfig
from maxdiffusion_b200.trainers.wan_trainer import wan_train_tflops


def _close(a, b, rel=5e-2):
  return abs(a - b) / max(abs(a), abs(b)) <= rel


def test_wan_14b_720p_training_tflops_match_the_reference_value():
  # 720 x 1280 x 81 frames -> 21 x 45 x 80 latent patches = 75 600 tokens, one sample: 19 573 TFLOPs per step
  # (flop_calculations_test.py:50-75, 5 % tolerance there)
  cfg = WanConfig(**WAN_PRESETS["wan2.1-t2v-14b"])
  tokens = ((81 - 1) // 4 + 1) * (720 // 16) * (1280 // 16)
  assert tokens == 75600 and _close(wan_train_tflops(cfg, tokens, 1.0), 19_573, rel=1e-3)
  assert _close(wan_train_tflops(cfg, tokens, 2.0), 2 * 19_573, rel=1e-3)


def test_dense_layers():
  model = torch.nn.Sequential(torch.nn.Linear(10, 20), torch.nn.Linear(20, 15), torch.nn.Linear(15, 1))
  macs = 10 * 20 + 20 * 15 + 15 * 1
  assert _close(calculate_model_tflops(model, torch.randn(1, 10), train=True), 3 * 2 * macs / 1e12)
  assert _close(calculate_model_tflops(model, torch.randn(1, 10)), 2 * macs / 1e12)


def test_convolution_layers():
  class Net(torch.nn.Module):
    def __init__(self):
      super().__init__()
      self.a, self.b = torch.nn.Conv2d(1, 16, 3, padding=1), torch.nn.Conv2d(16, 32, 3, padding=1)
      self.c = torch.nn.Linear(32, 10)

    def forward(self, x):
      return self.c(self.b(self.a(x)).permute(0, 2, 3, 1))

  macs = 3 * 3 * 28 * 28 * 16 + 3 * 3 * 28 * 28 * 32 * 16 + 28 * 28 * 32 * 10
  assert _close(calculate_model_tflops(Net(), torch.randn(1, 1, 28, 28), train=True), 3 * 2 * macs / 1e12)


def test_attention_layer():
  class Attn(torch.nn.Module):
    def __init__(self, dim=320, heads=5):
      super().__init__()
      self.heads = heads
      self.q, self.k, self.v, self.o = (torch.nn.Linear(dim, dim, bias=False) for _ in range(4))

    def forward(self, x):
      B, S, C = x.shape
      split = lambda t: t.view(B, S, self.heads, C // self.heads).transpose(1, 2)
      out = torch.nn.functional.scaled_dot_product_attention(split(self.q(x)), split(self.k(x)), split(self.v(x)))
      return self.o(out.transpose(1, 2).reshape(B, S, C))

  S = 2304
  want = (2 * 3 * 320 * 320 * S + 4 * 320 * S ** 2 + 2 * 320 * 320 * S) / 1e12
  assert _close(calculate_model_tflops(Attn(), torch.randn(1, S, 320), train=True), 3 * want)


def test_products_on_the_kernel_path_are_counted_at_their_entry_points(monkeypatch):
  """On a GPU the GEMM, attention and 3x3 convolution kernels are called through ctypes and are invisible to PyTorch's
  counter; their entry points in `ops.functional` count them instead. Emulated here by declaring CPU tensors fast and
  standing plain PyTorch in for the kernels."""
  from maxdiffusion_b200 import max_utils
  from maxdiffusion_b200.ops import functional as OF

  F = torch.nn.functional
  monkeypatch.setattr(OF, "_fast", lambda t: True)
  monkeypatch.setattr(OF, "linear", lambda x, w, b=None, activation=None, residual=None: F.linear(x, w, b))
  monkeypatch.setattr(OF, "linear_gated_residual", lambda x, w, b, res, gate: res + gate * F.linear(x, w, b))
  monkeypatch.setattr(OF, "attention", lambda q, k, v, scale=None, fixed_m=None, keep_mask=None: q)
  monkeypatch.setattr(OF, "conv2d", lambda x, w, b=None, stride=1, padding=1, upsample=False:
                      F.conv2d(F.interpolate(x, scale_factor=2.0) if upsample else x, w, b, stride=stride, padding=padding))
  stubs = {n: getattr(OF, n) for n in ("linear", "linear_gated_residual", "attention", "conv2d")}
  total = [0]
  x = torch.randn(2, 24, 64)
  w = torch.randn(128, 64)
  q = torch.randn(2, 24, 4, 32)
  img, cw = torch.randn(1, 8, 16, 16), torch.randn(16, 8, 3, 3)
  with max_utils._count_kernel_path_flops(total):
    assert OF.linear is not stubs["linear"]
    OF.linear(x, w)
    OF.linear_gated_residual(x, torch.randn(64, 64), None, x, torch.ones(64))
    OF.attention(q, [q, q[:, :8]], [q, q[:, :8]])
    OF.conv2d(img, cw)
    OF.conv2d(img, cw, stride=2)
    OF.conv2d(img, cw, upsample=True)
    OF.conv2d(img, torch.randn(16, 8, 5, 5), padding=2)   # not a kernel shape: left to PyTorch's counter
  want = (2 * 48 * 128 * 64 + 2 * 48 * 64 * 64 + 4 * 2 * 4 * 24 * 32 * 32 +
          2 * 16 * 8 * 9 * (16 * 16 + 8 * 8 + 32 * 32))
  assert total[0] == want
  assert all(getattr(OF, n) is fn for n, fn in stubs.items())   # the entry points are restored
