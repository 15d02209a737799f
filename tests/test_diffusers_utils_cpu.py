"""Plumbing utilities: optional-dependency probing, logger, outputs, PIL helpers, deprecation, LoRA naming, adapters."""
import dataclasses
import os
import warnings

import numpy as np
import pytest
import torch


def test_import_utils():
  from maxdiffusion_b200.utils import import_utils as I

  assert I.is_torch_available() and not I.is_available("surely_not_a_package_xyz")
  with pytest.raises(I.OptionalDependencyNotAvailable):
    I.requires_backends("thing", ["surely_not_a_package_xyz"])

  class Needs(metaclass=I.DummyObject):
    _backends = ["surely_not_a_package_xyz"]

  with pytest.raises(ImportError):
    Needs()
  with pytest.raises(ImportError):
    Needs.from_pretrained


def test_logging_levels(capsys):
  from maxdiffusion_b200.utils import logging as L

  log = L.get_logger("maxdiffusion_b200.test")
  L.set_verbosity_error()
  log.warning("hidden")
  L.set_verbosity_info()
  log.info("shown")
  L.warning_once(log, "once")
  L.warning_once(log, "once")
  err = capsys.readouterr().err
  assert "hidden" not in err and "shown" in err and err.count("once") == 1
  L.set_verbosity_warning()


def test_base_output():
  from maxdiffusion_b200.utils.outputs import BaseOutput

  @dataclasses.dataclass
  class Out(BaseOutput):
    images: torch.Tensor
    flags: object = None

  o = Out(images=torch.ones(2))
  assert o[0] is o.images and o["images"] is o.images and len(o.to_tuple()) == 1
  o.flags = [True]
  assert o.to_tuple()[1] == [True]
  with pytest.raises(TypeError):
    o.pop("images")


def test_pil_and_grid():
  from maxdiffusion_b200.utils.pil_utils import make_image_grid, numpy_to_pil, pt_to_pil

  ims = numpy_to_pil(np.random.rand(4, 8, 8, 3))
  assert len(ims) == 4 and ims[0].size == (8, 8)
  assert make_image_grid(ims, 2, 2).size == (16, 16)
  assert pt_to_pil(torch.zeros(1, 3, 4, 4))[0].getpixel((0, 0)) == (128, 128, 128)
  assert numpy_to_pil(np.zeros((5, 5, 1)))[0].mode == "L"


def test_deprecate():
  from maxdiffusion_b200.utils.deprecation_utils import deprecate

  kw = {"old": 3}
  with warnings.catch_warnings(record=True) as w:
    warnings.simplefilter("always")
    assert deprecate("old", "9.0.0", "use new", take_from=kw) == 3
  assert not kw and "deprecated" in str(w[0].message)
  with pytest.raises(ValueError):
    deprecate("old", "0.0.1", "gone")
  with pytest.raises(TypeError):
    deprecate("old", "9.0.0", "x", take_from={"other": 1})


def test_randn_tensor_reproducible():
  from maxdiffusion_b200.utils.torch_utils import fourier_filter, randn_tensor

  a = randn_tensor((2, 3), torch.Generator().manual_seed(1))
  b = randn_tensor((2, 3), torch.Generator().manual_seed(1), dtype=torch.bfloat16)
  assert torch.equal(a.to(torch.bfloat16), b)
  c = randn_tensor((2, 3), [torch.Generator().manual_seed(5), torch.Generator().manual_seed(5)])
  assert torch.equal(c[0], c[1])
  x = torch.randn(1, 2, 8, 8)
  assert torch.allclose(fourier_filter(x, 2, 1.0), x, atol=1e-5)


def test_lora_naming_round_trip():
  from maxdiffusion_b200.utils.state_dict_utils import (StateDictType, convert_state_dict_to_diffusers, convert_state_dict_to_kohya,
                                                         convert_state_dict_to_peft, detect_state_dict_type)

  old = {"unet.down.attn.to_q_lora.down.weight": torch.zeros(4, 8), "unet.down.attn.to_q_lora.up.weight": torch.zeros(8, 4),
         "unet.down.attn.to_out_lora.down.weight": torch.zeros(4, 8), "unet.down.attn.to_out_lora.up.weight": torch.zeros(8, 4)}
  assert detect_state_dict_type(old) == StateDictType.DIFFUSERS_OLD
  peft = convert_state_dict_to_peft(old)
  assert set(peft) == {"unet.down.attn.to_q.lora_A.weight", "unet.down.attn.to_q.lora_B.weight",
                       "unet.down.attn.to_out.0.lora_A.weight", "unet.down.attn.to_out.0.lora_B.weight"}
  assert detect_state_dict_type(peft) == StateDictType.PEFT
  diff = convert_state_dict_to_diffusers(peft)
  assert "unet.down.attn.to_q.lora.up.weight" in diff
  ko = convert_state_dict_to_kohya(peft)
  assert "lora_unet_down_attn_to_q.lora_down.weight" in ko and float(ko["lora_unet_down_attn_to_q.alpha"]) == 4.0
  assert detect_state_dict_type(ko) == StateDictType.KOHYA_SS


def test_adapter_management():
  from maxdiffusion_b200.loaders.lora_loader import LoRALinear
  from maxdiffusion_b200.utils import peft_utils as P

  torch.manual_seed(0)
  net = torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.ReLU(), torch.nn.Linear(8, 4))
  x = torch.randn(3, 8)
  base = net(x)
  for i in (0, 2):
    w = LoRALinear(net[i])
    w.add_adapter("a", torch.randn(2, 8), torch.randn(net[i].out_features, 2), 0.5)
    w.add_adapter("b", torch.randn(2, 8), torch.randn(net[i].out_features, 2), 0.25)
    net[i] = w
  both = net(x)
  assert not torch.allclose(both, base)
  P.set_adapters(net, ["a"], [0.5])
  only_a = net(x)
  P.delete_adapter(net, "b")
  assert torch.allclose(net(x), only_a)
  assert P.set_adapter_scale(net, "a", 0.0) == 2 and torch.allclose(net(x), base, atol=1e-6)
  P.set_adapter_scale(net, "a", 0.5)
  assert P.fuse_adapters(net) == 2 and isinstance(net[0], torch.nn.Linear)
  assert torch.allclose(net(x), only_a, atol=1e-5)
  sd = {"x.to_q.lora_A.weight": torch.zeros(4, 8), "x.to_q.lora_B.weight": torch.zeros(8, 4), "x.to_k.lora_A.weight": torch.zeros(2, 8),
        "x.to_k.lora_B.weight": torch.zeros(8, 2), "x.to_v.lora_A.weight": torch.zeros(4, 8), "x.to_v.lora_B.weight": torch.zeros(8, 4)}
  kw = P.get_peft_kwargs(P.get_rank_dict(sd), {}, sd)
  assert kw["r"] == 4 and kw["rank_pattern"] == {"x.to_k": 2} and "x.to_q" in kw["target_modules"]


def test_hub_utils_local(tmp_path):
  from maxdiffusion_b200.utils.hub_utils import populate_model_card, resolve_model_path

  snap = tmp_path / "hub" / "models--org--name" / "snapshots" / "abc"
  (snap / "unet").mkdir(parents=True)
  assert resolve_model_path("org/name", "unet", cache_dir=str(tmp_path / "hub")) == str(snap / "unet")
  assert resolve_model_path(str(snap)) == str(snap)
  with pytest.raises(FileNotFoundError):
    resolve_model_path("org/missing", cache_dir=str(tmp_path / "hub"))
  assert os.path.exists(populate_model_card(str(tmp_path / "card"), "demo", "org/name", ["lora"]))


def test_custom_pipeline_files_are_loaded_from_a_local_folder(tmp_path):
  """A pipeline shipped as Python files next to a checkpoint: the file and its relative imports are copied into the
  modules cache and imported from there; an edited file becomes a new module; missing packages are named."""
  import pytest

  from maxdiffusion_b200.utils import dynamic_modules_utils as DM

  folder = tmp_path / "my-pipeline"
  folder.mkdir()
  (folder / "helpers.py").write_text("def double(x):\n  return 2 * x\n")
  (folder / "pipeline.py").write_text(
      "from .helpers import double\n\nclass MyPipeline:\n  @classmethod\n  def from_config(cls, config):\n    return cls()\n"
      "  def __call__(self, x):\n    return double(x)\n\nclass NotAPipeline:\n  pass\n")
  cache = str(tmp_path / "cache")
  assert DM.get_relative_imports(str(folder / "pipeline.py")) == ["helpers"]
  cls = DM.get_class_from_dynamic_module(str(folder), "pipeline.py", cache_root=cache)
  assert cls.__name__ == "MyPipeline" and cls()(21) == 42
  assert DM.get_class_from_dynamic_module(str(folder), "pipeline.py", "NotAPipeline", cache_root=cache).__name__ == "NotAPipeline"
  first = DM.get_cached_module_file(str(folder), "pipeline.py", cache)
  (folder / "helpers.py").write_text("def double(x):\n  return 3 * x\n")
  second = DM.get_cached_module_file(str(folder), "pipeline.py", cache)
  assert first != second and DM.get_class_from_dynamic_module(str(folder), "pipeline.py", cache_root=cache)()(1) == 3
  (folder / "broken.py").write_text("import a_package_that_does_not_exist_anywhere\n")
  with pytest.raises(ImportError, match="a_package_that_does_not_exist_anywhere"):
    DM.get_cached_module_file(str(folder), "broken.py", cache)
  with pytest.raises(FileNotFoundError):
    DM.get_cached_module_file(str(folder), "absent.py", cache)


def test_doc_and_offload_hook_helpers():
  import pytest

  from maxdiffusion_b200.utils.accelerate_utils import apply_forward_hook
  from maxdiffusion_b200.utils.doc_utils import replace_example_docstring

  @replace_example_docstring("    >>> pipe('a cat')")
  def call():
    """Runs the pipeline.

    Examples:

    Returns: frames."""

  assert ">>> pipe('a cat')" in call.__doc__ and "Examples:" not in call.__doc__ and "Returns: frames." in call.__doc__
  with pytest.raises(ValueError, match="placeholder"):
    replace_example_docstring("x")(lambda: None)

  seen = []

  class Vae:
    @apply_forward_hook
    def decode(self, z):
      return z + 1

  v = Vae()
  assert v.decode(1) == 2 and Vae.decode.__name__ == "decode"
  v._hf_hook = type("Hook", (), {"pre_forward": lambda self, module: seen.append(module)})()
  assert v.decode(2) == 3 and seen == [v]


def test_local_hub_helpers(tmp_path):
  import pytest

  from maxdiffusion_b200.utils import hub_utils as H

  h = "0123456789abcdef0123456789abcdef01234567"
  assert H.extract_commit_hash(f"/c/models--a--b/snapshots/{h}/unet/config.json") == h
  assert H.extract_commit_hash("/c/models--a--b/snapshots/main/x") is None and H.extract_commit_hash(None, "abc") == "abc"
  assert H.add_variant("diffusion_pytorch_model.safetensors", "fp16") == "diffusion_pytorch_model.fp16.safetensors"
  assert H.add_variant("model.bin") == "model.bin"
  (tmp_path / "unet").mkdir()
  (tmp_path / "unet" / "w.fp16.safetensors").write_bytes(b"x")
  (tmp_path / "w.safetensors").write_bytes(b"y")
  assert H.get_model_file(str(tmp_path), "w.safetensors", subfolder="unet", variant="fp16").endswith("unet/w.fp16.safetensors")
  assert H.get_model_file(str(tmp_path), "w.safetensors", subfolder="unet") == str(tmp_path / "w.safetensors")
  assert H.get_model_file(str(tmp_path / "w.safetensors"), "ignored") == str(tmp_path / "w.safetensors")
  with pytest.raises(EnvironmentError, match="no file named"):
    H.get_model_file(str(tmp_path), "missing.safetensors")
  assert H.http_user_agent({"pipeline": "wan"}).startswith("maxdiffusion_b200/") and "pipeline/wan" in H.http_user_agent({"pipeline": "wan"})

  class Thing(H.PushToHubMixin):
    def save_pretrained(self, folder):
      open(os.path.join(folder, "config.json"), "w").write("{}")

  out = Thing().push_to_hub("org/my-model", output_dir=str(tmp_path / "export"), commit_message="first version")
  assert sorted(os.listdir(out)) == ["README.md", "config.json"] and "first version" in open(os.path.join(out, "README.md")).read()
  with pytest.raises(EnvironmentError, match="network"):
    Thing().push_to_hub("org/my-model", upload=True)
