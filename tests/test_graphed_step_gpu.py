"""Forward + backward replayed from a CUDA graph must give the loss and the gradients of the eager step, step after
step, with the optimizer running eagerly in between."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

CFG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "maxdiffusion_b200", "configs")


def _trainer(graph: bool):
  from maxdiffusion_b200 import pyconfig
  from maxdiffusion_b200.parallel.mesh import create_device_mesh
  from maxdiffusion_b200.trainers.stable_diffusion_trainer import StableDiffusionXLTrainer

  c = pyconfig.initialize(["t", os.path.join(CFG, "base_xl.yml"), "run_name=t", "random_init=True", "log_config=false",
                           "write_metrics=false", "dataset_type=synthetic", "resolution=256", "per_device_batch_size=2",
                           "unet_preset=tiny", "learning_rate=1e-4", "max_train_steps=100",
                           f"cuda_graph_train_step={'true' if graph else 'false'}"], unittest=True)
  return StableDiffusionXLTrainer(c, mesh=create_device_mesh(c))


def test_graphed_sdxl_step_follows_the_eager_step():
  eager, graphed = _trainer(False), _trainer(True)
  assert graphed._graphed is not None and eager._graphed is None
  la, lb = [], []
  for i in range(6):
    la.append(float(eager.train_step(eager.synthetic_batch(i))["learning/loss"]))
    lb.append(float(graphed.train_step(graphed.synthetic_batch(i))["learning/loss"]))
  assert graphed._graphed.replays == 4  # two eager warm-up calls, one capture + replay, three more replays
  assert lb == pytest.approx(la, rel=2e-2, abs=1e-3)
  # the first two steps are the same code path: equal bit for bit; weights stay close afterwards
  assert la[:2] == lb[:2]
  for (n, p), (_, q) in zip(eager.unet.named_parameters(), graphed.unet.named_parameters()):
    assert (p.float() - q.float()).abs().max() <= 5e-3 * (1 + p.float().abs().max()), n
