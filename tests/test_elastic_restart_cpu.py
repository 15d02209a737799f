"""Fail -> tear down -> restart -> resume, end to end on CPU: two gloo ranks under `torch.distributed.run
--max-restarts 1` train a tiny SDXL UNet; rank 1 raises (host-side injection) before step 3 in the first incarnation;
rank 0 learns of it through the health monitor before its next step and leaves too; the launcher starts both again;
the trainers restore the step-2 checkpoint and finish. The final weights equal those of an uninterrupted 2-rank run."""
import os
import socket
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = os.path.join(ROOT, "maxdiffusion_b200", "configs", "base_xl.yml")


def _run(out_dir, extra, restarts):
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
         "--master-port", str(port), "--max-restarts", str(restarts), "-m", "maxdiffusion_b200.train_sdxl", CFG, "run_name=r",
         f"output_dir={out_dir}", "random_init=True", "log_config=false", "write_metrics=false", "dataset_type=synthetic",
         "save_optimizer=true", "learning_rate=1e-3", "checkpoint_every=2", "enable_async_checkpointing=false",
         "resolution=32", "per_device_batch_size=1", "unet_preset=tiny", "max_train_steps=4", "ici_data_parallelism=2",
         "ici_fsdp_parallelism=1", "ici_context_parallelism=1", "health_timeout_s=30", *extra]
  env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
  return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=240)


def _final_unet(out_dir):
  from safetensors.torch import load_file

  ckpt = os.path.join(out_dir, "r", "checkpoints")
  steps = sorted(int(d) for d in os.listdir(ckpt) if d.isdigit())
  return steps, load_file(os.path.join(ckpt, str(steps[-1]), "unet_state", "state.safetensors"))


def test_injected_failure_restarts_from_the_last_checkpoint(tmp_path):
  clean = _run(tmp_path / "clean", [], 0)
  assert clean.returncode == 0, clean.stderr[-3000:]
  failed = _run(tmp_path / "failed", ["inject_failure_at_step=3", "inject_failure_rank=1"], 0)
  assert failed.returncode != 0 and "injected host failure" in failed.stderr  # without restarts the job ends
  again = _run(tmp_path / "again", ["inject_failure_at_step=3", "inject_failure_rank=1"], 1)
  assert again.returncode == 0, again.stderr[-3000:]
  assert "injected host failure" in again.stderr  # the first incarnation did fail
  steps_a, a = _final_unet(str(tmp_path / "clean"))
  steps_b, b = _final_unet(str(tmp_path / "again"))
  assert steps_a == steps_b == [2, 4]

  assert a.keys() == b.keys() and len(a) > 10
  for k in a:
    assert torch.allclose(a[k].float(), b[k].float(), atol=1e-6), k
