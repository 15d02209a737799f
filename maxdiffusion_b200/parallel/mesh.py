"""The 4-axis device mesh `(data, fsdp, context, tensor)` mapped onto torch.distributed ranks.

The reference builds a `jax.sharding.Mesh` from `ici_*_parallelism` x `dcn_*_parallelism` and lets GSPMD
derive the collectives (src/maxdiffusion/max_utils.py:426-506). Here the mesh is plain rank arithmetic: the
axes are laid out row-major with `tensor` fastest, every axis gets a process group, and the 2-D
Ulysses x ring split of the context axis keeps the Ulysses ranks adjacent (the reference puts Ulysses
innermost too, src/maxdiffusion/models/attention_flax.py:182-197). On an NVSwitch box every pair of GPUs has
the same bandwidth, so the assignment is free of topology constraints.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..common_types import CONTEXT, DATA, FSDP, MESH_AXES, TENSOR


def fill_unspecified_mesh_axes(sizes: Sequence[int], num_devices: int, what: str = "ICI") -> list[int]:
  """Replaces the single -1 entry by whatever makes the product equal `num_devices`."""
  sizes = [int(s) for s in sizes]
  if sizes.count(-1) > 1:
    raise ValueError(f"{what}: at most one parallelism axis may be -1, got {sizes}")
  if -1 in sizes:
    known = 1
    for s in sizes:
      if s != -1:
        known *= s
    if known == 0 or num_devices % known != 0:
      raise ValueError(f"{what}: {num_devices} devices cannot be split by the fixed axes {sizes}")
    sizes[sizes.index(-1)] = num_devices // known
  prod = 1
  for s in sizes:
    prod *= s
  if prod != num_devices:
    raise ValueError(f"{what}: mesh {sizes} has {prod} devices but {num_devices} are available")
  return sizes


def mesh_shape_from_config(config, num_devices: int) -> dict[str, int]:
  """Axis sizes from `ici_*` x `dcn_*` keys (`dcn_*` spans nodes; on one box they are all 1)."""
  nodes = max(1, int(os.environ.get("NNODES", "1")))
  per_node = num_devices // nodes
  ici = [int(config.get(f"ici_{a}_parallelism", 1)) for a in MESH_AXES]
  dcn = [int(config.get(f"dcn_{a}_parallelism", 1)) for a in MESH_AXES]
  if nodes == 1:
    dcn = [1 if d == -1 else d for d in dcn]
  ici = fill_unspecified_mesh_axes(ici, per_node, "ICI")
  dcn = fill_unspecified_mesh_axes(dcn, nodes, "DCN")
  return {a: i * d for a, i, d in zip(MESH_AXES, ici, dcn)}


def rank_to_coords(rank: int, shape: dict[str, int]) -> dict[str, int]:
  coords = {}
  for axis in reversed(MESH_AXES):
    coords[axis] = rank % shape[axis]
    rank //= shape[axis]
  return coords


def coords_to_rank(coords: dict[str, int], shape: dict[str, int]) -> int:
  rank = 0
  for axis in MESH_AXES:
    rank = rank * shape[axis] + coords[axis]
  return rank


def axis_groups(shape: dict[str, int], axes: Sequence[str]) -> list[list[int]]:
  """All rank lists that vary only along `axes` (in mesh order), one list per setting of the other axes."""
  world = 1
  for a in MESH_AXES:
    world *= shape[a]
  groups: dict[tuple, list[int]] = {}
  for r in range(world):
    c = rank_to_coords(r, shape)
    key = tuple(c[a] for a in MESH_AXES if a not in axes)
    groups.setdefault(key, []).append(r)
  return list(groups.values())


def split_context(context_ranks: Sequence[int], ulysses_shards: int) -> tuple[list[list[int]], list[list[int]]]:
  """Splits one context group into Ulysses groups (adjacent ranks) and ring groups (strided ranks)."""
  n = len(context_ranks)
  u = ulysses_shards if ulysses_shards and ulysses_shards > 0 else 1
  if n == 1:
    u = 1
  if n % u != 0:
    raise ValueError(f"ulysses_shards={u} does not divide the context axis ({n})")
  ulysses = [list(context_ranks[i:i + u]) for i in range(0, n, u)]
  ring = [list(context_ranks[i::u]) for i in range(u)]
  return ulysses, ring


@dataclass
class DeviceMesh:
  shape: dict[str, int]
  rank: int
  world_size: int
  coords: dict[str, int] = field(default_factory=dict)
  groups: dict[str, Optional[dist.ProcessGroup]] = field(default_factory=dict)
  group_ranks: dict[str, list[int]] = field(default_factory=dict)

  def size(self, axis: str) -> int:
    return self.shape[axis]

  def group(self, name: str):
    return self.groups.get(name)

  def ranks(self, name: str) -> list[int]:
    return self.group_ranks.get(name, [self.rank])

  def index_in(self, name: str) -> int:
    return self.ranks(name).index(self.rank)


def create_device_mesh(config=None, shape: Optional[dict[str, int]] = None, ulysses_shards: int = -1) -> DeviceMesh:
  """Builds the mesh and its process groups. Works without torch.distributed (single process).

  Groups: one per axis (`data`, `fsdp`, `context`, `tensor`), `shard` = fsdp x context (the ranks a Wan
  weight is sharded over: the reference maps `embed -> ('context', 'fsdp')`, configs/base_wan_14b.yml:217),
  `replica` = data (gradient averaging), `batch` = data x fsdp (ranks that hold different samples), and `ulysses` / `ring` inside the context axis.
  """
  initialized = dist.is_available() and dist.is_initialized()
  world = dist.get_world_size() if initialized else 1
  rank = dist.get_rank() if initialized else 0
  if shape is None:
    if config is None:
      shape = {DATA: 1, FSDP: 1, CONTEXT: world, TENSOR: 1}
    else:
      shape = mesh_shape_from_config(config, world)
      if ulysses_shards <= 0:
        ulysses_shards = int(config.get("ulysses_shards", -1))
  mesh = DeviceMesh(shape=dict(shape), rank=rank, world_size=world, coords=rank_to_coords(rank, shape))

  def make(name: str, axes: Sequence[str]):
    for ranks in axis_groups(shape, axes):
      pg = dist.new_group(ranks) if (initialized and len(ranks) > 1) else None
      if rank in ranks:
        mesh.groups[name] = pg
        mesh.group_ranks[name] = ranks

  for axis in MESH_AXES:
    make(axis, (axis,))
  make("shard", (FSDP, CONTEXT))
  make("replica", (DATA,))
  make("model", (FSDP, CONTEXT, TENSOR))
  make("batch", (DATA, FSDP))
  for ctx_ranks in axis_groups(shape, (CONTEXT,)):
    ul, rg = split_context(ctx_ranks, ulysses_shards)
    for name, sub in (("ulysses", ul), ("ring", rg)):
      for ranks in sub:
        pg = dist.new_group(ranks) if (initialized and len(ranks) > 1) else None
        if rank in ranks:
          mesh.groups[name] = pg
          mesh.group_ranks[name] = ranks
  return mesh


def init_distributed(backend: Optional[str] = None) -> tuple[int, int, int]:
  """Initialises torch.distributed from torchrun-style env (the reference's JAX_COORDINATOR_* / NODE_RANK
  names are accepted as aliases, gpu_multi_process_run.sh:18-77). Returns (rank, world_size, local_rank)."""
  env = os.environ
  if "MASTER_ADDR" not in env and "JAX_COORDINATOR_IP" in env:
    env["MASTER_ADDR"] = env["JAX_COORDINATOR_IP"]
    env["MASTER_PORT"] = env.get("JAX_COORDINATOR_PORT", "29500")
  if "WORLD_SIZE" not in env and "NNODES" in env and "GPUS_PER_NODE" in env:
    env["WORLD_SIZE"] = str(int(env["NNODES"]) * int(env["GPUS_PER_NODE"]))
  world = int(env.get("WORLD_SIZE", "1"))
  rank = int(env.get("RANK", "0"))
  local_rank = int(env.get("LOCAL_RANK", str(rank % max(1, torch.cuda.device_count() or 1))))
  if torch.cuda.is_available():
    torch.cuda.set_device(local_rank)
  if world > 1 and not dist.is_initialized():
    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    kwargs = {}
    if backend == "nccl":
      kwargs["device_id"] = torch.device("cuda", local_rank)
    if env.get("TORCHELASTIC_USE_AGENT_STORE") == "True" and "MASTER_PORT" in env:
      # Under a launcher that restarts failed jobs (`torch.distributed.run --max-restarts`) with a fixed master
      # address, the launcher's store outlives an incarnation and still holds the addresses its ranks published.
      # Every incarnation therefore works under its own key prefix (sub-groups inherit it from the default group).
      from datetime import timedelta

      base = dist.TCPStore(env["MASTER_ADDR"], int(env["MASTER_PORT"]), world, is_master=False, timeout=timedelta(minutes=10))
      kwargs["store"] = dist.PrefixStore(f"/mdb/attempt_{env.get('TORCHELASTIC_RESTART_COUNT', '0')}", base)
    dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
  return rank, world, local_rank
