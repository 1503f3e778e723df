"""Context-parallel process-group plumbing, mirroring ``pithtrain/modules/distributed.py``.

Same names and meaning as the reference for the parts ring attention depends on: ``DistributedCfg``
(``context_parallel_size`` at distributed.py:33), ``DistributedCtx``, ``setup_default_process_group`` (:127),
``setup_device_mesh`` with the ``(pp, dp, cp, ep)`` mesh (:151-179), plus the helpers the reference spreads over
its training code: the CP group lookup (pithtrain/modules/training.py:294), the divisibility check (:302-304),
the slicing of tokens/labels (pithtrain/tasks/pretrain_language_model.py:128-133), position ids
(pithtrain/models/qwen3_30b_a3b.py:817-821) and the loss average over CP ranks (pretrain_language_model.py:384-389).
The sharding-aware helpers take ``sharding="contiguous" | "zigzag"``; contiguous reproduces the reference.
"""

from __future__ import annotations

import atexit
import os
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Generator, Optional

import torch
import torch.distributed as dist

from ..operators.ring_attention.sharding import check_sharding, local_positions, shard_sequence


@dataclass
class DistributedCfg:
    pipeline_parallel_size: int = 1
    context_parallel_size: int = 1
    expert_parallel_size: int = 1
    context_parallel_sharding: str = "contiguous"
    backend: Optional[str] = None  # None: "nccl" with CUDA, else "gloo"


@dataclass
class DistributedCtx:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    local_world_size: int = 1
    dp_rank: int = 0
    dp_size: int = 1
    pp_rank: int = 0
    pp_size: int = 1
    cp_rank: int = 0
    cp_size: int = 1
    ep_rank: int = 0
    ep_size: int = 1
    device_mesh: Optional["dist.DeviceMesh"] = None


def setup_default_process_group(cfg: DistributedCfg, ctx: DistributedCtx) -> None:
    """Initialises the default process group from torchrun's environment (one process per GPU)."""
    assert "RANK" in os.environ and "WORLD_SIZE" in os.environ, "Not launched with torchrun."
    ctx.rank = int(os.environ["RANK"])
    ctx.world_size = int(os.environ["WORLD_SIZE"])
    ctx.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    ctx.local_world_size = int(os.environ.get("LOCAL_WORLD_SIZE", str(ctx.world_size)))
    backend = cfg.backend or ("nccl" if torch.cuda.is_available() else "gloo")
    if not dist.is_initialized():
        kwargs = dict(backend=backend)
        if backend == "nccl":
            torch.cuda.set_device(ctx.local_rank)
            kwargs["device_id"] = torch.device("cuda", ctx.local_rank)
        dist.init_process_group(**kwargs)
        atexit.register(_destroy)


def _destroy() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()


def setup_device_mesh(cfg: DistributedCfg, ctx: DistributedCtx) -> None:
    """Mesh ``(pp, dp, cp, ep)``; CP and EP innermost so that their traffic stays on NVLink."""
    ctx.ep_size = cfg.expert_parallel_size
    ctx.pp_size = cfg.pipeline_parallel_size
    ctx.cp_size = cfg.context_parallel_size
    denom = ctx.ep_size * ctx.pp_size * ctx.cp_size
    assert ctx.world_size % denom == 0, (
        f"world_size ({ctx.world_size}) must be divisible by pp*cp*ep ({denom})"
    )
    ctx.dp_size = ctx.world_size // denom
    device_type = "cuda" if dist.get_backend() == "nccl" else "cpu"
    ctx.device_mesh = dist.init_device_mesh(device_type, (ctx.pp_size, ctx.dp_size, ctx.cp_size, ctx.ep_size),
                                            mesh_dim_names=("pp", "dp", "cp", "ep"))
    ctx.dp_rank = ctx.device_mesh.get_local_rank("dp")
    ctx.pp_rank = ctx.device_mesh.get_local_rank("pp")
    ctx.cp_rank = ctx.device_mesh.get_local_rank("cp")
    ctx.ep_rank = ctx.device_mesh.get_local_rank("ep")


@contextmanager
def distributed_context(cfg: object, ctx: object) -> Generator[DistributedCtx, None, None]:
    """Brings the distributed runtime up for a task (reference: distributed.py:182-194): ``cfg.distributed`` and
    ``ctx.distributed`` hold the configuration and the context; the default group and the device mesh exist inside
    the ``with`` body. The matmul precision switches are the reference's and only matter where CUDA is present."""
    assert hasattr(cfg, "distributed") and isinstance(cfg.distributed, DistributedCfg)
    assert hasattr(ctx, "distributed") and isinstance(ctx.distributed, DistributedCtx)
    if torch.cuda.is_available():
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.set_float32_matmul_precision("high")
    setup_default_process_group(cfg.distributed, ctx.distributed)
    setup_device_mesh(cfg.distributed, ctx.distributed)
    yield ctx.distributed


def get_cp_group(ctx: DistributedCtx):
    """The CP process group, or ``None`` when context parallelism is off (reference: training.py:294)."""
    return ctx.device_mesh.get_group("cp") if ctx.cp_size > 1 else None


def check_sequence_length(sequence_length: int, cp_size: int, sharding: str = "contiguous") -> None:
    check_sharding(sharding)
    unit = cp_size if sharding == "contiguous" else 2 * cp_size
    assert sequence_length % unit == 0, (
        f"sequence_length ({sequence_length}) must be divisible by "
        f"{'context_parallel_size' if sharding == 'contiguous' else '2 * context_parallel_size'} ({unit})"
    )


def shard_batch_for_cp(tokens: torch.Tensor, labels: torch.Tensor, cp_rank: int, cp_size: int,
                       sharding: str = "contiguous"):
    """Slices ``[batch, sequence]`` tokens and labels to this CP rank's part of the sequence."""
    if cp_size == 1:
        return tokens, labels
    check_sequence_length(tokens.shape[1], cp_size, sharding)
    return (shard_sequence(tokens, cp_size, cp_rank, sharding, seq_dim=1),
            shard_sequence(labels, cp_size, cp_rank, sharding, seq_dim=1))


def cp_position_ids(local_seq_len: int, cp_rank: int, cp_size: int, sharding: str = "contiguous",
                    device=None) -> torch.Tensor:
    """Global position of every local token, shape [1, local_seq_len] (contiguous: ``cp_rank*len + arange``)."""
    return local_positions(local_seq_len * cp_size, cp_size, cp_rank, sharding, device=device).unsqueeze(0)


def average_loss_over_cp(loss: Optional[torch.Tensor], cp_group, cp_size: int):
    """All-reduce + divide, in place, so that every CP rank logs the loss of the whole sequence."""
    if loss is not None and cp_size > 1:
        dist.all_reduce(loss, group=cp_group)
        loss /= cp_size
    return loss


def use_ring_attn(cp_group) -> bool:
    """The models' switch (pithtrain/models/qwen3_30b_a3b.py:372): ring attention iff a CP group of size > 1."""
    return cp_group is not None and cp_group.size() > 1
