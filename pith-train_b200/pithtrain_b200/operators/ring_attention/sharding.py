"""Sequence sharding layouts for context parallelism.

``contiguous`` is what PithTrain ships (pithtrain/tasks/pretrain_language_model.py:128-133 slices
``[cp_rank*chunk, (cp_rank+1)*chunk)``; position ids are ``cp_rank*seq_len + arange``,
pithtrain/models/qwen3_30b_a3b.py:817-821). ``zigzag`` is the load-balanced layout the reference
names as future work (pithtrain/operators/ring_attention/standard.py:16-18): the sequence is cut
into ``2*cp_size`` chunks and rank ``r`` holds chunks ``r`` and ``2*cp_size-1-r``, in that order.
"""

from __future__ import annotations

import torch

SHARDINGS = ("contiguous", "zigzag")


def check_sharding(sharding: str) -> str:
    if sharding not in SHARDINGS:
        raise ValueError(f"unknown sharding {sharding!r}; expected one of {SHARDINGS}")
    return sharding


def local_positions(seq_len: int, cp_size: int, cp_rank: int, sharding: str = "contiguous",
                    device=None) -> torch.Tensor:
    """Global token positions held by ``cp_rank``, in local storage order (int64 [seq_len // cp_size])."""
    check_sharding(sharding)
    if not 0 <= cp_rank < cp_size:
        raise ValueError(f"cp_rank {cp_rank} outside [0, {cp_size})")
    if sharding == "contiguous":
        if seq_len % cp_size:
            raise ValueError(f"sequence length {seq_len} is not divisible by cp_size {cp_size}")
        c = seq_len // cp_size
        return torch.arange(cp_rank * c, (cp_rank + 1) * c, device=device)
    if seq_len % (2 * cp_size):
        raise ValueError(f"zigzag sharding needs seq_len % (2*cp_size) == 0, got {seq_len} and cp_size {cp_size}")
    c = seq_len // (2 * cp_size)
    lo = torch.arange(cp_rank * c, (cp_rank + 1) * c, device=device)
    hi = torch.arange((2 * cp_size - 1 - cp_rank) * c, (2 * cp_size - cp_rank) * c, device=device)
    return torch.cat([lo, hi])


def shard_sequence(x: torch.Tensor, cp_size: int, cp_rank: int, sharding: str = "contiguous",
                   seq_dim: int = 1) -> torch.Tensor:
    """Slice of a full-sequence tensor owned by ``cp_rank`` (copy for zigzag, view for contiguous)."""
    n = x.shape[seq_dim]
    if sharding == "contiguous":
        c = n // cp_size
        if n % cp_size:
            raise ValueError(f"sequence length {n} is not divisible by cp_size {cp_size}")
        return x.narrow(seq_dim, cp_rank * c, c)
    check_sharding(sharding)
    if n % (2 * cp_size):
        raise ValueError(f"zigzag sharding needs seq_len % (2*cp_size) == 0, got {n} and cp_size {cp_size}")
    c = n // (2 * cp_size)
    return torch.cat([x.narrow(seq_dim, cp_rank * c, c), x.narrow(seq_dim, (2 * cp_size - 1 - cp_rank) * c, c)],
                     dim=seq_dim)


def unshard_sequence(shards: list[torch.Tensor], sharding: str = "contiguous", seq_dim: int = 1) -> torch.Tensor:
    """Inverse of :func:`shard_sequence` given every rank's shard in rank order."""
    cp_size = len(shards)
    if sharding == "contiguous":
        return torch.cat(shards, dim=seq_dim)
    check_sharding(sharding)
    chunks: list[torch.Tensor | None] = [None] * (2 * cp_size)
    for r, s in enumerate(shards):
        c = s.shape[seq_dim] // 2
        chunks[r] = s.narrow(seq_dim, 0, c)
        chunks[2 * cp_size - 1 - r] = s.narrow(seq_dim, c, c)
    return torch.cat(chunks, dim=seq_dim)


# Work a rank has when the key/value block of rank ``src`` visits it.
STEP_SKIP = "skip"                    # nothing visible (contiguous sharding, src > rank)
STEP_CAUSAL = "causal"                # own block: causal over the local order
STEP_FULL = "full"                    # every local query sees every key of the block
STEP_KV_FIRST_HALF = "kv_first_half"  # every local query sees the first half of the block only
STEP_Q_SECOND_HALF = "q_second_half"  # only the second half of the local queries sees the block (all of it)


def step_kind(sharding: str, cp_rank: int, src_rank: int) -> str:
    """Which part of (local Q) x (KV block of ``src_rank``) is inside the causal mask."""
    if src_rank == cp_rank:
        return STEP_CAUSAL
    if sharding == "contiguous":
        # pithtrain/operators/ring_attention/standard.py:89-90: compute iff kv_rank <= cp_rank
        return STEP_FULL if src_rank < cp_rank else STEP_SKIP
    check_sharding(sharding)
    return STEP_KV_FIRST_HALF if src_rank < cp_rank else STEP_Q_SECOND_HALF
