"""Sequence sharding layouts and the per-step work classification of the ring."""

import pytest
import torch

from pithtrain_b200.operators.ring_attention import sharding as sh
from oracle import attention_oracle as O


@pytest.mark.parametrize("cp", [1, 2, 4, 8])
@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
def test_shard_unshard_roundtrip(cp, layout):
    x = torch.arange(2 * 64 * 3).view(2, 64, 3)
    shards = [sh.shard_sequence(x, cp, r, layout) for r in range(cp)]
    assert all(s.shape[1] == 64 // cp for s in shards)
    assert torch.equal(sh.unshard_sequence(shards, layout), x)
    for r in range(cp):
        pos = sh.local_positions(64, cp, r, layout)
        assert torch.equal(x[:, pos], shards[r])


def test_zigzag_positions_match_oracle_and_definition():
    for cp in (2, 4, 8):
        for r in range(cp):
            pos = sh.local_positions(32 * cp, cp, r, "zigzag")
            assert torch.equal(pos, O.zigzag_indices(32 * cp, cp, r))
            c = 16
            assert pos[0] == r * c and pos[c] == (2 * cp - 1 - r) * c


def test_contiguous_positions_are_rank_offset_arange():
    assert torch.equal(sh.local_positions(64, 4, 2, "contiguous"), torch.arange(32, 48))


def test_step_kinds_cover_exactly_the_causal_mask():
    """For every (rank, src) the rows/columns a step kind touches are exactly the visible (q, k) pairs."""
    for layout in ("contiguous", "zigzag"):
        for cp in (2, 4):
            S = 8 * cp
            for r in range(cp):
                qpos = sh.local_positions(S, cp, r, layout)
                for src in range(cp):
                    kpos = sh.local_positions(S, cp, src, layout)
                    vis = kpos.unsqueeze(0) <= qpos.unsqueeze(1)
                    n, c = len(qpos), len(qpos) // 2
                    kind = sh.step_kind(layout, r, src)
                    exp = torch.zeros(n, n, dtype=torch.bool)
                    if kind == sh.STEP_CAUSAL:
                        exp = torch.tril(torch.ones(n, n, dtype=torch.bool))
                    elif kind == sh.STEP_FULL:
                        exp[:] = True
                    elif kind == sh.STEP_KV_FIRST_HALF:
                        exp[:, :c] = True
                    elif kind == sh.STEP_Q_SECOND_HALF:
                        exp[c:, :] = True
                    assert torch.equal(vis, exp), (layout, cp, r, src, kind)


def test_zigzag_is_balanced_and_contiguous_is_not():
    cp = 8
    work = lambda layout, r: sum({sh.STEP_SKIP: 0, sh.STEP_CAUSAL: 2, sh.STEP_FULL: 4, sh.STEP_KV_FIRST_HALF: 2,  # noqa: E731
                                  sh.STEP_Q_SECOND_HALF: 2}[sh.step_kind(layout, r, s)] for s in range(cp))
    assert len({work("zigzag", r) for r in range(cp)}) == 1
    assert work("contiguous", 0) < work("contiguous", cp - 1)


def test_bad_arguments():
    with pytest.raises(ValueError):
        sh.check_sharding("striped")
    with pytest.raises(ValueError):
        sh.local_positions(30, 4, 0, "zigzag")
    with pytest.raises(ValueError):
        sh.shard_sequence(torch.zeros(1, 10), 4, 0, "contiguous")
    with pytest.raises(ValueError):
        sh.local_positions(32, 4, 4, "contiguous")
