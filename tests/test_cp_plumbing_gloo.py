"""The context-parallel plumbing with real process groups: four gloo ranks on CPU, cp = 2 (so dp = 2).

Covers what the reference does at pithtrain/modules/distributed.py:127-194 (default group, device mesh,
`distributed_context`), pithtrain/modules/training.py:294 (CP group lookup),
pithtrain/tasks/pretrain_language_model.py:384-389 (loss average over the CP ranks) and
pithtrain/operators/ring_attention/standard.py:29-50 (`_ring_send_recv_kv` between ring neighbours given by their
GLOBAL ranks)."""

import datetime
import os
import socket
import types

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pithtrain_b200.modules import distributed as D
from pithtrain_b200.operators.ring_attention.standard import _ring_send_recv_kv


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world))
    torch.set_num_threads(1)
    cfg = types.SimpleNamespace(distributed=D.DistributedCfg(context_parallel_size=2, backend="gloo"))
    ctx = types.SimpleNamespace(distributed=D.DistributedCtx())
    with D.distributed_context(cfg, ctx) as dctx:
        assert dctx is ctx.distributed and dist.is_initialized()
        assert (dctx.rank, dctx.world_size) == (rank, world)
        # mesh (pp, dp, cp, ep) = (1, 2, 2, 1): cp is the fastest-moving of the non-trivial dimensions
        assert (dctx.pp_size, dctx.dp_size, dctx.cp_size, dctx.ep_size) == (1, 2, 2, 1)
        assert (dctx.dp_rank, dctx.cp_rank) == (rank // 2, rank % 2)
        group = D.get_cp_group(dctx)
        assert D.use_ring_attn(group) and group.size() == 2 and group.rank() == dctx.cp_rank
        members = [dist.get_global_rank(group, r) for r in range(2)]
        assert members == [2 * dctx.dp_rank, 2 * dctx.dp_rank + 1]

        # loss average over the CP ranks only: the two dp replicas keep different values
        loss = torch.tensor([float(rank)])
        D.average_loss_over_cp(loss, group, dctx.cp_size)
        assert loss.item() == 2 * dctx.dp_rank + 0.5
        assert D.average_loss_over_cp(None, group, dctx.cp_size) is None

        # blocking K/V exchange with the ring neighbours, addressed by global rank
        nxt, prv = members[(dctx.cp_rank + 1) % 2], members[(dctx.cp_rank - 1) % 2]
        k = torch.full((1, 4, 2, 8), float(rank))
        v = torch.full((1, 4, 2, 8), float(rank) + 0.25)
        rk, rv = _ring_send_recv_kv(k, v, nxt, prv)
        assert rk.shape == k.shape and rv.shape == v.shape
        assert torch.equal(rk, torch.full_like(k, float(prv))) and torch.equal(rv, torch.full_like(v, prv + 0.25))
        try:
            _ring_send_recv_kv(k.transpose(1, 2), v, nxt, prv)
            raised = False
        except AssertionError as e:
            raised = "not contiguous" in str(e)
        assert raised

        # sequence slicing and position ids agree with the group's rank
        tokens = torch.arange(32).view(1, 32)
        t_loc, l_loc = D.shard_batch_for_cp(tokens, tokens + 1, dctx.cp_rank, dctx.cp_size, "zigzag")
        pos = D.cp_position_ids(t_loc.shape[1], dctx.cp_rank, dctx.cp_size, "zigzag")
        assert torch.equal(t_loc, pos) and torch.equal(l_loc, pos + 1)
        dist.barrier()
    with open(os.path.join(path, f"ok{rank}"), "w") as f:
        f.write("ok")
    dist.destroy_process_group()


def test_cp_plumbing_over_gloo(tmp_path):
    world = 4
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(p.name for p in tmp_path.iterdir()) == [f"ok{r}" for r in range(world)]


def test_single_process_has_no_cp_group():
    ctx = D.DistributedCtx()
    assert ctx.cp_size == 1 and D.get_cp_group(ctx) is None and not D.use_ring_attn(None)
    loss = torch.tensor([3.0])
    assert D.average_loss_over_cp(loss, None, 1) is loss and loss.item() == 3.0
