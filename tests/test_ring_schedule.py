"""The ring schedule (forward and backward, contiguous and zigzag) with the oracle doing the block arithmetic:
in-process with simulated ranks, and as real ``torch.distributed`` ranks over gloo on CPU."""

import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import LazyPullRing, OracleBlockBackend, OraclePartialsBackend, ThreadRing
from oracle import attention_oracle as O
from pithtrain_b200.operators.ring_attention import _ring
from pithtrain_b200.operators.ring_attention import sharding as sh


def _problem(S, hq=4, hkv=2, dqk=32, dv=16, seed=42, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, S, hq, dqk, generator=g, dtype=dtype)
    k = torch.randn(1, S, hkv, dqk, generator=g, dtype=dtype)
    v = torch.randn(1, S, hkv, dv, generator=g, dtype=dtype)
    do = torch.randn(1, S, hq, dv, generator=g, dtype=dtype)
    return q, k, v, do


def _rank_fwd_bwd(rank, cp, comm, layout, q, k, v, do, scale, dtype):
    be = OracleBlockBackend(dtype)
    loc = lambda t: sh.shard_sequence(t, cp, rank, layout).contiguous()  # noqa: E731
    ql, kl, vl, dol = loc(q), loc(k), loc(v), loc(do)
    out, lse = _ring.ring_forward(be, comm, ql, kl, vl, scale, rank, cp, layout)
    dq, dk, dv = _ring.ring_backward(be, comm, ql, kl, vl, out, lse, dol, scale, rank, cp, layout)
    return out, lse, dq, dk, dv


def _check_against_full(results, cp, layout, q, k, v, do, scale, atol):
    full = O.full_attention_fwd_bwd(q, k, v, do, scale, torch.float64)
    for name, i, dim in (("o", 0, 1), ("lse_log2", 1, 2), ("dq", 2, 1), ("dk", 3, 1), ("dv", 4, 1)):
        got = sh.unshard_sequence([r[i].double() for r in results], layout, seq_dim=dim)
        assert torch.allclose(got, full[name], atol=atol), (layout, cp, name, (got - full[name]).abs().max())


@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
@pytest.mark.parametrize("cp", [1, 2, 3, 4, 8])
def test_schedule_in_process(cp, layout):
    S = 16 * cp * 2
    q, k, v, do = _problem(S, dtype=torch.float64)
    ring = ThreadRing(cp)
    res = ring.run(lambda r, comm: _rank_fwd_bwd(r, cp, comm, layout, q, k, v, do, 0.25, torch.float64))
    _check_against_full(res, cp, layout, q, k, v, do, 0.25, 5e-6)


@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
@pytest.mark.parametrize("cp", [2, 3, 8])
def test_forward_with_one_pass_merge(cp, layout):
    """A backend that offers ``combine_partials`` gets one un-merged partial per visible step (the zigzag
    ``q_second_half`` steps cover the second half of the rows only, contiguous ``skip`` steps none) and one merge."""
    S = 16 * cp * 2
    q, k, v, do = _problem(S, dtype=torch.float64)
    ring = ThreadRing(cp)
    backends = [OraclePartialsBackend(torch.float64) for _ in range(cp)]

    def rank(r, comm):
        loc = lambda t: sh.shard_sequence(t, cp, r, layout).contiguous()  # noqa: E731
        return _ring.ring_forward(backends[r], comm, loc(q), loc(k), loc(v), 0.25, r, cp, layout)

    res = ring.run(rank)
    full = O.full_attention_fwd_bwd(q, k, v, do, 0.25, torch.float64)
    for name, i, dim in (("o", 0, 1), ("lse_log2", 1, 2)):
        got = sh.unshard_sequence([x[i].double() for x in res], layout, seq_dim=dim)
        assert torch.allclose(got, full[name], atol=5e-6), (layout, cp, name, (got - full[name]).abs().max())
    assert all(b.merges == 1 for b in backends)


@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
@pytest.mark.parametrize("cp", [2, 3, 8])
def test_schedule_under_pull_exchange(cp, layout):
    """The buffer discipline the copy-engine exchange needs: receivers read the sender's live buffer as late as the
    protocol allows, so a buffer reused before its exchange was waited for would corrupt the result."""
    S = 16 * cp * 2
    q, k, v, do = _problem(S, dtype=torch.float64)
    res = LazyPullRing(cp).run(lambda r, comm: _rank_fwd_bwd(r, cp, comm, layout, q, k, v, do, 0.25, torch.float64))
    _check_against_full(res, cp, layout, q, k, v, do, 0.25, 5e-6)


def test_every_ring_step_opens_a_named_range():
    """One NVTX range per ring step and direction, named by step index and kind, so that a profile of a DualPipeV run
    shows them nested under the caller's ``layerNN.stage1_f`` / ``stage1_b`` ranges (pithtrain/dualpipe/execution.py:71,101)."""
    cp, S = 2, 64
    q, k, v, do = _problem(S, dtype=torch.float64)
    _ring.nvtx_log = log = []
    try:
        ThreadRing(1).run(lambda r, comm: _rank_fwd_bwd(1, cp, _OneRankOfTwo(), "zigzag", q, k, v, do, 0.25, torch.float64))
    finally:
        _ring.nvtx_log = None
    assert log == ["ring_attn.f.step0.causal", "ring_attn.f.step1.kv_first_half",
                   "ring_attn.b.step0.causal", "ring_attn.b.step1.kv_first_half", "ring_attn.b.home"]


class _OneRankOfTwo:
    """Stand-in communicator for a schedule-only run: the 'received' block is whatever the buffer holds."""

    def exchange(self, send, recv):
        recv.copy_(send)
        return None

    @staticmethod
    def wait(h):
        return None


def test_schedule_mla_shapes_in_process():
    """q/k width 192, v width 128, 16 heads without grouping (the DeepSeek-V2-Lite attention layout)."""
    cp, S = 4, 64
    q, k, v, do = _problem(S, hq=16, hkv=16, dqk=192, dv=128, dtype=torch.float64)
    res = ThreadRing(cp).run(lambda r, comm: _rank_fwd_bwd(r, cp, comm, "zigzag", q, k, v, do, 192 ** -0.5, torch.float64))
    _check_against_full(res, cp, "zigzag", q, k, v, do, 192 ** -0.5, 5e-6)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_worker(rank, world, port, layout, path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    try:
        torch.set_num_threads(1)
        q, k, v, do = _problem(32 * world)
        comm = _ring.RingComm(rank, world, list(range(world)), torch.device("cpu"))
        res = _rank_fwd_bwd(rank, world, comm, layout, q, k, v, do, 0.25, torch.float32)
        torch.save([t.clone() for t in res], os.path.join(path, f"rank{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("layout,world", [("zigzag", 2), ("contiguous", 2), ("zigzag", 4)])
def test_schedule_over_gloo(tmp_path, layout, world):
    mp.spawn(_gloo_worker, args=(world, _free_port(), layout, str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    q, k, v, do = _problem(32 * world)
    _check_against_full(res, world, layout, q, k, v, do, 0.25, 2e-5)


def _dying_peer_worker(rank, world, port, path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    if rank == 1:
        os._exit(0)  # leaves between steps, before posting its send
    comm = _ring.RingComm(rank, world, list(range(world)), torch.device("cpu"))
    try:
        comm.wait(comm.exchange(torch.zeros(4), torch.empty(4)))
        outcome = "completed"
    except Exception as e:  # noqa: BLE001
        outcome = f"raised {type(e).__name__}"
    with open(os.path.join(path, "outcome.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)


def test_lost_peer_surfaces_as_an_exception(tmp_path):
    """A ring neighbour that exits between steps must turn into a Python exception on the survivor,
    not a hang (host-side failure; no GPU involved)."""
    mp.spawn(_dying_peer_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "outcome.txt").read_text().startswith("raised")
