"""Ring attention on the real kernels: simulated ranks on one GPU (threads + mailboxes instead of NCCL), and, when
the box has at least two GPUs, real NCCL ranks through the public operator API."""

import os
import socket
import time

import pytest
import torch

from helpers import ThreadRing, assert_bf16_close, assert_lse_close
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


def _problem(S, hq, hkv, dqk, seed=42):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, S, hq, dqk, generator=g).bfloat16()
    k = torch.randn(1, S, hkv, dqk, generator=g).bfloat16()
    v = torch.randn(1, S, hkv, 128, generator=g).bfloat16()
    do = torch.randn(1, S, hq, 128, generator=g).bfloat16()
    return q, k, v, do


def _check(results, layout, full):
    from pithtrain_b200.operators.ring_attention import sharding as sh
    for name, i, dim in (("o", 0, 1), ("dq", 2, 1), ("dk", 3, 1), ("dv", 4, 1)):
        got = sh.unshard_sequence([r[i].cpu() for r in results], layout, seq_dim=dim)  # bf16 outputs
        assert_bf16_close(got, full[name], f"{layout} {name}")
    lse = sh.unshard_sequence([r[1].cpu() for r in results], layout, seq_dim=2)
    assert_lse_close(lse, full["lse_log2"])


@pytest.mark.parametrize("cp,layout,S,hq,hkv,dqk", [
    (2, "zigzag", 1024, 8, 2, 128),
    (4, "zigzag", 2048, 8, 2, 128),
    (4, "contiguous", 1024, 4, 4, 128),
    (8, "zigzag", 2048, 4, 1, 128),
    (4, "zigzag", 1024, 16, 16, 192),
    (2, "contiguous", 512, 16, 16, 192),
])
def test_ring_on_one_gpu_with_simulated_ranks(cuda_device, cp, layout, S, hq, hkv, dqk):
    from pithtrain_b200 import kernels
    from pithtrain_b200.operators.ring_attention import _ring
    from pithtrain_b200.operators.ring_attention import sharding as sh
    q, k, v, do = _problem(S, hq, hkv, dqk)
    scale = dqk ** -0.5
    full = O.full_attention_fwd_bwd(q, k, v, do, scale)

    def rank_fn(r, comm):
        torch.cuda.set_device(cuda_device)
        be = _ring.CudaBlockBackend()
        loc = lambda t: sh.shard_sequence(t, cp, r, layout).contiguous().to(cuda_device)  # noqa: E731
        ql, kl, vl, dol = loc(q), loc(k), loc(v), loc(do)
        out, lse = _ring.ring_forward(be, comm, ql, kl, vl, scale, r, cp, layout)
        dq, dk, dv = _ring.ring_backward(be, comm, ql, kl, vl, out, lse, dol, scale, r, cp, layout)
        return out, lse, dq, dk, dv

    res = ThreadRing(cp).run(rank_fn)
    torch.cuda.synchronize()
    kernels.check_device_status(cuda_device)
    _check(res, layout, full)


def test_cp1_operator_equals_full_attention(cuda_device):
    """cp_size = 1 through the autograd functions (no process group needed)."""
    from pithtrain_b200.operators.ring_attention import RingAttentionFunc, RingMLAAttentionFunc
    for fn, (hq, hkv, dqk) in ((RingAttentionFunc, (8, 2, 128)), (RingMLAAttentionFunc, (16, 16, 192))):
        q, k, v, do = (t.to(cuda_device) for t in _problem(512, hq, hkv, dqk))
        q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
        out = fn.apply(q, k, v, dqk ** -0.5, 0, 1, [0])
        out.backward(do)
        full = O.full_attention_fwd_bwd(q.detach().cpu(), k.detach().cpu(), v.detach().cpu(), do.cpu(), dqk ** -0.5)
        assert_bf16_close(out, full["o"], "O")
        assert_bf16_close(q.grad, full["dq"], "dQ")
        assert_bf16_close(k.grad, full["dk"], "dK")
        assert_bf16_close(v.grad, full["dv"], "dV")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_worker(rank, world, port, path):
    import torch.distributed as dist
    from pithtrain_b200 import kernels
    from pithtrain_b200.operators.ring_attention import ring_attention_func, ring_mla_attention_func
    from pithtrain_b200.operators.ring_attention import sharding as sh
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        group = dist.new_group(list(range(world)))
        results = {}
        for tag, fn, (hq, hkv, dqk), layout in (("gqa_zigzag", ring_attention_func, (8, 2, 128), "zigzag"),
                                                 ("gqa_contiguous", ring_attention_func, (8, 2, 128), "contiguous"),
                                                 ("mla_zigzag", ring_mla_attention_func, (16, 16, 192), "zigzag")):
            q, k, v, do = _problem(512 * world, hq, hkv, dqk)
            loc = lambda t: sh.shard_sequence(t, world, rank, layout).contiguous().to(dev)  # noqa: E731
            ql, kl, vl, dol = loc(q).requires_grad_(), loc(k).requires_grad_(), loc(v).requires_grad_(), loc(do)
            out = fn(ql, kl, vl, dqk ** -0.5, group, layout)
            out.backward(dol)
            torch.cuda.synchronize()
            kernels.check_device_status(dev)
            results[tag] = [t.detach().cpu() for t in (out, ql.grad, kl.grad, vl.grad)]
            if tag == "gqa_zigzag":
                # the same ring replayed from CUDA graphs (captured at the first call, replayed at the second)
                from pithtrain_b200.operators.ring_attention import enable_cuda_graphs, release_cuda_graphs
                enable_cuda_graphs(True)
                for _ in range(2):
                    ql.grad = kl.grad = vl.grad = None
                    out_g = fn(ql, kl, vl, dqk ** -0.5, group, layout)
                    out_g.backward(dol)
                torch.cuda.synchronize()
                kernels.check_device_status(dev)
                results["gqa_zigzag_graph"] = [t.detach().cpu() for t in (out_g, ql.grad, kl.grad, vl.grad)]
                enable_cuda_graphs(False)
                release_cuda_graphs()
        torch.save(results, os.path.join(path, f"rank{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_ring_over_nccl(cuda_device, tmp_path):
    import torch.multiprocessing as mp
    from pithtrain_b200.operators.ring_attention import sharding as sh
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    mp.spawn(_nccl_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    for tag, (hq, hkv, dqk), layout in (("gqa_zigzag", (8, 2, 128), "zigzag"),
                                        ("gqa_zigzag_graph", (8, 2, 128), "zigzag"),
                                        ("gqa_contiguous", (8, 2, 128), "contiguous"),
                                        ("mla_zigzag", (16, 16, 192), "zigzag")):
        q, k, v, do = _problem(512 * world, hq, hkv, dqk)
        full = O.full_attention_fwd_bwd(q, k, v, do, dqk ** -0.5)
        for i, name in enumerate(("o", "dq", "dk", "dv")):
            got = sh.unshard_sequence([r[tag][i] for r in res], layout, seq_dim=1)  # bf16 outputs
            assert_bf16_close(got, full[name], f"{tag} {name}")
            # the reference's own ring test metric (tests/test_ring_attention.py:91): cosine error < 1e-5
            assert O.cosine_error(got, full[name]) < 1e-5, (tag, name)


def test_flag_wait_is_bounded_and_reports(cuda_device):
    """A wait on a flag that nothing sets gives up after its limit and records code 3; the context stays usable.
    A signal followed by a wait on the same stream (stream order, so nothing spins) passes silently."""
    from pithtrain_b200 import _lib, kernels
    lib = _lib.load()
    flag = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    ctr = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(3):  # signal n, then wait for n: already satisfied
        _lib.check(lib.pith_flag_signal(flag.data_ptr(), ctr.data_ptr(), s), "signal")
        _lib.check(lib.pith_flag_wait(flag.data_ptr(), ctr.data_ptr() + 4, 0.2, status.data_ptr(), s), "wait")
    torch.cuda.synchronize()
    assert flag[0].item() == 3 and ctr[:2].tolist() == [3, 3] and status.item() == 0
    t0 = time.perf_counter()
    _lib.check(lib.pith_flag_wait(flag.data_ptr() + 4, ctr.data_ptr() + 8, 0.2, status.data_ptr(), s), "wait")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    word = status.item() & 0xFFFFFFFF
    assert word >> 24 == 3 and (word & 0xFFFFFF) == 1
    assert b"neighbour" in lib.pith_status_string(word)
    t0 = time.perf_counter()  # with the status word set, later waits return at once (counters still advance)
    for _ in range(20):
        _lib.check(lib.pith_flag_wait(flag.data_ptr() + 4, ctr.data_ptr() + 8, 0.2, status.data_ptr(), s), "wait")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0 and ctr[2].item() == 21
    assert lib.pith_flag_wait(0, ctr.data_ptr(), 0.2, 0, s) != 0  # null flag rejected on the host
    assert lib.pith_flag_wait(flag.data_ptr(), ctr.data_ptr(), 1e9, 0, s) != 0  # unbounded wait rejected
    assert torch.ones(4, device=cuda_device).sum().item() == 4.0


def _peer_worker(rank, world, port, path):
    import torch.distributed as dist
    from pithtrain_b200 import kernels
    from pithtrain_b200.operators import ring_attention as ra
    from pithtrain_b200.operators.ring_attention import sharding as sh
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        group = dist.new_group(list(range(world)))
        ra.enable_peer_copies(True, group)
        results = {}
        for tag, fn, (hq, hkv, dqk), layout in (("gqa_zigzag", ra.ring_attention_func, (8, 2, 128), "zigzag"),
                                                 ("mla_contiguous", ra.ring_mla_attention_func, (16, 16, 192),
                                                  "contiguous")):
            q, k, v, do = _problem(512 * world, hq, hkv, dqk)
            loc = lambda t: sh.shard_sequence(t, world, rank, layout).contiguous().to(dev)  # noqa: E731
            ql, kl, vl, dol = loc(q).requires_grad_(), loc(k).requires_grad_(), loc(v).requires_grad_(), loc(do)
            for graphs in (False, True):
                ra.enable_cuda_graphs(graphs)
                for _ in range(3 if graphs else 2):  # with graphs: capture at the first call, then two replays
                    ql.grad = kl.grad = vl.grad = None
                    out = fn(ql, kl, vl, dqk ** -0.5, group, layout)
                    out.backward(dol)
                torch.cuda.synchronize()
                kernels.check_device_status(dev)
                results[tag + ("_graph" if graphs else "")] = [t.detach().cpu()
                                                               for t in (out, ql.grad, kl.grad, vl.grad)]
            ra.enable_cuda_graphs(False)
        torch.save(results, os.path.join(path, f"rank{rank}.pt"))
        ra.release_peer_copies()
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_ring_over_peer_copies(cuda_device, tmp_path):
    """Ring blocks moved by the copy engines over IPC-mapped peer memory, eager and replayed from CUDA graphs."""
    import torch.multiprocessing as mp
    from pithtrain_b200.operators.ring_attention import sharding as sh
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    mp.spawn(_peer_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    for base, (hq, hkv, dqk), layout in (("gqa_zigzag", (8, 2, 128), "zigzag"),
                                         ("mla_contiguous", (16, 16, 192), "contiguous")):
        q, k, v, do = _problem(512 * world, hq, hkv, dqk)
        full = O.full_attention_fwd_bwd(q, k, v, do, dqk ** -0.5)
        for tag in (base, base + "_graph"):
            for i, name in enumerate(("o", "dq", "dk", "dv")):
                got = sh.unshard_sequence([r[tag][i] for r in res], layout, seq_dim=1)
                assert_bf16_close(got, full[name], f"{tag} {name}")
                assert O.cosine_error(got, full[name]) < 1e-5, (tag, name)
