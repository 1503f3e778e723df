"""Ring schedule shared by the GQA and MLA context-parallel attention operators.

The schedule is the reference's (pithtrain/operators/ring_attention/standard.py:86-102 forward,
:116-187 backward) with three changes made for B200:

* the exchange of step ``t+1`` is issued BEFORE the attention kernel of step ``t`` and joined after
  it, so NCCL's copy over NVLink runs under the tensor-core work instead of after it (the reference
  waits on the requests right away, standard.py:46-50);
* partial results are merged inside the attention kernel's epilogue into one fp32 running (O, LSE)
  instead of ~10 elementwise kernels per step (standard.py:53-66, :94);
* the backward circulates K/V again together with a travelling fp32 dK/dV accumulator that visits
  every rank and is home after ``cp_size`` hops, instead of keeping every visited K/V block alive
  and redistributing dK/dV by distance afterwards (standard.py:97-99, :164-187). Gradients are
  accumulated in fp32 across steps and rounded to bf16 once.

Besides the reference's contiguous sharding the schedule knows the zigzag layout (see ``sharding``).

The arithmetic is delegated to a *block backend*; the shipped one (:class:`CudaBlockBackend`) calls the
sm_100a kernels. Tests drive the same schedule over gloo with a backend of their own.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import sharding as sh


class CudaBlockBackend:
    """Block arithmetic on the sm_100a kernels of ``libpith_b200.so``. CUDA tensors only."""

    def __init__(self):
        from ... import kernels  # deferred so that importing the operators never needs the library
        self.k = kernels

    def fwd_block(self, q, k, v, scale, causal, out, lse, merge):
        self.k.attn_fwd(q, k, v, scale, causal, 0, out=out, lse=lse,
                        prev_o=out if merge else None, prev_lse=lse if merge else None)

    def delta(self, o, do):
        return self.k.bwd_preprocess(o, do)

    def bwd_block(self, q, k, v, do, lse, delta, scale, causal, dq_acc, dk_acc, dv_acc):
        self.k.attn_bwd(q, k, v, do, lse, delta, scale, causal, 0, dq_acc, dk_acc, dv_acc)

    def cast(self, acc):
        return self.k.cast_to_bf16(acc)


class RingComm:
    """send-to-next / receive-from-previous over ``torch.distributed`` P2P, joined later.

    On CUDA the requests are issued from a side stream ordered after the caller's stream, so the
    transfer overlaps whatever the caller enqueues next; ``wait`` makes the caller's stream wait for
    it. Every rank must call ``exchange`` the same number of times in the same order.
    """

    _streams: dict[int, "torch.cuda.Stream"] = {}

    def __init__(self, cp_rank: int, cp_size: int, global_ranks, device: torch.device):
        self.next_global = global_ranks[(cp_rank + 1) % cp_size]
        self.prev_global = global_ranks[(cp_rank - 1) % cp_size]
        self.device = device
        self.stream = None
        if device.type == "cuda":
            idx = device.index if device.index is not None else torch.cuda.current_device()
            if idx not in RingComm._streams:
                RingComm._streams[idx] = torch.cuda.Stream(device=idx)
            self.stream = RingComm._streams[idx]

    def exchange(self, send: torch.Tensor, recv: torch.Tensor):
        assert send.is_contiguous() and recv.is_contiguous(), "ring attention send or recv buffer is not contiguous"
        ops = [dist.P2POp(dist.isend, send, self.next_global), dist.P2POp(dist.irecv, recv, self.prev_global)]
        if self.stream is None:
            return dist.batch_isend_irecv(ops)
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            reqs = dist.batch_isend_irecv(ops)
        return reqs

    @staticmethod
    def wait(reqs) -> None:
        for r in reqs:
            r.wait()


def _pack_kv(k, v):
    """Two ping-pong buffers holding [K | V] back to back; the first is filled from (k, v)."""
    nk, nv = k.numel(), v.numel()
    bufs = [torch.empty(nk + nv, dtype=k.dtype, device=k.device) for _ in range(2)]
    bufs[0][:nk].view(k.shape).copy_(k)
    bufs[0][nk:].view(v.shape).copy_(v)
    return bufs, nk


def _views(buf, nk, k_shape, v_shape):
    return buf[:nk].view(k_shape), buf[nk:].view(v_shape)


def ring_forward(backend, comm: RingComm, q, k, v, scale: float, cp_rank: int, cp_size: int, sharding: str):
    """Returns (O [B,S,Hq,Dv] in q.dtype, LSE_log2 fp32 [B,Hq,S]) for this rank's queries."""
    sh.check_sharding(sharding)
    B, S, Hq, _ = q.shape
    Dv = v.shape[-1]
    lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
    if cp_size == 1:
        out = torch.empty((B, S, Hq, Dv), dtype=q.dtype, device=q.device)
        backend.fwd_block(q, k, v, scale, True, out, lse, False)
        return out, lse
    if sharding == "zigzag" and S % 2:
        raise ValueError(f"zigzag sharding needs an even local sequence length, got {S}")
    c = S // 2
    bufs, nk = _pack_kv(k, v)
    acc = torch.empty((B, S, Hq, Dv), dtype=torch.float32, device=q.device)
    cur = 0
    for t in range(cp_size):
        src = (cp_rank - t) % cp_size
        reqs = comm.exchange(bufs[cur], bufs[cur ^ 1]) if t < cp_size - 1 else None
        kc, vc = _views(bufs[cur], nk, k.shape, v.shape)
        kind = sh.step_kind(sharding, cp_rank, src)
        if kind == sh.STEP_CAUSAL:  # always step 0: initialises the running (O, LSE)
            backend.fwd_block(q, kc, vc, scale, True, acc, lse, False)
        elif kind == sh.STEP_FULL:
            backend.fwd_block(q, kc, vc, scale, False, acc, lse, True)
        elif kind == sh.STEP_KV_FIRST_HALF:
            backend.fwd_block(q, kc[:, :c], vc[:, :c], scale, False, acc, lse, True)
        elif kind == sh.STEP_Q_SECOND_HALF:
            backend.fwd_block(q[:, c:], kc, vc, scale, False, acc[:, c:], lse[:, :, c:], True)
        if reqs is not None:
            comm.wait(reqs)
            cur ^= 1
    return backend.cast(acc).to(q.dtype), lse


def ring_backward(backend, comm: RingComm, q, k, v, out, lse, dout, scale: float, cp_rank: int, cp_size: int,
                  sharding: str):
    """Returns (dQ, dK, dV) in the input dtype for this rank's shard."""
    sh.check_sharding(sharding)
    B, S, Hq, Dqk = q.shape
    delta = backend.delta(out, dout)
    dq_acc = torch.zeros((B, S, Hq, Dqk), dtype=torch.float32, device=q.device)
    nk, nv = k.numel(), v.numel()
    if cp_size == 1:
        dkv = torch.zeros(nk + nv, dtype=torch.float32, device=q.device)
        dk_acc, dv_acc = _views(dkv, nk, k.shape, v.shape)
        backend.bwd_block(q, k, v, dout, lse, delta, scale, True, dq_acc, dk_acc, dv_acc)
        return backend.cast(dq_acc).to(q.dtype), backend.cast(dk_acc).to(k.dtype), backend.cast(dv_acc).to(v.dtype)
    c = S // 2
    bufs, _ = _pack_kv(k, v)
    grads = [torch.empty(nk + nv, dtype=torch.float32, device=q.device) for _ in range(3)]
    cur = 0
    for t in range(cp_size):
        src = (cp_rank - t) % cp_size
        kv_reqs = comm.exchange(bufs[cur], bufs[cur ^ 1]) if t < cp_size - 1 else None
        local, inbound, done = grads[t % 3], grads[(t + 1) % 3], grads[(t - 1) % 3]
        # the accumulator finished at the previous step travels on while this step computes
        g_reqs = comm.exchange(done, inbound) if t > 0 else None
        local.zero_()
        kc, vc = _views(bufs[cur], nk, k.shape, v.shape)
        dkc, dvc = _views(local, nk, k.shape, v.shape)
        kind = sh.step_kind(sharding, cp_rank, src)
        if kind == sh.STEP_CAUSAL:
            backend.bwd_block(q, kc, vc, dout, lse, delta, scale, True, dq_acc, dkc, dvc)
        elif kind == sh.STEP_FULL:
            backend.bwd_block(q, kc, vc, dout, lse, delta, scale, False, dq_acc, dkc, dvc)
        elif kind == sh.STEP_KV_FIRST_HALF:
            backend.bwd_block(q, kc[:, :c], vc[:, :c], dout, lse, delta, scale, False, dq_acc, dkc[:, :c], dvc[:, :c])
        elif kind == sh.STEP_Q_SECOND_HALF:
            backend.bwd_block(q[:, c:], kc, vc, dout[:, c:], lse[:, :, c:], delta[:, :, c:], scale, False,
                              dq_acc[:, c:], dkc, dvc)
        if g_reqs is not None:
            comm.wait(g_reqs)
            local.add_(inbound)
        if kv_reqs is not None:
            comm.wait(kv_reqs)
            cur ^= 1
    # last hop: the accumulator this rank just completed belongs to rank+1; ours arrives from rank-1
    last = grads[(cp_size - 1) % 3]
    home = grads[cp_size % 3]
    comm.wait(comm.exchange(last, home))
    dk_acc, dv_acc = _views(home, nk, k.shape, v.shape)
    return backend.cast(dq_acc).to(q.dtype), backend.cast(dk_acc).to(k.dtype), backend.cast(dv_acc).to(v.dtype)
