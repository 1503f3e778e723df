"""Ring schedule shared by the GQA and MLA context-parallel attention operators.

The schedule is the reference's (pithtrain/operators/ring_attention/standard.py:86-102 forward,
:116-187 backward) with three changes made for B200:

* the exchange of step ``t+1`` is issued BEFORE the attention kernel of step ``t`` and joined after
  it, so NCCL's copy over NVLink (on the process group's own stream) runs under the tensor-core work
  instead of after it (the reference waits on the requests right away, standard.py:46-50);
* every step writes its own bf16 partial (O, LSE) and one kernel merges all of them at the end (LSE-weighted mean in
  fp32, rounded once) instead of ~10 elementwise kernels per step (standard.py:53-66, :94). Rings longer than that
  kernel takes, and backends without it, merge inside the attention kernel's epilogue into an fp32 running (O, LSE);
* the backward circulates K/V again together with a travelling fp32 dK/dV accumulator that visits
  every rank and is home after ``cp_size`` hops, instead of keeping every visited K/V block alive
  and redistributing dK/dV by distance afterwards (standard.py:97-99, :164-187). Gradients are
  accumulated in fp32 across steps and rounded to bf16 once.

Besides the reference's contiguous sharding the schedule knows the zigzag layout (see ``sharding``).

The arithmetic is delegated to a *block backend*; the shipped one (:class:`CudaBlockBackend`) calls the
sm_100a kernels. Tests drive the same schedule over gloo with a backend of their own.
"""

from __future__ import annotations

import os as _os

import torch
import torch.distributed as dist

from . import sharding as sh


# NVTX ranges: one per ring, one per ring step and direction. They nest under whatever range the caller has open, so
# under DualPipeV a step shows up as "layerNN.stage1_f / ring_attn.f / step3.kv_first_half" (the reference opens
# "layerNN.stage1_f" and "...stage1_b" around attention at pithtrain/dualpipe/execution.py:71,88,101,111).
# PITH_B200_NVTX=0 turns them off; they are skipped for CPU tensors.
_nvtx_enabled = _os.environ.get("PITH_B200_NVTX", "1") != "0"
nvtx_log: list | None = None  # tests set this to a list to record the range names instead of asking a profiler


class _Range:
    def __init__(self, name: str, on: bool):
        self.name, self.on = name, on and _nvtx_enabled

    def __enter__(self):
        if nvtx_log is not None:
            nvtx_log.append(self.name)
        if self.on:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if self.on:
            torch.cuda.nvtx.range_pop()


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

    max_partials = 16
    partial_dtype = torch.bfloat16

    def combine_partials(self, parts, B, S, H, D):
        """``parts``: (O bf16 [B,rows,H,D], LSE [B,H,rows], first row) per ring step -> (O bf16 [B,S,H,D], LSE)."""
        return self.k.combine_partials(parts, B, S, H, D)

    def bwd_single(self, q, k, v, do, lse, delta, scale, dk_acc, dv_acc):
        """The whole backward is this one causal block (CP = 1): returns dQ. At head_dim 128 the dQ pass stores its
        bf16 result directly (no zeroed fp32 accumulator, no rounding pass)."""
        if q.shape[-1] == 128 and q.dtype == torch.bfloat16:
            dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
            self.k.attn_bwd(q, k, v, do, lse, delta, scale, True, 0, None, dk_acc, dv_acc, dq_out=dq)
            return dq
        dq_acc = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        self.k.attn_bwd(q, k, v, do, lse, delta, scale, True, 0, dq_acc, dk_acc, dv_acc)
        return self.k.cast_to_bf16(dq_acc).to(q.dtype)


class RingComm:
    """send-to-next / receive-from-previous over ``torch.distributed`` P2P, joined later.

    With NCCL the transfer runs on the process group's own communication stream: it is ordered after
    everything already enqueued on the caller's current stream, overlaps whatever the caller enqueues
    next, and ``wait`` makes the caller's stream wait for it. Every rank must call ``exchange`` the same
    number of times in the same order.
    """

    def __init__(self, cp_rank: int, cp_size: int, global_ranks, device: torch.device):
        self.next_global = global_ranks[(cp_rank + 1) % cp_size]
        self.prev_global = global_ranks[(cp_rank - 1) % cp_size]
        self.device = device

    def exchange(self, send: torch.Tensor, recv: torch.Tensor):
        assert send.is_contiguous() and recv.is_contiguous(), "ring attention send or recv buffer is not contiguous"
        return dist.batch_isend_irecv([dist.P2POp(dist.isend, send, self.next_global),
                                       dist.P2POp(dist.irecv, recv, self.prev_global)])

    @staticmethod
    def wait(reqs) -> None:
        for r in reqs:
            r.wait()


def _begin(comm, nbytes: int) -> None:
    """Tells a communicator that owns its ring buffers how much one ring needs."""
    if hasattr(comm, "begin"):
        comm.begin(nbytes)


def _ring_buffer(comm, numel: int, dtype, device):
    """A buffer that takes part in exchanges: from the communicator's arena if it has one."""
    if hasattr(comm, "empty"):
        return comm.empty(numel, dtype)
    return torch.empty(numel, dtype=dtype, device=device)


def _pack_kv(comm, k, v):
    """Two ping-pong buffers holding [K | V] back to back; the first is filled from (k, v)."""
    nk, nv = k.numel(), v.numel()
    bufs = [_ring_buffer(comm, nk + nv, k.dtype, k.device) for _ in range(2)]
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
    _begin(comm, 2 * (k.numel() + v.numel()) * k.element_size())
    bufs, nk = _pack_kv(comm, k, v)
    # One partial per step, merged after the last one: the attention kernels then store bf16 rows and nothing else (the
    # fp32 merge in their epilogue costs a quarter of a 4096 x 2048 step: 160 us against 127 us).
    lazy = hasattr(backend, "combine_partials") and cp_size <= getattr(backend, "max_partials", 0)
    if lazy:
        pdtype = getattr(backend, "partial_dtype", torch.bfloat16)
        parts = []
        cur = 0
        for t in range(cp_size):
            kind = sh.step_kind(sharding, cp_rank, (cp_rank - t) % cp_size)
            with _Range(f"ring_attn.f.step{t}.{kind}", q.is_cuda):
                reqs = comm.exchange(bufs[cur], bufs[cur ^ 1]) if t < cp_size - 1 else None
                kc, vc = _views(bufs[cur], nk, k.shape, v.shape)
                if kind != sh.STEP_SKIP:
                    row0 = c if kind == sh.STEP_Q_SECOND_HALF else 0
                    po = torch.empty((B, S - row0, Hq, Dv), dtype=pdtype, device=q.device)
                    pl = torch.empty((B, Hq, S - row0), dtype=torch.float32, device=q.device)
                    if kind == sh.STEP_KV_FIRST_HALF:
                        kc, vc = kc[:, :c], vc[:, :c]
                    backend.fwd_block(q[:, row0:], kc, vc, scale, kind == sh.STEP_CAUSAL, po, pl, False)
                    parts.append((po, pl, row0))
                if reqs is not None:
                    comm.wait(reqs)
                    cur ^= 1
        with _Range("ring_attn.f.merge", q.is_cuda):
            return backend.combine_partials(parts, B, S, Hq, Dv)
    acc = torch.empty((B, S, Hq, Dv), dtype=torch.float32, device=q.device)
    cur = 0
    for t in range(cp_size):
        kind = sh.step_kind(sharding, cp_rank, (cp_rank - t) % cp_size)
        with _Range(f"ring_attn.f.step{t}.{kind}", q.is_cuda):
            reqs = comm.exchange(bufs[cur], bufs[cur ^ 1]) if t < cp_size - 1 else None
            kc, vc = _views(bufs[cur], nk, k.shape, v.shape)
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
    nk, nv = k.numel(), v.numel()
    if cp_size == 1:
        dkv = torch.zeros(nk + nv, dtype=torch.float32, device=q.device)
        dk_acc, dv_acc = _views(dkv, nk, k.shape, v.shape)
        if hasattr(backend, "bwd_single"):
            dq = backend.bwd_single(q, k, v, dout, lse, delta, scale, dk_acc, dv_acc)
        else:
            dq_acc = torch.zeros((B, S, Hq, Dqk), dtype=torch.float32, device=q.device)
            backend.bwd_block(q, k, v, dout, lse, delta, scale, True, dq_acc, dk_acc, dv_acc)
            dq = backend.cast(dq_acc).to(q.dtype)
        return dq, backend.cast(dk_acc).to(k.dtype), backend.cast(dv_acc).to(v.dtype)
    dq_acc = torch.zeros((B, S, Hq, Dqk), dtype=torch.float32, device=q.device)
    c = S // 2
    _begin(comm, (nk + nv) * (2 * k.element_size() + 3 * 4))
    bufs, _ = _pack_kv(comm, k, v)
    grads = [_ring_buffer(comm, nk + nv, torch.float32, q.device) for _ in range(3)]
    cur = 0
    for t in range(cp_size):
        kind = sh.step_kind(sharding, cp_rank, (cp_rank - t) % cp_size)
        with _Range(f"ring_attn.b.step{t}.{kind}", q.is_cuda):
            kv_reqs = comm.exchange(bufs[cur], bufs[cur ^ 1]) if t < cp_size - 1 else None
            local, inbound, done = grads[t % 3], grads[(t + 1) % 3], grads[(t - 1) % 3]
            # the accumulator finished at the previous step travels on while this step computes
            g_reqs = comm.exchange(done, inbound) if t > 0 else None
            local.zero_()
            kc, vc = _views(bufs[cur], nk, k.shape, v.shape)
            dkc, dvc = _views(local, nk, k.shape, v.shape)
            if kind == sh.STEP_CAUSAL:
                backend.bwd_block(q, kc, vc, dout, lse, delta, scale, True, dq_acc, dkc, dvc)
            elif kind == sh.STEP_FULL:
                backend.bwd_block(q, kc, vc, dout, lse, delta, scale, False, dq_acc, dkc, dvc)
            elif kind == sh.STEP_KV_FIRST_HALF:
                backend.bwd_block(q, kc[:, :c], vc[:, :c], dout, lse, delta, scale, False, dq_acc, dkc[:, :c],
                                  dvc[:, :c])
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
    with _Range("ring_attn.b.home", q.is_cuda):
        comm.wait(comm.exchange(last, home))
    dk_acc, dv_acc = _views(home, nk, k.shape, v.shape)
    return backend.cast(dq_acc).to(q.dtype), backend.cast(dk_acc).to(k.dtype), backend.cast(dv_acc).to(v.dtype)


# ----------------------------------------------------------------------------- CUDA-graph replay of a whole ring
# At high CP degrees one ring step is 100-300 us of GPU work while issuing it from Python (two exchanges, two kernel
# launches, a memset and an add per backward step) costs about as much, so the host becomes the bottleneck. With
# graphs enabled the complete forward (and backward) ring of one shape is captured once, NCCL exchanges included, and
# replayed with a single launch. Opt-in, because a capture allocates static input/output buffers per shape and every
# rank must take the same decision at the same call.
_graphs_enabled = _os.environ.get("PITH_B200_RING_CUDA_GRAPHS", "0") == "1"
_graph_cache: dict = {}


def enable_cuda_graphs(flag: bool = True) -> None:
    """Replay ring attention from CUDA graphs (one per shape and direction). Call on every rank alike."""
    global _graphs_enabled
    _graphs_enabled = bool(flag)


def cuda_graphs_enabled() -> bool:
    return _graphs_enabled


def release_cuda_graphs() -> None:
    """Drops every captured graph and its buffers. Call before destroying the process group: a live graph that
    holds NCCL work keeps the communicator busy at teardown."""
    if _graph_cache:
        torch.cuda.synchronize()
        _graph_cache.clear()
        torch.cuda.synchronize()


class _GraphedCall:
    """``fn(*tensors) -> tuple of tensors`` captured once on static buffers; calls copy in, replay, copy out."""

    def __init__(self, fn, example_inputs):
        self.static_in = [torch.empty(t.shape, dtype=t.dtype, device=t.device) for t in example_inputs]
        for s, t in zip(self.static_in, example_inputs):
            s.copy_(t)
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):  # warm-up outside the capture (allocator, NCCL channels, function attributes)
            for _ in range(2):
                fn(*self.static_in)
        cur.wait_stream(side)
        torch.cuda.synchronize()
        from ... import kernels
        self._kernels = kernels
        launched = kernels.launch_count
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_out = tuple(fn(*self.static_in))
        self.launches = kernels.launch_count - launched  # kernels of libpith_b200.so inside one replay

    def __call__(self, *inputs):
        for s, t in zip(self.static_in, inputs):
            s.copy_(t)
        self.graph.replay()
        self._kernels._count(self.launches)
        return tuple(o.clone() for o in self.static_out)


# ----------------------------------------------------------------------------- copy-engine exchanges (opt-in)
_peer_enabled = _os.environ.get("PITH_B200_RING_PEER_COPIES", "0") == "1"
_peer_group = None
_peer_comms: dict = {}
_ring_groups: dict = {}


def enable_peer_copies(flag: bool = True, group=None) -> None:
    """Move ring blocks with the copy engines over peer-mapped memory instead of NCCL send/recv (single node).

    ``group`` is the process group used once per ring to exchange memory handles. Default: the ``cp_group`` given
    to ``ring_attention_func`` / ``ring_mla_attention_func``, or the world group when the autograd functions are
    called directly. It must contain the ring's ranks, and all its ranks must make the first ring call together."""
    global _peer_enabled, _peer_group
    _peer_enabled = bool(flag)
    _peer_group = group


def register_group(global_ranks, group) -> None:
    """Remembers the process group of a ring so that the peer exchange can set itself up over exactly its ranks."""
    _ring_groups[tuple(global_ranks)] = group


def peer_copies_enabled() -> bool:
    return _peer_enabled


def release_peer_copies() -> None:
    """Unmaps the neighbours' buffers (collective). Call before destroying the process group."""
    release_cuda_graphs()
    for comm in _peer_comms.values():
        comm.close()
    _peer_comms.clear()


def _make_comm(cp_rank, cp_size, global_ranks, device):
    if not (_peer_enabled and cp_size > 1 and device.type == "cuda"):
        return RingComm(cp_rank, cp_size, global_ranks, device)
    key = (cp_rank, cp_size, tuple(global_ranks), device.index)
    comm = _peer_comms.get(key)
    if comm is None:
        from ._peer import PeerRingComm
        wait_seconds = float(_os.environ.get("PITH_B200_RING_WAIT_SECONDS", "30"))
        comm = _peer_comms[key] = PeerRingComm(cp_rank, cp_size, global_ranks, device, group=_peer_group if _peer_group is not None else _ring_groups.get(tuple(global_ranks)),
                                               wait_seconds=wait_seconds)
    return comm


class RingFunction(torch.autograd.Function):
    """Causal ring attention as an autograd function, shared by the GQA and the MLA operator (the kernels pick
    their instantiation from the head dimensions): ``apply(q, k, v, softmax_scale, cp_rank, cp_size,
    global_ranks[, sharding])``. Mirrors pithtrain/operators/ring_attention/standard.py:69-189 and mla.py:43-149:
    backward returns one gradient per forward argument."""

    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, cp_rank, cp_size, global_ranks, *extra):
        sharding = extra[0] if extra else "contiguous"
        ctx.n_extra = len(extra)
        assert k.is_contiguous() and v.is_contiguous(), "ring attention k or v is not contiguous"
        sh.check_sharding(sharding)
        if q.is_cuda:  # an anomaly an earlier step reported surfaces here, without a synchronisation
            from ... import kernels
            kernels.poll_device_status(q.device)
        out, lse = ring_forward_auto(q, k, v, softmax_scale, cp_rank, cp_size, global_ranks, sharding)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.softmax_scale = softmax_scale
        ctx.cp_rank, ctx.cp_size, ctx.global_ranks, ctx.sharding = cp_rank, cp_size, global_ranks, sharding
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        dq, dk, dv = ring_backward_auto(q, k, v, out, lse, dout, ctx.softmax_scale, ctx.cp_rank, ctx.cp_size,
                                        ctx.global_ranks, ctx.sharding)
        if q.is_cuda:
            from ... import kernels
            kernels.post_status_copy(q.device)
        return (dq, dk, dv, None, None, None, None) + (None,) * ctx.n_extra


def _use_graph(q) -> bool:
    return _graphs_enabled and q.is_cuda and not torch.cuda.is_current_stream_capturing()


def _key(kind, tensors, scale, cp_rank, cp_size, global_ranks, sharding):
    return (kind, tuple((tuple(t.shape), t.dtype) for t in tensors), tensors[0].device.index, float(scale), cp_rank,
            cp_size, tuple(global_ranks), sharding)


def ring_forward_auto(q, k, v, scale, cp_rank, cp_size, global_ranks, sharding):
    """ring_forward on the CUDA backend, replayed from a graph when graphs are enabled and CP > 1."""
    backend = CudaBlockBackend()
    comm = _make_comm(cp_rank, cp_size, global_ranks, q.device)
    if cp_size == 1 or not _use_graph(q):
        with _Range("ring_attn.f", q.is_cuda):
            return ring_forward(backend, comm, q, k, v, scale, cp_rank, cp_size, sharding)
    key = _key("fwd", (q, k, v), scale, cp_rank, cp_size, global_ranks, sharding)
    g = _graph_cache.get(key)
    if g is None:
        g = _GraphedCall(lambda q_, k_, v_: ring_forward(backend, comm, q_, k_, v_, scale, cp_rank, cp_size, sharding),
                         (q, k, v))
        _graph_cache[key] = g
    return g(q, k, v)


def ring_backward_auto(q, k, v, out, lse, dout, scale, cp_rank, cp_size, global_ranks, sharding):
    """ring_backward on the CUDA backend, replayed from a graph when graphs are enabled and CP > 1."""
    backend = CudaBlockBackend()
    comm = _make_comm(cp_rank, cp_size, global_ranks, q.device)
    if cp_size == 1 or not _use_graph(q):
        with _Range("ring_attn.b", q.is_cuda):
            return ring_backward(backend, comm, q, k, v, out, lse, dout, scale, cp_rank, cp_size, sharding)
    key = _key("bwd", (q, k, v, out, lse, dout), scale, cp_rank, cp_size, global_ranks, sharding)
    g = _graph_cache.get(key)
    if g is None:
        g = _GraphedCall(lambda q_, k_, v_, o_, l_, d_: ring_backward(backend, comm, q_, k_, v_, o_, l_, d_, scale,
                                                                     cp_rank, cp_size, sharding),
                         (q, k, v, out, lse, dout))
        _graph_cache[key] = g
    return g(q, k, v, out, lse, dout)
