"""Test-only helpers: golden loaders, error metrics, an oracle-backed block backend and in-process ring comms."""

from __future__ import annotations

import threading
from pathlib import Path

import numpy as np
import torch

from oracle import attention_oracle as O

GOLDEN = Path(__file__).resolve().parent / "golden"

# Parity bars of the path (bf16 tensors: max-abs and mean-abs; LSE in fp32).
TOL_MAX_ABS = 2e-2
TOL_MEAN_ABS = 2e-3
TOL_LSE = 1e-3


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def load_golden_attention(name: str):
    z = np.load(GOLDEN / "golden_attention.npz")
    b, s, h, dq, dv, causal = (int(x) for x in z[f"{name}.meta"])
    t = {k: bf16_from_bits(z[f"{name}.{k}"]) for k in ("q", "k", "v", "do")}
    t.update({k: torch.from_numpy(z[f"{name}.{k}"]) for k in ("o", "dq", "dk", "dv")})
    t["causal"] = bool(causal)
    t["scale"] = dq ** -0.5
    return t


def assert_bf16_close(actual: torch.Tensor, expected: torch.Tensor, what: str,
                      max_abs: float = TOL_MAX_ABS, mean_abs: float = TOL_MEAN_ABS):
    """|actual - expected| <= max_abs (+ rounding allowance) everywhere and <= mean_abs on average.

    The absolute bar is below one bf16 ulp once |x| >= 8 (ulp 2^-4 there), so a tensor that has been ROUNDED to
    bf16 cannot meet it however exact the arithmetic was. Each side that is stored in bf16 therefore gets half a
    bf16 ulp of its own magnitude (2^-8 relative) on top of the bar; fp32 results get none.
    """
    half_ulps = int(actual.dtype == torch.bfloat16) + int(expected.dtype == torch.bfloat16)
    a = actual.detach().float().cpu()
    e = expected.detach().float().cpu()
    assert a.shape == e.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(e.shape)}"
    assert not torch.isnan(a).any(), f"{what}: NaN in result"
    d = (a - e).abs()
    excess = d - (max_abs + half_ulps * (2.0 ** -8) * e.abs())
    assert excess.max().item() <= 0, (f"{what}: |diff| exceeds {max_abs} + {half_ulps} bf16 half-ulp by "
                                      f"{excess.max().item():.3e} (max-abs diff {d.max().item():.3e})")
    assert d.mean().item() <= mean_abs, f"{what}: mean-abs {d.mean().item():.3e} > {mean_abs}"


def assert_lse_close(actual: torch.Tensor, expected: torch.Tensor, what: str = "lse", tol: float = TOL_LSE):
    a = actual.detach().float().cpu()
    e = expected.detach().float().cpu()
    fin = torch.isfinite(e)
    assert torch.equal(torch.isfinite(a), fin), f"{what}: finiteness pattern differs"
    d = (a[fin] - e[fin]).abs()
    if d.numel():
        assert d.max().item() <= tol, f"{what}: max-abs {d.max().item():.3e} > {tol}"


class OracleBlockBackend:
    """Block backend for the ring schedule that computes with the CPU oracle (tests only)."""

    def __init__(self, dtype=torch.float32):
        self.dtype = dtype

    def fwd_block(self, q, k, v, scale, causal, out, lse, merge):
        o, l = O.attention_fwd(q, k, v, scale, causal, 0, self.dtype)
        if merge:
            o, l = O.combine(out.to(self.dtype), lse.to(self.dtype), o, l, log2=True)
        out.copy_(o)
        lse.copy_(l)

    def delta(self, o, do):
        return O.delta(o, do, self.dtype).float()

    def bwd_block(self, q, k, v, do, lse, delta, scale, causal, dq_acc, dk_acc, dv_acc):
        dq, dk, dv = O.attention_bwd(q, k, v, do, lse, delta, scale, causal, 0, self.dtype)
        dq_acc += dq.float()
        dk_acc += dk.float()
        dv_acc += dv.float()

    def cast(self, acc):
        return acc.clone()


class OraclePartialsBackend(OracleBlockBackend):
    """The same, offering the one-pass merge of per-step partial results that the forward ring prefers."""

    max_partials = 16

    def __init__(self, dtype=torch.float32):
        super().__init__(dtype)
        self.partial_dtype = dtype
        self.merges = 0

    def fwd_block(self, q, k, v, scale, causal, out, lse, merge):
        assert not merge, "with combine_partials on offer the ring must not merge in the block"
        super().fwd_block(q, k, v, scale, causal, out, lse, False)

    def combine_partials(self, parts, B, S, H, D):
        self.merges += 1
        out = torch.zeros((B, S, H, D), dtype=self.dtype)
        lse = torch.full((B, H, S), -float("inf"), dtype=self.dtype)
        for o, l, r0 in parts:
            rows = o.shape[1]
            old = lse[:, :, r0:r0 + rows]
            co, cl = O.combine(out[:, r0:r0 + rows], old, o.to(self.dtype), l.to(self.dtype), log2=True)
            dead = torch.isinf(old) & torch.isinf(l.to(self.dtype))  # both sides saw no key: the formula gives NaN
            out[:, r0:r0 + rows] = torch.where(dead.permute(0, 2, 1).unsqueeze(-1), torch.zeros_like(co), co)
            lse[:, :, r0:r0 + rows] = torch.where(dead, torch.full_like(cl, -float("inf")), cl)
        return out, lse.float() if self.dtype != torch.float64 else lse


class ThreadRing:
    """In-process stand-in for the ring's P2P: ``cp_size`` threads, one per simulated rank, exchanging
    tensors through mailboxes. Lets the schedule (and on a GPU the real kernels) run on a single device.
    Like real P2P, the n-th send of a rank pairs with the n-th receive of its successor, whatever the
    order in which the requests are waited for."""

    def __init__(self, cp_size: int):
        self.cp_size = cp_size
        self.cond = threading.Condition()
        self.mail = [dict() for _ in range(cp_size)]  # mail[r][n]: n-th message addressed to rank r

    def comm(self, rank: int):
        ring = self
        state = {"seq": 0}

        class _Comm:
            def exchange(self, send, recv):
                n = state["seq"]
                state["seq"] += 1
                with ring.cond:
                    # a snapshot, because the sender may reuse its buffer before the receiver has copied it
                    ring.mail[(rank + 1) % ring.cp_size][n] = send.clone()
                    ring.cond.notify_all()
                return recv, n

            @staticmethod
            def wait(handle):
                recv, n = handle
                with ring.cond:
                    if not ring.cond.wait_for(lambda: n in ring.mail[rank], timeout=120):
                        raise TimeoutError(f"simulated rank {rank}: message {n} never arrived")
                    msg = ring.mail[rank].pop(n)
                recv.copy_(msg)

        return _Comm()

    def run(self, fn):
        """Runs ``fn(rank, comm)`` on every simulated rank; returns the results in rank order."""
        results = [None] * self.cp_size
        errors = []

        def target(r):
            try:
                results[r] = fn(r, self.comm(r))
            except BaseException as e:  # noqa: BLE001 - reported to the main thread
                errors.append((r, e))

        threads = [threading.Thread(target=target, args=(r,)) for r in range(self.cp_size)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0][1]
        return results


class LazyPullRing(ThreadRing):
    """Stand-in for the copy-engine exchange (``PeerRingComm``): nothing is snapshotted. The receiver PULLS from
    the sender's live buffer, and here it does so at the latest moment the protocol allows (inside its ``wait``),
    while the sender's ``wait`` blocks until that pull has happened. A schedule that overwrites a send buffer before
    waiting for its exchange, or reads a receive buffer early, computes with wrong data under this model and fails
    the comparison with the oracle. Send buffers must come from ``empty`` (the arena), as with the real thing."""

    def __init__(self, cp_size: int):
        super().__init__(cp_size)
        self.read = [set() for _ in range(cp_size)]  # read[r]: sequence numbers of rank r's sends already pulled

    def comm(self, rank: int):
        ring = self
        state = {"seq": 0, "arena": []}

        class _Comm:
            def begin(self, nbytes):
                state["arena"] = []

            def empty(self, numel, dtype):
                t = torch.empty(numel, dtype=dtype)
                state["arena"].append(t)
                return t

            def exchange(self, send, recv):
                assert any(send.data_ptr() == t.data_ptr() for t in state["arena"]), "send buffer is not arena memory"
                n = state["seq"]
                state["seq"] += 1
                with ring.cond:
                    ring.mail[(rank + 1) % ring.cp_size][n] = send  # the live buffer, not a copy
                    ring.cond.notify_all()
                return recv, n

            @staticmethod
            def wait(handle):
                recv, n = handle
                prev = (rank - 1) % ring.cp_size
                with ring.cond:
                    if not ring.cond.wait_for(lambda: n in ring.mail[rank], timeout=120):
                        raise TimeoutError(f"simulated rank {rank}: buffer {n} was never published")
                    recv.copy_(ring.mail[rank].pop(n))  # pull now: whatever the sender's buffer holds at this time
                    ring.read[prev].add(n)
                    ring.cond.notify_all()
                    if not ring.cond.wait_for(lambda: n in ring.read[rank], timeout=120):
                        raise TimeoutError(f"simulated rank {rank}: buffer {n} was never read by its successor")

        return _Comm()
