#!/usr/bin/env python
"""Benchmark of the context-parallel attention path: causal forward + backward, TFLOP/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload ...]

N = 1 runs the Qwen3-30B-A3B attention layer at S = 8192 on one GPU; N > 1 (launched with torchrun, one rank
per GPU) runs the same layer at global S = 32768 under zigzag context parallelism of degree N. One step is one
forward + backward of the public ring-attention operator on seeded synthetic bf16 inputs. FLOPs follow the
reference's convention (benchmarks/operators/mla/test_triton.py:7-14): causal forward = B*H*S^2*(Dqk+Dv),
backward = 2.5 x forward. Rank 0 prints one JSON line.

At N = 8 the same run also measures the DeepSeek-V2-Lite MLA ring and the S = 131072 ring and embeds both under
``workloads``. At every N > 1 the result of the ring is checked, outside the timed region, against an fp32 PyTorch
reference evaluated on slices of the sequence (``parity``).

``--impl reference`` times the reference's CPU attention arithmetic (the oracle's restatement) on the host cores.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (ROOT, ROOT / "pith-train_b200"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import torch  # noqa: E402

WORKLOADS = {
    # name: (S_global at N=1, S_global at N>1, Hq, Hkv, Dqk, Dv, description)
    "qwen3": (8192, 32768, 32, 4, 128, 128, "Qwen3-30B-A3B attention layer, B=1, Hq=32, Hkv=4, head_dim=128"),
    "mla": (8192, 32768, 16, 16, 192, 128, "DeepSeek-V2-Lite MLA attention, B=1, 16 heads, q/k dim 192, v dim 128"),
    "long": (16384, 131072, 32, 4, 128, 128, "Qwen3-30B-A3B attention layer, long context"),
}
METRIC = "causal fwd+bwd attention TFLOP/s (whole job)"
BRACKETS = 10  # the timed bracket of `steps` steps is repeated this many times; the median bracket is reported


def fwd_bwd_flops(S, Hq, Dqk, Dv):
    return 3.5 * Hq * float(S) * S * (Dqk + Dv)


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        p = json.loads(f.read_text())
        return {"bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


# DRAM read + write bytes per launch of a kernel at an exact workload, taken from the ncu summary committed beside
# it. Keyed by (workload, n_gpus, kernel substring); anything else reports null.
NCU_TRAFFIC = {
    ("qwen3", 1, "dK/dV"): (343.2e6, "profiles/attention_kernels_qwen3_s8192.md (attn_bwd128_kernel<kDkDv>, S = 8192)"),
}


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only) while the timed region runs: a thread every
    20 ms plus one explicit sample taken while the timed work is still in flight."""

    def __init__(self, index: int):
        self.rows = []
        self.index = index
        self.nv = self.handle = None
        self.stop = threading.Event()
        self.thread = None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv, self.handle = pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
        except Exception:  # no NVML: the summary says so (samples = 0)
            self.nv = None
        return self

    def sample(self):
        nv = self.nv
        if nv is None:
            return
        try:
            sm = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
            mx = nv.nvmlDeviceGetMaxClockInfo(self.handle, nv.NVML_CLOCK_SM)
            bits = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
        except Exception:
            return
        flag = lambda name: "Active" if bits & getattr(nv, name, 0) else "Not Active"  # noqa: E731
        self.rows.append([str(sm), str(mx), flag("nvmlClocksEventReasonHwSlowdown"),
                          flag("nvmlClocksEventReasonHwThermalSlowdown"),
                          flag("nvmlClocksEventReasonSwThermalSlowdown"), flag("nvmlClocksEventReasonSwPowerCap")])

    def _loop(self):
        while not self.stop.is_set():
            self.sample()
            self.stop.wait(0.02)

    def __exit__(self, *exc):
        self.stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def check_heads(Hq, Hkv):
    """The kv head (and its group of query heads) whose results the multi-GPU parity check recomputes: the last."""
    g = Hq // Hkv
    return Hkv - 1, list(range(Hq - g, Hq))


def make_inputs(S_global, Hq, Hkv, Dqk, Dv, cp, rank, sharding, seed=42, keep_check_heads=False):
    """Seeded N(0,1) bf16 Q, K, V, dO at the global shape, sliced to this rank's shard (pinned host tensors).

    With keep_check_heads the full-sequence slices of one kv head and its query heads are returned as well
    ([S, G, Dqk], [S, Dqk], [S, Dv], [S, G, Dv], bf16 on the CPU) for the parity check."""
    from pithtrain_b200.operators.ring_attention import sharding as sh
    g = torch.Generator().manual_seed(seed)
    kvh, qhs = check_heads(Hq, Hkv)
    out, kept = [], []
    for shape, heads in (((1, S_global, Hq, Dqk), qhs), ((1, S_global, Hkv, Dqk), kvh), ((1, S_global, Hkv, Dv), kvh),
                         ((1, S_global, Hq, Dv), qhs)):
        full = torch.randn(shape, generator=g, dtype=torch.float32).bfloat16()
        loc = sh.shard_sequence(full, cp, rank, sharding).contiguous() if cp > 1 else full
        out.append(loc.pin_memory() if torch.cuda.is_available() else loc)
        if keep_check_heads:
            kept.append(full[0][:, heads].clone())
        del full
    return (out, kept) if keep_check_heads else out


@torch.no_grad()
def reference_slices(qg, kg, vg, dog, scale, rows, cols, chunk):
    """Causal attention forward + backward of one kv head and its G query heads in fp32 PyTorch on the GPU
    (cuBLAS SGEMM, TF32 off), evaluated over the whole sequence in row chunks; keeps O, LSE (log2), dQ at the query
    positions `rows` and dK, dV at the key positions `cols` (sorted int64 tensors of global positions)."""
    S, G, Dqk = qg.shape
    Dv = vg.shape[-1]
    dev = qg.device
    o_rows = torch.empty(len(rows), G, Dv, device=dev)
    lse_rows = torch.empty(len(rows), G, device=dev)
    dq_rows = torch.empty(len(rows), G, Dqk, device=dev)
    dk = torch.zeros(len(cols), Dqk, device=dev)
    dv = torch.zeros(len(cols), Dv, device=dev)
    pos = torch.arange(S, device=dev)
    for m0 in range(0, S, chunk):
        m1 = min(S, m0 + chunk)
        csel = cols < m1
        rsel = (rows >= m0) & (rows < m1)
        if not bool(rsel.any()) and not bool(csel.any()):
            continue
        kk, vv, qc, doc = kg[:m1], vg[:m1], qg[m0:m1], dog[m0:m1]
        s = torch.einsum("cgd,nd->gcn", qc, kk) * scale
        s.masked_fill_(pos[None, None, :m1] > pos[None, m0:m1, None], float("-inf"))
        lse = torch.logsumexp(s, dim=-1)             # [G, c], natural log
        p = torch.exp(s - lse[..., None])
        del s
        o = torch.einsum("gcn,nd->cgd", p, vv)
        dl = (o * doc).sum(-1)                        # [c, G]
        if bool(rsel.any()):
            idx = rows[rsel] - m0
            o_rows[rsel] = o[idx]
            lse_rows[rsel] = lse.T[idx] * math.log2(math.e)
            dp = torch.einsum("cgd,nd->gcn", doc[idx], vv)
            ds = p[:, idx] * (dp - dl[idx].T[..., None])
            dq_rows[rsel] = torch.einsum("gcn,nd->cgd", ds, kk) * scale
            del dp, ds
        if bool(csel.any()):
            cc = cols[csel]
            pc = p[:, :, cc]
            dv[csel] += torch.einsum("gcn,cgd->nd", pc, doc)
            dpc = torch.einsum("cgd,nd->gcn", doc, vg[cc])
            dk[csel] += torch.einsum("gcn,cgd->nd", pc * (dpc - dl.T[..., None]), qc) * scale
        del p
    return o_rows, lse_rows, dq_rows, dk, dv


def parity_record(dev, kept, local_pos, results, Hq, Hkv, scale, world):
    """Compares this rank's slices of O, dQ (first / last 128 local query positions, the check heads) and dK, dV
    (first / last 128 local key positions, the check kv head) with `reference_slices`; the worst figures over all
    ranks are returned. Bars: max-abs <= 2e-2 + half a bf16 ulp of the value (the results are rounded to bf16),
    mean-abs <= 2e-3, LSE <= 1e-3, and the reference's ring-test criterion 1 - cosine < 1e-5."""
    import torch.distributed as dist
    torch.backends.cuda.matmul.allow_tf32 = False
    qg, kg, vg, dog = (t.to(dev).float() for t in kept)
    kvh, qhs = check_heads(Hq, Hkv)
    n = min(128, local_pos.numel() // 2)
    sel = torch.cat([torch.arange(n), torch.arange(local_pos.numel() - n, local_pos.numel())])
    gpos = local_pos[sel].to(dev)
    order = torch.argsort(gpos)
    rows = gpos[order]
    S = qg.shape[0]
    ro, rl, rdq, rdk, rdv = reference_slices(qg, kg, vg, dog, scale, rows, rows, chunk=1024 if S <= 32768 else 512)
    out, lse, dq, dk, dv = results
    pick = sel.to(dev)[order]
    got = {
        "o": (out.detach()[0][pick][:, qhs].float(), ro), "dq": (dq.detach()[0][pick][:, qhs].float(), rdq),
        "dk": (dk.detach()[0][pick][:, kvh].float(), rdk), "dv": (dv.detach()[0][pick][:, kvh].float(), rdv),
    }
    rec, ok = {}, True
    for name, (a, b) in got.items():
        err = (a - b).abs()
        excess = float((err - (2e-2 + 2.0 ** -8 * b.abs())).max())
        cos = 1.0 - float(torch.nn.functional.cosine_similarity(a.flatten().double(), b.flatten().double(), dim=0))
        vals = torch.tensor([float(err.max()), float(err.mean()), excess, cos], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        mx, mean, excess, cos = (float(x) for x in vals)
        rec[name] = {"max_abs": mx, "mean_abs": mean, "one_minus_cosine": cos}
        ok = ok and excess <= 0 and mean <= 2e-3 and cos < 1e-5
    lerr = torch.tensor([float((lse[0][qhs][:, pick].T - rl).abs().max())], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(lerr, op=dist.ReduceOp.MAX)
    rec["lse"] = {"max_abs": float(lerr)}
    ok = ok and float(lerr) <= 1e-3
    rec["passed"] = bool(ok)
    rec["checked"] = (f"per rank: first and last {n} local positions; O, LSE, dQ of query heads {qhs[0]}..{qhs[-1]}, dK, dV of "
                      f"kv head {kvh}; against fp32 PyTorch attention (cuBLAS SGEMM, TF32 off) over the whole sequence; "
                      "worst rank reported")
    rec["bars"] = "max_abs <= 2e-2 + 2^-8 |x|, mean_abs <= 2e-3, lse <= 1e-3, 1 - cosine < 1e-5"
    return rec


def cpu_attention_sample(S, heads, group, Dqk, Dv, seed=42):
    """The reference's fp32 attention arithmetic, forward + backward, on `heads` query heads (kv heads = heads/group)
    of a causal sequence of length S, run by the CPU oracle. Returns (seconds, flops)."""
    from oracle import attention_oracle as O
    g = torch.Generator().manual_seed(seed)
    kvh = max(1, heads // group)
    q = torch.randn(1, S, heads, Dqk, generator=g)
    k = torch.randn(1, S, kvh, Dqk, generator=g)
    v = torch.randn(1, S, kvh, Dv, generator=g)
    do = torch.randn(1, S, heads, Dv, generator=g)
    t0 = time.perf_counter()
    O.full_attention_fwd_bwd(q, k, v, do, Dqk ** -0.5)
    return time.perf_counter() - t0, fwd_bwd_flops(S, heads, Dqk, Dv)


def host_threads() -> int:
    """The CPU arm uses every host core it may run on, whatever OMP_NUM_THREADS the launcher exported."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def run_reference(args, rank):
    """Reference arm: CPU attention (oracle port of the reference's PyTorch math) on the host cores."""
    if rank != 0:
        return
    threads = host_threads()
    name = args.workload
    S1, SN, Hq, Hkv, Dqk, Dv, desc = WORKLOADS[name]
    S = S1 if args.gpus == 1 else SN
    group = Hq // Hkv
    # bounded sample: a shorter sequence of the same layer; attention cost grows with S^2, the rate does not
    S_s, heads = min(S, 2048), min(Hq, group)
    times = []
    for i in range(args.warmup + args.steps):
        dt, fl = cpu_attention_sample(S_s, heads, group, Dqk, Dv)
        if i >= args.warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    tflops = fl / sec / 1e12
    sample = f"{heads} query heads ({max(1, heads // group)} kv head) x S={S_s} causal fwd+bwd in fp32 per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{desc}; S={S}; CPU sample: {sample}"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": sample, "host_cpus": os.cpu_count()},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- the reference's GPU kernels, same box
def gpu_reference_child(kind: str):
    """Runs in a child process (Triton's autotuning of the reference's MLA kernels compiles ~150 variants; a child
    can be given a time limit): times the reference's own GPU attention at S = 8192 with CUDA events and prints one
    JSON object. kind = 'flash' (flash_attn_func, the arithmetic behind the reference's GQA path, config 2 shape)
    or 'triton_mla' (the reference's Triton MLA custom op from an installed copy under baseline/_ref)."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    S = 8192
    g = torch.Generator().manual_seed(42)
    if kind == "flash":
        from flash_attn import flash_attn_func
        import flash_attn
        Hq, Hkv, Dqk, Dv = 32, 4, 128, 128
        what = f"flash_attn_func {flash_attn.__version__} (pithtrain/models/qwen3_30b_a3b.py:424)"
    else:
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        from pithtrain.operators.mla.triton import _mla_triton_fwd
        Hq, Hkv, Dqk, Dv = 16, 16, 192, 128
        what = "pithtrain::mla_triton_fwd / _bwd custom ops (pithtrain/operators/mla/triton.py:445-508), autotuned"
    scale = Dqk ** -0.5
    q = torch.randn(1, S, Hq, Dqk, generator=g).bfloat16().to(dev).requires_grad_()
    k = torch.randn(1, S, Hkv, Dqk, generator=g).bfloat16().to(dev).requires_grad_()
    v = torch.randn(1, S, Hkv, Dv, generator=g).bfloat16().to(dev).requires_grad_()
    do = torch.randn(1, S, Hq, Dv, generator=g).bfloat16().to(dev)

    def step():
        q.grad = k.grad = v.grad = None
        if kind == "flash":
            out = flash_attn_func(q, k, v, softmax_scale=scale, causal=True)
        else:
            out, _ = _mla_triton_fwd(q, k, v, scale)
        out.backward(do)

    t0 = time.perf_counter()
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    warm_s = time.perf_counter() - t0
    times = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            step()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / 5)
    ms = statistics.median(times)
    print(json.dumps({"what": what, "S": S, "Hq": Hq, "Hkv": Hkv, "Dqk": Dqk, "Dv": Dv, "ms_per_step": ms,
                      "tflops": fwd_bwd_flops(S, Hq, Dqk, Dv) / (ms * 1e-3) / 1e12, "warmup_seconds": warm_s}), flush=True)


def gpu_reference(kind: str, limit_s: int):
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    try:
        r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--gpu-reference-child", kind], capture_output=True,
                           text=True, timeout=limit_s, env=env, cwd=str(ROOT))
    except subprocess.TimeoutExpired:
        return {"unavailable": f"did not finish within {limit_s} s"}
    for line in reversed(r.stdout.splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    return {"unavailable": (r.stderr.strip().splitlines() or ["no output"])[-1][:300]}


# ----------------------------------------------------------------------------- our arm
class Bench:
    def __init__(self, args, rank, world, local_rank):
        import torch.distributed as dist
        from pithtrain_b200 import build, kernels
        from pithtrain_b200.operators import ring_attention as ring
        self.args, self.rank, self.world = args, rank, world
        self.dist, self.kernels, self.ring = dist, kernels, ring
        if world == 1 or local_rank == 0:
            build.build_library()
        self.dev = torch.device("cuda", local_rank)
        self.local_rank = local_rank
        torch.cuda.set_device(self.dev)
        if world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)
            dist.barrier()  # the library is in place on every rank
        self.pk = peaks()
        self.exchange_note = None
        self.use_graphs = world > 1 and args.graphs
        ring.enable_cuda_graphs(self.use_graphs)  # public switch: whole rings are captured once and replayed
        self.use_peer = world > 1 and args.exchange == "peer"
        ring.enable_peer_copies(self.use_peer)    # public switch: exchanges run on the copy engines, not in NCCL

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def timed(self, run, steps, brackets=1, in_flight=None, finish=None, queue_ahead=False):
        """Device time of `steps` calls of run(), max over ranks, in ms per call: the median of `brackets` brackets,
        each bracketed by a barrier + synchronize on both sides.

        queue_ahead (single kernels only): a spin kernel of a few ms runs first, so that the host has enqueued all
        launches before the first one starts and the events bracket GPU execution, not Python call overhead."""
        per = []
        for b in range(brackets):
            self.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if queue_ahead:
                torch.cuda._sleep(int(6e6))
            e0.record()
            for _ in range(steps):
                run()
            if finish is not None:
                finish()
            e1.record()
            if in_flight is not None and b == brackets // 2:
                in_flight()  # called while the last steps still run on the GPU
            self.barrier()
            ms = torch.tensor([e0.elapsed_time(e1) / steps], device=self.dev)
            if self.world > 1:
                self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
            per.append(float(ms.item()))
        return statistics.median(per), per

    def probe_exchange(self, step):
        """The copy-engine exchange needs CUDA IPC between the ranks' processes; where the host forbids it, every rank
        fails alike while mapping its neighbour's memory, and all of them fall back to the NCCL exchange together."""
        if not self.use_peer:
            return
        ok = torch.ones(1, device=self.dev)
        try:
            step()
            torch.cuda.synchronize()
            self.kernels.check_device_status(self.dev)
        except Exception as e:  # noqa: BLE001 - reported in the JSON line
            ok.zero_()
            self.exchange_note = f"copy-engine exchange unavailable ({type(e).__name__}: {str(e)[:120]}); NCCL send/recv used"
        self.dist.all_reduce(ok, op=self.dist.ReduceOp.MIN)
        if ok.item() == 0:
            self.use_peer = False
            self.ring.enable_peer_copies(False)
            self.exchange_note = self.exchange_note or "copy-engine exchange unavailable on another rank; NCCL send/recv used"

    def measure(self, name, headline, S_override=None):
        args, rank, world, dev, kernels, ring = self.args, self.rank, self.world, self.dev, self.kernels, self.ring
        _ring = ring._ring
        S1, SN, Hq, Hkv, Dqk, Dv, desc = WORKLOADS[name]
        S = S_override or (S1 if world == 1 else SN)
        S_loc = S // world
        scale = Dqk ** -0.5
        fn = ring.RingMLAAttentionFunc if Dqk == 192 else ring.RingAttentionFunc
        global_ranks = list(range(world))
        check = world > 1 or args.parity
        made = make_inputs(S, Hq, Hkv, Dqk, Dv, world, rank, args.sharding, keep_check_heads=check)
        (hq, hk, hv, hdo), kept = made if check else (made, None)
        q, k, v, do = (t.to(dev) for t in (hq, hk, hv, hdo))
        for t in (q, k, v):
            t.requires_grad_()

        def step(q_=q, k_=k, v_=v, do_=do):
            q_.grad = k_.grad = v_.grad = None
            out = fn.apply(q_, k_, v_, scale, rank, world, global_ranks, args.sharding)
            out.backward(do_)
            return out, q_.grad, k_.grad, v_.grad

        if headline:
            self.probe_exchange(step)

        # ---- resident-input measurement (`value`)
        warm = max(3, args.warmup)
        for _ in range(warm):
            step()
        kernels.check_device_status(dev)
        launches0 = kernels.launch_count
        with ClockSampler(self.local_rank) as clk:
            ms, brackets = self.timed(step, args.steps, BRACKETS if headline else 3, clk.sample)
        launches = (kernels.launch_count - launches0) // (args.steps * len(brackets))
        kernels.check_device_status(dev)
        flops_total = fwd_bwd_flops(S, Hq, Dqk, Dv)
        tflops_total = flops_total / (ms * 1e-3) / 1e12
        pk = self.pk
        rec = {
            "workload": f"{desc}; global S={S}, causal; " + (
                f"zigzag context parallel CP={world} ({S_loc} tokens per GPU)" if world > 1 and args.sharding == "zigzag"
                else f"{args.sharding} CP={world}" if world > 1 else "single GPU (CP=1)"),
            "value": tflops_total, "unit": "TFLOP/s", "ms_per_step": ms, "ms_per_step_brackets": brackets,
            "tflops_per_gpu": tflops_total / world,
            "frac_of_measured_bf16_peak": tflops_total / world / pk["bf16_tflops"],
            # the timed region is hundreds of steps long and runs under the power cap: the sustained GEMM figure is the
            # like-for-like denominator, the burst one above the stricter
            "frac_of_measured_sustained_peak": (tflops_total / world / pk["bf16_tflops_sustained"]
                                                if pk.get("bf16_tflops_sustained") else None),
            "frac_of_nominal_2250": tflops_total / world / 2250.0,
            "tokens_per_s": S / (ms * 1e-3), "gpu_launches": launches, "clocks": clk.summary(),
        }

        # ---- parity of this very computation, outside the timed region
        if check:
            from pithtrain_b200.operators.ring_attention import sharding as sh
            out, dq, dk, dv = step()
            # the operator keeps the LSE to itself: recompute it with the forward half of the ring
            o2, lse = _ring.ring_forward_auto(q.detach(), k.detach(), v.detach(), scale, rank, world, global_ranks,
                                              args.sharding)
            torch.cuda.synchronize()
            kernels.check_device_status(dev)
            lpos = sh.local_positions(S, world, rank, args.sharding) if world > 1 else torch.arange(S)
            rec["parity"] = parity_record(dev, kept, lpos, (out, lse, dq, dk, dv), Hq, Hkv, scale, world)
            del kept, out, dq, dk, dv, o2, lse

        # ---- the same ring with the NCCL send/recv exchange (the transport the operator uses by default)
        if world > 1 and self.use_peer and not args.no_nccl_compare:
            ring.release_cuda_graphs()
            ring.enable_peer_copies(False)
            for _ in range(3):
                step()
            ms_nccl, _ = self.timed(step, max(3, args.steps // 2), 3)
            ring.release_cuda_graphs()
            ring.enable_peer_copies(True)
            step()
            rec["nccl_exchange"] = {"ms_per_step": ms_nccl,
                                    "tflops_per_gpu": flops_total / (ms_nccl * 1e-3) / 1e12 / world}

        # ---- comm / compute overlap of one ring (N > 1): compute alone, exchanges alone, both
        if world > 1 and not args.no_overlap:
            rec["overlap"] = self.overlap(q.detach(), k.detach(), v.detach(), do, scale, global_ranks)

        if not headline:
            return rec

        # ---- end to end through the public operator with host buffers (H2D of inputs, D2H of results, every step).
        # The copies run on their own streams with two sets of device input buffers, the way a training loop prefetches:
        # step i's inputs arrive while step i-1 computes and step i-1's results leave while step i computes. Every step
        # still copies all of its inputs from pinned memory and all of its results back inside the timed region.
        host_in = (hq, hk, hv, hdo)
        host_out = [torch.empty_like(t).pin_memory() for t in (hdo, hq, hk, hv)]
        h2d_stream, d2h_stream = torch.cuda.Stream(), torch.cuda.Stream()
        slots = [{"dev": [torch.empty(t.shape, dtype=t.dtype, device=dev) for t in host_in],
                  "free": torch.cuda.Event(), "ready": torch.cuda.Event()} for _ in range(2)]
        state = {"i": 0}

        def e2e_step():
            slot = slots[state["i"] % 2]
            state["i"] += 1
            cur = torch.cuda.current_stream()
            h2d_stream.wait_event(slot["free"])  # the compute that last read these buffers is done
            with torch.cuda.stream(h2d_stream):
                for d, h in zip(slot["dev"], host_in):
                    d.copy_(h, non_blocking=True)
                slot["ready"].record()
            cur.wait_event(slot["ready"])
            qd, kd, vd = (t.detach().requires_grad_() for t in slot["dev"][:3])
            res = step(qd, kd, vd, slot["dev"][3])
            slot["free"].record(cur)
            d2h_stream.wait_stream(cur)
            with torch.cuda.stream(d2h_stream):
                for h, r in zip(host_out, res):
                    h.copy_(r, non_blocking=True)
                    r.record_stream(d2h_stream)

        def e2e_finish():  # the last results must have reached the host before the closing event
            torch.cuda.current_stream().wait_stream(d2h_stream)

        for _ in range(3):
            e2e_step()
        ms_e2e, _ = self.timed(e2e_step, args.steps, 5, finish=e2e_finish)
        kernels.check_device_status(dev)
        rec["e2e"] = {"value": flops_total / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                      "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host_in),
                      "d2h_bytes_per_step": sum(t.numel() * t.element_size() for t in host_out),
                      "copies": "pinned host memory, own H2D and D2H streams, double-buffered device inputs: the "
                                "copies of neighbouring steps overlap the compute"}
        del slots, host_out

        rec["roofline"] = self.roofline(name, q.detach(), k.detach(), v.detach(), do, scale, S_loc, Hq, Hkv, Dqk, Dv)
        return rec

    def overlap(self, qd, kd, vd, do, scale, global_ranks):
        _ring = self.ring._ring
        rank, world, sharding = self.rank, self.world, self.args.sharding

        class NoComm:
            def exchange(self, send, recv):
                return None

            @staticmethod
            def wait(h):
                return None

        class NoCompute:
            def fwd_block(self, *a):
                pass

            def bwd_block(self, *a):
                pass

            def delta(self, o, d):
                return torch.empty((o.shape[0], o.shape[2], o.shape[1]), dtype=torch.float32, device=o.device)

            def cast(self, acc):
                return torch.empty(acc.shape, dtype=torch.bfloat16, device=acc.device)

            def add_into(self, a, b):
                pass

            def zero(self, a):
                pass

        be, nocompute = _ring.CudaBlockBackend(), NoCompute()
        comm, nocomm = _ring._make_comm(rank, world, global_ranks, self.dev), NoComm()

        def ring(b, c):
            o, l = _ring.ring_forward(b, c, qd, kd, vd, scale, rank, world, sharding)
            _ring.ring_backward(b, c, qd, kd, vd, o, l, do, scale, rank, world, sharding)

        for b_, c_ in ((be, comm), (be, nocomm), (nocompute, comm)):  # warm the allocator for each variant
            ring(b_, c_)
            ring(b_, c_)
        t_both, _ = self.timed(lambda: ring(be, comm), 5, 3)
        t_comp, _ = self.timed(lambda: ring(be, nocomm), 5, 3)
        t_comm, _ = self.timed(lambda: ring(nocompute, comm), 5, 3)
        return {"ms_both": t_both, "ms_compute_only": t_comp, "ms_comm_only": t_comm,
                "hidden_fraction": max(0.0, min(1.0, 1.0 - (t_both - t_comp) / t_comm)) if t_comm > 0 else None}

    def roofline(self, name, qd, kd, vd, do, scale, S_loc, Hq, Hkv, Dqk, Dv):
        kernels, dev, pk = self.kernels, self.dev, self.pk
        # ---- each attention kernel timed alone through the C ABI on the local causal block
        out_d, lse_d = kernels.attn_fwd(qd, kd, vd, scale, True, 0)
        delta_d = kernels.bwd_preprocess(out_d, do)
        dk_acc = torch.zeros(kd.shape, dtype=torch.float32, device=dev)
        dv_acc = torch.zeros(vd.shape, dtype=torch.float32, device=dev)
        dq_acc = torch.zeros(qd.shape, dtype=torch.float32, device=dev)
        runs = {
            "attn_fwd": (lambda: kernels.attn_fwd(qd, kd, vd, scale, True, 0, out=out_d, lse=lse_d), 1.0),
            "attn_bwd dK/dV pass": (lambda: kernels.attn_bwd(qd, kd, vd, do, lse_d, delta_d, scale, True, 0, None, dk_acc, dv_acc), 2.0),
            "attn_bwd dQ pass": (lambda: kernels.attn_bwd(qd, kd, vd, do, lse_d, delta_d, scale, True, 0, dq_acc, None, None), 0.5),
        }
        kern = {}
        fwd_fl_local = float(Hq) * S_loc * S_loc * (Dqk + Dv)  # causal forward FLOPs of the local block
        for kname, (run, mult) in runs.items():
            for _ in range(3):
                run()
            kms, _ = self.timed(run, 10, 3, queue_ahead=True)
            kern[kname] = {"ms": kms, "tflops": mult * fwd_fl_local / (kms * 1e-3) / 1e12}
        dom = max(kern, key=lambda n: kern[n]["ms"])
        traffic = None
        for (w, n, sub), val in NCU_TRAFFIC.items():
            if w == name and n == self.world and sub in dom:
                traffic = val
        roofline = {
            "bound": "tensor", "kernel": dom, "achieved": kern[dom]["tflops"], "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
            "frac": kern[dom]["tflops"] / pk["bf16_tflops"], "peak_source": pk["source"] + " burst (kernel timed alone)",
            "traffic": traffic[0] if traffic else None, "traffic_source": traffic[1] if traffic else None,
            "traffic_unit": "DRAM bytes per launch (ncu)", "kernels": kern,
            "note": "algorithmic FLOPs per launch: causal block B*H*S^2*(Dqk+Dv) x {fwd 1, dK/dV 2, dQ 0.5}; "
                    "the dQ launch recomputes S and dP (not counted)",
        }

        # ---- HBM-bound kernels of the path, timed alone: algorithmic bytes / time against the measured copy bandwidth
        n_row = S_loc * Hq
        acc_f32 = torch.randn(1, S_loc, Hq, Dv, device=dev)
        parts8 = [(torch.randn(1, S_loc, Hq, Dv, device=dev).bfloat16(), torch.randn(1, Hq, S_loc, device=dev), 0)
                  for _ in range(8)]  # eight distinct partial results, as the forward ring leaves them at CP = 8
        hbm_runs = {
            "combine_kernel (fp32 + bf16 -> fp32, log2)": (
                lambda: kernels.combine(acc_f32, lse_d, out_d, lse_d, natural=False), n_row * Dv * (4 + 2 + 4) + 12 * n_row),
            "combine_partials_kernel (8 x bf16 -> bf16, log2)": (
                lambda: kernels.combine_partials(parts8, 1, S_loc, Hq, Dv), 9 * n_row * (Dv * 2 + 4)),
            "delta_kernel": (lambda: kernels.bwd_preprocess(out_d, do, delta_d), n_row * Dv * 4 + 4 * n_row),
            "cast_kernel (dQ)": (lambda: kernels.cast_to_bf16(dq_acc), n_row * Dqk * 6),
        }
        if Dqk == 128:  # the fused q/k RMSNorm + rotary step in front of the operator (head_dim 128 models)
            w_n = torch.ones(Dqk, dtype=torch.bfloat16, device=dev)
            pos = torch.arange(S_loc, device=dev, dtype=torch.float32)
            inv = 1.0 / (1e6 ** (torch.arange(0, Dqk, 2, device=dev, dtype=torch.float32) / Dqk))
            emb = torch.outer(pos, inv).repeat(1, 2)[None]
            cos_t, sin_t = emb.cos().bfloat16(), emb.sin().bfloat16()
            rows_qk = S_loc * (Hq + Hkv) * Dqk
            hbm_runs["qk_norm_rope_kernel fwd (q, k bf16 -> bf16)"] = (
                lambda: kernels.qk_norm_rope_fwd(qd, kd, w_n, w_n, cos_t, sin_t, 1e-6), rows_qk * 4 + S_loc * Dqk * 4)
            hbm_runs["qk_norm_rope_kernel bwd"] = (
                lambda: kernels.qk_norm_rope_bwd(qd, kd, w_n, w_n, cos_t, sin_t, 1e-6, do if Dv == Dqk else qd, kd),
                rows_qk * 6 + S_loc * Dqk * 4)
        if Dqk == 192:  # the rotary + input assembly step in front of the MLA operator
            q_in = torch.randn(1, S_loc, Hq, 192, device=dev).bfloat16()
            kv_in = torch.randn(1, S_loc, Hq, 256, device=dev).bfloat16()
            kpe_in = torch.randn(1, S_loc, 64, device=dev).bfloat16()
            ang = torch.outer(torch.arange(S_loc, device=dev, dtype=torch.float32),
                              1.0 / (1e4 ** (torch.arange(0, 64, 2, device=dev, dtype=torch.float32) / 64))).repeat(1, 2)[None]
            cos_m, sin_m = ang.cos().bfloat16(), ang.sin().bfloat16()
            asm_bytes = S_loc * (Hq * (192 + 256 + 192 + 192 + 128) * 2 + 64 * 2 + 64 * 4)
            hbm_runs["mla_assemble_kernel fwd"] = (lambda: kernels.mla_assemble_fwd(q_in, kv_in, kpe_in, cos_m, sin_m),
                                                   asm_bytes)
            hbm_runs["mla_assemble_kernel bwd"] = (lambda: kernels.mla_assemble_bwd(cos_m, sin_m, qd, kd, vd), asm_bytes)
        hbm = {}
        for hname, (run, nbytes) in hbm_runs.items():
            for _ in range(3):
                run()
            kms, _ = self.timed(run, 10, 3, queue_ahead=True)
            hbm[hname] = {"us": kms * 1e3, "gbs": nbytes / (kms * 1e-3) / 1e9,
                          "frac_of_measured_hbm": nbytes / (kms * 1e-3) / 1e9 / pk["hbm_gbs"]}
        roofline["hbm_kernels"] = hbm
        return roofline

    def cpu_baseline(self, name):
        """The oracle on the host cores of this box, bounded sample (rank 0, N = 1)."""
        _, _, Hq, Hkv, Dqk, Dv, _ = WORKLOADS[name]
        threads = host_threads()
        group = Hq // Hkv
        heads, S_s = min(Hq, group), 2048
        cpu_attention_sample(512, heads, group, Dqk, Dv)
        reps, t_acc, fl = 0, 0.0, 0.0
        while t_acc < 10.0 and reps < 50:
            dt, f1 = cpu_attention_sample(S_s, heads, group, Dqk, Dv)
            t_acc += dt; fl += f1; reps += 1
        return {"value": fl / t_acc / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                "host_cpus": os.cpu_count(),
                "sample": f"{reps} x ({heads} query heads / 1 kv head, S={S_s}) causal fwd+bwd in fp32 with the oracle"}

    def run(self):
        args, rank, world = self.args, self.rank, self.world
        head = self.measure(args.workload, headline=True)
        extra = {}
        if world == 8 and not args.single_workload:  # configs 4 and 5 are quoted at CP = 8
            for name in ("mla", "long"):
                if name != args.workload:
                    extra[name] = self.measure(name, headline=False)
        anchor = None
        if world == 1 and not args.no_anchor and args.workload == "qwen3":
            # the N > 1 runs split S = 32768 over the ranks: the same problem on one GPU anchors strong scaling
            a = self.measure(args.workload, headline=False, S_override=WORKLOADS[args.workload][1])
            anchor = {k: a[k] for k in ("workload", "value", "unit", "ms_per_step", "frac_of_measured_bf16_peak",
                                         "tokens_per_s", "parity") if k in a}
        cpu = gpu_ref = None
        if rank == 0 and world == 1:
            if not args.no_cpu_baseline:
                cpu = self.cpu_baseline(args.workload)
            if not args.no_gpu_reference:
                torch.cuda.synchronize()
                gpu_ref = {"flash_attn": gpu_reference("flash", 180),
                           "reference_triton_mla": gpu_reference("triton_mla", args.triton_limit)}
        if rank == 0:
            pk = self.pk
            line = {
                "metric": METRIC, "value": head["value"], "unit": "TFLOP/s",
                "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": head["ms_per_step"],
                "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic",
                "config": {
                    "workload": head["workload"],
                    "sharding": args.sharding if world > 1 else "none",
                    "ring_cuda_graphs": self.use_graphs,
                    "ring_exchange": self.exchange_note or ("copy engines over peer-mapped memory" if self.use_peer
                                                            else "NCCL send/recv" if world > 1 else "none (CP=1)"),
                    "l2": "inputs + gradients per step exceed the 126 MB L2 (no flush needed)",
                    "flops_convention": "fwd B*H*S^2*(Dqk+Dv), bwd 2.5x fwd",
                    "timing": f"median of {BRACKETS} brackets of {args.steps} steps, each between barrier + synchronize; "
                              "max over ranks per bracket",
                },
                "peak_source": pk["source"],
            }
            for key in ("ms_per_step_brackets", "tflops_per_gpu", "frac_of_measured_bf16_peak",
                        "frac_of_measured_sustained_peak", "frac_of_nominal_2250",
                        "tokens_per_s", "e2e", "gpu_launches", "clocks", "roofline", "parity", "overlap", "nccl_exchange"):
                if key in head:
                    line[key] = head[key]
            line["cpu_baseline"] = cpu
            if gpu_ref is not None:
                line["gpu_reference"] = gpu_ref
            if extra:
                line["workloads"] = extra
            if anchor is not None:
                line["strong_scaling_anchor"] = anchor
            print(json.dumps(line), flush=True)
        if world > 1:
            self.ring.release_cuda_graphs()
            self.ring.release_peer_copies()
            self.dist.barrier()
            self.dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="qwen3")
    ap.add_argument("--sharding", choices=["zigzag", "contiguous"], default="zigzag")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gpu-reference", action="store_true",
                    help="skip timing flash-attn and the reference's Triton MLA kernels on this GPU (N = 1)")
    ap.add_argument("--triton-limit", type=int, default=420,
                    help="seconds the reference's Triton MLA kernels may take to autotune and run before they are "
                         "reported as unavailable")
    ap.add_argument("--no-anchor", action="store_true", help="skip the CP = 1 run at the N > 1 sequence length (N = 1)")
    ap.add_argument("--parity", action="store_true", help="run the slice parity check at N = 1 as well")
    ap.add_argument("--no-overlap", action="store_true", help="skip the comm/compute overlap measurement (N > 1)")
    ap.add_argument("--no-nccl-compare", action="store_true", help="skip re-timing the ring over NCCL send/recv (N > 1)")
    ap.add_argument("--single-workload", action="store_true", help="at N = 8, do not add the MLA and long-context rings")
    ap.add_argument("--graphs", action="store_true",
                    help="replay each ring from a CUDA graph instead of issuing every step from Python (N > 1)")
    ap.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                    help="how ring blocks travel at N > 1: copy engines over peer-mapped memory (one node), or NCCL "
                         "send/recv")
    ap.add_argument("--gpu-reference-child", choices=["flash", "triton_mla"], help=argparse.SUPPRESS)
    args = ap.parse_args()

    if args.gpu_reference_child:
        gpu_reference_child(args.gpu_reference_child)
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus:
        if args.gpus == 1 or world > 1:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
        raise SystemExit(f"--gpus {args.gpus} needs torchrun --nproc-per-node {args.gpus}")
    Bench(args, rank, world, local_rank).run()


if __name__ == "__main__":
    main()
