#!/usr/bin/env python
"""Benchmark of the context-parallel attention path: causal forward + backward, TFLOP/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload ...]

N = 1 runs the Qwen3-30B-A3B attention layer at S = 8192 on one GPU; N > 1 (launched with torchrun, one rank
per GPU) runs the same layer at global S = 32768 under zigzag context parallelism of degree N. One step is one
forward + backward of the public ring-attention operator on seeded synthetic bf16 inputs. FLOPs follow the
reference's convention (benchmarks/operators/mla/test_triton.py:7-14): causal forward = B*H*S^2*(Dqk+Dv),
backward = 2.5 x forward. Rank 0 prints one JSON line.

``--impl reference`` times the reference's CPU attention arithmetic (the oracle's restatement) on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
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


def fwd_bwd_flops(S, Hq, Dqk, Dv):
    return 3.5 * Hq * float(S) * S * (Dqk + Dv)


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        p = json.loads(f.read_text())
        return {"bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


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


def make_inputs(S_global, Hq, Hkv, Dqk, Dv, cp, rank, sharding, seed=42):
    """Seeded N(0,1) bf16 Q, K, V, dO at the global shape, sliced to this rank's shard (pinned host tensors)."""
    from pithtrain_b200.operators.ring_attention import sharding as sh
    g = torch.Generator().manual_seed(seed)
    out = []
    for shape in ((1, S_global, Hq, Dqk), (1, S_global, Hkv, Dqk), (1, S_global, Hkv, Dv), (1, S_global, Hq, Dv)):
        full = torch.randn(shape, generator=g, dtype=torch.float32).bfloat16()
        loc = sh.shard_sequence(full, cp, rank, sharding).contiguous() if cp > 1 else full
        out.append(loc.pin_memory() if torch.cuda.is_available() else loc)
        del full
    return out


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


def run_reference(args, rank):
    """Reference arm: CPU attention (oracle port of the reference's PyTorch math) on the host cores."""
    if rank != 0:
        return
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
        "impl": "reference", "metric": "causal fwd+bwd attention TFLOP/s (whole job)", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{desc}; S={S}; CPU sample: {sample}"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample, "host_cpus": os.cpu_count()},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="qwen3")
    ap.add_argument("--sharding", choices=["zigzag", "contiguous"], default="zigzag")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-overlap", action="store_true", help="skip the comm/compute overlap measurement (N > 1)")
    ap.add_argument("--graphs", action="store_true",
                    help="replay each ring from a CUDA graph instead of issuing every step from Python (N > 1)")
    ap.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                    help="how ring blocks travel at N > 1: copy engines over peer-mapped memory (one node), or NCCL "
                         "send/recv")
    args = ap.parse_args()

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

    import torch.distributed as dist
    from pithtrain_b200 import build, kernels
    from pithtrain_b200.operators.ring_attention import (RingAttentionFunc, RingMLAAttentionFunc, _ring,
                                                         enable_cuda_graphs, enable_peer_copies,
                                                         release_cuda_graphs, release_peer_copies)

    build.build_library()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    use_graphs = world > 1 and args.graphs
    enable_cuda_graphs(use_graphs)  # public switch of the operator: whole rings are captured once and replayed
    use_peer = world > 1 and args.exchange == "peer"
    enable_peer_copies(use_peer)    # public switch: exchanges run on the copy engines, not in NCCL kernels
    S1, SN, Hq, Hkv, Dqk, Dv, desc = WORKLOADS[args.workload]
    S = S1 if world == 1 else SN
    S_loc = S // world
    scale = Dqk ** -0.5
    fn = RingMLAAttentionFunc if Dqk == 192 else RingAttentionFunc
    global_ranks = list(range(world))
    hq, hk, hv, hdo = make_inputs(S, Hq, Hkv, Dqk, Dv, world, rank, args.sharding)
    q, k, v, do = (t.to(dev) for t in (hq, hk, hv, hdo))

    def step(q_, k_, v_, do_):
        q_.grad = k_.grad = v_.grad = None
        out = fn.apply(q_, k_, v_, scale, rank, world, global_ranks, args.sharding)
        out.backward(do_)
        return out, q_.grad, k_.grad, v_.grad

    for t in (q, k, v):
        t.requires_grad_()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(run, steps, in_flight=None, finish=None, queue_ahead=False):
        """Device time of `steps` calls of run(), max over ranks, in ms per call.

        queue_ahead (single kernels only): a spin kernel of a few ms runs first, so that the host has enqueued all
        launches before the first one starts and the events bracket GPU execution, not Python call overhead."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if queue_ahead:
            torch.cuda._sleep(int(6e6))
        e0.record()
        for _ in range(steps):
            run()
        if finish is not None:
            finish()
        e1.record()
        if in_flight is not None:
            in_flight()  # called while the last steps still run on the GPU
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # ---- the copy-engine exchange needs CUDA IPC between the ranks' processes; where the host forbids it, every rank
    # fails alike while mapping its neighbour's memory, and all of them fall back to the NCCL exchange together
    exchange_note = None
    if use_peer:
        ok = torch.ones(1, device=dev)
        try:
            step(q, k, v, do)
            torch.cuda.synchronize()
            kernels.check_device_status(dev)
        except Exception as e:  # noqa: BLE001 - reported in the JSON line
            ok.zero_()
            exchange_note = f"copy-engine exchange unavailable ({type(e).__name__}: {str(e)[:120]}); NCCL send/recv used"
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            use_peer = False
            enable_peer_copies(False)
            exchange_note = exchange_note or "copy-engine exchange unavailable on another rank; NCCL send/recv used"

    # ---- resident-input measurement (headline `value`)
    for _ in range(max(3, args.warmup)):
        step(q, k, v, do)
    kernels.check_device_status(dev)
    launches0 = kernels.launch_count
    with ClockSampler(local_rank) as clk:
        ms = timed(lambda: step(q, k, v, do), args.steps, clk.sample)
    launches = (kernels.launch_count - launches0) // args.steps
    kernels.check_device_status(dev)
    flops_total = fwd_bwd_flops(S, Hq, Dqk, Dv)
    tflops_total = flops_total / (ms * 1e-3) / 1e12
    pk = peaks()

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
    ms_e2e = timed(e2e_step, args.steps, finish=e2e_finish)
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo))
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    # ---- dominant kernel, timed alone through the C ABI: backward dK/dV (4 of the 5 backward GEMMs)
    out_d, lse_d = kernels.attn_fwd(q.detach(), k.detach(), v.detach(), scale, True, 0)
    delta_d = kernels.bwd_preprocess(out_d, do)
    dk_acc = torch.zeros(k.shape, dtype=torch.float32, device=dev)
    dv_acc = torch.zeros(v.shape, dtype=torch.float32, device=dev)
    dq_acc = torch.zeros(q.shape, dtype=torch.float32, device=dev)
    qd, kd, vd = q.detach(), k.detach(), v.detach()
    bwd_label = " (attn_bwd128_kernel at head_dim 128)" if Dqk == 128 else " (Dqk = 192 instantiation)"
    runs = {
        "attn_fwd_kernel": (lambda: kernels.attn_fwd(qd, kd, vd, scale, True, 0, out=out_d, lse=lse_d), 1.0),
        "attn_bwd_kernel<kDkDv>" + bwd_label: (lambda: kernels.attn_bwd(qd, kd, vd, do, lse_d, delta_d, scale, True, 0, None, dk_acc, dv_acc), 2.0),
        "attn_bwd_kernel<kDq>" + bwd_label: (lambda: kernels.attn_bwd(qd, kd, vd, do, lse_d, delta_d, scale, True, 0, dq_acc, None, None), 0.5),
    }
    kern = {}
    fwd_fl_local = float(Hq) * S_loc * S_loc * (Dqk + Dv)  # causal forward FLOPs of the local block
    for name, (run, mult) in runs.items():
        for _ in range(3):
            run()
        kms = timed(run, 10, queue_ahead=True)
        kern[name] = {"ms": kms, "tflops": mult * fwd_fl_local / (kms * 1e-3) / 1e12}
    dom = max(kern, key=lambda n: kern[n]["ms"])
    roofline = {
        "bound": "tensor", "kernel": dom, "achieved": kern[dom]["tflops"], "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
        "frac": kern[dom]["tflops"] / pk["bf16_tflops"], "peak_source": pk["source"] + " burst (kernel timed alone)",
        # DRAM read + write bytes of one dK/dV launch at this exact workload, from the ncu capture summarised in
        # profiles/attention_kernels_qwen3_s8192.md (only known for the N = 1 Qwen3 case)
        "traffic": 208.1e6 if (world == 1 and args.workload == "qwen3" and "kDkDv" in dom) else None,
        "traffic_unit": "DRAM bytes per launch (ncu)", "kernels": kern,
        "note": "algorithmic FLOPs per launch: causal block B*H*S^2*(Dqk+Dv) x {fwd 1, dK/dV 2, dQ 0.5}; "
                "the dQ launch recomputes S and dP (not counted)",
    }

    # ---- HBM-bound kernels of the path, timed alone: algorithmic bytes / time against the measured copy bandwidth
    n_row = S_loc * Hq
    acc_f32 = torch.randn(1, S_loc, Hq, Dv, device=dev)
    hbm_runs = {
        "combine_kernel (fp32 + bf16 -> fp32, log2)": (
            lambda: kernels.combine(acc_f32, lse_d, out_d, lse_d, natural=False), n_row * Dv * (4 + 2 + 4) + 12 * n_row),
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
    for name, (run, nbytes) in hbm_runs.items():
        for _ in range(3):
            run()
        kms = timed(run, 10, queue_ahead=True)
        hbm[name] = {"us": kms * 1e3, "gbs": nbytes / (kms * 1e-3) / 1e9, "frac_of_measured_hbm": nbytes / (kms * 1e-3) / 1e9 / pk["hbm_gbs"]}
    roofline["hbm_kernels"] = hbm

    # ---- comm / compute overlap of one ring (N > 1): compute alone, exchanges alone, both
    overlap = None
    if world > 1 and not args.no_overlap:
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

        be, nocompute = _ring.CudaBlockBackend(), NoCompute()
        comm, nocomm = _ring._make_comm(rank, world, global_ranks, dev), NoComm()

        def ring(b, c):
            o, l = _ring.ring_forward(b, c, qd, kd, vd, scale, rank, world, args.sharding)
            _ring.ring_backward(b, c, qd, kd, vd, o, l, do, scale, rank, world, args.sharding)

        for b_, c_ in ((be, comm), (be, nocomm), (nocompute, comm)):  # warm the allocator for each variant
            ring(b_, c_)
            ring(b_, c_)
        t_both = timed(lambda: ring(be, comm), 5)
        t_comp = timed(lambda: ring(be, nocomm), 5)
        t_comm = timed(lambda: ring(nocompute, comm), 5)
        overlap = {"ms_both": t_both, "ms_compute_only": t_comp, "ms_comm_only": t_comm,
                   "hidden_fraction": max(0.0, min(1.0, 1.0 - (t_both - t_comp) / t_comm)) if t_comm > 0 else None}

    # ---- CPU baseline (rank 0, N = 1): the oracle on the host cores, bounded sample
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        group = Hq // Hkv
        heads, S_s = min(Hq, group), 2048
        cpu_attention_sample(512, heads, group, Dqk, Dv)
        reps, t_acc, fl = 0, 0.0, 0.0
        while t_acc < 10.0 and reps < 50:
            dt, f1 = cpu_attention_sample(S_s, heads, group, Dqk, Dv)
            t_acc += dt; fl += f1; reps += 1
        cpu = {"value": fl / t_acc / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
               "host_cpus": os.cpu_count(),
               "sample": f"{reps} x ({heads} query heads / 1 kv head, S={S_s}) causal fwd+bwd in fp32 with the oracle"}

    if rank == 0:
        line = {
            "metric": "causal fwd+bwd attention TFLOP/s (whole job)", "value": tflops_total, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": f"{desc}; global S={S}, causal; " + (
                    f"zigzag context parallel CP={world} ({S_loc} tokens per GPU)" if world > 1 and args.sharding == "zigzag"
                    else f"{args.sharding} CP={world}" if world > 1 else "single GPU (CP=1)"),
                "sharding": args.sharding if world > 1 else "none",
                "ring_cuda_graphs": use_graphs,
                "ring_exchange": exchange_note or ("copy engines over peer-mapped memory" if use_peer
                                                   else "NCCL send/recv"),
                "l2": "inputs + gradients per step exceed the 126 MB L2 (no flush needed)",
                "flops_convention": "fwd B*H*S^2*(Dqk+Dv), bwd 2.5x fwd",
            },
            "tflops_per_gpu": tflops_total / world,
            "frac_of_measured_bf16_peak": tflops_total / world / pk["bf16_tflops"],
            "frac_of_nominal_2250": tflops_total / world / 2250.0,
            "peak_source": pk["source"],
            "tokens_per_s": S / (ms * 1e-3),
            "e2e": {"value": flops_total / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "copies": "pinned host memory, own H2D and D2H streams, double-buffered device inputs: the "
                              "copies of neighbouring steps overlap the compute"},
            "gpu_launches": launches,
            "clocks": clk.summary(),
            "roofline": roofline,
            "cpu_baseline": cpu,
        }
        if overlap is not None:
            line["overlap"] = overlap
        print(json.dumps(line), flush=True)
    if world > 1:
        release_cuda_graphs()
        release_peer_copies()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
