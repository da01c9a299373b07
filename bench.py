#!/usr/bin/env python
"""Benchmark of the quantized-weight matmul hot path on B200.

Metric: Q4_K grouped-MMQ forward + input-gradient throughput in logical TFLOP/s
(2 * routed_rows * N * K per direction, the reference's own definition:
bench/grouped_mmq_benchmark_common.py:228-239), on the MoE expert-projection configuration:
256 experts of Q4_K 512 x 2048, 8192 tokens per GPU, top-8 routing from Gaussian logits
(65536 routed rows per GPU).  Inputs are seeded synthetic tensors of that shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one forward pass plus one input-gradient pass over the routed rows.

* N = 1: the grouped operators on one GPU.  ``value`` is timed with the expert-sorted rows
  resident in HBM (C-ABI calls, CUDA events per launch).
* N > 1 (under torchrun): expert-parallel.  Each rank owns 256/N experts and 8192 tokens; a token's
  row goes once to every GPU that owns one of its experts and results come back, moved by this
  library's peer-memory kernels over NVLink; the forward matmul's epilogue stores its rows
  straight into the token owner's memory; counts and phase barriers go over peer memory too
  (NCCL only for the host-side setup and the scalar reductions around the timed region, or with
  ``--fences nccl``).  Weak scaling: per-GPU tokens are fixed.  ``ep_phases_ms`` is the CUDA-event
  time of every phase of one extra, untimed step.
* every N: ``e2e`` is the expert-parallel step (tokens + top-k ids in, per-pair forward rows and
  per-token gradients out; routing sort, dispatch and combine inside) with pinned host buffers
  copied in and results copied out inside the timed region; ``parity`` compares sampled tokens of
  every rank with the CPU oracle after the timed region; ``config5`` times and checks the
  expert-parallel MoE feed-forward configuration (IQ2_S gate/up + Q6_K down, 65536 tokens split
  over the GPUs).
* ``--impl reference``: the reference semantics on the host CPU (dequantise the GGUF blocks, fp32
  ``torch.matmul`` per group) on a bounded sample of the same workload.  The reference's own
  kernels are ROCm-only and cannot run here.

Prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

Q4_K = 12
BLOCK_BYTES = {11: 110, 12: 144, 13: 176, 14: 210, 22: 82}
FP16_FIELDS = {12: (0, 2), 13: (0, 2), 14: (208,), 11: (108,), 22: (0,)}

WORKLOAD = {
    "name": "grouped Q4_K 256 experts x (512 x 2048), 8192 tokens/GPU, top-8 Gaussian-logit routing, fwd + dX",
    "quant": "Q4_K", "qt": Q4_K, "experts": 256, "N": 512, "K": 2048, "tokens": 8192, "top_k": 8, "sigma": 2.0,
}


# ------------------------------------------------------------------------------ synthetic inputs
def synthetic_expert_weights(qt, experts, n, k, seed, lo=0, hi=None):
    """uint8 [hi-lo, n, row_bytes] of random valid super-blocks (uniform payload bytes, fp16
    super-scales |N(0,1)| * 2e-3); expert e is drawn from its own stream so shards agree."""
    hi = experts if hi is None else hi
    bb = BLOCK_BYTES[qt]
    nb = n * (k // 256)
    out = np.empty((hi - lo, nb, bb), dtype=np.uint8)
    for e in range(lo, hi):
        rng = np.random.Generator(np.random.PCG64([seed, e]))
        blk = rng.integers(0, 256, size=(nb, bb), dtype=np.uint8)
        for off in FP16_FIELDS[qt]:
            d = (np.abs(rng.standard_normal(nb)) * 2e-3).astype(np.float16)
            blk[:, off:off + 2] = d.view(np.uint8).reshape(nb, 2)
        out[e - lo] = blk
    return out.reshape(hi - lo, n, (k // 256) * bb)


def synthetic_routing(tokens, experts, top_k, sigma, seed):
    """Top-k of Gaussian logits (+ a fixed per-expert popularity bias, so counts are skewed)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    logits = rng.standard_normal((tokens, experts), dtype=np.float32) * np.float32(sigma)
    bias = np.random.Generator(np.random.PCG64(12345)).standard_normal(experts, dtype=np.float32)
    logits += bias * np.float32(sigma * 0.25)
    return np.argsort(-logits, axis=1, kind="stable")[:, :top_k].astype(np.int64)


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        for line in open(self.path).read().splitlines():
            f = [c.strip() for c in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def keep_busy_for(seconds, fn):
    """Repeat fn for about `seconds` so the clock sampler sees the GPU under this load.  The number
    of repetitions is agreed between the ranks first: fn may contain collectives, and ranks that
    each watched their own clock would leave the loop after different counts and deadlock."""
    import torch.distributed as dist

    fn()
    torch.cuda.synchronize()
    t0 = time.time()
    fn()
    torch.cuda.synchronize()
    n = torch.tensor([max(1, min(20000, int(seconds / max(time.time() - t0, 1e-5))))], device="cuda", dtype=torch.int64)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(n, op=dist.ReduceOp.MAX)
    for _ in range(int(n.item())):
        fn()
    torch.cuda.synchronize()


# ------------------------------------------------------------------------------ CPU arm
def cpu_reference_arm(wl, steps, warmup, sample_experts=32, seed=2024):
    """The reference semantics on the host: dequantise + fp32 matmul per group, forward and input
    gradient, over the groups of the first `sample_experts` experts of the workload."""
    from oracle import ref  # CPU oracle: the checker / baseline, never the product path

    qt, E, N, K = wl["qt"], wl["experts"], wl["N"], wl["K"]
    ids = synthetic_routing(wl["tokens"], E, wl["top_k"], wl["sigma"], seed)
    counts = np.bincount(ids.reshape(-1), minlength=E)[:sample_experts]
    w = synthetic_expert_weights(qt, E, N, K, seed, 0, sample_experts)
    g = torch.Generator().manual_seed(seed)
    rows = int(counts.sum())
    x = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    dy = torch.randn(rows, N, generator=g).to(torch.bfloat16)
    threads = ref.cpu_threads()
    torch.set_num_threads(threads)
    ends = np.cumsum(counts)

    def step():
        W = torch.from_numpy(ref.dequantize(w, qt, threads).reshape(sample_experts, N, K))
        xf, dyf = x.float(), dy.float()
        y = torch.empty(rows, N)
        dx = torch.empty(rows, K)
        b = 0
        for e in range(sample_experts):
            end = int(ends[e])
            if end > b:
                torch.matmul(xf[b:end], W[e].t(), out=y[b:end])
                torch.matmul(dyf[b:end], W[e], out=dx[b:end])
            b = end
        return y, dx

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    flops = 2 * 2.0 * rows * N * K
    return {"value": flops / dt / 1e12, "ms_per_step": dt * 1e3, "cores": threads,
            "sample": f"groups of experts 0..{sample_experts - 1} of {E} ({rows} of {wl['tokens'] * wl['top_k']} routed rows), "
                      f"dequantise + fp32 matmul fwd + dX, {steps} timed passes"}


# ------------------------------------------------------------------------------ helpers of the GPU arm
def bind_to_gpu_numa_node(gpu_index: int):
    """Best effort: run this process (and so place its pinned host buffers) on the CPUs of the NUMA
    node the GPU hangs off.  Returns the node, or None when the topology cannot be read."""
    try:
        bus = subprocess.run(["nvidia-smi", f"--id={gpu_index}", "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20).stdout.strip().lower()
        if not bus:
            return None
        bus = bus[-12:] if len(bus) > 12 else bus          # 00000000:1b:00.0 -> 0000:1b:00.0
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
        return node
    except Exception:
        return None


def routing_weights(tokens, top_k, seed):
    """Seeded positive routing weights that sum to one per token (stand-in for the router's softmax)."""
    g = torch.Generator().manual_seed(seed)
    w = torch.rand(tokens, top_k, generator=g) + 0.25
    return w / w.sum(1, keepdim=True)


def oracle_expert(qt, experts, n, k, seed, e):
    """fp32 [n, k] weight of expert e of the synthetic stack (CPU oracle: the checker only)."""
    from oracle import ref

    raw = synthetic_expert_weights(qt, experts, n, k, seed, e, e + 1)
    return torch.from_numpy(ref.dequantize(raw, qt).reshape(n, k))


def rel_err(got, want):
    return float(torch.linalg.vector_norm(got.double() - want.double()) / torch.linalg.vector_norm(want.double()))


def projection_parity(wl, seed, ids_cpu, x_tok, dy_rows, y_rows, dx_tok, n_check):
    """Forward rows and token gradients of `n_check` sampled tokens of this rank against the fp32
    oracle (dequantise + matmul) on the experts those tokens hit."""
    qt, E, N, K, top_k = wl["qt"], wl["experts"], wl["N"], wl["K"], wl["top_k"]
    T = ids_cpu.shape[0]
    pick = np.random.Generator(np.random.PCG64(99)).choice(T, size=min(n_check, T), replace=False)
    cache = {}
    got_y, want_y, got_dx, want_dx = [], [], [], []
    for t in pick:
        xt = x_tok[t].float().cpu()
        acc = torch.zeros(K)
        for s in range(top_k):
            e = int(ids_cpu[t, s])
            if e not in cache:
                cache[e] = oracle_expert(qt, E, N, K, seed, e)
            W = cache[e]
            want_y.append(W @ xt)
            got_y.append(y_rows[t * top_k + s].float().cpu())
            acc += dy_rows[t * top_k + s].float().cpu() @ W
        want_dx.append(acc)
        got_dx.append(dx_tok[t].float().cpu())
    return {"fwd_rel_err": rel_err(torch.stack(got_y), torch.stack(want_y)),
            "dx_rel_err": rel_err(torch.stack(got_dx), torch.stack(want_dx)), "tokens_checked": int(len(pick)),
            "experts_dequantised": len(cache)}


def mlp_parity(c5, seed, ids_cpu, gate_w, x_tok, dy_tok, y_tok, dx_tok, n_check):
    """The MoE feed-forward step of `n_check` sampled tokens against the fp32 oracle chain."""
    E, H, F, top_k = c5["experts"], c5["hidden"], c5["ffn"], c5["top_k"]
    T = ids_cpu.shape[0]
    pick = np.random.Generator(np.random.PCG64(77)).choice(T, size=min(n_check, T), replace=False)
    silu = lambda v: v * torch.sigmoid(v)  # noqa: E731
    cache = {}
    want_y, want_dx = [], []
    for t in pick:
        xt, dyt = x_tok[t].float().cpu(), dy_tok[t].float().cpu()
        y, dx = torch.zeros(H), torch.zeros(H)
        for s in range(top_k):
            e = int(ids_cpu[t, s])
            if e not in cache:
                cache[e] = (oracle_expert(c5["qt_gate_up"], E, F, H, seed + 1, e), oracle_expert(c5["qt_gate_up"], E, F, H, seed + 2, e),
                            oracle_expert(c5["qt_down"], E, H, F, seed + 3, e))
            Wg, Wu, Wd = cache[e]
            w = float(gate_w[t, s])
            g, u = Wg @ xt, Wu @ xt
            y += w * (Wd @ (silu(g) * u))
            dh = w * (dyt @ Wd)
            sg = torch.sigmoid(g)
            dx += (dh * u * (sg * (1 + g * (1 - sg)))) @ Wg + (dh * silu(g)) @ Wu
        want_y.append(y)
        want_dx.append(dx)
    idx = torch.from_numpy(pick.astype(np.int64))
    return {"fwd_rel_err": rel_err(y_tok.float().cpu()[idx], torch.stack(want_y)),
            "dx_rel_err": rel_err(dx_tok.float().cpu()[idx], torch.stack(want_dx)), "tokens_checked": int(len(pick)),
            "experts_dequantised": len(cache)}


# ------------------------------------------------------------------------------ GPU arm
def gpu_arm(args):
    import torch.distributed as dist

    import torch_ggml_ops_b200 as tgo
    from torch_ggml_ops_b200 import native
    from torch_ggml_ops_b200.expert_parallel import ExpertParallel
    from torch_ggml_ops_b200.moe_parallel import PeerMoEMLP
    from torch_ggml_ops_b200.peer_parallel import PeerExpertParallel

    wl = WORKLOAD
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    numa = bind_to_gpu_numa_node(local_rank)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL serves the host-side setup and the few scalar reductions around the timed region only;
        # without NVLS it binds no NVLink multicast object to the buffers (a rank that dies while one
        # is bound can fault its peers)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    qt, E, N, K, T, top_k = wl["qt"], wl["experts"], wl["N"], wl["K"], wl["tokens"], wl["top_k"]
    seed = 2024
    EL = E // world
    w = torch.from_numpy(synthetic_expert_weights(qt, E, N, K, seed, rank * EL, (rank + 1) * EL)).to(dev)
    ids_cpu = synthetic_routing(T, E, top_k, wl["sigma"], seed + rank)
    ids = torch.from_numpy(ids_cpu).to(dev)
    ids32 = ids.to(torch.int32)
    g = torch.Generator(device=dev).manual_seed(seed + rank)
    x_tok = torch.randn(T, K, generator=g, device=dev).to(torch.bfloat16)
    dy_rows = torch.randn(T * top_k, N, generator=g, device=dev).to(torch.bfloat16)  # per routed row, token-major
    R = T * top_k
    flops_step = 2 * 2.0 * R * N * K * world  # forward + dX, all ranks

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_steps(fn, steps):
        """`steps` calls of fn between barriers, CUDA events on the current stream, max over ranks (ms per call)."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / steps)

    # ---------------------------------------------------------------- the expert-parallel step (every N)
    # tokens + top-k expert ids in, per-pair forward rows and per-token input gradients out: device
    # routing sort, dispatch to the owning GPU, grouped matmuls, return.  Receive buffers hold twice
    # the mean load when experts are spread over several GPUs (the routing is skewed).
    cap = R if world == 1 else 2 * R
    pep = PeerExpertParallel(w, qt, E, N, K, capacity_rows=cap, tokens_per_rank=T if args.token_level else None, top_k=top_k,
                             fences=args.fences)
    y_out = [torch.empty(R, N, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    dx_out = [torch.empty(T, K, dtype=torch.bfloat16, device=dev) for _ in range(2)]

    def step_ep(x=x_tok, dy=dy_rows, b=0, keep=False):
        """One step.  The forward rows arrive in this rank's peer-addressable result buffer (the
        matmul epilogues of the experts' GPUs store them there); ``keep`` copies them to a private
        buffer, for a reader that overlaps the next step (the end-to-end loop's copy-out stream)."""
        plan = pep.plan(ids32)
        # the barrier after the forward is the one inside grad_input (the rows are complete after it)
        y = pep.forward(plan, x, out=y_out[b] if keep else None, fence=False)
        pep.grad_input(plan, dy, out=dx_out[b])
        return y, dx_out[b]

    result = {}
    if not args.profile:
        for _ in range(max(args.warmup, 3)):
            step_ep()
    barrier()
    if world == 1:
        # ---------------------------------------------------------------- kernel-resident timing
        ep = ExpertParallel(E)
        plan1 = ep.plan(ids)
        x_rows = ep.dispatch_tokens(plan1, x_tok)              # [R, K] expert-major (local gather only)
        dy_sorted = ep.dispatch_rows(plan1, dy_rows)
        ei, eo = plan1.expert_indices, plan1.expert_offsets
        y = torch.empty(R, N, dtype=torch.bfloat16, device=dev)
        dx = torch.empty(R, K, dtype=torch.bfloat16, device=dev)
        ws = torch.empty(native.grouped_workspace_bytes(R, EL), dtype=torch.uint8, device=dev)

        def step_resident():
            native.grouped_fwd(x_rows, w, None, y, None, ei, eo, EL, R, N, K, qt, ws)
            native.grouped_dx(dy_sorted, None, w, None, dx, ei, eo, EL, R, N, K, qt, ws)

        for _ in range(args.warmup if args.profile else max(args.warmup, 3)):
            step_resident()
        barrier()
        if args.profile:
            # minimal launch sequence for a profiler: no clock sampling, no end-to-end leg
            for _ in range(args.steps):
                step_resident()
            barrier()
            print(json.dumps({"profile": True, "steps": args.steps, "device_status": native.device_status()}))
            return
        sampler = ClockSampler(local_rank)
        sampler.start()
        keep_busy_for(1.0, step_resident)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps + 1)]
        barrier()
        ev[0].record()
        for i in range(args.steps):
            native.grouped_fwd(x_rows, w, None, y, None, ei, eo, EL, R, N, K, qt, ws)
            ev[2 * i + 1].record()
            native.grouped_dx(dy_sorted, None, w, None, dx, ei, eo, EL, R, N, K, qt, ws)
            ev[2 * i + 2].record()
        barrier()
        clocks = sampler.stop()
        total_ms = ev[0].elapsed_time(ev[2 * args.steps])
        fwd_ms = float(np.mean([ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(args.steps)]))
        bwd_ms = float(np.mean([ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) for i in range(args.steps)]))
        ms_step = total_ms / args.steps
        result["ep_step_ms"] = timed_steps(step_ep, args.steps)   # the same work through routing + dispatch + combine
        launches = 4  # tile builder + GEMM, forward and backward
        peaks = json.load(open(ROOT / "MEASURED_PEAKS.json")) if (ROOT / "MEASURED_PEAKS.json").exists() else None
        # The launches are timed back to back inside a power-capped loop (a second of the same load
        # runs first), so the sustained cuBLAS figure is the denominator; the burst one is given too.
        peak_tf = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) if peaks else 1400.0
        burst_tf = peaks["bf16_tflops"] if peaks else 1590.0
        peak_hbm = peaks["hbm_gbs"] if peaks else 6650.0
        flops_dir = 2.0 * R * N * K
        bytes_dir = R * K * 2 + R * N * 2 + w.numel()  # activations once, packed experts once, outputs once
        roof = lambda ms: {  # noqa: E731
            "bound": "tensor", "achieved": flops_dir / (ms * 1e-3) / 1e12, "peak": peak_tf, "unit": "TFLOP/s",
            "frac": flops_dir / (ms * 1e-3) / 1e12 / peak_tf,
            "peak_source": "measured, sustained bf16 cuBLAS (MEASURED_PEAKS.json)" if peaks else "fallback",
            "frac_of_burst_peak": flops_dir / (ms * 1e-3) / 1e12 / burst_tf, "burst_peak": burst_tf,
            "hbm_gbs": bytes_dir / (ms * 1e-3) / 1e9, "hbm_frac": bytes_dir / (ms * 1e-3) / 1e9 / peak_hbm,
            "ms_per_launch": ms}
        result["roofline"] = dict(roof(fwd_ms), kernel="mmq_gemm_kernel<Q4_K, forward> (+ tile builder)",
                                  traffic=MEASURED_DRAM_TRAFFIC.get("fwd"), traffic_source=MEASURED_DRAM_TRAFFIC["source"])
        result["roofline_dx"] = dict(roof(bwd_ms), kernel="mmq_gemm_kernel<Q4_K, input gradient> (+ tile builder)",
                                     traffic=MEASURED_DRAM_TRAFFIC.get("bwd"), traffic_source=MEASURED_DRAM_TRAFFIC["source"])
        executor = "one GPU: grouped operators on expert-sorted rows resident in HBM"
    else:
        sampler = ClockSampler(local_rank)
        sampler.start()
        keep_busy_for(1.0, step_ep)
        ms_step = timed_steps(step_ep, args.steps)
        clocks = sampler.stop()
        # this library's kernels per step: GEMMs + tile builders (4), routing sort (3), plan (2, + 1 for the
        # token maps, zeroing of dropped rows), exchange (pair level 4; token level 6: dispatch, expand, row
        # pointers, dispatch dy, reduce, pull - the forward rows are returned by the matmul's own epilogue)
        launches = 4 + 3 + (4 + 6 if args.token_level else 2 + 4) + (5 if args.fences == "peer" else 0)   # + count exchange, 4 barriers
        executor = (f"{world} GPUs: experts sharded; dispatch/combine by peer-memory kernels over NVLink, forward rows "
                    "stored into the token owner's memory by the matmul epilogue (NCCL only for the host-side setup; "
                    "counts and phase barriers by peer memory too unless --fences nccl)")
    result["device_status"] = native.device_status()
    result["ep_overflow"] = int(pep.overflow.item())

    # ---------------------------------------------------------------- parity on this rank's own results (not timed)
    yb, dxb = step_ep()
    torch.cuda.synchronize()
    par = projection_parity(wl, seed, ids_cpu, x_tok, dy_rows, yb, dxb, args.parity_tokens)
    par["fwd_rel_err"], par["dx_rel_err"] = max_over_ranks(par["fwd_rel_err"]), max_over_ranks(par["dx_rel_err"])
    par["tolerance"] = {"fwd": 1e-2, "dx": 5e-3}
    par["ranks_checked"] = world
    result["parity"] = par
    if pep.push:
        # one more step, not timed, with a CUDA event after every phase (max over ranks, ms)
        ph = pep.phase_times(step_ep)
        result["ep_phases_ms"] = {k: round(max_over_ranks(v), 4) for k, v in ph.items()}

    # ---------------------------------------------------------------- end to end with host buffers (every N)
    # Tokens and per-pair cotangents come from pinned host memory, per-pair forward rows and
    # per-token gradients go back to it, every step.  Three streams and two sets of device buffers:
    # the copy-in of step i+1 and the copy-out of step i-1 overlap the work of step i.
    xh, dyh = x_tok.cpu().pin_memory(), dy_rows.cpu().pin_memory()
    yh = torch.empty(R, N, dtype=torch.bfloat16).pin_memory()
    dxh = torch.empty(T, K, dtype=torch.bfloat16).pin_memory()
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    xd = [torch.empty_like(x_tok) for _ in range(2)]
    dyd = [torch.empty_like(dy_rows) for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def step_e2e(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_cmp[b])          # the step that last read these input buffers is done
            xd[b].copy_(xh, non_blocking=True)
            dyd[b].copy_(dyh, non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_cmp):
            s_cmp.wait_event(ev_in[b])
            s_cmp.wait_event(ev_out[b])         # the copy-out that last read these output buffers is done
            step_ep(xd[b], dyd[b], b, keep=True)
            ev_cmp[b].record(s_cmp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_cmp[b])
            yh.copy_(y_out[b], non_blocking=True)
            dxh.copy_(dx_out[b], non_blocking=True)
            ev_out[b].record(s_out)

    def run_e2e(n):
        for st in (s_in, s_cmp, s_out):
            st.wait_stream(torch.cuda.current_stream())
        for i in range(n):
            step_e2e(i)
        for st in (s_in, s_cmp, s_out):
            torch.cuda.current_stream().wait_stream(st)

    run_e2e(3)
    e2e_ms = timed_steps(lambda: run_e2e(args.steps), 1) / args.steps
    h2d = xh.numel() * 2 + dyh.numel() * 2
    d2h = yh.numel() * 2 + dxh.numel() * 2
    e2e = {"value": flops_step / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "numa_node": numa,
           "form": "tokens + top-k ids + per-pair cotangents in, per-pair forward rows + per-token gradients out; "
                   "routing sort, dispatch and combine inside the timed region"}

    # ---------------------------------------------------------------- the expert-parallel MoE feed-forward configuration
    if not args.no_config5:
        result["config5"] = config5_step(args, world, rank, dev, seed, PeerMoEMLP, native, barrier, max_over_ranks, timed_steps)

    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        cpu = cpu_reference_arm(wl, steps=1, warmup=1)
        result["cpu_baseline"] = {"value": cpu["value"], "unit": "TFLOP/s", "cores": cpu["cores"], "kind": "port",
                                  "sample": cpu["sample"]}

    if rank == 0:
        value = flops_step / (ms_step * 1e-3) / 1e12
        line = {
            "metric": "Q4_K grouped-MMQ fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": bench_config(wl, world), "executor": executor,
            "tokens_per_s": T * world / (ms_step * 1e-3),
            "e2e": e2e, "gpu_launches": launches * args.steps, "clocks": clocks,
        }
        line.update(result)
        print(json.dumps(line))
    failed = par["fwd_rel_err"] > 1e-2 or par["dx_rel_err"] > 5e-3
    if world > 1:
        dist.destroy_process_group()
    if failed:
        raise SystemExit(f"parity check failed: {par}")


def bench_config(wl, n_gpus):
    """The `config` object: the workload, identical in both arms."""
    return {"workload": wl["name"], "quant": wl["quant"], "experts": wl["experts"], "out_features": wl["N"],
            "in_features": wl["K"], "tokens_per_gpu": wl["tokens"], "top_k": wl["top_k"],
            "routed_rows_per_gpu": wl["tokens"] * wl["top_k"],
            "parallelism": "single GPU" if n_gpus == 1 else f"ep{n_gpus}: experts sharded evenly, tokens data-parallel",
            "l2": "inputs larger than L2 (activations 268 MB + weights 151 MB per pass vs 126 MB L2)"}


CONFIG5 = {"name": "expert-parallel MoE feed-forward: 256 experts, IQ2_S gate/up 512 x 2048 + Q6_K down 2048 x 512, "
                   "65536 tokens over all GPUs, top-8 Gaussian-logit routing, fwd + dX",
           "experts": 256, "hidden": 2048, "ffn": 512, "tokens_total": 65536, "top_k": 8, "qt_gate_up": 22, "qt_down": 14}


def config5_step(args, world, rank, dev, seed, PeerMoEMLP, native, barrier, max_over_ranks, timed_steps):
    """BASELINE configuration 5: the whole MoE feed-forward step (gate/up pair, silu * up, down,
    weighted combine; forward + input gradient) with the experts sharded over the GPUs and the
    65536 tokens split evenly between them (strong scaling).  Returns its timing and parity."""
    c5 = CONFIG5
    E, H, F, top_k = c5["experts"], c5["hidden"], c5["ffn"], c5["top_k"]
    T = c5["tokens_total"] // world
    EL = E // world
    lo, hi = rank * EL, (rank + 1) * EL
    wg = torch.from_numpy(synthetic_expert_weights(c5["qt_gate_up"], E, F, H, seed + 1, lo, hi)).to(dev)
    wu = torch.from_numpy(synthetic_expert_weights(c5["qt_gate_up"], E, F, H, seed + 2, lo, hi)).to(dev)
    wd = torch.from_numpy(synthetic_expert_weights(c5["qt_down"], E, H, F, seed + 3, lo, hi)).to(dev)
    ids_cpu = synthetic_routing(T, E, top_k, 2.0, seed + 100 + rank)
    ids32 = torch.from_numpy(ids_cpu).to(dev).to(torch.int32)
    gate_w = routing_weights(T, top_k, seed + 200 + rank)
    gate_wd = gate_w.to(dev)
    g = torch.Generator(device=dev).manual_seed(seed + 300 + rank)
    x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    dy = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    rows = T * top_k
    cap = rows if world == 1 else rows + rows // 2
    mlp = PeerMoEMLP(wg, wu, wd, c5["qt_gate_up"], c5["qt_down"], E, H, F, capacity_rows=cap, tokens_per_rank=T, top_k=top_k,
                     fences=args.fences)
    y = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    dx = torch.empty(T, H, dtype=torch.bfloat16, device=dev)

    def step():
        mlp.plan(ids32, gate_wd)
        mlp.forward(x, out=y)
        mlp.grad_input(dy, out=dx)

    for _ in range(3):
        step()
    steps = max(3, min(args.steps, 10))
    ms = timed_steps(step, steps)
    torch.cuda.synchronize()
    par = mlp_parity(c5, seed, ids_cpu, gate_w, x, dy, y, dx, args.parity_tokens_mlp)
    par["fwd_rel_err"], par["dx_rel_err"] = max_over_ranks(par["fwd_rel_err"]), max_over_ranks(par["dx_rel_err"])
    par["tolerance"] = {"fwd": 1e-2, "dx": 1e-2, "note": "chain of three matmuls with bf16 results between them"}
    overflow = int(mlp.r.plan["overflow"].item())
    flops = 2 * 6.0 * F * H * c5["tokens_total"] * top_k     # gate + up + down, forward + input gradient
    out = {"workload": c5["name"], "tokens_per_gpu": T, "steps": steps, "ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12,
           "tokens_per_s": c5["tokens_total"] / (ms * 1e-3), "scaling": "strong", "parity": par, "ep_overflow": overflow,
           "device_status": native.device_status()}
    del mlp
    if par["fwd_rel_err"] > 1e-2 or par["dx_rel_err"] > 1e-2:
        raise SystemExit(f"MoE feed-forward parity check failed: {par}")
    return out


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the GEMM kernel on this
# workload, from the ncu capture summarised in the file named here; not measured by this run.
MEASURED_DRAM_TRAFFIC = {"fwd": 475.9e6, "bwd": 442.1e6, "source": "profiles/mmq_gemm_q4k_grouped_ncu_full.txt"}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = WORKLOAD
    steps, warmup = max(1, args.steps), max(1, min(args.warmup, 3))
    cpu = cpu_reference_arm(wl, steps=steps, warmup=warmup)
    line = {
        "impl": "reference", "metric": "Q4_K grouped-MMQ fwd+bwd TFLOP/s", "value": cpu["value"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": cpu["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(wl, args.gpus), "executor": "host CPU, all cores (rank 0 only)",
        "cpu_baseline": {"value": cpu["value"], "unit": "TFLOP/s", "cores": cpu["cores"], "kind": "port",
                         "sample": cpu["sample"]},
        "e2e": {"value": cpu["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's kernels are ROCm/HIP-only; this arm times its dequantise + matmul semantics "
                "(CPU restatement, checked against gguf-py) on the host cores",
    }
    print(json.dumps(line))


def sweep_arm(args):
    """Kernel-level TFLOP/s of the other benchmark configurations (dense config 1 and 2 for all
    five quant types, grouped config 3, pair + down projection of config 4), device-resident,
    CUDA events, one JSON line per case.  Not the contract line: a table for the design notes."""
    from torch_ggml_ops_b200 import native

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        tot = 0.0
        for _ in range(n):
            flush.zero_()   # evict the operands from L2 between repeats
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            tot += a.elapsed_time(b)
        return tot / n

    def report(name, flops, f_ms, b_ms):
        print(json.dumps({"case": name, "fwd_ms": round(f_ms, 4), "fwd_tflops": round(flops / f_ms / 1e9, 1),
                          "dx_ms": round(b_ms, 4), "dx_tflops": round(flops / b_ms / 1e9, 1)}), flush=True)

    def bf16(rows, cols, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        return torch.randn(rows, cols, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)

    names = {11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 22: "IQ2_S"}
    dense = [(12, 512, 2048, 2048)] + [(qt, 4096, n, k) for qt in (22, 11, 12, 13, 14) for (n, k) in ((4096, 2048), (2048, 4096))]
    for qt, M, N, K in dense:
        w = torch.from_numpy(synthetic_expert_weights(qt, 1, N, K, 11)).to(dev)[0]
        x, dy = bf16(M, K, 1), bf16(M, N, 2)
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        dx = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
        f = timed(lambda: native.mmq_fwd(x, w, y, M, N, K, qt), args.steps)
        b = timed(lambda: native.mmq_dx(dy, w, dx, M, N, K, qt), args.steps)
        report(f"dense {names[qt]} M={M} N={N} K={K}", 2.0 * M * N * K, f, b)

    # the LM-head shape of the reference's chunked loss loop (docs/mmq_bwd_optimization.md:442-446, 502-524)
    V, Kh = 248320, 2048
    wh = torch.from_numpy(synthetic_expert_weights(14, 1, V, Kh, 12)).to(dev)[0]
    for M in (64, 128, 256):
        x, dy = bf16(M, Kh, 1), bf16(M, V, 2)
        y = torch.empty(M, V, dtype=torch.bfloat16, device=dev)
        dx = torch.empty(M, Kh, dtype=torch.bfloat16, device=dev)
        f = timed(lambda: native.mmq_fwd(x, wh, y, M, V, Kh, 14), args.steps)
        b = timed(lambda: native.mmq_dx_split(dy, wh, dx, M, V, Kh, 14), args.steps)
        report(f"LM head Q6_K M={M} N={V} K={Kh} (weight 417 MB read per call; dX with the split reduction)", 2.0 * M * V * Kh, f, b)
    del wh

    def grouped(qt, E, N, K, tokens, top_k, pair, label):
        ids = synthetic_routing(tokens, E, top_k, 2.0, 2024)
        counts = np.bincount(ids.reshape(-1), minlength=E)
        eo = torch.tensor(np.cumsum(counts), dtype=torch.int32, device=dev)
        ei = torch.arange(E, dtype=torch.int64, device=dev)
        R = tokens * top_k
        w0 = torch.from_numpy(synthetic_expert_weights(qt, E, N, K, 21)).to(dev)
        w1 = torch.from_numpy(synthetic_expert_weights(qt, E, N, K, 22)).to(dev) if pair else None
        x, dy0 = bf16(R, K, 3), bf16(R, N, 4)
        dy1 = bf16(R, N, 5) if pair else None
        y0 = torch.empty(R, N, dtype=torch.bfloat16, device=dev)
        y1 = torch.empty(R, N, dtype=torch.bfloat16, device=dev) if pair else None
        dx = torch.empty(R, K, dtype=torch.bfloat16, device=dev)
        ws = torch.empty(native.grouped_workspace_bytes(R, E), dtype=torch.uint8, device=dev)
        f = timed(lambda: native.grouped_fwd(x, w0, w1, y0, y1, ei, eo, E, R, N, K, qt, ws), args.steps)
        b = timed(lambda: native.grouped_dx(dy0, dy1, w0, w1, dx, ei, eo, E, R, N, K, qt, ws), args.steps)
        report(label, 2.0 * R * N * K * (2 if pair else 1), f, b)

    grouped(12, 256, 512, 2048, 8192, 8, False, "config 3: grouped Q4_K 256 x (512 x 2048), 65536 routed rows")
    grouped(13, 256, 512, 2048, 16384, 8, True, "config 4: gate/up pair Q5_K 256 x (512 x 2048), 131072 routed rows")
    grouped(14, 256, 2048, 512, 16384, 8, False, "config 4: down Q6_K 256 x (2048 x 512), 131072 routed rows")
    grouped(22, 256, 512, 2048, 16384, 8, True, "config 5 shapes on one GPU: gate/up pair IQ2_S, 131072 routed rows")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--parity-tokens", type=int, default=32, help="tokens per rank checked against the oracle (not timed)")
    ap.add_argument("--parity-tokens-mlp", type=int, default=6, help="tokens per rank checked in the MoE feed-forward step")
    ap.add_argument("--fences", choices=["peer", "nccl"], default="peer",
                    help="multi-GPU: order the ranks' phases by this library's peer-memory barrier kernel or by NCCL collectives")
    ap.add_argument("--no-config5", action="store_true", help="skip the expert-parallel MoE feed-forward configuration")
    ap.add_argument("--pair-level", dest="token_level", action="store_false",
                    help="multi-GPU peer exchange: move one row per routed pair instead of one per (token, destination GPU)")
    ap.add_argument("--profile", action="store_true",
                    help="single GPU only: run warm-up + steps of the device-resident step and exit (for ncu)")
    ap.add_argument("--sweep", action="store_true",
                    help="single GPU only: kernel-level TFLOP/s of the other benchmark configurations, one JSON line each")
    args = ap.parse_args()
    if args.sweep:
        sweep_arm(args)
    elif args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
