#!/usr/bin/env python
"""Benchmark of the fused-MoE layer (routing + XpuFusedMoe.apply) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg2_mixtral_bf16] [--tokens T]

A step is one pass of the layer over one batch of T synthetic tokens: top-k
routing followed by the eight stages of ``XpuFusedMoe.apply``.  The default
workload is the Mixtral-8x7B-shaped bf16 layer at T=4096 tokens per GPU.  With
N > 1 (launched under torch.distributed.run) every rank runs its own replica on
its own tokens; no collective is on the data path, so scaling is weak.

Rank 0 prints one JSON line: whole-job tokens/s with inputs resident in HBM
(``value``), the same metric through the public API with host buffers and the
copies inside the timed region (``e2e``), the roofline of the grouped GEMM
kernel measured live with CUDA events, SM clocks sampled during the timed
region, and - at N=1 - the CPU oracle timed on a bounded sample of the same
workload.  ``--impl reference`` times that CPU path alone, with all host
threads.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "vllm-xpu-kernels_b200"))

import torch  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum of the two grouped-GEMM launches of one
# step, from one ncu capture per workload (see the summaries under profiles/).
NCU_TRAFFIC_BYTES = {("cfg2_mixtral_bf16", 4096): 3.956e9,
                     ("cfg3_qwen3_fp8", 4096): 0.884e9,   # profiles/grouped_gemm_fp8t256_cfg3_T4096.md
                     ("cfg5_gptoss_mxfp4", 2048): 1.883e9}   # profiles/grouped_gemm_mx_mxfp4_cfg5_T2048.md


def _gemm_kernel_name(cfg, T):
    """The kernel b200moe_grouped_gemm picks for the 16-bit / block-fp8 recipes: fp8 segments of
    12 rows per expert or more on average run the token-major kernel."""
    if cfg.recipe == "fp8block" and (T * cfg.K + cfg.E - 1) // cfg.E >= 12:
        return "grouped_gemm_fp8t256_kernel"
    return "grouped_gemm_tc_kernel"

METRIC = "fused_moe_layer_tokens_per_s"
UNIT = "tokens/s"


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=float(d["hbm_gbs"]), tensor=float(d["bf16_tflops_sustained"]),
                    tensor_burst=float(d["bf16_tflops"]), source="measured")
    return dict(hbm=6650.0, tensor=1400.0, tensor_burst=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only)."""

    def __init__(self, index: int):
        self.index, self.samples, self.reasons = index, [], set()
        self.max_mhz, self._stop, self._thr = None, threading.Event(), None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40,
                 "sw_thermal_slowdown": 0x20, "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.004)

    def __enter__(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()

    def summary(self):
        s = sorted(self.samples)
        med = s[len(s) // 2] if s else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def _physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ----------------------------------------------------------------------------- CPU arm
def cpu_layer_tokens_per_s(cfg, seconds_budget: float, steps: int, warmup: int):
    """Times the oracle's whole-layer restatement on the host cores.  Each step
    processes a bounded sample of T_s tokens of the workload; returns
    (tokens/s, T_s, ms per step, cores)."""
    from oracle import torch_oracle as to
    from oracle import workloads as wl
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    w = wl.make_weights(cfg, seed=0)
    d13, d2 = wl.dequant_weights(cfg, w)  # fp32 once, outside the timed steps

    def run(T):
        x, logits, bias = wl.make_inputs(cfg, T, seed=0)
        t0 = time.perf_counter()
        tw, ids = wl.route_cpu(cfg, logits, bias)
        if cfg.recipe == "bf16":
            to.fused_moe_bf16(x, d13, w["w13_bias"], d2, w["w2_bias"], tw, ids, cfg.E)
        else:
            to.fused_moe_staged(x, d13, w["w13_bias"], d2, w["w2_bias"], tw, ids, cfg.E,
                                activation=cfg.activation, act_quant=cfg.recipe == "fp8block")
        return time.perf_counter() - t0

    run(4)
    t_small = run(16)
    per_tok = max(t_small / 16, 1e-6)
    per_step = seconds_budget / max(1, steps + warmup)
    T_s = int(max(8, min(4096, per_step / per_tok)))
    for _ in range(warmup):
        run(T_s)
    t = [run(T_s) for _ in range(steps)]
    total = sum(t)
    return T_s * steps / total, T_s, 1e3 * total / steps, cores


# ----------------------------------------------------------------------------- GPU arm
def launches_per_step(M: int, quant: bool) -> int:
    """Kernels of ours launched by one step: routing 1; permute bookkeeping 1
    (<= 2048 routed slots) or 3, row copy 1; GEMM 2; activation 1; (fp8: act
    quant 1); gather 1."""
    return 1 + (1 if M <= 2048 else 3) + 1 + 2 + 1 + (1 if quant else 0) + 1


def build_gpu_workload(cfg, T, dev, ep_world=1, ep_rank=0, ep_chunks=None, ep_sm_reserve=20, ep_groups=None,
                       ep_sorted=False, ep_per_rank=True):
    """Synthetic weights on the device (this rank's experts only when the experts
    are sharded) and the host-side inputs of one step."""
    import vllm_xpu_kernels.fused_moe_interface as fmi
    from oracle import workloads as wl
    assert fmi.FUSEDMOE_AVAILABLE, fmi.FUSEDMOE_UNAVAILABLE_REASON
    g = torch.Generator(device=dev).manual_seed(1234 + ep_rank)
    E, H, I = cfg.E // ep_world, cfg.H, cfg.I
    if cfg.recipe == "bf16":
        # op layout [E,K,N], drawn on the device expert by expert
        w13 = torch.empty(E, H, 2 * I, dtype=torch.bfloat16, device=dev)
        w2 = torch.empty(E, I, H, dtype=torch.bfloat16, device=dev)
        for e in range(E):
            w13[e] = (torch.randn(H, 2 * I, generator=g, device=dev) * H ** -0.5).to(torch.bfloat16)
            w2[e] = (torch.randn(I, H, generator=g, device=dev) * I ** -0.5).to(torch.bfloat16)
        s13 = s2 = b13 = b2 = None
    elif cfg.recipe == "fp8block":
        from oracle import torch_oracle as to
        w13 = torch.empty(E, 2 * I, H, dtype=torch.float8_e4m3fn, device=dev)
        w2 = torch.empty(E, H, I, dtype=torch.float8_e4m3fn, device=dev)
        s13 = torch.empty(E, 2 * I // 128, H // 128, dtype=torch.float32, device=dev)
        s2 = torch.empty(E, H // 128, I // 128, dtype=torch.float32, device=dev)
        for e in range(E):  # quantised from N(0, 1/fan_in), amax/448 per 128x128 block
            w13[e], s13[e] = to.quant_fp8_block_wei(torch.randn(2 * I, H, generator=g, device=dev) * H ** -0.5)
            w2[e], s2[e] = to.quant_fp8_block_wei(torch.randn(H, I, generator=g, device=dev) * I ** -0.5)
        b13 = b2 = None
    else:  # mxfp4: uniform e2m1 codes, e8m0 exponents in [-10, -4], bf16 biases N(0, 0.02)
        w13 = torch.randint(0, 256, (E, 2 * I, H // 2), generator=g, device=dev, dtype=torch.int32).to(torch.uint8).view(torch.float4_e2m1fn_x2)
        w2 = torch.randint(0, 256, (E, H, I // 2), generator=g, device=dev, dtype=torch.int32).to(torch.uint8).view(torch.float4_e2m1fn_x2)
        s13 = torch.randint(117, 124, (E, 2 * I, H // 32), generator=g, device=dev, dtype=torch.int32).to(torch.uint8)
        s2 = torch.randint(117, 124, (E, H, I // 32), generator=g, device=dev, dtype=torch.int32).to(torch.uint8)
        b13 = (torch.randn(E, 2 * I, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        b2 = (torch.randn(E, H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    if ep_world > 1:
        from vllm_xpu_kernels.ep_moe import EpFusedMoe
        layer = EpFusedMoe(w13, s13, b13, w2, s2, b2, cfg.K, cfg.activation, E,
                           overlap_chunks=ep_chunks, sm_reserve=ep_sm_reserve, expert_groups=ep_groups,
                           sorted_exchange=ep_sorted, per_rank_rows=ep_per_rank)
    else:
        layer = fmi.XpuFusedMoe(w13, s13, b13, w2, s2, b2, cfg.K, cfg.activation, E)
    x_cpu, logits_cpu, bias_cpu = wl.make_inputs(cfg, T, seed=ep_rank)
    return layer, x_cpu, logits_cpu, bias_cpu


def make_step(cfg, layer, dev, T):
    K, E = cfg.K, cfg.E
    tw = torch.empty(T, K, dtype=torch.float32, device=dev)
    ids = torch.empty(T, K, dtype=torch.int32, device=dev)
    src = torch.empty(T, K, dtype=torch.int32, device=dev)
    out = torch.empty(T, cfg.H, dtype=torch.bfloat16, device=dev)

    def step(x, logits, bias, out=out):
        if cfg.routing == "softmax":
            torch.ops._moe_C.topk_softmax(tw, ids, src, logits, cfg.renormalize, None)
            layer.apply(out, x, tw, ids)
        else:
            scores = torch.sigmoid(logits)
            v, i = torch.ops._moe_C.grouped_topk(scores, scores + bias, cfg.n_group, cfg.topk_group, K,
                                                 cfg.renormalize, cfg.routed_scaling_factor)
            layer.apply(out, x, v, i)
            ids.copy_(i)  # keep the routed ids for the roofline's row distribution
        return out

    return step, (tw, ids)


def time_gemms(cfg, layer, ids, T, dev, iters, ep_world=1, ep_rank=0):
    """Average duration of the two grouped-GEMM launches of a step, CUDA events
    on the launching stream, on this step's real row distribution (with sharded
    experts: the rows all ranks route to this rank's experts)."""
    H, I, K = cfg.H, cfg.I, cfg.K
    E = cfg.E // ep_world
    if ep_world > 1:
        import torch.distributed as dist
        gathered = [torch.empty_like(ids) for _ in range(ep_world)]
        dist.all_gather(gathered, ids)
        flat = torch.cat([g.reshape(-1) for g in gathered]).long()
        flat = flat[(flat >= ep_rank * E) & (flat < (ep_rank + 1) * E)] - ep_rank * E
        layer = layer.local
    else:
        flat = ids.reshape(-1).long()
    rows = torch.bincount(flat, minlength=E).to(torch.int32)
    M = int(flat.numel())
    fp8 = cfg.recipe == "fp8block"
    adt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    a1 = torch.randn(M, H, device=dev).to(adt)
    a2 = torch.randn(M, I, device=dev).to(adt)
    s1 = torch.rand(M, H // 128, device=dev) if fp8 else None
    s2 = torch.rand(M, I // 128, device=dev) if fp8 else None
    d1 = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=dev)
    d2 = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
    f = torch.ops._xpu_C.cutlass_grouped_gemm_interface
    if getattr(layer, "mx_acts", False):
        # block-scaled MXFP4 path: MXFP8 activations, SwigluOAI inside gemm1's epilogue
        a1, s1 = layer._quant_mx(a1)
        a2, s2 = layer._quant_mx(a2)
        d1 = torch.empty(M, I, dtype=torch.bfloat16, device=dev)
        g = torch.ops._xpu_C.b200_grouped_gemm

        def both():
            g(a1, s1, layer.w13, layer.gemm1_wei_scales, layer.w13_bias, d1, rows, 2 * I, H, E, 0, 2, 1.702,
              7.0, 0.0, 0, 0)
            g(a2, s2, layer.w2, layer.gemm2_wei_scales, layer.w2_bias, d2, rows, H, I, E, 0, 0, 1.702, 7.0,
              0.0, 0, 0)
    else:
        def both():
            f(a1, s1, layer.w13, layer.gemm1_wei_scales, layer.w13_bias, d1, rows, 2 * I, H, E)
            f(a2, s2, layer.w2, layer.gemm2_wei_scales, layer.w2_bias, d2, rows, H, I, E)

    for _ in range(3):
        both()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        both()
    e1.record()
    torch.cuda.synchronize()
    ms_pair = e0.elapsed_time(e1) / iters
    e_act = int((rows > 0).sum())
    return ms_pair, e_act, M


def weight_bytes_per_expert(cfg):
    n = 3 * cfg.H * cfg.I
    if cfg.recipe == "bf16":
        return 2 * n
    if cfg.recipe == "fp8block":
        return n + 4 * (3 * cfg.H * cfg.I // (128 * 128))
    return n // 2 + n // 32 + (2 * (2 * cfg.I + cfg.H) if cfg.has_bias else 0)


def run_ours(args):
    import torch.distributed as dist
    from oracle import workloads as wl
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = wl.CONFIGS[args.workload]
    T = args.tokens
    ep_world = world if (args.parallelism == "ep" and world > 1) else 1
    layer, x_cpu, logits_cpu, bias_cpu = build_gpu_workload(cfg, T, dev, ep_world, rank if ep_world > 1 else 0,
                                                            args.ep_chunks, args.ep_sm_reserve, args.ep_groups, args.ep_sorted,
                                                            # one row per (token, rank) pays off once the rows, not the launches, cost
                                                            not args.ep_per_expert_rows and T > 256)
    step, (tw, ids) = make_step(cfg, layer, dev, T)
    x, logits = x_cpu.to(dev), logits_cpu.to(dev)
    bias = bias_cpu.to(dev) if bias_cpu is not None else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput ------------------------------------------------
    for _ in range(max(3, args.warmup)):
        step(x, logits, bias)
    barrier()
    run_step = lambda: step(x, logits, bias)
    if args.cuda_graph and ep_world == 1:
        # replay the step's launches from a CUDA graph (what a serving engine does at
        # decode sizes, where eager launch overhead exceeds the kernels)
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step(x, logits, bias)
            with torch.cuda.graph(g, stream=side):
                step(x, logits, bias)
        torch.cuda.current_stream(dev).wait_stream(side)
        run_step = g.replay
        for _ in range(3):
            run_step()
        barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(_physical_gpu_index(local_rank)) as clocks:
        torch.cuda.nvtx.range_push("b200_timed")
        e0.record()
        for _ in range(args.steps):
            run_step()
        e1.record()
        barrier()
        torch.cuda.nvtx.range_pop()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms)
    ms_per_step = ms_total / args.steps
    value = world * T * args.steps / (ms_total * 1e-3)

    # ---- end to end: host buffers, copies inside the timed region -----------------------
    # Every step copies its inputs from pinned host memory and its result back; the copies of
    # neighbouring steps overlap the compute of the current one (two buffers, three streams),
    # as a serving loop would run it.
    x_pin, lg_pin = x_cpu.pin_memory(), logits_cpu.pin_memory()
    out_pin = [torch.empty(T, cfg.H, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    x_d = [torch.empty_like(x) for _ in range(2)]
    lg_d = [torch.empty_like(logits) for _ in range(2)]
    out_d = [torch.empty(T, cfg.H, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    s_in, s_out, cur = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.current_stream(dev)

    def e2e_loop(n):
        comp_done = [None, None]
        out_done = [None, None]
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(s_in):
                if comp_done[b] is not None:
                    s_in.wait_event(comp_done[b])       # step i-2 has consumed this input buffer
                x_d[b].copy_(x_pin, non_blocking=True)
                lg_d[b].copy_(lg_pin, non_blocking=True)
                in_ready = torch.cuda.Event()
                in_ready.record(s_in)
            cur.wait_event(in_ready)
            if out_done[b] is not None:
                cur.wait_event(out_done[b])             # step i-2's result has left this buffer
            step(x_d[b], lg_d[b], bias, out_d[b])
            comp_done[b] = torch.cuda.Event()
            comp_done[b].record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[b])
                out_pin[b].copy_(out_d[b], non_blocking=True)
                out_done[b] = torch.cuda.Event()
                out_done[b].record(s_out)
        for ev in out_done:
            if ev is not None:
                cur.wait_event(ev)

    e2e_loop(3)
    barrier()
    e0.record()
    e2e_loop(args.steps)
    e1.record()
    barrier()
    ms2 = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
    e2e_value = world * T * args.steps / (float(ms2) * 1e-3)
    h2d = x_pin.numel() * 2 + lg_pin.numel() * 4
    d2h = out_pin[0].numel() * 2

    # ---- roofline of the grouped GEMM kernel ---------------------------------------------
    peaks = _peaks()
    ms_pair, e_act, m_rows = time_gemms(cfg, layer, ids, T, dev, max(3, min(20, args.steps)), ep_world, rank)
    flops = 6.0 * m_rows * cfg.H * cfg.I
    wbytes = e_act * weight_bytes_per_expert(cfg)
    act_bytes = m_rows * (cfg.H + 2 * cfg.I + cfg.I + cfg.H) * 2  # A and D of both launches
    mx = getattr(layer.local if ep_world > 1 else layer, "mx_acts", False)
    if mx:  # per plane 1-byte codes + 1/32 scale byte in, 16-bit out; gemm1 writes the activated [M, I]
        planes = (layer.local if ep_world > 1 else layer).mx_planes
        act_bytes = m_rows * (planes * (cfg.H + cfg.I) * 33 // 32 + (cfg.I + cfg.H) * 2)
    t_tensor = flops / (peaks["tensor"] * 1e12)
    t_hbm = (wbytes + act_bytes) / (peaks["hbm"] * 1e9)
    if t_tensor >= t_hbm:
        ach = flops / (ms_pair * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": round(ach, 2), "peak": peaks["tensor"], "unit": "TFLOP/s",
                "frac": round(ach / peaks["tensor"], 4)}
    else:
        ach = (wbytes + act_bytes) / (ms_pair * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": round(ach, 1), "peak": peaks["hbm"], "unit": "GB/s",
                "frac": round(ach / peaks["hbm"], 4)}
    roof.update({"traffic": NCU_TRAFFIC_BYTES.get((cfg.name, T)) if ep_world == 1 else None, "kernel": (("grouped_gemm_mx_kernel" if mx else "grouped_gemm_dq_kernel") if cfg.recipe == "mxfp4" else _gemm_kernel_name(cfg, T))
                           + " (gemm1 + gemm2 of one step)",
                 "ms_per_launch_pair": round(ms_pair, 4), "peak_source": peaks["source"] + " (sustained)",
                 "experts_active": e_act})

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": {"bf16": "bf16", "fp8block": "fp8_e4m3",
                                                          "mxfp4": "mxfp4"}[cfg.recipe],
        "data": "synthetic",
        "config": {"workload": f"{cfg.name} T={T} per GPU", "H": cfg.H, "I": cfg.I, "E": cfg.E, "top_k": cfg.K,
                   "tokens_per_gpu": T, "routing": cfg.routing, "parallelism": (f"ep{world}: {cfg.E // world} experts per GPU, NCCL all-to-all dispatch/combine"
                                   if ep_world > 1 else f"replicas x{world}"),
                   "l2": "inputs exceed L2: the weights streamed per step are larger than the 126 MB L2"
                         if e_act * weight_bytes_per_expert(cfg) > 126e6 else "inputs smaller than L2",
                   "launch": "cuda graph replay" if (args.cuda_graph and ep_world == 1) else "eager torch ops",
                   "seed": 0},
        "e2e": {"value": round(e2e_value, 1), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_per_step(T * cfg.K, cfg.recipe == "fp8block") * args.steps,
        "clocks": clocks.summary(),
        "roofline": roof,
    }
    if world == 1 and not args.no_cpu_baseline:
        v, T_s, ms_cpu, cores = cpu_layer_tokens_per_s(cfg, 20.0, 2, 1)
        line["cpu_baseline"] = {"value": round(v, 2), "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"{T_s} tokens of the same layer per step, 2 timed steps, "
                                          f"weights pre-converted to fp32, {ms_cpu:.0f} ms per step"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_ops(args):
    """`--workload ops`: the standalone activation / quantisation / routing-side ops of the
    layer's neighbourhood, one JSON line each: CUDA-event time at a DeepSeek-sized
    activation (rows x 2*2048 gate|up, larger than L2 in total), algorithmic bytes,
    achieved GB/s against the measured copy bandwidth.  Not the headline: the
    default run reports the layer."""
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    import vllm_xpu_kernels.fused_moe_interface  # noqa: F401  (registers the ops)
    peaks = _peaks()
    rows, H = 65536, 2048
    g = torch.Generator(device=dev).manual_seed(0)
    x2 = torch.randn(rows, 2 * H, generator=g, device=dev).to(torch.bfloat16)
    x1 = torch.randn(rows, H, generator=g, device=dev).to(torch.bfloat16)
    q8 = torch.empty(rows, H, dtype=torch.float8_e4m3fn, device=dev)
    q4 = torch.empty(rows, H // 2, dtype=torch.uint8, device=dev)
    s128 = torch.empty(rows, H // 128, dtype=torch.float32, device=dev)
    s32 = torch.empty(rows, H // 32, dtype=torch.float32, device=dev)
    o16 = torch.empty(rows, H, dtype=torch.bfloat16, device=dev)
    qmx = torch.empty(2 * rows, H, dtype=torch.float8_e4m3fn, device=dev)
    smx = torch.empty(2, (H + 127) // 128, rows, dtype=torch.int32, device=dev)
    one = torch.tensor([0.5], device=dev)
    C = torch.ops._C
    cases = [
        ("silu_and_mul", lambda: C.silu_and_mul(o16, x2), rows * H * 6),
        ("swigluoai_and_mul", lambda: C.swigluoai_and_mul(o16, x2, 1.702, 7.0), rows * H * 6),
        ("per_token_group_fp8_quant", lambda: C.per_token_group_fp8_quant(x1, q8, s128, 128, 1e-10, -448., 448., False, False, False),
         rows * H * 3 + s128.numel() * 4),
        ("silu_and_mul_per_block_quant", lambda: C.silu_and_mul_per_block_quant(q8, x2, s128, 128, None, False, False),
         rows * H * 5 + s128.numel() * 4),
        ("silu_and_mul_quant", lambda: C.silu_and_mul_quant(q8, x2, one), rows * H * 5),
        ("silu_and_mul_mxfp4_quant", lambda: C.silu_and_mul_mxfp4_quant(q4, x2, s32, 32, 1e-10),
         rows * H * 4 + rows * H // 2 + s32.numel() * 4),
        ("per_token_group_quant_mxfp4", lambda: C.per_token_group_quant_mxfp4(x1, q4, s32, 32, 1e-10),
         rows * H * 2 + rows * H // 2 + s32.numel() * 4),
        ("b200_quant_mxfp8 (2 planes)", lambda: C.b200_quant_mxfp8(x1, qmx, smx), rows * H * 4 + smx.numel() * 4),
    ]
    for name, fn, nbytes in cases:
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        gbs = nbytes / (ms * 1e-3) / 1e9
        print(json.dumps({"op": name, "rows": rows, "hidden": H, "ms": round(ms, 4), "algorithmic_bytes": nbytes,
                          "achieved_GBps": round(gbs, 1), "peak_GBps": peaks["hbm"],
                          "frac": round(gbs / peaks["hbm"], 3), "peak_source": peaks["source"]}), flush=True)


def run_reference(args):
    """The reference's own CPU path for this layer (its pure-torch test
    reference, restated in oracle/), timed on the host cores of this box."""
    from oracle import workloads as wl
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    cfg = wl.CONFIGS[args.workload]
    v, T_s, ms_cpu, cores = cpu_layer_tokens_per_s(cfg, 120.0, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(v, 2), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_cpu, 2), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{cfg.name} T={args.tokens} per GPU", "H": cfg.H, "I": cfg.I, "E": cfg.E,
                   "top_k": cfg.K, "tokens_per_gpu": args.tokens, "routing": cfg.routing, "seed": 0},
        "cpu_baseline": {"value": round(v, 2), "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{T_s} tokens of the same layer per step"},
        "e2e": {"value": round(v, 2), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2_mixtral_bf16")
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--parallelism", default="replicas", choices=["replicas", "ep"],
                    help="N > 1: independent replicas (default) or experts sharded over the ranks "
                         "with all-to-all token dispatch / combine")
    ap.add_argument("--ep-groups", type=int, default=None,
                    help="expert parallelism: pipeline the two all-to-alls with the experts by splitting each "
                         "rank's experts into this many groups")
    ap.add_argument("--ep-per-expert-rows", action="store_true",
                    help="expert parallelism: ship one row per (token, expert) instead of one per (token, rank)")
    ap.add_argument("--ep-sorted", action="store_true",
                    help="expert parallelism: ship rows sorted by expert so the receiver multiplies them as they "
                         "arrive (prefill-sized batches)")
    ap.add_argument("--ep-chunks", type=int, default=None,
                    help="ep: token chunks whose exchange overlaps the experts (default: by batch size)")
    ap.add_argument("--ep-sm-reserve", type=int, default=20,
                    help="ep: SMs the GEMM kernels leave to the collective while chunks overlap")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="device-resident loop replays the step from a CUDA graph instead of eager ops")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.workload == "ops":
        run_ops(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
