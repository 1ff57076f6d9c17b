#!/usr/bin/env python
"""Benchmark of the fused-MoE layer (routing + the layer's apply) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg4_deepseek_fp8] [--tokens T] [--sweep]

A step is one pass of the layer over one batch of T synthetic tokens per GPU: top-k routing
followed by the stages of the layer.  The default workload is the DeepSeek-V3-shaped
block-fp8 layer (H=7168, I=2048, 256 experts, grouped sigmoid top-8) at 8192 tokens per GPU,
the configuration the 1/2/4/8-GPU metric is quoted on.  With N > 1 (launched under
torch.distributed.run) the experts are sharded evenly over the ranks and tokens are dispatched
to their experts' ranks and combined back over NVLink peer memory (``--parallelism ep``, the
default at N > 1; ``--ep-placement`` says which rank holds which experts: evened out by the expert
histogram of a calibration batch, or contiguous); ``--parallelism replicas`` runs N independent
copies instead.

Rank 0 prints one JSON line: whole-job tokens/s with inputs resident in HBM (``value``), the
same metric through the public API with host buffers and the copies inside the timed region
(``e2e``), the roofline of the grouped GEMM kernel measured live with CUDA events, per-stage
times, SM clocks sampled during the timed region, and - at N=1 - the CPU restatement of the
reference's torch path timed on a bounded sample of the same workload.  ``--impl reference``
times that CPU path alone, with all host threads.  ``--sweep`` (one GPU) prints one such line
for every (workload, T) point of the five benchmark layers.
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

import bench_workloads as bw  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum of the two grouped-GEMM launches of one step, from
# one ncu capture per workload on a smaller case of the same kernel, scaled by the rows processed.
# Not measured in the run: the line says "from capture".
CAPTURED_TRAFFIC_BYTES = {("cfg2_mixtral_bf16", 4096): 3.921e9,
                          ("cfg3_qwen3_fp8", 4096): 0.884e9,
                          ("cfg5_gptoss_mxfp4", 2048): 1.883e9}

FP8T_TRAFFIC_OVER_ALGORITHMIC = 0.947

METRIC = "fused_moe_layer_tokens_per_s"
UNIT = "tokens/s"


def _gemm_kernel_name(cfg, rows_per_expert_avg, mx):
    if cfg.recipe == "mxfp4":
        return "grouped_gemm_mx_kernel" if mx else "grouped_gemm_dq_kernel"
    if cfg.recipe == "fp8block" and rows_per_expert_avg >= 12:
        return "grouped_gemm_fp8t256_kernel"
    return "grouped_gemm_tc_kernel"


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=float(d["hbm_gbs"]), tensor=float(d["bf16_tflops"]),
                    tensor_sustained=float(d["bf16_tflops_sustained"]), source="measured")
    return dict(hbm=6650.0, tensor=1590.0, tensor_sustained=1400.0, source="fallback")


def measure_fp8_dense_tflops(dev):
    """Dense e4m3 x e4m3 GEMM rate of this GPU, as a yardstick for the fp8 kernels: the library
    GEMM (torch._scaled_mm, 8192^3, unit scales), best of 5 after warm-up.  None if unavailable."""
    try:
        n = 8192
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)
        f = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


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
    """Times the restatement of the reference's torch path for the whole layer on the host cores.
    Each step processes a bounded sample of T_s tokens of the workload; returns
    (tokens/s, T_s, ms per step, cores, note).  Layers with many large experts draw their
    experts from at most 8 distinct weight sets so that the fp32 copies fit host memory; the
    arithmetic per token is unchanged."""
    from oracle import torch_oracle as to
    from oracle import workloads as wl
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    distinct = cfg.E if cfg.E * bw.weight_bytes_per_expert(cfg) * 4 < 24e9 else 8
    w = wl.make_weights(cfg, seed=0, num_experts=distinct)
    d13, d2 = wl.dequant_weights(cfg, w)  # fp32 once, outside the timed steps
    note = ""
    b13, b2 = w["w13_bias"], w["w2_bias"]
    if distinct < cfg.E:
        d13 = wl.ExpertView(cfg.E, 2 * cfg.I, cfg.H, lambda e, d=d13: d[e % distinct])
        d2 = wl.ExpertView(cfg.E, cfg.H, cfg.I, lambda e, d=d2: d[e % distinct])
        note = f", the {cfg.E} experts drawn from {distinct} distinct weight sets (host memory)"

    def run(T):
        x, logits, bias = wl.make_inputs(cfg, T, seed=0)
        t0 = time.perf_counter()
        tw, ids = wl.route_cpu(cfg, logits, bias)
        if cfg.recipe == "bf16":
            to.fused_moe_bf16(x, d13, b13, d2, b2, tw, ids, cfg.E)
        else:
            to.fused_moe_staged(x, d13, b13, d2, b2, tw, ids, cfg.E,
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
    return T_s * steps / total, T_s, 1e3 * total / steps, cores, note


# ----------------------------------------------------------------------------- GPU arm
class StageTimer:
    """CUDA-event marks between the stages of a layer call (the per-stage timing of the
    reference's harness, benchmark/src/fused_moe_interface_.py:12-40 of vllm-xpu-kernels)."""

    def __init__(self):
        self.marks = []

    def mark(self, name):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.marks.append((name, ev))

    def durations_ms(self):
        out = {}
        for (_, e0), (name, e1) in zip(self.marks[:-1], self.marks[1:]):
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        return out


def route_on_device(cfg, logits, bias):
    """Top-k routing of the workload: (weights [T, K] f32, ids [T, K])."""
    T = logits.shape[0]
    if cfg.routing == "softmax":
        tw = torch.empty(T, cfg.K, dtype=torch.float32, device=logits.device)
        ids = torch.empty(T, cfg.K, dtype=torch.int32, device=logits.device)
        torch.ops._moe_C.topk_softmax(tw, ids, torch.empty_like(ids), logits, cfg.renormalize, None)
        return tw, ids
    scores = torch.sigmoid(logits)
    return torch.ops._moe_C.grouped_topk(scores, scores + bias, cfg.n_group, cfg.topk_group, cfg.K,
                                         cfg.renormalize, cfg.routed_scaling_factor)


CALIBRATION_SEED, CALIBRATION_TOKENS = 777_001, 8192


def balanced_placement(cfg, dev, ep_world, bias):
    """expert -> slot for the sharded experts, from the expert histogram of a calibration batch:
    tokens of the workload's distribution (a seed no timed batch uses) routed with the layer's
    own routing bias.  Deterministic, so every rank computes the same table."""
    from vllm_xpu_kernels.ep_moe import balanced_expert_slots
    _, logits, _ = bw.make_inputs(cfg, CALIBRATION_TOKENS, seed=CALIBRATION_SEED)
    _, ids = route_on_device(cfg, logits.to(dev), bias.to(dev) if bias is not None else None)
    load = torch.bincount(ids.reshape(-1).long().cpu(), minlength=cfg.E)
    return balanced_expert_slots(load, ep_world)


def build_gpu_workload(cfg, T, dev, ep_world=1, ep_rank=0, transport="peer", placement="balanced"):
    """Synthetic weights on the device (this rank's experts only when the experts are sharded)
    and the host-side inputs of one step."""
    import vllm_xpu_kernels.fused_moe_interface as fmi
    assert fmi.FUSEDMOE_AVAILABLE, fmi.FUSEDMOE_UNAVAILABLE_REASON
    E = cfg.E // ep_world
    w13, s13, b13, w2, s2, b2 = bw.make_device_weights(cfg, E, dev, seed=1234 + ep_rank)
    # every rank draws its own tokens and router logits; the routing bias belongs to the layer and is
    # the same on all ranks (the one the single-GPU run uses)
    x_cpu, logits_cpu, bias_cpu = bw.make_inputs(cfg, T, seed=ep_rank)
    if ep_rank != 0 and bias_cpu is not None:
        bias_cpu = bw.make_inputs(cfg, T, seed=0)[2]
    layer = None
    if ep_world > 1 and transport == "peer":
        # symmetric memory is a property of the box (driver, IPC permissions): if any rank cannot
        # set it up, all ranks fall back to the collective-library transport and the line says so
        import torch.distributed as dist
        from vllm_xpu_kernels.ep_moe import EpPeerFusedMoe, SymmetricPeerGroup
        ok = torch.ones(1, device=dev)
        try:
            slot = balanced_placement(cfg, dev, ep_world, bias_cpu) if placement == "balanced" else None
            layer = EpPeerFusedMoe(w13, s13, b13, w2, s2, b2, cfg.K, cfg.activation, E,
                                   SymmetricPeerGroup(dev), T, cfg.H, expert_slot=slot)
        except Exception as e:  # noqa: BLE001
            print(f"rank {ep_rank}: peer-memory transport unavailable ({e!r})", file=sys.stderr, flush=True)
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok) == 0.0:
            layer = None
    if layer is not None:
        pass
    elif ep_world > 1:
        from vllm_xpu_kernels.ep_moe import EpFusedMoe
        layer = EpFusedMoe(w13, s13, b13, w2, s2, b2, cfg.K, cfg.activation, E, per_rank_rows=T > 256)
    else:
        layer = fmi.XpuFusedMoe(w13, s13, b13, w2, s2, b2, cfg.K, cfg.activation, E)
    return layer, x_cpu, logits_cpu, bias_cpu


def _transport_of(layer):
    return "peer" if type(layer).__name__ == "EpPeerFusedMoe" else "nccl"


def make_step(cfg, layer, dev, T):
    K = cfg.K
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
    """Average duration of the two grouped-GEMM launches of a step, CUDA events on the launching
    stream, on this step's real row distribution (with sharded experts: the rows all ranks route
    to this rank's experts)."""
    H, I = cfg.H, cfg.I
    E = cfg.E // ep_world
    if ep_world > 1:
        import torch.distributed as dist
        gathered = [torch.empty_like(ids) for _ in range(ep_world)]
        dist.all_gather(gathered, ids)
        flat = torch.cat([g.reshape(-1) for g in gathered]).long()
        if getattr(layer, "expert_slot", None) is not None:
            flat = layer.expert_slot.long()[flat]
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
        layer.persistent_workspace = False
        a1, s1 = layer._quant_mx(a1)
        a2, s2 = layer._quant_mx(a2)
        layer.persistent_workspace = True
        d1 = torch.empty(M, I, dtype=torch.bfloat16, device=dev)
        g = torch.ops._xpu_C.b200_grouped_gemm

        def both():
            g(a1, s1, layer.w13, layer.gemm1_wei_scales, layer.w13_bias, d1, rows, 2 * I, H, E, 0, 2, 1.702,
              7.0, 0.0, 0, 0)
            g(a2, s2, layer.w2, layer.gemm2_wei_scales, layer.w2_bias, d2, rows, H, I, E, 0, 0, 1.702, 7.0,
              0.0, 0, 0)
    elif not fp8 and layer.fuses_activation(M) == "epilogue":
        # 16-bit layer with the gated activation inside gemm1's epilogue: time that form
        d1 = torch.empty(M, I, dtype=torch.bfloat16, device=dev)
        g = torch.ops._xpu_C.b200_grouped_gemm
        epi = 1 if cfg.activation == "silu" else 2

        def both():
            g(a1, None, layer.w13, None, layer.w13_bias, d1, rows, 2 * I, H, E, 0, epi, 1.702, 7.0, 0.0, 0, 0)
            f(a2, None, layer.w2, None, layer.w2_bias, d2, rows, H, I, E)
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


def launches_per_step(cfg, T, layer, ep_world, transport) -> int:
    """Kernels of this repository launched by one step, counted from the code path taken:
    routing 1; sort 1 (<= 2048 slots) or 3; row copy (+quant) 1; gemm1 1; activation (+quant) 1
    unless fused into gemm1; MX activation quantisers 2; gemm2 1; gather 1.  Expert parallelism
    over peer memory: routing 1, dispatch sort 1|3 + dispatch 1, mask 1, the local layer without
    its gather, combine 1, final gather 1."""
    local = layer.local if ep_world > 1 else layer
    act = 0 if local.fuses_activation(T * cfg.K) else 1
    mx = 2 if getattr(local, "mx_acts", False) else 0
    sort = lambda slots: 1 if slots <= 2048 else 3
    if ep_world == 1:
        return 1 + sort(T * cfg.K) + 1 + 1 + act + mx + 1 + 1
    if transport == "peer":
        return 1 + sort(T * ep_world) + 1 + 1 + sort(ep_world * T * cfg.K) + 1 + 1 + act + mx + 1 + 1 + 1
    return 1 + sort(T * ep_world) + 1 + sort(T * ep_world * cfg.K) + 1 + 1 + act + mx + 1 + 1 + 1


def stage_times(cfg, layer, step, x, logits, bias, reps=5):
    """Per-stage device time of a step (single GPU): the layer is given a hook that records a
    CUDA event after every stage; averaged over `reps` steps outside the timed region."""
    import torch.distributed as dist
    acc = {}
    for _ in range(reps):
        if dist.is_initialized():     # ranks start a step together, as they do inside the timed loop
            torch.cuda.synchronize()
            dist.barrier()
        timer = StageTimer()
        layer.stage_hook = timer.mark
        timer.mark("start")
        step(x, logits, bias)
        layer.stage_hook = None
        torch.cuda.synchronize()
        for k, v in timer.durations_ms().items():
            acc[k] = acc.get(k, 0.0) + v / reps
    return {k: round(v, 4) for k, v in acc.items()}


def run_point(args, cfg, T, world, rank, local_rank, dev, dist):
    """One (workload, T) measurement -> the JSON line as a dict."""
    ep_world = world if (args.parallelism == "ep" and world > 1) else 1
    layer, x_cpu, logits_cpu, bias_cpu = build_gpu_workload(cfg, T, dev, ep_world, rank if ep_world > 1 else 0,
                                                            args.ep_transport, args.ep_placement)
    if ep_world > 1:
        args.ep_transport = _transport_of(layer)     # what actually runs
    step, (tw, ids) = make_step(cfg, layer, dev, T)
    x, logits = x_cpu.to(dev), logits_cpu.to(dev)
    bias = bias_cpu.to(dev) if bias_cpu is not None else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput ------------------------------------------------
    warm = max(3, args.warmup)
    for _ in range(warm):
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
    local = layer.local if ep_world > 1 else layer
    ms_pair, e_act, m_rows = time_gemms(cfg, layer, ids, T, dev, max(3, min(20, args.steps)), ep_world, rank)
    flops = 6.0 * m_rows * cfg.H * cfg.I
    wbytes = e_act * bw.weight_bytes_per_expert(cfg)
    act_bytes = m_rows * (cfg.H + 2 * cfg.I + cfg.I + cfg.H) * 2  # A and D of both launches
    if cfg.recipe == "fp8block":  # e4m3 rows + fp32 scale per 128 in, 16-bit out
        act_bytes = m_rows * ((cfg.H + cfg.I) * (1 + 4 / 128) + (2 * cfg.I + cfg.H) * 2)
    mx = getattr(local, "mx_acts", False)
    if mx:  # per plane 1-byte codes + 1/32 scale byte in, 16-bit out; gemm1 writes the activated [M, I]
        act_bytes = m_rows * (local.mx_planes * (cfg.H + cfg.I) * 33 // 32 + (cfg.I + cfg.H) * 2)
    # tensor peak of the instruction kind the kernel issues: kind::f16 -> the measured bf16 GEMM
    # (burst: the pair is timed alone); kind::f8f6f4 / mxf8f6f4 -> a dense fp8 GEMM measured here
    fp8_kind = cfg.recipe != "bf16"
    tensor_peak, tensor_src = peaks["tensor"], peaks["source"] + " bf16 GEMM (burst)"
    if fp8_kind:
        fp8_peak = measure_fp8_dense_tflops(dev)
        if fp8_peak is not None:
            tensor_peak, tensor_src = fp8_peak, "measured in this run: torch._scaled_mm e4m3 8192^3 (burst)"
        else:
            tensor_peak, tensor_src = 2.0 * peaks["tensor"], "2 x " + tensor_src + ": no fp8 GEMM available"
    t_tensor = flops / (tensor_peak * 1e12)
    t_hbm = (wbytes + act_bytes) / (peaks["hbm"] * 1e9)
    tf = flops / (ms_pair * 1e-3) / 1e12
    gbs = (wbytes + act_bytes) / (ms_pair * 1e-3) / 1e9
    if t_tensor >= t_hbm:
        roof = {"bound": "tensor", "achieved": round(tf, 2), "peak": round(tensor_peak, 1), "unit": "TFLOP/s",
                "frac": round(tf / tensor_peak, 4), "peak_source": tensor_src}
    else:
        roof = {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm"], "unit": "GB/s",
                "frac": round(gbs / peaks["hbm"], 4), "peak_source": peaks["source"] + " copy bandwidth"}
    # both limits, whichever binds: the time the launch pair would take at each peak over its time
    roof.update({"tflops": round(tf, 2), "tensor_frac": round(tf / tensor_peak, 4), "tensor_peak": round(tensor_peak, 1),
                 "tensor_peak_source": tensor_src, "frac_of_bf16_peak": round(tf / peaks["tensor"], 4),
                 "gbs": round(gbs, 1), "hbm_frac": round(gbs / peaks["hbm"], 4)})
    traffic = CAPTURED_TRAFFIC_BYTES.get((cfg.name, T)) if ep_world == 1 else None
    traffic_source = "from capture" if traffic else None
    if traffic is None and cfg.recipe == "fp8block" and m_rows / max(1, cfg.E // ep_world) >= 12:
        # the token-major fp8 kernel: its small-case capture (cfg3, T=4096: 0.882 GB of DRAM traffic for
        # 0.931 GB of algorithmic bytes) scaled to this launch pair by the algorithmic bytes
        traffic = round(FP8T_TRAFFIC_OVER_ALGORITHMIC * (wbytes + act_bytes))
        traffic_source = "scaled from a small-case capture of the same kernel by the algorithmic bytes"
    roof.update({"traffic": traffic, "traffic_source": traffic_source,
                 "kernel": _gemm_kernel_name(cfg, m_rows / max(1, cfg.E // ep_world), mx) + " (gemm1 + gemm2 of one step)",
                 "ms_per_launch_pair": round(ms_pair, 4), "experts_active": e_act, "rows": m_rows})
    # the whole layer against its algorithmic bytes / flops (intermediates not counted)
    e_act_layer = e_act
    layer_t_hbm = bw.layer_bytes(cfg, T, e_act_layer) / (peaks["hbm"] * 1e9)
    layer_t_tensor = bw.layer_flops(cfg, T) / (tensor_peak * 1e12)
    layer_roof = {"hbm_frac": round(layer_t_hbm / (ms_per_step * 1e-3), 4),
                  "tensor_frac": round(layer_t_tensor / (ms_per_step * 1e-3), 4)} if ep_world == 1 else None

    par = (f"ep{world}: {cfg.E // world} experts per GPU"
           + (" placed by load" if getattr(layer, "expert_slot", None) is not None else "")
           + ", dispatch/combine "
           + ("by peer stores over NVLink (symmetric memory), two barriers per step"
              if args.ep_transport == "peer" else "by NCCL all-to-all")) if ep_world > 1 else (
        f"replicas x{world}" if world > 1 else "single GPU")
    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": {"bf16": "bf16", "fp8block": "fp8_e4m3",
                                                          "mxfp4": "mxfp4"}[cfg.recipe],
        "data": "synthetic",
        "config": {"workload": f"{cfg.name} T={T} per GPU", "H": cfg.H, "I": cfg.I, "E": cfg.E, "top_k": cfg.K,
                   "tokens_per_gpu": T, "routing": cfg.routing, "parallelism": par,
                   "l2": "inputs exceed L2: the weights streamed per step are larger than the 126 MB L2"
                         if e_act * bw.weight_bytes_per_expert(cfg) > 126e6 else "inputs smaller than L2",
                   "launch": "cuda graph replay" if (args.cuda_graph and ep_world == 1) else "eager torch ops",
                   "seed": 0},
        "e2e": {"value": round(e2e_value, 1), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_per_step(cfg, T, layer, ep_world, args.ep_transport) * args.steps,
        "clocks": clocks.summary(),
        "roofline": roof,
        "layer_roofline": layer_roof,
    }
    if (ep_world == 1 and world == 1) or (ep_world > 1 and args.ep_transport == "peer"):
        # (with sharded experts: rank 0's view; a barrier's time includes waiting for the slowest rank)
        line["stages_ms"] = stage_times(cfg, layer, step, x, logits, bias)
    if ep_world > 1 and args.ep_transport == "peer":
        # bytes one rank stores into its peers per step (rows + scales + ids + weights out, partial
        # sums back), from the counts of the last step
        sent = int(layer.send_counts.sum())
        remote = sent - int(layer.send_counts[rank])
        row = cfg.H + (cfg.H // 128) * 4 if layer.quant else 2 * cfg.H
        recvd = int(layer.recv_counts.sum()) - int(layer.recv_counts[rank])
        # routed (token, expert) slots every rank's experts received: the synthetic routing bias makes
        # experts unequally popular, and a step lasts as long as its busiest rank
        mine = torch.tensor([float((layer.recv_ids >= 0).sum())], device=dev)
        loads = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(loads, mine)
        loads = [float(v) for v in loads]
        # each rank's own work per step (its stage times without the waits at the barriers) and
        # the time of its two GEMM stages: tells a slow GPU from an uneven load
        st = line.get("stages_ms") or {}
        mine = torch.tensor([sum(v for k, v in st.items() if not k.startswith("barrier")),
                             st.get("local_gemm1", 0.0) + st.get("local_gemm2", 0.0),
                             st.get("dispatch", 0.0) + st.get("combine", 0.0)], device=dev)
        busy = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(busy, mine)
        line["ep"] = {"busy_ms_by_rank": [round(float(b[0]), 3) for b in busy],
                      "gemm_ms_by_rank": [round(float(b[1]), 3) for b in busy],
                      "exchange_ms_by_rank": [round(float(b[2]), 3) for b in busy],
                      "rows_sent": sent, "rows_sent_remote": remote,
                      "dispatch_bytes_remote": remote * (row + cfg.K * 8),
                      "combine_bytes_remote": recvd * cfg.H * 2,
                      "placement": ("experts placed by the load of a calibration batch (%d tokens, seed %d)"
                                    % (CALIBRATION_TOKENS, CALIBRATION_SEED)
                                    if layer.expert_slot is not None else "contiguous"),
                      "expert_slots_per_rank": [int(v) for v in loads],
                      "load_max_over_mean": round(max(loads) * world / max(1.0, sum(loads)), 3)}
    return line


def run_ours(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        dist.init_process_group("nccl", device_id=dev)
    if args.parallelism == "auto":
        args.parallelism = "ep" if world > 1 else "replicas"
    if args.sweep:
        assert world == 1, "--sweep runs on one GPU"
        for name, cfg in bw.CONFIGS.items():
            for T in cfg.tokens:
                line = run_point(args, cfg, T, 1, 0, local_rank, dev, dist)
                print(json.dumps(line), flush=True)
                from vllm_xpu_kernels.fused_moe_interface import _WORKSPACE
                _WORKSPACE.clear()
                torch.cuda.empty_cache()
        return
    cfg = bw.CONFIGS[args.workload]
    line = run_point(args, cfg, args.tokens, world, rank, local_rank, dev, dist)
    if world == 1 and not args.no_cpu_baseline:
        v, T_s, ms_cpu, cores, note = cpu_layer_tokens_per_s(cfg, 20.0, 2, 1)
        line["cpu_baseline"] = {"value": round(v, 2), "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"{T_s} tokens of the same layer per step, 2 timed steps, "
                                          f"weights pre-converted to fp32{note}, {ms_cpu:.0f} ms per step"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
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
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    cfg = bw.CONFIGS[args.workload]
    v, T_s, ms_cpu, cores, note = cpu_layer_tokens_per_s(cfg, 90.0, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(v, 2), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_cpu, 2), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{cfg.name} T={args.tokens} per GPU", "H": cfg.H, "I": cfg.I, "E": cfg.E,
                   "top_k": cfg.K, "tokens_per_gpu": args.tokens, "routing": cfg.routing, "seed": 0},
        "cpu_baseline": {"value": round(v, 2), "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{T_s} tokens of the same layer per step{note}"},
        "e2e": {"value": round(v, 2), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg4_deepseek_fp8")
    ap.add_argument("--tokens", type=int, default=8192, help="tokens per GPU and step")
    ap.add_argument("--parallelism", default="auto", choices=["auto", "replicas", "ep"],
                    help="N > 1: experts sharded over the ranks with token dispatch / combine (ep, the "
                         "default) or independent replicas")
    ap.add_argument("--ep-transport", default="peer", choices=["peer", "nccl"],
                    help="ep: dispatch / combine by this repository's kernels storing into peer memory over "
                         "NVLink (default) or by NCCL all-to-all (the comparison point)")
    ap.add_argument("--ep-placement", default="balanced", choices=["balanced", "contiguous"],
                    help="ep over peer memory: which rank holds which experts - placed so that the ranks' "
                         "loads even out, from the expert histogram of a calibration batch (default), or "
                         "expert g on rank g // (E / N)")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="device-resident loop replays the step from a CUDA graph instead of eager ops")
    ap.add_argument("--sweep", action="store_true",
                    help="one GPU: one JSON line for every (workload, T) point of the benchmark table")
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
