# SPDX-License-Identifier: Apache-2.0
"""Expert parallelism with token dispatch / combine over ``torch.distributed``.

The reference has no communication layer: its expert parallelism is a per-rank
``expert_map`` mask (``vllm_xpu_kernels/fused_moe_interface.py:256-271``,
``csrc/moe/init_expert_map.cpp:33-53``) that leaves every rank with the full
token batch and a partial sum for the caller to all-reduce.  ``XpuFusedMoe``
keeps that semantic untouched.  This module adds the other scheme on top of the
same kernels: experts are split contiguously and evenly over the ranks (expert
``g`` lives on rank ``g // E_local``, as ``init_expert_map`` encodes it), every
rank routes its own tokens, sends each routed row to the rank that owns its
expert (all-to-all), runs the local experts, and gets the rows back (all-to-all)
for the weighted top-k reduction.

``EpAllToAll`` is pure plumbing (counts, splits, the three exchanges) and works
on any backend (NCCL on GPUs; Gloo on CPU tensors in the tests).
``EpFusedMoe`` is the CUDA layer built from the registered ops.

The exact per-peer row counts are read back to the host once per call (one
small device-to-host copy) because ``all_to_all_single`` takes its split sizes
from the host.
"""
from typing import Optional

import torch
import torch.distributed as dist

FP8_BLOCK = 128


class EpAllToAll:
    """Variable-size row exchange between the ranks of one process group."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.ep_size = dist.get_world_size(group)
        self.ep_rank = dist.get_rank(group)

    def exchange_counts(self, send_counts: torch.Tensor):
        """send_counts [ep] (rows this rank sends to each peer) ->
        (send_splits, recv_splits) as host lists."""
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        both = torch.stack((send_counts, recv_counts)).cpu()
        return both[0].tolist(), both[1].tolist()

    def dispatch(self, tensors, send_splits, recv_splits):
        """Sends rows [sum(send_splits), ...] of every tensor in `tensors`
        (grouped by destination rank) and returns the received counterparts
        (grouped by source rank)."""
        n_recv = int(sum(recv_splits))
        out = []
        for t in tensors:
            if t is None:
                out.append(None)
                continue
            r = torch.empty((n_recv,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            # byte view: some backends lack the 8-bit float types
            tv = t.view(torch.uint8) if t.element_size() == 1 else t
            rv = r.view(torch.uint8) if r.element_size() == 1 else r
            dist.all_to_all_single(rv, tv, output_split_sizes=recv_splits,
                                   input_split_sizes=send_splits, group=self.group)
            out.append(r)
        return out

    def combine(self, rows, send_splits, recv_splits):
        """The way back: `rows` are in the order they were received; the result is
        in the order this rank sent its rows."""
        back, work = self.combine_async(rows, send_splits, recv_splits)
        work.wait()
        return back

    # Asynchronous forms: the collective is queued behind the work already on
    # the current stream and runs beside whatever is queued after it;
    # ``work.wait()`` makes the current stream wait for it (no host block).
    def dispatch_async(self, tensors, send_splits, recv_splits):
        n_recv = int(sum(recv_splits))
        out, works = [], []
        for t in tensors:
            if t is None:
                out.append(None)
                continue
            r = torch.empty((n_recv,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            tv = t.view(torch.uint8) if t.element_size() == 1 else t
            rv = r.view(torch.uint8) if r.element_size() == 1 else r
            works.append(dist.all_to_all_single(rv, tv, output_split_sizes=recv_splits,
                                                input_split_sizes=send_splits, group=self.group,
                                                async_op=True))
            out.append(r)
        return out, works

    def combine_async(self, rows, send_splits, recv_splits, out=None):
        n_send = int(sum(send_splits))
        back = out if out is not None else torch.empty((n_send,) + tuple(rows.shape[1:]), dtype=rows.dtype,
                                                       device=rows.device)
        work = dist.all_to_all_single(back, rows, output_split_sizes=send_splits,
                                      input_split_sizes=recv_splits, group=self.group, async_op=True)
        return back, work


def owner_map(num_experts_total: int, ep_size: int, device) -> torch.Tensor:
    """int32 [E_total]: the rank that owns each expert (contiguous even split)."""
    e_local = num_experts_total // ep_size
    return (torch.arange(num_experts_total, device=device) // e_local).to(torch.int32)


def group_bucket_map(num_experts_total: int, ep_size: int, groups: int, device) -> torch.Tensor:
    """int32 [E_total]: bucket ``g * ep_size + rank`` of each expert, where ``rank`` owns the
    expert and ``g`` is the group of the expert among its rank's experts (contiguous, as even as
    possible).  Sorting routed rows by this bucket puts, for every group, the rows of all ranks
    side by side: one contiguous slice of the send buffer per group, split by rank inside."""
    e_local = num_experts_total // ep_size
    e = torch.arange(num_experts_total, device=device)
    rank = e // e_local
    g = (e % e_local) * groups // e_local
    return (g * ep_size + rank).to(torch.int32)


class EpFusedMoe:
    """Fused-MoE layer with all-to-all expert parallelism (CUDA).

    ``w13`` / ``w2`` (and scales, biases) hold this rank's ``num_local_experts``
    experts in the layouts ``XpuFusedMoe`` takes.  ``apply`` has the signature
    of ``XpuFusedMoe.apply`` with *global* expert ids in ``topk_ids``.
    """

    def __init__(self, w13, w13_scales, w13_bias, w2, w2_scales, w2_bias,
                 n_experts_per_token, activation, num_local_experts,
                 group: Optional[dist.ProcessGroup] = None,
                 gemm1_clamp_limit: Optional[float] = None,
                 overlap_chunks: Optional[int] = None, sm_reserve: int = 20,
                 expert_groups: Optional[int] = None, sorted_exchange: bool = False,
                 per_rank_rows: bool = True):
        from .fused_moe_interface import XpuFusedMoe
        self.a2a = EpAllToAll(group)
        self.ep_size, self.ep_rank = self.a2a.ep_size, self.a2a.ep_rank
        self.num_local_experts = num_local_experts
        self.num_experts_total = num_local_experts * self.ep_size
        self.topk = n_experts_per_token
        # every received row is one routed slot of one local expert: top-1 locally
        self.local = XpuFusedMoe(w13, w13_scales, w13_bias, w2, w2_scales, w2_bias, 1, activation,
                                 num_local_experts, gemm1_clamp_limit=gemm1_clamp_limit)
        self.owner = owner_map(self.num_experts_total, self.ep_size, w13.device)
        self.quant = self.local.is_block_fp8
        # Default schedule (`per_rank_rows`): a token's row travels once to every rank that owns
        # at least one of its experts, with the token's local expert ids and routing weights; the
        # owner runs its experts as a top-k layer on the received tokens (slots of other ranks
        # are id -1 and skipped) and returns one partial sum per (token, rank), which the source
        # adds up.  Against one row per (token, expert) this divides both exchanges by the mean
        # number of experts a token has on one rank (DeepSeek-V3 routing: 4 at 2 ranks, 2 at 8).
        # Each partial sum is rounded to the output type before the final addition, as in the
        # reference's own scheme (partial outputs all-reduced by the caller).
        self.per_rank_rows = bool(per_rank_rows) and not sorted_exchange and not (
            expert_groups is not None and expert_groups > 1) and overlap_chunks is None
        if self.per_rank_rows:
            self.local_topk = XpuFusedMoe(w13, w13_scales, w13_bias, w2, w2_scales, w2_bias,
                                          n_experts_per_token, activation, num_local_experts,
                                          gemm1_clamp_limit=gemm1_clamp_limit)
        # Optional: cut the batch into `overlap_chunks` token chunks so that the
        # exchange of one chunk runs beside the experts of another (the persistent
        # GEMM kernels then leave `sm_reserve` SMs to the collective's kernels).
        # Off by default: every chunk streams the local experts' weights again,
        # which on B200 cost more than the overlap saved (DeepSeek-V3 shape,
        # 8192 tokens per GPU, 2 GPUs: 12.0 ms unchunked, 13.7 ms with 2 chunks,
        # 15.2 ms with 4).
        self.overlap_chunks = overlap_chunks
        self.sm_reserve = sm_reserve
        # Optional: split the local experts into `expert_groups` contiguous groups and run the
        # exchange group by group, so that the rows of group g+1 arrive and the results of group
        # g-1 leave while group g's experts compute.  Unlike token chunks this streams every
        # weight once: a group's GEMMs touch only that group's experts.
        # Optional (`sorted_exchange`): the sender sorts its routed rows by (group, destination
        # rank, expert) and ships the per-expert counts along, so the rows arrive grouped by source
        # rank and by expert inside a source.  The grouped GEMMs take those segments as they are
        # (segment s -> expert s % experts, `XpuFusedMoe.apply_sorted`): the receiver neither permutes
        # the rows again nor un-permutes the result, and no expert ids travel.  Every source's
        # segments walk the weights once more, which costs nothing while a segment has enough
        # rows to be compute-bound: for prefill-sized batches.  Must be set alike on all ranks.
        self.sorted_exchange = bool(sorted_exchange)
        if self.sorted_exchange:
            G = expert_groups if (expert_groups is not None and expert_groups > 1) else 1
            while num_local_experts % G:
                G -= 1
            self.sorted_groups = G
            eg = num_local_experts // G
            e = torch.arange(self.num_experts_total, device=w13.device)
            rank, le = e // num_local_experts, e % num_local_experts
            # bucket order: group-major, then destination rank, then expert inside the group
            self.sorted_bucket = ((le // eg) * (self.ep_size * eg) + rank * eg + le % eg).to(torch.int32)
            sl = lambda t, g: t[g * eg:(g + 1) * eg] if t is not None else None
            self.group_layers = [XpuFusedMoe(sl(w13, g), sl(w13_scales, g), sl(w13_bias, g), sl(w2, g),
                                             sl(w2_scales, g), sl(w2_bias, g), 1, activation, eg,
                                             gemm1_clamp_limit=gemm1_clamp_limit) for g in range(G)]
            expert_groups = None
        self.expert_groups = None
        if expert_groups is not None and expert_groups > 1:
            self.expert_groups = min(expert_groups, num_local_experts)
            self.group_bucket = group_bucket_map(self.num_experts_total, self.ep_size, self.expert_groups,
                                                 w13.device)
        self._sm_count = torch.cuda.get_device_properties(w13.device).multi_processor_count

    def _num_chunks(self, T):
        if self.overlap_chunks is None:
            return 1
        return max(1, min(self.overlap_chunks, T))

    def apply(self, output, hidden_states, topk_weights, topk_ids):
        if self.sorted_exchange:
            return self._apply_sorted(output, hidden_states, topk_weights, topk_ids)
        if self.expert_groups is not None:
            return self._apply_grouped(output, hidden_states, topk_weights, topk_ids)
        if self.per_rank_rows and self._num_chunks(hidden_states.shape[0]) == 1:
            return self._apply_per_rank(output, hidden_states, topk_weights, topk_ids)
        nc = self._num_chunks(hidden_states.shape[0])
        if nc > 1:
            return self._apply_chunked(output, hidden_states, topk_weights, topk_ids, nc)
        T, H = hidden_states.shape
        K = self.topk
        dev = hidden_states.device
        ep = self.ep_size
        M = T * K
        ops = torch.ops._moe_C

        # 1. group this rank's routed rows by destination rank (stable), quantising
        #    them on the way when the experts take fp8 activations
        send_counts = torch.empty((ep,), dtype=torch.int32, device=dev)
        send_pos = torch.empty((T, K), dtype=torch.int32, device=dev)
        if self.quant:
            send_rows = torch.empty((M, H), dtype=torch.float8_e4m3fn, device=dev)
            send_scales = torch.empty((M, H // FP8_BLOCK), dtype=torch.float32, device=dev)
            ops.b200_remap_quant_fp8(hidden_states, send_rows, send_scales, self.owner, send_counts,
                                     send_pos, topk_ids, self.num_experts_total, ep)
        else:
            send_rows = torch.empty((M, H), dtype=hidden_states.dtype, device=dev)
            send_scales = None
            ops.remap_hidden_states(hidden_states, None, send_rows, None, self.owner, send_counts,
                                    send_pos, topk_ids, self.num_experts_total, ep)
        send_eids = torch.empty((M,), dtype=torch.int32, device=dev)
        send_eids[send_pos.reshape(-1).long()] = (topk_ids.reshape(-1) % self.num_local_experts).to(torch.int32)

        # 2. exchange
        send_splits, recv_splits = self.a2a.exchange_counts(send_counts)
        recv_rows, recv_scales, recv_eids = self.a2a.dispatch((send_rows, send_scales, send_eids),
                                                              send_splits, recv_splits)

        # 3. local experts on the received rows (top-1, unit weight), result in
        #    the received order
        R = recv_rows.shape[0]
        local_out = torch.empty((R, H), dtype=output.dtype, device=dev)
        if R > 0:
            ones = torch.ones((R, 1), dtype=torch.float32, device=dev)
            self.local.apply(local_out, recv_rows, ones, recv_eids.view(R, 1),
                             a1q_scale=recv_scales if self.quant else None)

        # 4. rows travel back; weighted top-k reduction on the source rank
        back = self.a2a.combine(local_out, send_splits, recv_splits)
        ops.moe_gather(output, back, topk_weights, send_pos, self.num_experts_total)

    def _permute_for_send(self, hidden_states, topk_ids):
        """Groups one token range's routed rows by destination rank."""
        T, H = hidden_states.shape
        K, ep, dev = self.topk, self.ep_size, hidden_states.device
        M = T * K
        ops = torch.ops._moe_C
        send_counts = torch.empty((ep,), dtype=torch.int32, device=dev)
        send_pos = torch.empty((T, K), dtype=torch.int32, device=dev)
        if self.quant:
            send_rows = torch.empty((M, H), dtype=torch.float8_e4m3fn, device=dev)
            send_scales = torch.empty((M, H // FP8_BLOCK), dtype=torch.float32, device=dev)
            ops.b200_remap_quant_fp8(hidden_states, send_rows, send_scales, self.owner, send_counts,
                                     send_pos, topk_ids, self.num_experts_total, ep)
        else:
            send_rows = torch.empty((M, H), dtype=hidden_states.dtype, device=dev)
            send_scales = None
            ops.remap_hidden_states(hidden_states, None, send_rows, None, self.owner, send_counts,
                                    send_pos, topk_ids, self.num_experts_total, ep)
        send_eids = torch.empty((M,), dtype=torch.int32, device=dev)
        send_eids[send_pos.reshape(-1).long()] = (topk_ids.reshape(-1) % self.num_local_experts).to(torch.int32)
        return send_rows, send_scales, send_eids, send_counts, send_pos

    def _apply_chunked(self, output, hidden_states, topk_weights, topk_ids, nc):
        T, H = hidden_states.shape
        dev = hidden_states.device
        ep = self.ep_size
        bounds = [(T * c) // nc for c in range(nc + 1)]
        # phase 1: permute every chunk, exchange all counts, read them back once
        prep = []
        for c in range(nc):
            t0, t1 = bounds[c], bounds[c + 1]
            prep.append(self._permute_for_send(hidden_states[t0:t1], topk_ids[t0:t1]))
        counts = torch.stack([p[3] for p in prep], dim=1).contiguous()       # [ep, nc]
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=self.a2a.group)     # [ep(src), nc]
        both = torch.stack((counts, recv_counts)).cpu()
        send_spl = [both[0][:, c].tolist() for c in range(nc)]
        recv_spl = [both[1][:, c].tolist() for c in range(nc)]

        # phase 2: dispatch(c+1) and combine(c-1) run beside the experts of chunk c
        self.local.gemm_max_ctas = max(1, self._sm_count - self.sm_reserve)
        try:
            inflight = [None] * nc
            inflight[0] = self.a2a.dispatch_async(prep[0][:3], send_spl[0], recv_spl[0])
            pending = None  # (chunk, back rows, work) of the previous chunk's combine
            keep = []

            def finish(c, back, work):
                work.wait()
                t0, t1 = bounds[c], bounds[c + 1]
                torch.ops._moe_C.moe_gather(output[t0:t1], back, topk_weights[t0:t1], prep[c][4],
                                            self.num_experts_total)

            for c in range(nc):
                if c + 1 < nc:
                    inflight[c + 1] = self.a2a.dispatch_async(prep[c + 1][:3], send_spl[c + 1], recv_spl[c + 1])
                (recv_rows, recv_scales, recv_eids), works = inflight[c]
                for w in works:
                    w.wait()
                R = recv_rows.shape[0]
                local_out = torch.empty((R, H), dtype=output.dtype, device=dev)
                if R > 0:
                    ones = torch.ones((R, 1), dtype=torch.float32, device=dev)
                    self.local.apply(local_out, recv_rows, ones, recv_eids.view(R, 1),
                                     a1q_scale=recv_scales if self.quant else None)
                back, work = self.a2a.combine_async(local_out, send_spl[c], recv_spl[c])
                keep.append((recv_rows, recv_scales, recv_eids, local_out, back))
                if pending is not None:
                    finish(*pending)
                pending = (c, back, work)
            finish(*pending)
        finally:
            self.local.gemm_max_ctas = 0

    def _apply_grouped(self, output, hidden_states, topk_weights, topk_ids):
        T, H = hidden_states.shape
        K, ep, G, dev = self.topk, self.ep_size, self.expert_groups, hidden_states.device
        M = T * K
        ops = torch.ops._moe_C
        # 1. one stable sort of the routed rows by (group, destination rank)
        counts = torch.empty((G * ep,), dtype=torch.int32, device=dev)
        send_pos = torch.empty((T, K), dtype=torch.int32, device=dev)
        if self.quant:
            send_rows = torch.empty((M, H), dtype=torch.float8_e4m3fn, device=dev)
            send_scales = torch.empty((M, H // FP8_BLOCK), dtype=torch.float32, device=dev)
            ops.b200_remap_quant_fp8(hidden_states, send_rows, send_scales, self.group_bucket, counts,
                                     send_pos, topk_ids, self.num_experts_total, G * ep)
        else:
            send_rows = torch.empty((M, H), dtype=hidden_states.dtype, device=dev)
            send_scales = None
            ops.remap_hidden_states(hidden_states, None, send_rows, None, self.group_bucket, counts,
                                    send_pos, topk_ids, self.num_experts_total, G * ep)
        send_eids = torch.empty((M,), dtype=torch.int32, device=dev)
        send_eids[send_pos.reshape(-1).long()] = (topk_ids.reshape(-1) % self.num_local_experts).to(torch.int32)

        # 2. all counts in one exchange, read back once: [ep (peer), G]
        by_peer = counts.view(G, ep).t().contiguous()
        recv_counts = torch.empty_like(by_peer)
        dist.all_to_all_single(recv_counts, by_peer, group=self.a2a.group)
        both = torch.stack((by_peer, recv_counts)).cpu()
        send_spl = [both[0][:, g].tolist() for g in range(G)]
        recv_spl = [both[1][:, g].tolist() for g in range(G)]
        starts = [0]
        for g in range(G):
            starts.append(starts[-1] + int(sum(send_spl[g])))

        def chunk(g):
            a, b = starts[g], starts[g + 1]
            return (send_rows[a:b], send_scales[a:b] if send_scales is not None else None, send_eids[a:b])

        # 3. dispatch(g+1) and combine(g-1) run beside the experts of group g
        back_all = torch.empty((M, H), dtype=output.dtype, device=dev)
        self.local.gemm_max_ctas = max(1, self._sm_count - self.sm_reserve)
        try:
            inflight = [None] * G
            inflight[0] = self.a2a.dispatch_async(chunk(0), send_spl[0], recv_spl[0])
            works, keep = [], []
            for g in range(G):
                if g + 1 < G:
                    inflight[g + 1] = self.a2a.dispatch_async(chunk(g + 1), send_spl[g + 1], recv_spl[g + 1])
                (recv_rows, recv_scales, recv_eids), ws = inflight[g]
                for w in ws:
                    w.wait()
                R = recv_rows.shape[0]
                local_out = torch.empty((R, H), dtype=output.dtype, device=dev)
                if R > 0:
                    ones = torch.ones((R, 1), dtype=torch.float32, device=dev)
                    self.local.apply(local_out, recv_rows, ones, recv_eids.view(R, 1),
                                     a1q_scale=recv_scales if self.quant else None)
                _, work = self.a2a.combine_async(local_out, send_spl[g], recv_spl[g],
                                                 out=back_all[starts[g]:starts[g + 1]])
                works.append(work)
                keep.append((recv_rows, recv_scales, recv_eids, local_out))
            for w in works:
                w.wait()
        finally:
            self.local.gemm_max_ctas = 0
        # 4. weighted top-k reduction on the source rank
        ops.moe_gather(output, back_all, topk_weights, send_pos, self.num_experts_total)

    def _apply_sorted(self, output, hidden_states, topk_weights, topk_ids):
        T, H = hidden_states.shape
        K, ep, G, dev = self.topk, self.ep_size, self.sorted_groups, hidden_states.device
        E_t = self.num_experts_total
        eg = self.num_local_experts // G
        M = T * K
        ops = torch.ops._moe_C
        # 1. one stable sort of the routed rows by (group, destination rank, expert)
        counts = torch.empty((E_t,), dtype=torch.int32, device=dev)
        send_pos = torch.empty((T, K), dtype=torch.int32, device=dev)
        if self.quant:
            send_rows = torch.empty((M, H), dtype=torch.float8_e4m3fn, device=dev)
            send_scales = torch.empty((M, H // FP8_BLOCK), dtype=torch.float32, device=dev)
            ops.b200_remap_quant_fp8(hidden_states, send_rows, send_scales, self.sorted_bucket, counts,
                                     send_pos, topk_ids, E_t, E_t)
        else:
            send_rows = torch.empty((M, H), dtype=hidden_states.dtype, device=dev)
            send_scales = None
            ops.remap_hidden_states(hidden_states, None, send_rows, None, self.sorted_bucket, counts,
                                    send_pos, topk_ids, E_t, E_t)
        # 2. per-expert counts to their owners: [ep (peer), G, eg]; split sizes read back once
        by_peer = counts.view(G, ep, eg).permute(1, 0, 2).contiguous()
        recv_seg = torch.empty_like(by_peer)                       # [ep (source), G, eg]
        dist.all_to_all_single(recv_seg, by_peer, group=self.a2a.group)
        both = torch.stack((by_peer.sum(dim=2), recv_seg.sum(dim=2))).cpu()     # [2, ep, G]
        send_spl = [both[0][:, g].tolist() for g in range(G)]
        recv_spl = [both[1][:, g].tolist() for g in range(G)]
        starts = [0]
        for g in range(G):
            starts.append(starts[-1] + int(sum(send_spl[g])))

        def chunk(g):
            a, b = starts[g], starts[g + 1]
            return (send_rows[a:b], send_scales[a:b] if send_scales is not None else None)

        # 3. dispatch(g+1) and combine(g-1) run beside the experts of group g
        back_all = torch.empty((M, H), dtype=output.dtype, device=dev)
        cap = max(1, self._sm_count - self.sm_reserve) if G > 1 else 0
        inflight = [None] * G
        inflight[0] = self.a2a.dispatch_async(chunk(0), send_spl[0], recv_spl[0])
        works, keep = [], []
        for g in range(G):
            if g + 1 < G:
                inflight[g + 1] = self.a2a.dispatch_async(chunk(g + 1), send_spl[g + 1], recv_spl[g + 1])
            (recv_rows, recv_scales), ws = inflight[g]
            for w in ws:
                w.wait()
            R = recv_rows.shape[0]
            local_out = torch.empty((R, H), dtype=output.dtype, device=dev)
            layer = self.group_layers[g]
            layer.gemm_max_ctas = cap
            layer.apply_sorted(local_out, recv_rows, recv_seg[:, g, :].reshape(-1),
                               a1q_scale=recv_scales if self.quant else None)
            _, work = self.a2a.combine_async(local_out, send_spl[g], recv_spl[g],
                                             out=back_all[starts[g]:starts[g + 1]])
            works.append(work)
            keep.append((recv_rows, recv_scales, local_out))
        for w in works:
            w.wait()
        # 4. weighted top-k reduction on the source rank
        ops.moe_gather(output, back_all, topk_weights, send_pos, E_t)

    def _apply_per_rank(self, output, hidden_states, topk_weights, topk_ids):
        T, H = hidden_states.shape
        K, ep, dev = self.topk, self.ep_size, hidden_states.device
        E_l = self.num_local_experts
        ops = torch.ops._moe_C
        cap = T * ep                                                   # slots (token, rank)

        # 1. which ranks a token needs, and what each of them has to know about it
        ids = topk_ids.to(torch.int64)
        dest = ids // E_l                                              # [T, K]
        ranks = torch.arange(ep, device=dev)
        hit = dest.unsqueeze(1) == ranks.view(1, ep, 1)                # [T, ep, K]
        rank_ids = torch.where(hit.any(dim=2), ranks.view(1, ep), -1).to(torch.int32).contiguous()
        loc_ids = torch.where(hit, (ids % E_l).unsqueeze(1), -1).to(torch.int32)
        loc_w = torch.where(hit, topk_weights.unsqueeze(1), 0.0).to(torch.float32)

        # 2. token rows grouped by destination rank (stable), quantised on the way for fp8 experts;
        #    slots of ranks a token does not need carry id -1 and are dropped
        send_counts = torch.empty((ep,), dtype=torch.int32, device=dev)
        send_pos = torch.empty((T, ep), dtype=torch.int32, device=dev)
        if self.quant:
            send_rows = torch.empty((cap, H), dtype=torch.float8_e4m3fn, device=dev)
            send_scales = torch.empty((cap, H // FP8_BLOCK), dtype=torch.float32, device=dev)
            ops.b200_remap_quant_fp8(hidden_states, send_rows, send_scales, None, send_counts, send_pos,
                                     rank_ids, ep, ep)
        else:
            send_rows = torch.empty((cap, H), dtype=hidden_states.dtype, device=dev)
            send_scales = None
            ops.remap_hidden_states(hidden_states, None, send_rows, None, None, send_counts, send_pos,
                                    rank_ids, ep, ep)
        pos = send_pos.reshape(-1).long()
        pos = torch.where(pos >= 0, pos, cap)                          # dropped slots -> spare row
        send_ids = torch.empty((cap + 1, K), dtype=torch.int32, device=dev)
        send_w = torch.empty((cap + 1, K), dtype=torch.float32, device=dev)
        send_ids.index_copy_(0, pos, loc_ids.reshape(cap, K))
        send_w.index_copy_(0, pos, loc_w.reshape(cap, K))

        # 3. exchange
        send_splits, recv_splits = self.a2a.exchange_counts(send_counts)
        n = int(sum(send_splits))
        recv_rows, recv_scales, recv_ids, recv_w = self.a2a.dispatch(
            (send_rows[:n], send_scales[:n] if send_scales is not None else None, send_ids[:n], send_w[:n]),
            send_splits, recv_splits)

        # 4. this rank's experts on the received tokens: top-k layer, foreign slots skipped
        R = recv_rows.shape[0]
        local_out = torch.empty((R, H), dtype=output.dtype, device=dev)
        if R > 0:
            self.local_topk.apply(local_out, recv_rows, recv_w, recv_ids,
                                  a1q_scale=recv_scales if self.quant else None)

        # 5. partial sums travel back; the source adds the (at most ep) partial sums of a token
        back = self.a2a.combine(local_out, send_splits, recv_splits)
        ones = torch.ones((T, ep), dtype=torch.float32, device=dev)
        ops.moe_gather(output, back, ones, send_pos, ep)
