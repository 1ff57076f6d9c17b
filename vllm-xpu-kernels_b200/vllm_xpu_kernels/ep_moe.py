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
        n_send = int(sum(send_splits))
        back = torch.empty((n_send,) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
        dist.all_to_all_single(back, rows, output_split_sizes=send_splits,
                               input_split_sizes=recv_splits, group=self.group)
        return back


def owner_map(num_experts_total: int, ep_size: int, device) -> torch.Tensor:
    """int32 [E_total]: the rank that owns each expert (contiguous even split)."""
    e_local = num_experts_total // ep_size
    return (torch.arange(num_experts_total, device=device) // e_local).to(torch.int32)


class EpFusedMoe:
    """Fused-MoE layer with all-to-all expert parallelism (CUDA).

    ``w13`` / ``w2`` (and scales, biases) hold this rank's ``num_local_experts``
    experts in the layouts ``XpuFusedMoe`` takes.  ``apply`` has the signature
    of ``XpuFusedMoe.apply`` with *global* expert ids in ``topk_ids``.
    """

    def __init__(self, w13, w13_scales, w13_bias, w2, w2_scales, w2_bias,
                 n_experts_per_token, activation, num_local_experts,
                 group: Optional[dist.ProcessGroup] = None,
                 gemm1_clamp_limit: Optional[float] = None):
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

    def apply(self, output, hidden_states, topk_weights, topk_ids):
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
