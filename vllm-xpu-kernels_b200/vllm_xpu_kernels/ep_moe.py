# SPDX-License-Identifier: Apache-2.0
"""Expert parallelism with token dispatch / combine, one process per GPU.

The reference has no communication layer: its expert parallelism is a per-rank
``expert_map`` mask (``vllm_xpu_kernels/fused_moe_interface.py:256-271``,
``csrc/moe/init_expert_map.cpp:33-53``) that leaves every rank with the full
token batch and a partial sum for the caller to all-reduce.  ``XpuFusedMoe``
keeps that semantic untouched.  This module adds the other scheme on top of the
same kernels: experts are split contiguously and evenly over the ranks (expert
``g`` lives on rank ``g // E_local``, as ``init_expert_map`` encodes it), every
rank routes its own tokens, each token's row travels once to every rank that
owns at least one of its experts, the owner runs its experts on the received
tokens as a top-k layer and returns one partial sum per (token, rank), and the
source rank adds the partial sums.

Two transports:

* ``EpPeerFusedMoe`` (the one to use on NVLink-connected GPUs): the dispatch and
  combine kernels store rows straight into the peers' receive buffers
  (symmetric memory) with ordinary global stores; the phases are ordered by two
  small barriers per call; nothing is read back to the host.
* ``EpFusedMoe``: the same schedule over ``torch.distributed.all_to_all_single``
  (NCCL on GPUs, Gloo on CPU tensors in the tests).  It needs the exact split
  sizes on the host, so it reads the counts back once per call.
"""
import os
from typing import Optional

import torch
import torch.distributed as dist

FP8_BLOCK = 128


# --------------------------------------------------------------------------- helpers
def owner_map(num_experts_total: int, ep_size: int, device) -> torch.Tensor:
    """int32 [E_total]: the rank that owns each expert (contiguous even split)."""
    e_local = num_experts_total // ep_size
    return (torch.arange(num_experts_total, device=device) // e_local).to(torch.int32)


def balanced_expert_slots(expert_load, ep_size: int, tolerance: float = 1.02) -> torch.Tensor:
    """An expert placement that evens out the ranks' load: int32 [E] (CPU), a permutation
    ``expert -> slot`` in which rank ``r`` holds the experts of slots ``[r * E_local, (r + 1) *
    E_local)``.  ``expert_load`` [E] is a load estimate per expert (e.g. the routed-slot histogram
    of a calibration batch).

    Starts from the contiguous split and swaps one expert of the busiest rank with one of the
    idlest until the busiest rank is within ``tolerance`` of the mean: few experts move, so a
    router that picks a token's experts from a few groups of neighbouring experts still finds
    most of them on one rank and a token's row travels to few ranks.  If swapping stalls above the
    tolerance, the result of a longest-processing-time greedy (experts in descending load, each to
    the least loaded rank with a free slot) is returned when it is better balanced."""
    load = torch.as_tensor(expert_load, dtype=torch.float64).cpu()
    E = load.numel()
    if E % ep_size:
        raise ValueError("the expert count must be divisible by the expert-parallel size")
    e_local = E // ep_size

    def imbalance(slot):
        per_rank = torch.zeros(ep_size, dtype=torch.float64).index_add_(0, slot.long() // e_local, load)
        return float(per_rank.max() / per_rank.mean().clamp(min=1e-30))

    # (a) swaps from the contiguous split
    slot = torch.arange(E, dtype=torch.int64)
    for _ in range(4 * E):
        owner = slot // e_local
        per_rank = torch.zeros(ep_size, dtype=torch.float64).index_add_(0, owner, load)
        hi, lo = int(per_rank.argmax()), int(per_rank.argmin())
        if per_rank[hi] <= tolerance * per_rank.mean():
            break
        gap = (per_rank[hi] - per_rank[lo]) / 2
        e_hi, e_lo = (owner == hi).nonzero().flatten(), (owner == lo).nonzero().flatten()
        moved = load[e_hi].unsqueeze(1) - load[e_lo].unsqueeze(0)      # load a swap takes from hi to lo
        score = torch.where((moved > 0) & (moved < 2 * gap), (moved - gap).abs(),
                            torch.full_like(moved, float("inf")))
        if not bool(torch.isfinite(score.min())):
            break
        i, j = divmod(int(score.argmin()), score.shape[1])
        a, b = int(e_hi[i]), int(e_lo[j])
        slot[a], slot[b] = slot[b].clone(), slot[a].clone()
    swapped = slot.to(torch.int32)
    if imbalance(swapped) <= tolerance:
        return swapped

    # (b) longest-processing-time greedy
    rank_load, rank_fill = [0.0] * ep_size, [0] * ep_size
    greedy = torch.empty(E, dtype=torch.int32)
    for e in torch.argsort(load, descending=True, stable=True).tolist():
        r = min((r for r in range(ep_size) if rank_fill[r] < e_local), key=lambda r: (rank_load[r], r))
        greedy[e] = r * e_local + rank_fill[r]
        rank_fill[r] += 1
        rank_load[r] += float(load[e])
    return greedy if imbalance(greedy) < imbalance(swapped) else swapped


def experts_in_slots(expert_slot: torch.Tensor, rank: int, num_local_experts: int) -> torch.Tensor:
    """int64 [E_local]: the global expert held in each local slot of ``rank`` (the order in which
    that rank's weights are stacked) for a placement ``expert -> slot``."""
    inverse = torch.empty_like(expert_slot, dtype=torch.int64)
    inverse[expert_slot.long()] = torch.arange(expert_slot.numel(), dtype=torch.int64)
    return inverse[rank * num_local_experts:(rank + 1) * num_local_experts]


def check_count_matrix(sent: torch.Tensor, received: torch.Tensor, rank: int, capacity: Optional[int] = None):
    """Consistency of one exchange: ``sent`` [ep, ep] holds what every rank says it sent to
    every rank (row = source), ``received`` [ep] what this rank was told it received from
    every source.  Raises ``RuntimeError`` naming the first source whose announced count
    differs - a lost or short message - or exceeds the receive capacity."""
    sent, received = sent.cpu().long(), received.cpu().long()
    col = sent[:, rank]
    for s in range(sent.shape[0]):
        if int(col[s]) != int(received[s]):
            raise RuntimeError(f"expert-parallel exchange: rank {s} sent {int(col[s])} rows to rank {rank}, "
                               f"which was told to expect {int(received[s])}")
        if capacity is not None and not 0 <= int(col[s]) <= capacity:
            raise RuntimeError(f"expert-parallel exchange: {int(col[s])} rows from rank {s} exceed the "
                               f"capacity {capacity} of rank {rank}'s receive region")


# --------------------------------------------------------------------------- peer memory
class SymmetricPeerGroup:
    """Peer-addressable buffers through ``torch.distributed._symmetric_memory`` and a
    stream-ordered barrier (a one-element all-reduce on the current stream: the peers' earlier
    kernels, and with them their stores into this rank's buffers, have finished when it
    completes).  ``alloc`` is collective: every rank calls it in the same order."""

    def __init__(self, device, group: Optional[dist.ProcessGroup] = None):
        # NVLink multicast objects are not needed for plain peer stores; leaving memory unbound
        # keeps a rank that dies from disturbing its peers' GPUs.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group if group is not None else dist.group.WORLD
        self.ep_size = dist.get_world_size(self.group)
        self.ep_rank = dist.get_rank(self.group)
        self.device = torch.device(device)
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._handles = []

    def alloc(self, nbytes: int):
        import torch.distributed._symmetric_memory as symm
        block = symm.empty(int(nbytes), dtype=torch.uint8, device=self.device)
        handle = symm.rendezvous(block, self.group)
        self._handles.append(handle)
        return block, [int(p) for p in handle.buffer_ptrs]

    def addresses(self, token):
        return token

    def barrier(self):
        dist.all_reduce(self._token, group=self.group)


class LocalPeerWorld:
    """All ranks of an expert-parallel group inside ONE process on one GPU: every rank's
    buffers are ordinary allocations of that GPU and a "peer store" is a local store.  The
    phases of all ranks are run one after the other on one stream, which is all the ordering
    the protocol needs - so the dispatch, mask, combine and gather kernels, their index
    arithmetic and the pointer tables can be checked where only one GPU is available."""

    def __init__(self, ep_size: int, device):
        self.ep_size, self.device = ep_size, torch.device(device)
        self.blocks = [[] for _ in range(ep_size)]

    def member(self, rank: int):
        return _LocalPeerGroup(self, rank)


class _LocalPeerGroup:
    def __init__(self, world: LocalPeerWorld, rank: int):
        self.world, self.ep_rank, self.ep_size, self.device = world, rank, world.ep_size, world.device

    def alloc(self, nbytes: int):
        block = torch.empty(int(nbytes), dtype=torch.uint8, device=self.device)
        index = len(self.world.blocks[self.ep_rank])
        self.world.blocks[self.ep_rank].append(block)
        return block, index

    def addresses(self, token):
        blocks = self.world.blocks
        if any(len(b) <= token for b in blocks):
            raise RuntimeError("LocalPeerWorld: construct the layers of all ranks before the first call")
        return [int(b[token].data_ptr()) for b in blocks]

    def barrier(self):
        pass  # one stream: launch order is the order


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class EpPeerFusedMoe:
    """Fused-MoE layer with expert parallelism over peer memory (CUDA).

    ``w13`` / ``w2`` (and scales, biases) hold this rank's ``num_local_experts`` experts in
    the layouts ``XpuFusedMoe`` takes.  Expert ``g`` is local expert ``g % E_local`` of rank
    ``g // E_local``, or - with ``expert_slot`` (int32 [E] on the device, the same permutation
    ``expert -> slot`` on every rank, e.g. from ``balanced_expert_slots``) - local expert
    ``slot % E_local`` of rank ``slot // E_local``.  ``apply`` has the signature of ``XpuFusedMoe.apply``
    with *global* expert ids in ``topk_ids``; all ranks call it together.  ``max_tokens`` is
    the largest token count any rank passes to one call (the receive regions are sized for
    it); ``peers`` provides the peer-addressable memory and the barrier
    (``SymmetricPeerGroup``, or a member of ``LocalPeerWorld`` in single-GPU tests).

    One call = three phases with a barrier between them:

    1. ``dispatch``: one stable counting sort of the (token, rank) slots, then one kernel that
       reads each token once, quantises it to e4m3 with 1x128 scales when the experts are
       block-scaled fp8, and stores row, scales, local expert ids and routing weights into
       region ``ep_rank`` of every destination rank's receive buffers;
    2. ``experts_and_combine``: the local experts run as a top-k layer over all receive regions
       (rows nobody sent carry id -1); the top-k reduction kernel stores each partial sum into
       region ``ep_rank`` of the source rank's return buffer;
    3. ``finish``: the source adds the partial sums of a token (at most one per rank).

    Each partial sum is rounded to the output type before the last addition, as in the
    reference's own scheme (partial outputs all-reduced by the caller).
    """

    def __init__(self, w13, w13_scales, w13_bias, w2, w2_scales, w2_bias, n_experts_per_token, activation,
                 num_local_experts, peers, max_tokens: int, hidden_size: int,
                 gemm1_clamp_limit: Optional[float] = None, out_dtype=torch.bfloat16,
                 expert_slot: Optional[torch.Tensor] = None):
        from .fused_moe_interface import XpuFusedMoe
        self.peers = peers
        if expert_slot is not None:
            if expert_slot.numel() != num_local_experts * peers.ep_size:
                raise ValueError("expert_slot must have one entry per expert of the whole group")
            expert_slot = expert_slot.to(device=w13.device, dtype=torch.int32).contiguous()
        self.expert_slot = expert_slot
        self.ep_size, self.ep_rank = peers.ep_size, peers.ep_rank
        self.num_local_experts = num_local_experts
        self.topk = n_experts_per_token
        self.hidden = hidden_size
        self.capacity = int(max_tokens)
        self.out_dtype = out_dtype
        self.local = XpuFusedMoe(w13, w13_scales, w13_bias, w2, w2_scales, w2_bias, n_experts_per_token,
                                 activation, num_local_experts, gemm1_clamp_limit=gemm1_clamp_limit)
        self.quant = self.local.is_block_fp8
        dev = w13.device
        ep, cap, K, H = self.ep_size, self.capacity, self.topk, self.hidden
        if self.quant and H % FP8_BLOCK:
            raise ValueError("block-scaled fp8 experts need a hidden size divisible by 128")
        row_bytes = H if self.quant else 2 * H
        sizes = [ep * cap * row_bytes,                                   # recv_rows
                 ep * cap * (H // FP8_BLOCK) * 4 if self.quant else 16,  # recv_scales
                 ep * cap * K * 4,                                       # recv_ids
                 ep * cap * K * 4,                                       # recv_weights
                 ep * 4,                                                 # recv_counts
                 ep * cap * H * 2]                                       # comb_rows
        self._offsets = [0]
        for s in sizes:
            self._offsets.append(self._offsets[-1] + _align(s))
        self._block, self._token = peers.alloc(self._offsets[-1])
        self._block[self._offsets[4]:self._offsets[4] + ep * 4].zero_()
        self._tables = None
        o = self._offsets
        blk = self._block
        row_dtype = torch.float8_e4m3fn if self.quant else out_dtype
        self.recv_rows = blk[o[0]:o[0] + sizes[0]].view(row_dtype).view(ep * cap, H)
        self.recv_scales = (blk[o[1]:o[1] + sizes[1]].view(torch.float32).view(ep * cap, H // FP8_BLOCK)
                            if self.quant else None)
        self.recv_ids = blk[o[2]:o[2] + sizes[2]].view(torch.int32).view(ep * cap, K)
        self.recv_weights = blk[o[3]:o[3] + sizes[3]].view(torch.float32).view(ep * cap, K)
        self.recv_counts = blk[o[4]:o[4] + sizes[4]].view(torch.int32)
        self.comb_rows = blk[o[5]:o[5] + sizes[5]].view(out_dtype).view(ep * cap, H)
        self.send_counts = torch.zeros((ep,), dtype=torch.int32, device=dev)
        self.send_pos = torch.empty((cap, ep), dtype=torch.int32, device=dev)
        self._ones = torch.ones((cap, ep), dtype=torch.float32, device=dev)
        # scratch of the dispatch sort (b200moe_ep_dispatch_workspace_bytes): one histogram cell per
        # rank and 256-slot chunk, then ep + 1 bucket offsets
        chunks = (cap * ep + 255) // 256
        self._workspace = torch.empty((ep * chunks + ep + 1) * 4 + 256, dtype=torch.uint8, device=dev)
        self._tokens = 0
        # optional callable(name) called after every stage (see XpuFusedMoe.stage_hook)
        self.stage_hook = None

    def _mark(self, name):
        if self.stage_hook is not None:
            self.stage_hook(name)

    # ---- plumbing ------------------------------------------------------------------------
    def _peer_tables(self):
        if self._tables is None:
            bases = self.peers.addresses(self._token)
            self._tables = torch.tensor([[b + self._offsets[i] for b in bases] for i in range(6)],
                                        dtype=torch.int64)
        return self._tables

    def _common(self):
        return (self.ep_rank, self.num_local_experts, self.capacity, self.quant)

    # ---- the three phases ------------------------------------------------------------------
    def dispatch(self, hidden_states, topk_weights, topk_ids):
        T = hidden_states.shape[0]
        if T > self.capacity:
            raise ValueError(f"{T} tokens exceed max_tokens={self.capacity} this layer was built for")
        self._tokens = T
        self._mark("routing")
        torch.ops._moe_C.b200_ep_dispatch(hidden_states, topk_ids, topk_weights, self.send_counts,
                                          self.send_pos[:T], self._workspace, self._peer_tables(), *self._common(),
                                          self.expert_slot)
        self._mark("dispatch")

    def experts_and_combine(self):
        ep, cap, K, H = self.ep_size, self.capacity, self.topk, self.hidden
        rank, E_l, _, quant = self._common()
        torch.ops._moe_C.b200_ep_mask_unused(self.recv_ids, self._peer_tables(), rank, E_l, K, H, cap, quant)
        self._mark("mask")
        self.local.stage_hook = (lambda name: self._mark("local_" + name) if name != "routing" else None) \
            if self.stage_hook is not None else None
        # on average a rank receives as many routed slots as it sends
        self.local.rows_hint = max(1, self._tokens * K)
        moe_out, row_map = self.local._apply_kernel(None, self.recv_rows, self.recv_weights, self.recv_ids,
                                                    a1q_scale=self.recv_scales, gather=False,
                                                    out_dtype=self.out_dtype)
        torch.ops._moe_C.b200_ep_combine(moe_out, row_map, self._peer_tables(), rank, E_l, cap, quant)
        self._mark("combine")

    def finish(self, output):
        T = self._tokens
        torch.ops._moe_C.moe_gather(output, self.comb_rows, self._ones[:T], self.send_pos[:T], self.ep_size)
        self._mark("finish")

    def apply(self, output, hidden_states, topk_weights, topk_ids):
        self.dispatch(hidden_states, topk_weights, topk_ids)
        self.peers.barrier()      # every rank's rows have arrived
        self._mark("barrier1")
        self.experts_and_combine()
        self.peers.barrier()      # every rank's partial sums have arrived
        self._mark("barrier2")
        self.finish(output)

    def check_counts(self):
        """Debugging aid (synchronises): gathers every rank's send counts and compares them with
        what this rank was told it received in the last call."""
        ep = self.ep_size
        sent = torch.empty((ep, ep), dtype=torch.int32, device=self.send_counts.device)
        dist.all_gather_into_tensor(sent, self.send_counts, group=getattr(self.peers, "group", None))
        check_count_matrix(sent, self.recv_counts, self.ep_rank, self.capacity)


# --------------------------------------------------------------------------- collective-library transport
class EpAllToAll:
    """Variable-size row exchange between the ranks of one process group."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.ep_size = dist.get_world_size(group)
        self.ep_rank = dist.get_rank(group)

    def exchange_counts(self, send_counts: torch.Tensor, verify: bool = False):
        """send_counts [ep] (rows this rank sends to each peer) ->
        (send_splits, recv_splits) as host lists.  With ``verify`` every rank's counts are
        gathered as well and compared with what arrived (``check_count_matrix``)."""
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        if verify:
            sent = [torch.empty_like(send_counts) for _ in range(self.ep_size)]
            dist.all_gather(sent, send_counts, group=self.group)
            check_count_matrix(torch.stack(sent), recv_counts, self.ep_rank)
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


class EpFusedMoe:
    """The same expert-parallel layer over ``all_to_all_single`` (CUDA; the comparison point
    for ``EpPeerFusedMoe`` and the form that runs wherever a process group exists).

    ``per_rank_rows`` (default): one row per (token, destination rank) as described in the
    module docstring.  ``per_rank_rows=False``: one row per (token, expert), top-1 on the
    owner, weighted reduction on the source - more traffic, fewer small launches.
    ``expert_slot``: a placement ``expert -> slot`` as for ``EpPeerFusedMoe`` (the routed ids are
    relabelled through it before anything else).
    """

    def __init__(self, w13, w13_scales, w13_bias, w2, w2_scales, w2_bias,
                 n_experts_per_token, activation, num_local_experts,
                 group: Optional[dist.ProcessGroup] = None,
                 gemm1_clamp_limit: Optional[float] = None, per_rank_rows: bool = True,
                 expert_slot: Optional[torch.Tensor] = None):
        from .fused_moe_interface import XpuFusedMoe
        self.a2a = EpAllToAll(group)
        if expert_slot is not None:
            if expert_slot.numel() != num_local_experts * self.a2a.ep_size:
                raise ValueError("expert_slot must have one entry per expert of the whole group")
            expert_slot = expert_slot.to(device=w13.device, dtype=torch.int64).contiguous()
        self.expert_slot = expert_slot
        self.ep_size, self.ep_rank = self.a2a.ep_size, self.a2a.ep_rank
        self.num_local_experts = num_local_experts
        self.num_experts_total = num_local_experts * self.ep_size
        self.topk = n_experts_per_token
        self.per_rank_rows = bool(per_rank_rows)
        self.local = XpuFusedMoe(w13, w13_scales, w13_bias, w2, w2_scales, w2_bias,
                                 n_experts_per_token if self.per_rank_rows else 1, activation,
                                 num_local_experts, gemm1_clamp_limit=gemm1_clamp_limit)
        self.owner = owner_map(self.num_experts_total, self.ep_size, w13.device)
        self.quant = self.local.is_block_fp8

    def apply(self, output, hidden_states, topk_weights, topk_ids):
        if self.expert_slot is not None:
            ids = topk_ids.long()
            topk_ids = torch.where(ids >= 0, self.expert_slot[ids.clamp(min=0)], ids).to(topk_ids.dtype)
        if self.per_rank_rows:
            return self._apply_per_rank(output, hidden_states, topk_weights, topk_ids)
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
            self.local.apply(local_out, recv_rows, recv_w, recv_ids,
                             a1q_scale=recv_scales if self.quant else None)

        # 5. partial sums travel back; the source adds the (at most ep) partial sums of a token
        back = self.a2a.combine(local_out, send_splits, recv_splits)
        ones = torch.ones((T, ep), dtype=torch.float32, device=dev)
        ops.moe_gather(output, back, ones, send_pos, ep)
