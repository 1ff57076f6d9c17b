"""Worker bodies of the multi-rank expert-parallel tests (spawned processes)."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "vllm-xpu-kernels_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def _case(rank, T, cfg_name, dims, seed):
    from oracle import workloads as wl
    cfg = wl.scaled(wl.CONFIGS[cfg_name], **dims)
    w = wl.make_weights(cfg, seed=seed)                     # all experts, same on every rank
    x, logits, bias = wl.make_inputs(cfg, T, seed=seed * 10 + rank)   # this rank's own tokens
    tw, ids = wl.route_cpu(cfg, logits, bias)
    return cfg, w, x, tw, ids


def _oracle_full(cfg, w, x, tw, ids):
    from oracle import torch_oracle as to
    from oracle import workloads as wl
    d13, d2 = wl.dequant_weights(cfg, w)
    return to.fused_moe_staged(x, d13, w["w13_bias"], d2, w["w2_bias"], tw, ids, cfg.E,
                               activation=cfg.activation, act_quant=cfg.recipe == "fp8block")


def cpu_worker(rank, world, port, T, result_queue):
    """Gloo ranks on CPU: the exchange plumbing (EpAllToAll) around the oracle's
    permutation and experts must reproduce the single-process oracle."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import torch_oracle as to
        from oracle import workloads as wl
        from vllm_xpu_kernels.ep_moe import EpAllToAll, owner_map
        cfg, w, x, tw, ids = _case(rank, T + 3 * rank, "cfg1_small_bf16", dict(H=64, I=32, E=8), 5)
        E_local = cfg.E // world
        a2a = EpAllToAll()
        owner = owner_map(cfg.E, world, "cpu")
        send_rows, _, send_counts, send_pos = to.remap_hidden_states(x, None, ids, owner, world)
        M = ids.numel()
        send_eids = torch.empty(M, dtype=torch.int32)
        send_eids[send_pos.reshape(-1).long()] = (ids.reshape(-1) % E_local).to(torch.int32)
        s_spl, r_spl = a2a.exchange_counts(send_counts, verify=True)
        assert sum(s_spl) == M
        recv_rows, none, recv_eids = a2a.dispatch((send_rows, None, send_eids), s_spl, r_spl)
        assert none is None and recv_rows.shape[0] == sum(r_spl) == recv_eids.numel()
        # local experts = this rank's slice of the weights, top-1 with unit weight
        lo = rank * E_local
        d13, d2 = wl.dequant_weights(cfg, w)
        R = recv_rows.shape[0]
        local_out = to.fused_moe_staged(recv_rows, d13[lo:lo + E_local], None, d2[lo:lo + E_local], None,
                                        torch.ones(R, 1), recv_eids.view(R, 1), E_local)
        back = a2a.combine(local_out, s_spl, r_spl)
        out = to.moe_gather(back, tw, send_pos, x.dtype)
        ref = _oracle_full(cfg, w, x, tw, ids)
        err = float((out.float() - ref.float()).abs().max())

        # the default schedule: one row per (token, destination rank) with the token's local expert
        # ids and weights, top-k layer on the owner, one partial sum per (token, rank) back.
        # `slots` [T, K] says where each routed expert lives (slot // E_local = rank, slot % E_local
        # = local expert), `held` which global experts this rank stacks, in local order.
        def per_rank_schedule(slots, held):
            K = slots.shape[1]
            dest = slots.long() // E_local
            hit = dest.unsqueeze(1) == torch.arange(world).view(1, world, 1)            # [T, ep, K]
            rank_ids = torch.where(hit.any(dim=2), torch.arange(world).view(1, world), -1).int()
            loc_ids = torch.where(hit, (slots.long() % E_local).unsqueeze(1), -1).int()
            loc_w = torch.where(hit, tw.unsqueeze(1), 0.0).float()
            p_rows, _, p_counts, p_pos = to.remap_hidden_states(x, None, rank_ids, None, world)
            Tn = x.shape[0]
            pos = p_pos.reshape(-1).long()
            pos = torch.where(pos >= 0, pos, Tn * world)
            s_ids = torch.empty(Tn * world + 1, K, dtype=torch.int32)
            s_w = torch.empty(Tn * world + 1, K)
            s_ids.index_copy_(0, pos, loc_ids.reshape(-1, K))
            s_w.index_copy_(0, pos, loc_w.reshape(-1, K))
            ps, pr = a2a.exchange_counts(p_counts)
            n = sum(ps)
            assert n <= M and n == int((rank_ids >= 0).sum())
            r_rows, _, r_ids, r_w = a2a.dispatch((p_rows[:n], None, s_ids[:n], s_w[:n]), ps, pr)
            part = to.fused_moe_staged(r_rows, d13[held], None, d2[held], None, r_w, r_ids,
                                       E_local) if r_rows.shape[0] else r_rows
            back = a2a.combine(part, ps, pr)
            return to.moe_gather(back, torch.ones(Tn, world), p_pos, x.dtype)

        out_p = per_rank_schedule(ids, torch.arange(lo, lo + E_local))
        # every partial sum is rounded to 16 bits before the last addition
        err = max(err, float((out_p.float() - ref.float()).abs().max()))

        # the same with the experts placed by a load estimate instead of contiguously: ids are
        # relabelled through the placement, every rank stacks the experts of its slots
        from vllm_xpu_kernels.ep_moe import balanced_expert_slots, experts_in_slots
        slot = balanced_expert_slots(torch.arange(cfg.E, dtype=torch.float64) ** 2 + 1, world)
        assert not torch.equal(slot.long(), torch.arange(cfg.E))
        out_s = per_rank_schedule(slot.long()[ids.long()], experts_in_slots(slot, rank, E_local))
        err = max(err, float((out_s.float() - ref.float()).abs().max()))
        result_queue.put((rank, err, s_spl, r_spl))
    finally:
        dist.destroy_process_group()


def cpu_failure_worker(rank, world, port, result_queue):
    """Gloo ranks on CPU, failures made on the host: (1) a count message that arrives short is
    caught by the consistency check before any row moves; (2) a rank that leaves between two
    steps ends the next exchange of the others with an error inside the group's timeout."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from vllm_xpu_kernels.ep_moe import EpAllToAll, check_count_matrix
    outcome = {}
    try:
        a2a = EpAllToAll()
        # step 1: a healthy exchange
        send_counts = torch.tensor([3 + rank, 5 - rank], dtype=torch.int32)
        s_spl, r_spl = a2a.exchange_counts(send_counts, verify=True)
        outcome["healthy"] = (s_spl, r_spl)
        # step 2: rank 1's count message is tampered with on its way (one row short)
        recv = torch.empty_like(send_counts)
        dist.all_to_all_single(recv, send_counts)
        sent = [torch.empty_like(send_counts) for _ in range(world)]
        dist.all_gather(sent, send_counts)
        if rank == 0:
            recv[1] -= 1   # the dropped row
        try:
            check_count_matrix(torch.stack(sent), recv, rank, capacity=16)
            outcome["short_count_caught"] = rank != 0
        except RuntimeError as e:
            outcome["short_count_caught"] = rank == 0 and "rank 1 sent" in str(e)
        dist.barrier()
        # step 3: rank 1 leaves between steps; rank 0's next exchange must fail, not hang
        if rank == 1:
            outcome["left"] = True
        else:
            import time
            time.sleep(1.0)   # the peer is gone by now
            t0 = time.time()
            try:
                a2a.exchange_counts(send_counts)
                outcome["peer_loss_raised"] = False
            except Exception as e:  # the backend's error type is not part of the contract
                outcome["peer_loss_raised"] = True
                outcome["peer_loss_seconds"] = time.time() - t0
        result_queue.put((rank, outcome))
    finally:
        if rank == 1:
            dist.destroy_process_group()
        # rank 0's group is broken after the failed exchange: nothing left to tear down cleanly


def gpu_worker(rank, world, port, T, cfg_name, dims, result_queue):
    """NCCL ranks, one GPU each: EpFusedMoe against the single-process oracle."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from oracle import workloads as wl
        from vllm_xpu_kernels.ep_moe import EpFusedMoe
        cfg, w, x, tw, ids = _case(rank, T + 5 * rank, cfg_name, dims, 7)
        E_local = cfg.E // world
        sl = slice(rank * E_local, (rank + 1) * E_local)
        wr = {k: (v[sl] if v is not None else None) for k, v in w.items()}
        w13, s13, w2, s2 = wl.to_op_layout(cfg, wr)
        mv = lambda t: t.to(dev) if t is not None else None
        layer = EpFusedMoe(mv(w13), mv(s13), mv(wr["w13_bias"]), mv(w2), mv(s2), mv(wr["w2_bias"]), cfg.K,
                           cfg.activation, E_local)
        out = torch.empty(x.shape, dtype=torch.bfloat16, device=dev)
        for _ in range(2):  # twice: the second call reuses cached state
            layer.apply(out, x.to(dev), tw.to(dev), ids.to(dev))
        torch.cuda.synchronize()
        ref = _oracle_full(cfg, w, x, tw, ids)
        err = float((out.cpu().float() - ref.float()).abs().max())
        scale = float(ref.float().abs().max())
        # one row per (token, expert) instead of per (token, rank)
        plain = EpFusedMoe(mv(w13), mv(s13), mv(wr["w13_bias"]), mv(w2), mv(s2), mv(wr["w2_bias"]), cfg.K,
                           cfg.activation, E_local, per_rank_rows=False)
        out1 = torch.empty_like(out)
        plain.apply(out1, x.to(dev), tw.to(dev), ids.to(dev))
        torch.cuda.synchronize()
        err = max(err, float((out1.cpu().float() - ref.float()).abs().max()))
        # the peer-memory transport: symmetric buffers, stores over NVLink, two barriers per call
        from vllm_xpu_kernels.ep_moe import EpPeerFusedMoe, SymmetricPeerGroup
        peers = SymmetricPeerGroup(dev)
        cap = T + 5 * (world - 1)
        peer_layer = EpPeerFusedMoe(mv(w13), mv(s13), mv(wr["w13_bias"]), mv(w2), mv(s2), mv(wr["w2_bias"]), cfg.K,
                                    cfg.activation, E_local, peers, cap, cfg.H)
        out2 = torch.full_like(out, float("nan"))
        for _ in range(3):
            peer_layer.apply(out2, x.to(dev), tw.to(dev), ids.to(dev).to(torch.int32))
        peer_layer.check_counts()
        torch.cuda.synchronize()
        err = max(err, float((out2.cpu().float() - ref.float()).abs().max()))
        result_queue.put((rank, err, scale))
    finally:
        dist.destroy_process_group()
