"""GPU: expert parallelism over peer memory (EpPeerFusedMoe).

All ranks of the group run inside this one process on one GPU (LocalPeerWorld): their
receive buffers are ordinary allocations and the phases of all ranks run one after the other
on one stream, which is the only ordering the protocol needs.  The dispatch bookkeeping is
compared exactly with its sequential restatement, the layer output with the single-process
CPU oracle of the whole layer.  (The same layer between real GPUs, over symmetric memory and
NVLink, is covered by test_gpu_ep.py where two GPUs are present.)"""
import pytest
import torch

from oracle import torch_oracle as to
from oracle import workloads as wl

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _build(native, cfg, ep, cap, seed, slot=None):
    from vllm_xpu_kernels.ep_moe import EpPeerFusedMoe, LocalPeerWorld, experts_in_slots
    w = wl.make_weights(cfg, seed=seed)
    E_local = cfg.E // ep
    world = LocalPeerWorld(ep, DEV)
    layers = []
    for r in range(ep):
        # the experts this rank holds, in the order of its local slots
        sl = slice(r * E_local, (r + 1) * E_local) if slot is None else experts_in_slots(slot, r, E_local)
        wr = {k: (v[sl] if v is not None else None) for k, v in w.items()}
        w13, s13, w2, s2 = wl.to_op_layout(cfg, wr)
        mv = lambda t: t.to(DEV) if t is not None else None
        layers.append(EpPeerFusedMoe(mv(w13), mv(s13), mv(wr["w13_bias"]), mv(w2), mv(s2), mv(wr["w2_bias"]),
                                     cfg.K, cfg.activation, E_local, world.member(r), cap, cfg.H,
                                     expert_slot=slot))
    return w, layers


def _oracle_full(cfg, w, x, tw, ids):
    d13, d2 = wl.dequant_weights(cfg, w)
    return to.fused_moe_staged(x, d13, w["w13_bias"], d2, w["w2_bias"], tw, ids, cfg.E,
                               activation=cfg.activation, act_quant=cfg.recipe == "fp8block")


@pytest.mark.parametrize("cfg_name,dims,ep,tokens,tol,placed", [
    ("cfg1_small_bf16", dict(H=256, I=128, E=8), 2, (40, 45), 2e-2, False),
    ("cfg1_small_bf16", dict(H=256, I=128, E=8), 4, (33, 0, 64, 7), 2e-2, False),       # an idle rank, a full one
    ("cfg1_small_bf16", dict(H=256, I=128, E=8), 4, (33, 0, 64, 7), 2e-2, True),        # experts placed by load
    ("cfg4_deepseek_fp8", dict(H=512, I=256, E=64), 4, (50, 64, 1, 23), 5e-2, False),
    ("cfg4_deepseek_fp8", dict(H=512, I=256, E=64), 4, (50, 64, 1, 23), 5e-2, True),
    ("cfg4_deepseek_fp8", dict(H=512, I=256, E=64), 8, (300, 290, 310, 5, 300, 0, 299, 320), 5e-2, False),  # multi-block sort
])
def test_peer_ep_layer_matches_the_single_process_oracle(native, cfg_name, dims, ep, tokens, tol, placed):
    from vllm_xpu_kernels.ep_moe import balanced_expert_slots
    cfg = wl.scaled(wl.CONFIGS[cfg_name], **dims)
    cap = max(tokens)
    slot = None
    if placed:   # a placement from a made-up load estimate: any permutation must give the same layer
        slot = balanced_expert_slots(torch.rand(cfg.E, generator=torch.Generator().manual_seed(5)), ep)
        assert sorted(slot.tolist()) == list(range(cfg.E))
    w, layers = _build(native, cfg, ep, cap, seed=3, slot=slot)
    E_local = cfg.E // ep
    for call in range(2):  # the second call runs over the first one's leftovers in every buffer
        inputs = []
        for r, T in enumerate(tokens):
            if T == 0:
                inputs.append((torch.zeros(0, cfg.H, dtype=torch.bfloat16), torch.zeros(0, cfg.K),
                               torch.zeros(0, cfg.K, dtype=torch.int32)))
                continue
            x, logits, bias = wl.make_inputs(cfg, T, seed=100 * call + r)
            tw, ids = wl.route_cpu(cfg, logits, bias)
            inputs.append((x, tw.reshape(T, cfg.K), ids.reshape(T, cfg.K).to(torch.int32)))
        outs = [torch.full((T, cfg.H), float("nan"), dtype=torch.bfloat16, device=DEV) for T in tokens]
        dev_in = [(x.to(DEV), tw.to(DEV), ids.to(DEV)) for x, tw, ids in inputs]
        for r in range(ep):
            layers[r].dispatch(*dev_in[r])
        torch.cuda.synchronize()
        # bookkeeping: exact against the sequential restatement
        plans = [to.ep_dispatch_plan(inputs[r][2], ep, E_local, cap, slot) for r in range(ep)]
        for r in range(ep):
            counts, pos, loc = plans[r]
            T = tokens[r]
            assert torch.equal(layers[r].send_counts.cpu(), counts)
            assert torch.equal(layers[r].send_pos[:T].cpu(), pos)
        for d in range(ep):
            got_counts = layers[d].recv_counts.cpu()
            ids_d = layers[d].recv_ids.cpu().view(ep, cap, cfg.K)
            w_d = layers[d].recv_weights.cpu().view(ep, cap, cfg.K)
            for s in range(ep):
                counts, pos, loc = plans[s]
                assert int(got_counts[s]) == int(counts[d])
                sent = pos[:, d] >= 0
                idx = (pos[sent, d] - d * cap).long()
                assert torch.equal(ids_d[s][idx], loc[sent, d])
                exp_w = torch.where(loc[sent, d] >= 0, inputs[s][1][sent], 0.0)
                assert torch.equal(w_d[s][idx], exp_w)
                if not layers[d].quant:   # 16-bit rows travel unchanged
                    rows_d = layers[d].recv_rows.cpu().view(ep, cap, cfg.H)
                    assert torch.equal(rows_d[s][idx], inputs[s][0][sent])
        for r in range(ep):
            layers[r].experts_and_combine()
        for r in range(ep):
            layers[r].finish(outs[r])
        torch.cuda.synchronize()
        for r, T in enumerate(tokens):
            if T == 0:
                continue
            x, tw, ids = inputs[r]
            ref = _oracle_full(cfg, w, x, tw, ids)
            err = float((outs[r].cpu().float() - ref.float()).abs().max())
            scale = float(ref.float().abs().max())
            assert err <= tol * max(1.0, scale), f"call {call} rank {r}: max abs err {err} (scale {scale})"


def test_peer_ep_quantised_rows_are_the_group_quantiser(native):
    # what travels for fp8 experts is exactly per_token_group_fp8_quant of the token row
    cfg = wl.scaled(wl.CONFIGS["cfg4_deepseek_fp8"], H=512, I=256, E=64)
    ep, cap = 2, 48
    w, layers = _build(native, cfg, ep, cap, seed=5)
    x, logits, bias = wl.make_inputs(cfg, cap, seed=9)
    tw, ids = wl.route_cpu(cfg, logits, bias)
    layers[0].dispatch(x.to(DEV), tw.to(DEV), ids.to(DEV))
    torch.cuda.synchronize()
    q, s = to.per_token_group_fp8_quant(x, 128)
    counts, pos, _ = to.ep_dispatch_plan(ids, ep, cfg.E // ep, cap)
    for d in range(ep):
        sent = pos[:, d] >= 0
        idx = (pos[sent, d] - d * cap).long()
        rows = layers[d].recv_rows.cpu().view(torch.uint8).view(ep, cap, cfg.H)[0]
        scales = layers[d].recv_scales.cpu().view(ep, cap, cfg.H // 128)[0]
        assert torch.equal(rows[idx], q.view(torch.uint8)[sent])
        assert torch.equal(scales[idx], s[sent])


def test_peer_ep_rejects_more_tokens_than_its_regions_hold(native):
    cfg = wl.scaled(wl.CONFIGS["cfg1_small_bf16"], H=256, I=128, E=8)
    _, layers = _build(native, cfg, 2, 16, seed=1)
    x = torch.zeros(17, cfg.H, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError, match="exceed max_tokens"):
        layers[0].dispatch(x, torch.zeros(17, cfg.K, device=DEV), torch.zeros(17, cfg.K, dtype=torch.int32, device=DEV))
