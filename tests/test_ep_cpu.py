"""CPU, world_size 2 over Gloo: the expert-parallel dispatch / combine plumbing."""
import socket

import pytest

import torch
import torch.multiprocessing as mp

from ep_worker import cpu_failure_worker, cpu_worker


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_ep_all_to_all_two_gloo_ranks_match_the_oracle():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=cpu_worker, args=(r, 2, port, 11, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    results.sort()
    for rank, err, s_spl, r_spl in results:
        assert err <= 2e-2, f"rank {rank}: max abs err {err}"
    # what rank 0 sends to rank 1 is what rank 1 receives from rank 0, and vice versa
    assert results[0][2][1] == results[1][3][0] and results[1][2][0] == results[0][3][1]


def test_ep_host_side_failures_are_detected_not_hung():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=cpu_failure_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert results[0]["healthy"][0][1] == results[1]["healthy"][1][0]     # what 0 sent to 1 arrived at 1
    assert results[0]["short_count_caught"] and results[1]["short_count_caught"]
    assert results[1]["left"]
    assert results[0]["peer_loss_raised"], "the exchange after a peer left must raise"
    assert results[0]["peer_loss_seconds"] < 30


def test_check_count_matrix_names_the_offending_rank():
    import pytest
    from vllm_xpu_kernels.ep_moe import check_count_matrix
    sent = torch.tensor([[1, 2], [3, 4]], dtype=torch.int32)
    check_count_matrix(sent, torch.tensor([2, 4]), rank=1, capacity=4)
    with pytest.raises(RuntimeError, match="rank 0 sent 2 rows to rank 1"):
        check_count_matrix(sent, torch.tensor([1, 4]), rank=1)
    with pytest.raises(RuntimeError, match="exceed the capacity"):
        check_count_matrix(sent, torch.tensor([2, 4]), rank=1, capacity=3)


def test_owner_map_is_the_contiguous_even_split():
    from vllm_xpu_kernels.ep_moe import owner_map
    from oracle import c_oracle as co
    m = owner_map(256, 8, "cpu")
    assert m.tolist() == [g // 32 for g in range(256)]
    for r in range(8):  # consistent with init_expert_map: rank r maps exactly its own experts
        local = co.init_expert_map(32, r, 8)
        assert torch.equal(local >= 0, m == r)


def test_balanced_expert_slots_even_out_the_ranks():
    from vllm_xpu_kernels.ep_moe import balanced_expert_slots, experts_in_slots
    from oracle import torch_oracle as to
    g = torch.Generator().manual_seed(0)
    load = torch.rand(64, generator=g) ** 3 * 1000          # a few hot experts
    slot = balanced_expert_slots(load, 8)
    assert slot.dtype == torch.int32 and sorted(slot.tolist()) == list(range(64))
    per_rank = torch.zeros(8, dtype=torch.float64).index_add_(0, (slot // 8).long(), load.double())
    contiguous = load.double().view(8, 8).sum(1)
    assert float(per_rank.max() / per_rank.mean()) < 1.05 < float(contiguous.max() / contiguous.mean())
    # the experts a rank stacks, slot by slot, and the table agree
    for r in range(8):
        held = experts_in_slots(slot, r, 8)
        assert slot[held].tolist() == list(range(r * 8, (r + 1) * 8))
    with pytest.raises(ValueError):
        balanced_expert_slots(torch.ones(10), 4)
    # the dispatch bookkeeping with a placement = the contiguous bookkeeping on relabelled ids
    ids = torch.randint(0, 64, (20, 4), generator=g).to(torch.int32)
    a = to.ep_dispatch_plan(ids, 8, 8, 32, slot)
    b = to.ep_dispatch_plan(slot[ids.long()], 8, 8, 32)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
