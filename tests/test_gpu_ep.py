"""GPU, 2 ranks over NCCL (one GPU each): the all-to-all expert-parallel layer
against the single-process CPU oracle.  Skipped on a single-GPU box."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

from ep_worker import gpu_worker

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("cfg_name,dims,tol", [
    ("cfg1_small_bf16", dict(H=256, I=128, E=8), 2e-2),
    ("cfg4_deepseek_fp8", dict(H=512, I=256, E=64), 5e-2),
])
def test_ep_fused_moe_two_ranks(cfg_name, dims, tol):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=gpu_worker, args=(r, 2, port, 40, cfg_name, dims, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, scale in results:
        assert err <= tol * max(1.0, scale), f"rank {rank}: max abs err {err} (ref scale {scale})"
