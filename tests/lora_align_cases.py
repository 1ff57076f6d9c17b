"""Seeded inputs for moe_lora_align_block_size, shaped like the ones the reference's test
builds (tests/test_moe_lora_align_sum.py:29-79, 119-222 of vllm-xpu-kernels): distinct
experts per token, one adapter id per token, output buffers pre-filled with out-of-domain
sentinels so untouched cells can be told from written ones."""
import torch

SENTINEL_EXPERT = -2
SENTINEL_TOKEN = -7
SENTINEL_NPAD = -13


def round_up(x, b):
    return (x + b - 1) // b * b


def padded_sizes(numel, num_experts, block_size):
    n = round_up(numel + num_experts * (block_size - 1), block_size)
    if numel < num_experts:
        n = numel * block_size
    return n, (n + block_size - 1) // block_size


def make_case(num_tokens, topk, num_experts, max_loras, block_size, seed=1, base_frac=0.0,
              disabled=(), lora_ids=None, with_map=False, index_dtype=torch.int32):
    g = torch.Generator().manual_seed(seed)
    if num_tokens * num_experts <= 1 << 18:
        ids = torch.stack([torch.randperm(num_experts, generator=g)[:topk] for _ in range(num_tokens)])
    else:
        ids = torch.randint(0, num_experts, (num_tokens, topk), generator=g)
    ids = ids.to(index_dtype)
    mapping = torch.randint(0, max_loras, (num_tokens,), generator=g, dtype=torch.int32)
    if base_frac > 0:
        mapping[torch.rand(num_tokens, generator=g) < base_frac] = -1
    n_pad, n_blocks = padded_sizes(ids.numel(), num_experts, block_size)
    if lora_ids is None:
        lora_ids = torch.full((max_loras + 1,), -1, dtype=torch.int32)
        u = torch.unique(mapping, sorted=True)
        lora_ids[: u.numel()] = u.int()
    enabled = torch.ones(max_loras + 1, dtype=torch.int32)
    for s in disabled:
        enabled[s] = 0
    emap = None
    if with_map:   # keep the even experts, renumbered
        emap = torch.full((num_experts,), -1, dtype=torch.int32)
        emap[::2] = torch.arange((num_experts + 1) // 2, dtype=torch.int32)
    return dict(topk_ids=ids, token_lora_mapping=mapping, num_experts=num_experts, block_size=block_size,
                max_loras=max_loras, max_num_tokens_padded=n_pad, max_num_m_blocks=n_blocks,
                adapter_enabled=enabled, lora_ids=lora_ids.int(), expert_map=emap)


def fresh_outputs(c, device="cpu"):
    return (torch.full((c["max_loras"] * c["max_num_tokens_padded"],), SENTINEL_TOKEN, dtype=torch.int32, device=device),
            torch.full((c["max_loras"] * c["max_num_m_blocks"],), SENTINEL_EXPERT, dtype=torch.int32, device=device),
            torch.full((c["max_loras"],), SENTINEL_NPAD, dtype=torch.int32, device=device))


def check_properties(c, sorted_ids, expert_ids, post_pad):
    """What the reference's tests assert, plus completeness: every block of an active adapter
    holds only slots of that block's expert and of tokens mapped to the adapter; every such
    slot appears exactly once; inactive adapters keep the sentinels."""
    ids = c["topk_ids"].reshape(-1).long()
    numel, bs, L = ids.numel(), c["block_size"], c["max_loras"]
    topk = c["topk_ids"].shape[1]
    emap = c["expert_map"]
    mapped = ids if emap is None else emap.long()[ids]
    active = set()
    for li in c["lora_ids"][: L + 1].tolist():
        if 0 <= li < L and c["adapter_enabled"][li] != 0:
            active.add(li)
    so = sorted_ids.view(L, -1)
    eo = expert_ids.view(L, -1)
    for l in range(L):
        if l not in active:
            assert (so[l] == SENTINEL_TOKEN).all() and (eo[l] == SENTINEL_EXPERT).all()
            assert int(post_pad[l]) == SENTINEL_NPAD
            continue
        n = int(post_pad[l])
        assert n % bs == 0 and 0 <= n <= c["max_num_tokens_padded"]
        assert (so[l] != SENTINEL_TOKEN).all() and (eo[l] != SENTINEL_EXPERT).all()
        assert (so[l][n:] == numel).all() and (eo[l][n // bs:] == -1).all()
        real = so[l][:n]
        slots = real[real != numel].long()
        want = torch.nonzero((c["token_lora_mapping"].long()[torch.arange(numel) // topk] == l) & (mapped >= 0)).flatten()
        assert torch.equal(torch.sort(slots).values, want)
        blk_expert = eo[l][: n // bs].long().repeat_interleave(bs)
        keep = real != numel
        assert torch.equal(mapped[real[keep].long()], blk_expert[keep])
