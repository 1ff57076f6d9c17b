"""GPU parity: moe_lora_align_block_size against the oracle (exact, including which cells
stay untouched), on the shapes of the reference's test
(tests/test_moe_lora_align_sum.py:43-106, 226-320 of vllm-xpu-kernels)."""
import pytest
import torch

from gpu_utils import DEV
from lora_align_cases import SENTINEL_NPAD, check_properties, fresh_outputs, make_case
from oracle import c_oracle as co

pytestmark = pytest.mark.gpu


def _both(c):
    s, e, p = fresh_outputs(c)
    co.moe_lora_align_block_size(c["topk_ids"], c["token_lora_mapping"], c["num_experts"], c["block_size"],
                                 c["max_loras"], c["max_num_tokens_padded"], c["max_num_m_blocks"], s, e, p,
                                 c["adapter_enabled"], c["lora_ids"], c["expert_map"])
    gs, ge, gp = fresh_outputs(c, DEV)
    emap = c["expert_map"].to(DEV) if c["expert_map"] is not None else None
    torch.ops._moe_C.moe_lora_align_block_size(
        c["topk_ids"].to(DEV), c["token_lora_mapping"].to(DEV), c["num_experts"], c["block_size"], c["max_loras"],
        c["max_num_tokens_padded"], c["max_num_m_blocks"], gs, ge, gp, c["adapter_enabled"].to(DEV),
        c["lora_ids"].to(DEV), emap)
    assert torch.equal(gp.cpu(), p)
    assert torch.equal(ge.cpu(), e)
    assert torch.equal(gs.cpu(), s)
    return gs.cpu(), ge.cpu(), gp.cpu()


@pytest.mark.parametrize("num_tokens", [100, 200, 1024, 4096])
@pytest.mark.parametrize("num_experts", [64, 128, 256, 512])
@pytest.mark.parametrize("max_loras", [2, 32])
def test_lora_align_exact(native, num_tokens, num_experts, max_loras):
    c = make_case(num_tokens, 6, num_experts, max_loras, 16)
    check_properties(c, *_both(c))


def test_lora_align_guards_map_dtypes(native):
    c = make_case(16, 6, 64, 2, 16, base_frac=0.5)          # -1 first in lora_ids
    check_properties(c, *_both(c))
    c = make_case(16, 6, 64, 1, 16, disabled=(0,))          # disabled adapter untouched
    s, e, p = _both(c)
    assert int(p[0]) == SENTINEL_NPAD
    c = make_case(16, 6, 64, 1, 16, lora_ids=torch.tensor([0, 5]))   # out-of-range id skipped
    s, e, p = _both(c)
    assert int(p[0]) != SENTINEL_NPAD
    c = make_case(300, 4, 32, 3, 8, with_map=True, base_frac=0.2)
    check_properties(c, *_both(c))
    c = make_case(2500, 8, 992, 4, 64, index_dtype=torch.int64)      # several rounds, most experts allowed
    check_properties(c, *_both(c))
    c = make_case(1, 2, 8, 1, 4)
    check_properties(c, *_both(c))
    ids = torch.zeros(4, 2, dtype=torch.int32, device=DEV)
    z = torch.zeros(64, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="block_size should be greater than 0"):
        torch.ops._moe_C.moe_lora_align_block_size(ids, z, 8, 0, 1, 16, 4, z, z, z, z, z, None)
    with pytest.raises(RuntimeError, match="padded_num_experts must be less than 1024"):
        torch.ops._moe_C.moe_lora_align_block_size(ids, z, 1000, 4, 1, 16, 4, z, z, z, z, z, None)


def test_lora_align_only_base_model_tokens(native):
    """Every token belongs to the base model (-1): lora_ids holds only -1 and no segment is written."""
    c = make_case(32, 4, 16, 2, 8, base_frac=1.1)
    assert (c["token_lora_mapping"] == -1).all() and (c["lora_ids"] == -1).all()
    s, e, p = _both(c)
    check_properties(c, s, e, p)
