"""CPU: the restated moe_lora_align_block_size against the properties the reference's own
test asserts (tests/test_moe_lora_align_sum.py:96-106, 226-320 of vllm-xpu-kernels).  The
reference holds no expected outputs for this op, only those properties."""
import pytest
import torch

from lora_align_cases import SENTINEL_NPAD, check_properties, fresh_outputs, make_case
from oracle import c_oracle as co


def _run(c):
    s, e, p = fresh_outputs(c)
    co.moe_lora_align_block_size(c["topk_ids"], c["token_lora_mapping"], c["num_experts"], c["block_size"],
                                 c["max_loras"], c["max_num_tokens_padded"], c["max_num_m_blocks"], s, e, p,
                                 c["adapter_enabled"], c["lora_ids"], c["expert_map"])
    return s, e, p


@pytest.mark.parametrize("num_tokens,num_experts,max_loras", [(100, 64, 2), (200, 128, 32), (1024, 256, 2),
                                                              (7, 512, 2), (1, 8, 1)])
def test_lora_align_oracle_properties(num_tokens, num_experts, max_loras):
    c = make_case(num_tokens, 6 if num_experts >= 6 else 2, num_experts, max_loras, 16)
    check_properties(c, *_run(c))


def test_lora_align_oracle_guards():
    # mixed base-model (-1) and adapter tokens: -1 sits first in lora_ids
    c = make_case(16, 6, 64, 2, 16, base_frac=0.5)
    assert int(c["lora_ids"][0]) == -1
    check_properties(c, *_run(c))
    # disabled adapter: nothing of its segment is written
    c = make_case(16, 6, 64, 1, 16, disabled=(0,))
    s, e, p = _run(c)
    assert int(p[0]) == SENTINEL_NPAD
    check_properties(c, s, e, p)
    # out-of-range adapter id in the extra slot is skipped
    c = make_case(16, 6, 64, 1, 16, lora_ids=torch.tensor([0, 5]))
    s, e, p = _run(c)
    assert int(p[0]) != SENTINEL_NPAD
    check_properties(c, s, e, p)
    # expert map drops the odd experts
    c = make_case(64, 4, 32, 3, 8, with_map=True, base_frac=0.2)
    check_properties(c, *_run(c))
