"""Helpers for the legacy prologue tests: run an implementation on a golden case and
compare the three regions the reference's test compares
(tests/fused_moe/test_moe_prologue.py:238-265 of vllm-xpu-kernels) plus the index maps."""
import torch

from oracle import c_oracle as co


def workspace_for(c):
    x = c["hidden_states"]
    sc = c["scales"]
    layout, total = co.prologue_layout(x.shape[0], c["topk"], c["num_experts"], x.shape[1], c["block_k"],
                                       x.element_size(), sc.element_size() if sc is not None else 0)
    return layout, total


def regions(c, ws, layout):
    """Views of a CPU uint8 workspace."""
    x, sc = c["hidden_states"], c["scales"]
    n = x.shape[0] * c["topk"]
    E = c["num_experts"]
    def cut(name, nbytes):
        return ws[layout[name]: layout[name] + nbytes]
    out = dict(
        p2u=cut("permuted_row_to_unpermuted_row", n * 4).view(torch.int32),
        pexp=cut("permuted_token_selected_experts", n * 4).view(torch.int32),
        u2p=cut("unpermuted_row_to_permuted_row", n * 4).view(torch.int32),
        first=cut("expert_first_token_offset", (E + 1) * 8).view(torch.int64),
        pscale=cut("permuted_token_final_scales", n * 4).view(torch.float32),
        rows=cut("overlapped_gemm1_gemm2_inputs", n * x.shape[1] * x.element_size()).view(x.dtype).view(n, x.shape[1]),
    )
    if sc is not None:
        out["srows"] = cut("permuted_act_scales", n * sc.shape[1] * sc.element_size()).view(sc.dtype).view(n, sc.shape[1])
    return out


def check_against_reference_vectors(c, r):
    E = c["num_experts"]
    n_ref = c["expert_offset"].numel()   # the reference's bincount stops at the largest id in use
    assert torch.equal(r["first"][1: 1 + n_ref], c["expert_offset"])
    assert (r["first"][n_ref:] == r["first"][E]).all()
    total = int(r["first"][E])
    assert int(r["first"][0]) == 0 and total == c["expand_input"].shape[0]
    assert torch.equal(r["rows"][:total].view(torch.uint8), c["expand_input"].contiguous().view(torch.uint8))
    if c["scales"] is not None:
        assert torch.equal(r["srows"][:total].view(torch.uint8), c["expand_scales"].contiguous().view(torch.uint8))
    # the index maps, from their definition
    T, K = c["topk_ids"].shape
    p2u = r["p2u"][:total].long()
    tok, k = p2u % T, p2u // T
    assert torch.equal(c["topk_ids"][tok, k].int(), r["pexp"][:total])
    assert torch.equal(c["topk_weights"][tok, k], r["pscale"][:total])
    assert torch.equal(r["u2p"][p2u], torch.arange(total, dtype=torch.int32))
