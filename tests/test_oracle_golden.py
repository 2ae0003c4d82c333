"""CPU: the oracle restatement against vectors produced by the reference's own naive path."""
import pytest
import torch

from helpers import NAMES, golden_cases, load_golden
from oracle import evo_oracle as oc


@pytest.mark.parametrize("path", golden_cases(), ids=lambda p: p.split("golden_")[-1][:-3])
def test_oracle_matches_reference_vectors_bitwise(path):
    g = load_golden(path)
    out = oc.attention_fwd_bwd(g["Q"], g["K"], g["V"], g["res_mask"], g["pair_bias"], g["dO"])
    for name, x in zip(NAMES, out):
        assert x.dtype == g[name].dtype, name
        assert torch.equal(x, g[name]), f"{name} differs from the reference's naive path"


@pytest.mark.parametrize("path", golden_cases(), ids=lambda p: p.split("golden_")[-1][:-3])
def test_chunked_oracle_equals_unchunked(path):
    g = load_golden(path)
    args = (g["Q"], g["K"], g["V"], g["res_mask"], g["pair_bias"], g["dO"])
    full = oc.attention_fwd_bwd(*args, upcast=torch.float64)
    part = oc.attention_fwd_bwd(*args, upcast=torch.float64, chunk=1)
    for name, a, b in zip(NAMES, full, part):
        assert oc.rel_err(b, a) < 1e-12, name


@pytest.mark.parametrize("path", golden_cases(), ids=lambda p: p.split("golden_")[-1][:-3])
def test_closed_form_backward_matches_autograd(path):
    """The hand-written backward formulas (the ones the CUDA kernels implement) against
    autograd through the naive path, both in fp64 on the golden inputs."""
    g = load_golden(path)
    args = (g["Q"], g["K"], g["V"], g["res_mask"], g["pair_bias"], g["dO"])
    auto = oc.attention_fwd_bwd(*args, upcast=torch.float64)
    hand = oc.attention_fwd_bwd_explicit(*args)
    for name, a, b in zip(NAMES, auto, hand):
        assert oc.rel_err(b, a) < 1e-10, name


def test_fully_masked_row_is_uniform_not_nan():
    g = load_golden([p for p in golden_cases() if "fullmask" in p][0])
    assert not g["res_mask"][0, 0].any()
    out = oc.attention_fwd_bwd(g["Q"], g["K"], g["V"], g["res_mask"], g["pair_bias"], g["dO"],
                               upcast=torch.float64)
    assert all(torch.isfinite(t).all() for t in out)
    B, S, R, H, D = g["Q"].shape
    v = g["V"].double().reshape(B, H, S, R, D)
    o = out[0].reshape(B, H, S, R, D)
    # attention-view row s=0 of every head has all keys dropped: O is the plain mean of V
    assert torch.allclose(o[:, :, 0], v[:, :, 0].mean(dim=-2, keepdim=True).expand_as(o[:, :, 0]), atol=1e-12)


def test_reinterpret_is_not_permute():
    x = torch.arange(2 * 3 * 4 * 5 * 6, dtype=torch.float32).reshape(2, 3, 4, 5, 6)
    assert not torch.equal(oc.kernel_view(x, "reinterpret"), oc.kernel_view(x, "true"))
    assert torch.equal(oc.label_view(oc.kernel_view(x, "true"), "true"), x)
    assert torch.equal(oc.label_view(oc.kernel_view(x, "reinterpret"), "reinterpret"), x)


def test_additive_mask_equals_bool_mask_when_rows_keep_a_key():
    from evoformer_triton_b200.workloads import WORKLOADS, additive_mask, make_inputs
    x = make_inputs(WORKLOADS["C1"])
    a = oc.attention_fwd_bwd(**x, upcast=torch.float64)
    x2 = dict(x)
    x2["res_mask"] = additive_mask(x["res_mask"], torch.float64)
    b = oc.attention_fwd_bwd(**x2, upcast=torch.float64)
    for name, u, v in zip(NAMES, a, b):
        assert oc.rel_err(v, u) < 1e-9, name
