"""GPU: the rows next to the reference's op: a sigmoid gate fused into the output, the pair bias in
the layout a linear layer emits ([B, N_res, N_res, H]), and a gradient for an additive mask.
The reference has none of them (its op ends at O, takes the bias as [B, 1, H, R, R] and returns
no mask gradient: evoformer.py:638, 735, 862); the yardstick is the oracle's composition of the
pinned naive attention with plain PyTorch, evaluated on the fp32-upcast inputs."""
import pytest
import torch

from oracle import evo_oracle as oc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("O", "dQ", "dK", "dV", "d_pair_bias", "d_gate", "d_mask")


def _inputs(B, S, R, H, D, dtype, seed, mask="bool"):
    g = torch.Generator().manual_seed(seed)
    shp = (B, S, R, H, D)
    x = {n: (torch.randn(shp, generator=g) * 0.5).to(dtype) for n in ("Q", "K", "V")}
    x["dO"] = torch.randn(shp, generator=g).to(dtype)
    x["gate"] = torch.randn(shp, generator=g).to(dtype)
    keep = torch.rand((B, S, 1, 1, R), generator=g) < 0.8
    keep[..., 0] = True
    x["res_mask"] = keep if mask == "bool" else torch.where(keep, 0.0, -30.0) + 0.1 * torch.randn((B, S, 1, 1, R), generator=g)
    x["pair_bias"] = torch.randn((B, 1, H, R, R), generator=g)
    return x


def _check(got, want, tol=1e-2):
    for name, a, b in zip(NAMES, got, want):
        if b is None:
            continue
        assert a is not None, name
        assert torch.isfinite(a).all(), name
        err = oc.rel_err(a, b)
        assert err <= tol, f"{name}: rel err {err:.3e}"


@pytest.mark.parametrize("cfg", [(1, 5, 200, 2, 32, torch.bfloat16), (1, 3, 256, 2, 64, torch.bfloat16),
                                 (1, 4, 136, 4, 8, torch.float16), (1, 2, 50, 2, 32, torch.float32)],
                         ids=lambda c: "B%dS%dR%dH%dD%d-%s" % (c[0], c[1], c[2], c[3], c[4], str(c[5]).split(".")[-1]))
def test_gated_output(cfg):
    import evoformer_triton_b200 as evo
    B, S, R, H, D, dtype = cfg
    x = _inputs(B, S, R, H, D, dtype, seed=R + D)
    want = oc.extended_attention_fwd_bwd(x["Q"], x["K"], x["V"], x["res_mask"], x["pair_bias"], x["dO"], gate=x["gate"],
                                         upcast=torch.float64 if dtype == torch.float32 else torch.float32)
    t = {n: x[n].to(DEV).requires_grad_() for n in ("Q", "K", "V", "gate", "pair_bias")}
    out = evo.GatedEvoformerAttention.apply(t["Q"], t["K"], t["V"], x["res_mask"].to(DEV), t["pair_bias"], t["gate"])
    out.backward(x["dO"].to(DEV))
    torch.cuda.synchronize()
    evo.check_device_status()
    got = (out, t["Q"].grad, t["K"].grad, t["V"].grad, t["pair_bias"].grad, t["gate"].grad, None)
    _check(got, want, tol=2e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("bias_dtype", [torch.float32, torch.bfloat16], ids=["fp32_bias", "bf16_bias"])
def test_pair_bias_heads_last(bias_dtype):
    import evoformer_triton_b200 as evo
    B, S, R, H, D, dtype = 2, 4, 200, 4, 32, torch.bfloat16
    x = _inputs(B, S, R, H, D, dtype, seed=7)
    bias_brrh = x["pair_bias"].reshape(B, H, R, R).permute(0, 2, 3, 1).contiguous().to(bias_dtype)
    want = oc.extended_attention_fwd_bwd(x["Q"], x["K"], x["V"], x["res_mask"], bias_brrh, x["dO"],
                                         pair_bias_layout="brrh", upcast=torch.float32)
    t = {n: x[n].to(DEV).requires_grad_() for n in ("Q", "K", "V")}
    b = bias_brrh.to(DEV).requires_grad_()
    out = evo.evoformer_attention(t["Q"], t["K"], t["V"], [x["res_mask"].to(DEV), b], layout="reinterpret",
                                  pair_bias_layout="brrh")
    out.backward(x["dO"].to(DEV))
    torch.cuda.synchronize()
    evo.check_device_status()
    assert b.grad.shape == (B, R, R, H) and b.grad.dtype == bias_dtype
    _check((out, t["Q"].grad, t["K"].grad, t["V"].grad, b.grad, None, None), want)


@pytest.mark.parametrize("D,dtype", [(32, torch.bfloat16), (16, torch.float16)])
def test_additive_mask_gets_a_gradient(D, dtype):
    import evoformer_triton_b200 as evo
    B, S, R, H = 1, 3, 136, 4
    x = _inputs(B, S, R, H, D, dtype, seed=11, mask="add")
    want = oc.extended_attention_fwd_bwd(x["Q"], x["K"], x["V"], x["res_mask"], x["pair_bias"], x["dO"], layout="true",
                                         upcast=torch.float32)
    t = {n: x[n].to(DEV).requires_grad_() for n in ("Q", "K", "V", "pair_bias")}
    m = x["res_mask"].to(DEV).requires_grad_()
    out = evo.evoformer_attention(t["Q"], t["K"], t["V"], [m, t["pair_bias"]])
    out.backward(x["dO"].to(DEV))
    torch.cuda.synchronize()
    evo.check_device_status()
    assert m.grad is not None and m.grad.shape == x["res_mask"].shape
    _check((out, t["Q"].grad, t["K"].grad, t["V"].grad, t["pair_bias"].grad, None, m.grad), want)
