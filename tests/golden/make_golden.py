"""Generate the golden vectors in this folder from the reference's own naive path.

Run once, in a container that has the reference checkout (it is not available
where the GPU tests run):

    python tests/golden/make_golden.py /path/to/reference/dsevoformer-triton

It imports the reference's ``speed_benchmark`` module *unmodified* and calls its
``_attention`` (speed_benchmark.py:10-16) on the CPU.  That module imports
``evoformer`` (Triton kernels that need a GPU driver at import time) and
``deepspeed`` (not installed) at its top, so empty stand-in modules are put in
``sys.modules`` first; nothing from them is executed.  Forward outputs come from
the reference function, gradients from autograd through it, exactly like
test.py:57-62.

Output: ``golden_<case>.pt`` files holding inputs and the reference's results.
"""
from __future__ import annotations

import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, B, H, S, R, D, dtype, mask kind)
CASES = [
    ("f32_r40_d16", 1, 2, 3, 40, 16, torch.float32, "bool"),
    ("f32_r64_d32_b2", 2, 2, 2, 64, 32, torch.float32, "bool"),
    ("bf16_r48_d32", 1, 2, 3, 48, 32, torch.bfloat16, "bool"),
    ("f16_r72_d8", 1, 4, 2, 72, 8, torch.float16, "bool"),
    ("bf16_r128_d64_fullmask", 1, 1, 2, 128, 64, torch.bfloat16, "fullrow"),
]


def import_reference_attention(ref_dir: str):
    evo = types.ModuleType("evoformer")
    evo.EvoformerAttention = object
    ds = types.ModuleType("deepspeed")
    ds_ops = types.ModuleType("deepspeed.ops")
    ds_sci = types.ModuleType("deepspeed.ops.deepspeed4science")
    ds_sci.DS4Sci_EvoformerAttention = object
    for name, mod in [("evoformer", evo), ("deepspeed", ds), ("deepspeed.ops", ds_ops),
                      ("deepspeed.ops.deepspeed4science", ds_sci)]:
        sys.modules[name] = mod
    sys.path.insert(0, ref_dir)
    import speed_benchmark  # the reference file itself
    return speed_benchmark._attention


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference/dsevoformer-triton")
    ref_dir = sys.argv[1]
    ref_attention = import_reference_attention(ref_dir)
    for idx, (name, B, H, S, R, D, dtype, mkind) in enumerate(CASES):
        g = torch.Generator().manual_seed(1234 + idx)
        shp = (B, S, R, H, D)
        Q = (torch.randn(shp, generator=g) * 0.5).to(dtype)
        K = (torch.randn(shp, generator=g) * 0.5).to(dtype)
        V = (torch.randn(shp, generator=g) * 0.5).to(dtype)
        mask = torch.randint(0, 2, (B, S, 1, 1, R), generator=g, dtype=torch.int32).bool()
        if mkind == "fullrow":
            mask[0, 0] = False  # one MSA row with every key dropped
        bias = torch.randn((B, 1, H, R, R), generator=g) * 0.5
        dO = torch.randn(shp, generator=g).to(dtype)

        # same views as the reference's "torch" provider (speed_benchmark.py:94-98)
        q = Q.reshape(B, H, S, R, D).clone().requires_grad_()
        k = K.reshape(B, H, S, R, D).clone().requires_grad_()
        v = V.reshape(B, H, S, R, D).clone().requires_grad_()
        b = bias.reshape(B, H, 1, R, R).clone().requires_grad_()
        m = mask.reshape(B, 1, S, 1, R)
        o = ref_attention(q, k, v, m, b)
        o = o.reshape(B, S, R, H, D)
        o.backward(dO)
        torch.save(
            dict(name=name, B=B, H=H, S=S, R=R, D=D, dtype=str(dtype),
                 Q=Q, K=K, V=V, res_mask=mask, pair_bias=bias, dO=dO,
                 O=o.detach(), dQ=q.grad.reshape(shp), dK=k.grad.reshape(shp),
                 dV=v.grad.reshape(shp), d_pair_bias=b.grad.reshape(B, 1, H, R, R)),
            os.path.join(HERE, f"golden_{name}.pt"))
        print("wrote", name)


if __name__ == "__main__":
    main()
