"""The module-name shims that let the reference's scripts run unmodified
(``from evoformer import EvoformerAttention``: test.py:2, speed_benchmark.py:4,
memory_benchmark.py:3; ``deepspeed.utils.timer`` and ``deepspeed.ops.deepspeed4science``:
memory_benchmark.py:2,4, speed_benchmark.py:5)."""
import importlib
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
COMPAT = os.path.join(ROOT, "evoformer_triton_b200", "compat")


def test_compat_modules_import_and_export_the_reference_names():
    code = (
        "import evoformer, unmasked_evoformer\n"
        "from deepspeed.utils.timer import SynchronizedWallClockTimer\n"
        "from deepspeed.ops.deepspeed4science import DS4Sci_EvoformerAttention\n"
        "import evoformer_triton_b200 as evo\n"
        "assert evoformer.EvoformerAttention is evo.EvoformerAttention\n"
        "assert unmasked_evoformer.EvoformerAttention is evo.EvoformerAttention\n"
        "assert callable(DS4Sci_EvoformerAttention)\n"
        "assert 'max_mem_allocated' in SynchronizedWallClockTimer.memory_usage()\n"
        "print('COMPAT-OK')\n")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([COMPAT, ROOT]))
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert "COMPAT-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_op_refuses_cpu_tensors():
    import evoformer_triton_b200 as evo
    x = torch.zeros(1, 1, 8, 1, 8, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        evo.EvoformerAttention.apply(x, x, x, None, None)


@pytest.mark.gpu
def test_ds4sci_style_call_matches_oracle():
    """``evoformer_attention(Q, K, V, [mask_bias, pair_bias])`` and the compat DS4Sci shim: true
    head semantics, additive 16-bit mask bias, 16-bit pair bias (speed_benchmark.py:82-84)."""
    from oracle import evo_oracle as oc
    import evoformer_triton_b200 as evo
    sys.path.insert(0, COMPAT)
    try:
        ds = importlib.import_module("deepspeed.ops.deepspeed4science")
    finally:
        sys.path.remove(COMPAT)
    g = torch.Generator().manual_seed(3)
    B, S, R, H, D = 1, 5, 200, 4, 32
    dt = torch.bfloat16
    x = {n: (torch.randn((B, S, R, H, D), generator=g) * 0.5).to(dt) for n in ("Q", "K", "V")}
    dO = torch.randn((B, S, R, H, D), generator=g).to(dt)
    keep = torch.rand((B, S, 1, 1, R), generator=g) < 0.8
    keep[..., 0] = True
    mask_bias = torch.where(keep, 0.0, -1e9).to(dt)
    pair_bias = torch.randn((B, 1, H, R, R), generator=g).to(dt)
    exact = oc.attention_fwd_bwd(x["Q"], x["K"], x["V"], mask_bias, pair_bias, dO, layout="true", upcast=torch.float32)
    for fn in (lambda q, k, v, b: evo.evoformer_attention(q, k, v, [mask_bias.cuda(), b]),
               lambda q, k, v, b: ds.DS4Sci_EvoformerAttention(q, k, v, [mask_bias.cuda(), b])):
        q, k, v = (x[n].cuda().requires_grad_() for n in ("Q", "K", "V"))
        b = pair_bias.cuda().requires_grad_()
        out = fn(q, k, v, b)
        out.backward(dO.cuda())
        torch.cuda.synchronize()
        evo.check_device_status()
        assert b.grad.dtype == dt
        for name, got, want in zip(("O", "dQ", "dK", "dV", "d_pair_bias"), (out, q.grad, k.grad, v.grad, b.grad), exact):
            assert oc.rel_err(got, want) < 1e-2, name
