"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle on identical inputs.

Bars: fp32 inputs within 2e-5 of the fp64 oracle; bf16/fp16 within 1e-2 maximum relative
error (max|x-ref|/max|ref|) of the fp32-upcast oracle, and the reference's own acceptance
(test.py:72-80: allclose atol 1e-2, rtol 1e-2 bf16 / 0 fp16) against the same-dtype oracle.
"""
import pytest
import torch

from helpers import NAMES, REL_TOL, golden_cases, load_golden, reference_allclose
from oracle import evo_oracle as oc

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _lib():
    from evoformer_triton_b200 import _lib
    return _lib


def run_op(x, layout="reinterpret", generic=False, want_path=None):
    """Forward + backward through the autograd boundary on the GPU."""
    import evoformer_triton_b200 as evo
    from evoformer_triton_b200 import attention
    fn = evo.EvoformerAttention if layout == "reinterpret" else evo.EvoformerAttentionTrueLayout
    Q, K, V = (x[n].to(DEV).requires_grad_() for n in ("Q", "K", "V"))
    mask = None if x["res_mask"] is None else x["res_mask"].to(DEV)
    bias = None if x["pair_bias"] is None else x["pair_bias"].to(DEV).requires_grad_()
    evo.force_generic(generic)
    try:
        out = fn.apply(Q, K, V, mask, bias)
        fwd_path = attention.last_path["fwd"]
        out.backward(x["dO"].to(DEV))
        bwd_path = attention.last_path["bwd"]
    finally:
        evo.force_generic(False)
    torch.cuda.synchronize()
    evo.check_device_status()
    if want_path is not None:
        assert fwd_path == want_path, f"forward ran on path {fwd_path}, wanted {want_path}"
    res = (out.detach(), Q.grad, K.grad, V.grad, None if bias is None else bias.grad)
    return tuple(None if t is None else t.cpu() for t in res), (fwd_path, bwd_path)


def check(got, x, layout="reinterpret", tol_scale=1.0, chunk=None, label=""):
    dtype = x["Q"].dtype
    up = torch.float64 if dtype == torch.float32 else torch.float32
    exact = oc.attention_fwd_bwd(x["Q"], x["K"], x["V"], x["res_mask"], x["pair_bias"], x["dO"],
                                 layout=layout, upcast=up, chunk=chunk)
    same = exact if dtype == torch.float32 else oc.attention_fwd_bwd(
        x["Q"], x["K"], x["V"], x["res_mask"], x["pair_bias"], x["dO"], layout=layout, chunk=chunk)
    errs = {}
    for name, g, e, s in zip(NAMES, got, exact, same):
        if e is None:
            assert g is None
            continue
        assert torch.isfinite(g).all(), f"{label}{name} has non-finite values"
        errs[name] = oc.rel_err(g, e)
    print(f"{label} rel.err vs upcast oracle:", {k: f"{v:.2e}" for k, v in errs.items()})
    for name, g, e, s in zip(NAMES, got, exact, same):
        if e is None:
            continue
        assert errs[name] <= REL_TOL[dtype] * tol_scale, f"{label}{name}: rel err {errs[name]:.3e}"
        if dtype != torch.float32:
            assert reference_allclose(g, s, dtype), f"{label}{name}: fails the reference's allclose"
            # never worse than the same-dtype naive path's own error against exact math (+ slack)
            own = oc.rel_err(s, e)
            assert errs[name] <= max(2.0 * own, 2e-3), f"{label}{name}: {errs[name]:.2e} vs naive path's {own:.2e}"
    return errs


def rand_inputs(B, S, R, H, D, dtype, seed, mask="bool", bias=True, keep_p=0.7):
    g = torch.Generator().manual_seed(seed)
    shp = (B, S, R, H, D)
    x = {n: (torch.randn(shp, generator=g) * 0.5).to(dtype) for n in ("Q", "K", "V")}
    x["dO"] = torch.randn(shp, generator=g).to(dtype)
    if mask == "none":
        x["res_mask"] = None
    else:
        keep = torch.rand((B, S, 1, 1, R), generator=g) < keep_p
        keep[..., 0] = True
        if mask == "bool":
            x["res_mask"] = keep
        else:
            x["res_mask"] = torch.where(keep, 0.0, -1e9).to(torch.float32 if mask == "add32" else dtype)
    x["pair_bias"] = torch.randn((B, 1, H, R, R), generator=g) if bias else None
    return x


@pytest.mark.parametrize("generic", [True, False], ids=["cuda_core", "default"])
@pytest.mark.parametrize("path", golden_cases(), ids=lambda p: p.split("golden_")[-1][:-3])
def test_golden_vectors(path, generic):
    g = load_golden(path)
    x = {k: g[k] for k in ("Q", "K", "V", "res_mask", "pair_bias", "dO")}
    got, _ = run_op(x, generic=generic)
    dtype = x["Q"].dtype
    for name, t in zip(NAMES, got):
        if dtype == torch.float32:
            assert oc.rel_err(t, g[name]) < 2e-5, name
        else:
            assert reference_allclose(t, g[name], dtype), f"{name} fails the reference's allclose vs golden"
    check(got, x, label=f"golden {g['name']} ")


@pytest.mark.parametrize("mask", ["bool", "add32"])
def test_c1_fp32(mask):
    from evoformer_triton_b200.workloads import WORKLOADS, additive_mask, make_inputs
    x = make_inputs(WORKLOADS["C1"])
    if mask == "add32":
        x["res_mask"] = additive_mask(x["res_mask"])
    got, paths = run_op(x)
    assert paths[0] == _lib().PATH_GENERIC  # fp32 stays on CUDA cores
    check(got, x, label=f"C1 {mask} ")


SHAPES = [
    # B, S, R, H, D, dtype, mask, bias
    (1, 2, 128, 2, 32, torch.bfloat16, "bool", True),
    (1, 3, 256, 2, 64, torch.bfloat16, "bool", True),
    (2, 2, 384, 2, 32, torch.bfloat16, "bool", True),
    (1, 2, 200, 2, 32, torch.bfloat16, "bool", True),      # ragged last tile
    (1, 2, 72, 4, 8, torch.float16, "bool", True),         # D=8, single ragged tile
    (1, 2, 384, 2, 8, torch.float16, "add32", True),
    (1, 2, 136, 2, 16, torch.float16, "addsame", True),
    (1, 2, 128, 2, 64, torch.float16, "none", True),
    (1, 2, 260, 2, 32, torch.bfloat16, "bool", False),     # no pair bias
    (1, 1, 640, 1, 64, torch.bfloat16, "none", False),
    (1, 2, 96, 2, 24, torch.bfloat16, "bool", True),       # D not a power of two
    (1, 2, 50, 2, 32, torch.bfloat16, "bool", True),       # R % 4 != 0: CUDA-core path
    (1, 4, 200, 2, 32, torch.bfloat16, "add32", True),     # additive masks at D=32 (sixteen-warp backward)
    (1, 5, 136, 2, 32, torch.float16, "addsame", True),
    (1, 7, 384, 3, 24, torch.bfloat16, "add32", False),    # D < 32 padded, no pair bias, ragged row group
]


@pytest.mark.parametrize("cfg", SHAPES, ids=lambda c: "B%dS%dR%dH%dD%d-%s-%s-%s" % (
    c[0], c[1], c[2], c[3], c[4], str(c[5]).split(".")[-1], c[6], "bias" if c[7] else "nobias"))
def test_shapes_default_path(cfg):
    B, S, R, H, D, dtype, mask, bias = cfg
    x = rand_inputs(B, S, R, H, D, dtype, seed=R * 7 + D, mask=mask, bias=bias)
    got, paths = run_op(x)
    print("paths", paths)
    if R % 4 == 0:
        assert paths == (_lib().PATH_TCGEN05, _lib().PATH_TCGEN05)
    check(got, x, label=f"{cfg} ")


@pytest.mark.parametrize("cfg", SHAPES[:6], ids=lambda c: "R%dD%d" % (c[2], c[4]))
def test_shapes_cuda_core_path(cfg):
    B, S, R, H, D, dtype, mask, bias = cfg
    x = rand_inputs(B, S, R, H, D, dtype, seed=R * 7 + D, mask=mask, bias=bias)
    got, paths = run_op(x, generic=True)
    assert paths == (_lib().PATH_GENERIC, _lib().PATH_GENERIC)
    check(got, x, label=f"generic {cfg} ")


def test_true_head_layout():
    x = rand_inputs(1, 3, 192, 4, 32, torch.bfloat16, seed=5)
    got, _ = run_op(x, layout="true")
    check(got, x, layout="true", label="true-layout ")


def test_fully_masked_row_default_path():
    x = rand_inputs(1, 2, 256, 2, 32, torch.bfloat16, seed=11)
    x["res_mask"][0, 1] = False
    got, _ = run_op(x)
    check(got, x, label="dead-row ")


def test_runs_are_reproducible():
    """O, dK, dV have a fixed summation order: bitwise equal between runs.  dQ and
    d(pair_bias) are summed across CTAs by fp32 reductions whose order is not fixed (the
    reference's atomics, evoformer.py:458, are not either): equal to rounding."""
    x = rand_inputs(1, 6, 384, 2, 32, torch.bfloat16, seed=3)
    a, _ = run_op(x)
    b, _ = run_op(x)
    for name, u, v in zip(NAMES, a, b):
        if name in ("O", "dK", "dV"):
            assert torch.equal(u, v), f"{name} changed between two identical runs"
        else:
            assert oc.rel_err(u, v) < 4e-3, name
    a, _ = run_op(x, generic=True)
    b, _ = run_op(x, generic=True)
    for name, u, v in zip(NAMES, a, b):
        assert torch.equal(u, v), f"cuda-core {name} changed between two identical runs"


def test_full_size_runs_are_reproducible():
    """The same at full size, where every persistent CTA walks several work items and the
    pair-bias buffers are refilled as soon as they are handed back: a buffer released before the
    shared loads from it had returned showed up here as a few dK/dV rows that changed from run
    to run."""
    from evoformer_triton_b200.workloads import WORKLOADS, make_inputs
    x = make_inputs(WORKLOADS["C2"])
    ref, _ = run_op(x)
    for _ in range(5):
        got, _ = run_op(x)
        for name, u, v in zip(NAMES, got, ref):
            if name in ("O", "dK", "dV"):
                assert torch.equal(u, v), f"{name} changed between two identical runs"


@pytest.mark.parametrize("name", ["C2"])
def test_full_size_config_against_oracle(name):
    from evoformer_triton_b200.workloads import WORKLOADS, make_inputs
    x = make_inputs(WORKLOADS[name])
    got, paths = run_op(x, want_path=_lib().PATH_TCGEN05)
    check(got, x, chunk=16, label=f"{name} ")


def test_full_size_properties_c5_rows():
    """At C5's full N_res/H/D (a slice of its MSA rows): size-independent properties.
    Rows of P sum to 1, so with V = const the output is that constant and dQ, dK, d_bias
    vanish; and the op is linear in V."""
    from evoformer_triton_b200.workloads import WORKLOADS, make_inputs
    w = WORKLOADS["C5"].with_rows(8)
    x = make_inputs(w)
    c = 0.75
    x1 = dict(x)
    x1["V"] = torch.full_like(x["V"], c)
    got, _ = run_op(x1, want_path=_lib().PATH_TCGEN05)
    assert (got[0].float() - c).abs().max() < 1e-2
    for n in (1, 2, 4):
        assert got[n].float().abs().max() < 2e-2, NAMES[n]
    a, _ = run_op(x)
    x2 = dict(x)
    x2["V"] = (x["V"].float() * 2).to(x["V"].dtype)
    b, _ = run_op(x2)
    assert oc.rel_err(b[0], 2 * a[0].float()) < 1e-2


# The reference's own shape matrix (test.py:82-101), (BATCH, HEAD, N_SEQ, SEQ_LEN, DIM), duplicates removed.
REFERENCE_SHAPES = [
    (1, 16, 1, 128, 64), (1, 4, 128, 128, 32), (5, 10, 200, 384, 64), (10, 5, 200, 384, 64),
    (1, 10, 200, 640, 64), (1, 15, 200, 640, 64), (1, 5, 100, 768, 64), (1, 10, 100, 768, 64),
    (1, 1, 100, 1280, 64), (1, 5, 300, 512, 64), (1, 5, 300, 384, 64),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("shape", REFERENCE_SHAPES, ids=lambda s: "B%dH%dS%dR%dD%d" % s)
def test_reference_shape_matrix(shape, dtype):
    """test.py:13-80 restated: same shapes, same input distributions, same acceptance.  At these
    sizes the naive path is evaluated with the oracle code on the GPU (the reference runs its
    naive path on the GPU as well), chunked over MSA rows."""
    import evoformer_triton_b200 as evo
    B, H, S, R, D = shape
    if dtype == torch.float16 and B * H * S * R > 4_000_000:
        pytest.skip("fp16 repeats only the smaller shapes")
    g = torch.Generator(device=DEV).manual_seed(B * 1000 + H * 100 + S + R)
    shp = (B, S, R, H, D)
    mk = lambda std: (torch.randn(shp, generator=g, device=DEV) * std).to(dtype)  # noqa: E731
    Q, K, V = mk(0.5), mk(0.5), mk(0.5)
    res_mask = torch.randint(0, 2, (B, S, 1, 1, R), generator=g, device=DEV, dtype=torch.int32).bool()
    pair_bias = torch.randn((B, 1, H, R, R), generator=g, device=DEV) * 0.5
    dO = torch.randn(shp, generator=g, device=DEV).to(dtype)
    ref = oc.attention_fwd_bwd(Q, K, V, res_mask, pair_bias, dO, chunk=max(1, 2_000_000_000 // (B * H * R * R * 16)))
    q, k, v, b = Q.clone().requires_grad_(), K.clone().requires_grad_(), V.clone().requires_grad_(), \
        pair_bias.clone().requires_grad_()
    out = evo.EvoformerAttention.apply(q, k, v, res_mask, b)
    out.backward(dO)
    torch.cuda.synchronize()
    evo.check_device_status()
    for name, got, want in zip(NAMES, (out, q.grad, k.grad, v.grad, b.grad), ref):
        assert reference_allclose(got, want, dtype), f"{name} fails the reference's allclose at {shape}"


def test_split_dbias_kernel_matches(monkeypatch):
    """The stand-alone d(pair_bias) kernel (opt-in with EVOATTN_SPLIT_DBIAS=1) against the oracle.
    The switch is read once per process, so the check runs in a child process."""
    import os
    import subprocess
    import sys
    code = (
        "import sys, torch; sys.path.insert(0, %r); sys.path.insert(0, %r)\n"
        "from test_parity_gpu import rand_inputs, run_op, check\n"
        "for cfg in [(1, 5, 384, 2, 32, torch.bfloat16), (1, 9, 200, 2, 64, torch.float16), (2, 3, 136, 2, 16, torch.bfloat16)]:\n"
        "    x = rand_inputs(*cfg, seed=17)\n"
        "    got, paths = run_op(x)\n"
        "    assert paths == (2, 2), paths\n"
        "    check(got, x, label='split-dbias %%s ' %% (cfg,))\n"
        "print('SPLIT-OK')\n") % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                 os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, EVOATTN_SPLIT_DBIAS="1")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert "SPLIT-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_eight_warp_backward_matches():
    """Head dimension 32 runs the sixteen-warp fused backward by default; EVOATTN_BWD_WARPS=8
    selects the eight-warp kernel (the one D <= 16 always uses).  The switch is read once per
    process, so the check runs in a child process; it includes a case with several work items per
    persistent CTA and a ragged last row group."""
    import os
    import subprocess
    import sys
    code = (
        "import sys, torch; sys.path.insert(0, %r); sys.path.insert(0, %r)\n"
        "from test_parity_gpu import rand_inputs, run_op, check\n"
        "for cfg in [(1, 5, 384, 2, 32, torch.bfloat16), (1, 64, 200, 8, 24, torch.float16), (2, 7, 136, 2, 32, torch.bfloat16)]:\n"
        "    x = rand_inputs(*cfg, seed=23)\n"
        "    got, paths = run_op(x)\n"
        "    assert paths == (2, 2), paths\n"
        "    check(got, x, label='eight-warp %%s ' %% (cfg,))\n"
        "print('EIGHT-OK')\n") % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                 os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, EVOATTN_BWD_WARPS="8")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert "EIGHT-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
