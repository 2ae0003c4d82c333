"""GPU: evoattn_bwd_static_scratch() against evoattn_bwd(), both called through the C ABI.

The static-scratch entry point exists for hosts that must not allocate device memory when
they run a backward pass (a fixed memory pool, a frozen memory plan): the scratch the
backward kernels need comes from an array inside the library instead of from the caller.
This file checks that it gives the same gradients as the ordinary entry point, twice in a
row (the second call finds the first call's leftovers in the shared array), and that it
refuses a request larger than the array.  It is named so that pytest collects it last.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _rel(x, ref):
    x, ref = x.double(), ref.double()
    den = ref.abs().max().item()
    return (x - ref).abs().max().item() / (den if den > 0 else 1.0)


def _make(B, H, S, R, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    shp = (B, H, S, R, D)  # attention view, contiguous
    q, k, v = ((torch.randn(shp, generator=g) * 0.5).to(dtype).to(DEV) for _ in range(3))
    d_o = torch.randn(shp, generator=g).to(dtype).to(DEV)
    keep = torch.rand((B, S, R), generator=g) < 0.8
    keep[..., 0] = True
    bias = torch.randn((B, H, R, R), generator=g).to(DEV)
    return q, k, v, d_o, keep.to(DEV), bias


def _bwd_params(q, k, v, o, lse, mask, bias, d_o, outs):
    from evoformer_triton_b200 import _lib, attention
    p = _lib.BwdParams()
    attention._fill_fwd(p.fwd, q, k, v, o, lse, mask, bias, q.shape[-1] ** -0.5)
    dq, dk, dv, dbias = outs
    p.d_o, p.dq, p.dk, p.dv, p.dbias = d_o.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dbias.data_ptr()
    p.do_stride, p.dq_stride = attention._strides4(d_o), attention._strides4(dq)
    p.dk_stride, p.dv_stride = attention._strides4(dk), attention._strides4(dv)
    return p


def _fresh_outs(q, bias):
    # filled with a marker so that anything the call fails to write shows up
    mk = lambda t: torch.full_like(t, 7.0)  # noqa: E731
    return mk(q), mk(q), mk(q), torch.full_like(bias, 7.0)


@pytest.mark.parametrize("cfg", [(1, 2, 5, 200, 32, torch.bfloat16), (1, 2, 3, 96, 32, torch.float32)],
                         ids=["bf16_tensor_core_path", "fp32_cuda_core_path"])
def test_static_scratch_backward_matches_ordinary_backward(cfg):
    from evoformer_triton_b200 import _lib, attention
    lib = _lib.load()
    B, H, S, R, D, dtype = cfg
    q, k, v, d_o, mask, bias = _make(B, H, S, R, D, dtype, seed=R + D)
    o, lse = attention.attention_forward(q, k, v, mask, bias, D ** -0.5)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    # ordinary entry point: the caller brings the workspace
    ref = _fresh_outs(q, bias)
    p = _bwd_params(q, k, v, o, lse, mask, bias, d_o, ref)
    need = lib.evoattn_bwd_workspace_bytes(C.byref(p))
    assert 0 < need <= _lib.STATIC_SCRATCH_BYTES
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    p.workspace, p.workspace_bytes = ws.data_ptr(), need
    assert lib.evoattn_bwd(C.byref(p), stream) == 0
    torch.cuda.synchronize()

    # static-scratch entry point, twice in a row, with no workspace in the parameters
    for attempt in range(2):
        got = _fresh_outs(q, bias)
        p2 = _bwd_params(q, k, v, o, lse, mask, bias, d_o, got)
        p2.workspace, p2.workspace_bytes = None, 0
        assert lib.evoattn_bwd_static_scratch(C.byref(p2), stream) == 0
        torch.cuda.synchronize()
        attention.check_device_status()
        for name, a, b in zip(("dq", "dk", "dv", "dbias"), got, ref):
            assert torch.isfinite(a).all(), (attempt, name)
            # dq and dbias are summed by fp32 reductions whose order varies between runs
            assert _rel(a, b) < 4e-3, (attempt, name, _rel(a, b))


def test_static_scratch_from_a_fresh_host_thread_and_near_the_limit():
    """Two things the small cases above do not reach: a call made from a host thread that has never
    touched CUDA (such a thread has no current context until the entry point binds one; PyTorch's
    autograd engine calls backward from a thread like that), and a request that fills most of the
    array (the headline workload: B=1, H=8, S=128, R=384, D=32 needs 51.9 MB of the 64 MiB)."""
    import threading
    from evoformer_triton_b200 import _lib, attention
    lib = _lib.load()
    B, H, S, R, D, dtype = 1, 8, 128, 384, 32, torch.bfloat16
    q, k, v, d_o, mask, bias = _make(B, H, S, R, D, dtype, seed=77)
    o, lse = attention.attention_forward(q, k, v, mask, bias, D ** -0.5)
    stream_handle = torch.cuda.current_stream().cuda_stream

    ref = _fresh_outs(q, bias)
    p = _bwd_params(q, k, v, o, lse, mask, bias, d_o, ref)
    need = lib.evoattn_bwd_workspace_bytes(C.byref(p))
    assert (48 << 20) < need <= _lib.STATIC_SCRATCH_BYTES
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    p.workspace, p.workspace_bytes = ws.data_ptr(), need
    assert lib.evoattn_bwd(C.byref(p), C.c_void_p(stream_handle)) == 0
    torch.cuda.synchronize()

    got = _fresh_outs(q, bias)
    p2 = _bwd_params(q, k, v, o, lse, mask, bias, d_o, got)
    p2.workspace, p2.workspace_bytes = None, 0
    rcs = []

    def call():  # no torch call in here: nothing else binds a context for this thread
        rcs.append(lib.evoattn_bwd_static_scratch(C.byref(p2), C.c_void_p(stream_handle)))

    for _ in range(2):  # the second thread finds the address table already filled
        t = threading.Thread(target=call)
        t.start()
        t.join(120)
        assert not t.is_alive()
        torch.cuda.synchronize()
    assert rcs == [0, 0], rcs
    attention.check_device_status()
    for name, a, b in zip(("dq", "dk", "dv", "dbias"), got, ref):
        assert torch.isfinite(a).all(), name
        assert _rel(a, b) < 4e-3, (name, _rel(a, b))


def test_static_scratch_rejects_requests_beyond_its_array():
    from evoformer_triton_b200 import _lib, attention
    lib = _lib.load()
    q, k, v, d_o, mask, bias = _make(1, 2, 2, 64, 32, torch.bfloat16, seed=1)
    o, lse = attention.attention_forward(q, k, v, mask, bias, 32 ** -0.5)
    outs = _fresh_outs(q, bias)
    p = _bwd_params(q, k, v, o, lse, mask, bias, d_o, outs)
    p.fwd.S = 1 << 20  # pretend there are a million MSA rows: far more scratch than the array holds
    assert lib.evoattn_bwd_workspace_bytes(C.byref(p)) > _lib.STATIC_SCRATCH_BYTES
    rc = lib.evoattn_bwd_static_scratch(C.byref(p), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 7 and "workspace" in _lib.strerror(rc)
    torch.cuda.synchronize()
    for t in outs:  # nothing was launched
        assert (t == 7.0).all()
