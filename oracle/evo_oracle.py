"""CPU oracle for Evoformer attention.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the naive attention that the
reference uses as its own correctness yardstick:

    dsevoformer-triton/test.py:47-62          (oracle inside test_full_step)
    dsevoformer-triton/speed_benchmark.py:10-16  (_attention, same math)

It is the checker for the CUDA kernels.  Nothing in the product package imports
it; only the test-suite, the smoke entry and the benchmark's CPU-baseline leg do.

Parity pin: ``tests/golden/make_golden.py`` imports the reference's own
``speed_benchmark._attention`` and stores its outputs; ``tests/test_oracle_golden.py``
checks this restatement against those stored vectors bit for bit.

Conventions (all taken from the reference):
  * Q, K, V, dO are labelled ``[B, N_seq, N_res, H, D]`` but are *reinterpreted*
    (``view``/``reshape``, no data movement) as ``[B, H, N_seq, N_res, D]``
    (test.py:48-50, evoformer.py:648-650).  ``layout="true"`` selects a genuine
    head permute instead (the DeepSpeed DS4Sci convention).
  * res_mask is a boolean keep-mask ``[B, N_seq, 1, 1, N_res]``; dropped keys are
    *replaced* by ``-finfo.max`` (test.py:54).  A floating mask is added instead.
  * pair_bias is ``[B, 1, H, N_res, N_res]`` and is shared by all N_seq rows.
  * softmax runs in fp32 and is cast back to the storage dtype (test.py:55).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def max_neg_value(t: torch.Tensor) -> float:
    """``-finfo(dtype).max`` of a tensor (test.py:4-10)."""
    return -torch.finfo(t.dtype).max


def kernel_view(x: torch.Tensor, layout: str = "reinterpret") -> torch.Tensor:
    """[B,S,R,H,D] label shape -> [B,H,S,R,D] as the attention math sees it.

    ``reinterpret`` follows test.py:48-50 (a view of the same memory);
    ``true`` permutes the head axis forward.
    """
    B, S, R, H, D = x.shape
    if layout == "reinterpret":
        return x.reshape(B, H, S, R, D)
    if layout == "true":
        return x.permute(0, 3, 1, 2, 4)
    raise ValueError(layout)


def label_view(x: torch.Tensor, layout: str = "reinterpret") -> torch.Tensor:
    """Inverse of :func:`kernel_view`: [B,H,S,R,D] -> [B,S,R,H,D]."""
    B, H, S, R, D = x.shape
    if layout == "reinterpret":
        return x.reshape(B, S, R, H, D)
    if layout == "true":
        return x.permute(0, 2, 3, 1, 4)
    raise ValueError(layout)


def attention_kernel_view(q, k, v, res_mask, pair_bias):
    """speed_benchmark.py:10-16 on pre-laid-out ``[B,H,S,R,D]`` tensors.

    res_mask: bool ``[B,1,S,1,R]`` (True = keep), or a floating tensor of the
    same shape that is added, or None.  pair_bias: ``[B,H,1,R,R]`` or None.
    """
    softmax_scale = 1 / (q.shape[-1] ** 0.5)
    p = torch.matmul(q * softmax_scale, k.transpose(3, 4))
    if pair_bias is not None:
        p = p + pair_bias
    if res_mask is not None:
        if res_mask.dtype == torch.bool:
            # fp64 is only used by the upcast yardstick: keep the fp32 fill value there so
            # that the softmax below stays finite
            fill = max_neg_value(p) if p.dtype != torch.float64 else -torch.finfo(torch.float32).max
            p = p.masked_fill(~res_mask, fill)
        else:
            p = p + res_mask
    p = torch.softmax(p if p.dtype == torch.float64 else p.float(), dim=-1).to(q.dtype)
    return torch.matmul(p, v)


def attention(Q, K, V, res_mask=None, pair_bias=None, layout: str = "reinterpret"):
    """Forward only, label shapes in and out (test.py:47-57)."""
    B, S, R, H, D = Q.shape
    q, k, v = (kernel_view(t, layout) for t in (Q, K, V))
    m = None if res_mask is None else res_mask.reshape(B, 1, S, 1, R)
    b = None if pair_bias is None else pair_bias.reshape(B, H, 1, R, R)
    o = attention_kernel_view(q, k, v, m, b)
    if layout == "reinterpret":
        return o.reshape(B, S, R, H, D)
    return o.permute(0, 2, 3, 1, 4)


def attention_fwd_bwd(
    Q, K, V, res_mask, pair_bias, dO, *,
    layout: str = "reinterpret",
    upcast: Optional[torch.dtype] = None,
    chunk: Optional[int] = None,
) -> Tuple[torch.Tensor, ...]:
    """Forward + autograd backward (test.py:47-62).

    Returns ``(O, dQ, dK, dV, d_pair_bias)``; d_pair_bias is None when
    pair_bias is None.  ``upcast`` first converts every floating input to that
    dtype (fp32 or fp64): the "what the exact math gives on these input bits"
    yardstick.  ``chunk`` processes that many kernel-view N_seq rows at a time so
    that large problems never materialise the whole score tensor; autograd sums
    the pair-bias gradient across chunks.
    """
    B, S, R, H, D = Q.shape

    def prep(t):
        t = t.detach()
        if upcast is not None and t.is_floating_point():
            t = t.to(upcast)
        return t

    Qd, Kd, Vd, dOd = prep(Q), prep(K), prep(V), prep(dO)
    bias = None if pair_bias is None else prep(pair_bias).clone().requires_grad_()
    mask = None if res_mask is None else prep(res_mask)

    qv = kernel_view(Qd, layout).clone().requires_grad_()
    kv = kernel_view(Kd, layout).clone().requires_grad_()
    vv = kernel_view(Vd, layout).clone().requires_grad_()
    dov = kernel_view(dOd, layout)
    mv = None if mask is None else mask.reshape(B, 1, S, 1, R)
    bv = None if bias is None else bias.reshape(B, H, 1, R, R)

    step = S if not chunk else int(chunk)
    outs = []
    for s0 in range(0, S, step):
        sl = slice(s0, min(S, s0 + step))
        o = attention_kernel_view(
            qv[:, :, sl], kv[:, :, sl], vv[:, :, sl],
            None if mv is None else mv[:, :, sl], bv)
        o.backward(dov[:, :, sl].to(o.dtype))
        outs.append(o.detach())
    o = torch.cat(outs, dim=2)
    back = (lambda t: label_view(t, layout).contiguous())
    return (back(o), back(qv.grad), back(kv.grad), back(vv.grad),
            None if bias is None else bias.grad)


def extended_attention_fwd_bwd(Q, K, V, res_mask, pair_bias, dO, *, gate=None, pair_bias_layout="b1hrr",
                               layout: str = "reinterpret", upcast: Optional[torch.dtype] = None):
    """The naive path with the extensions that lie just outside the reference's op, composed from
    plain PyTorch and differentiated by autograd: a sigmoid gate on the output
    (``sigmoid(gate) * O``, the step after the attention in a gated-attention block), a pair bias
    given as ``[B, N_res, N_res, H]`` (as a linear layer emits it; the reference takes
    ``[B, 1, H, N_res, N_res]``, evoformer.py:638), and a gradient for an additive mask (which
    DS4Sci returns and the reference does not, evoformer.py:862).  The reference has none of
    these, so nothing pins them beyond this composition of the pinned ``attention_kernel_view``.

    Returns ``(O, dQ, dK, dV, d_pair_bias, d_gate, d_mask)`` (None where not applicable);
    d_pair_bias is in the layout the bias came in.
    """
    B, S, R, H, D = Q.shape

    def prep(t, grad=False):
        if t is None:
            return None
        t = t.detach()
        if upcast is not None and t.is_floating_point():
            t = t.to(upcast)
        return t.clone().requires_grad_() if grad else t

    q, k, v = (prep(t, True) for t in (Q, K, V))
    bias = prep(pair_bias, True)
    g = prep(gate, True)
    mask_grad = res_mask is not None and res_mask.is_floating_point()
    mask = prep(res_mask, mask_grad)
    b5 = None
    if bias is not None:
        b5 = bias.permute(0, 3, 1, 2).reshape(B, H, 1, R, R) if pair_bias_layout == "brrh" else bias.reshape(B, H, 1, R, R)
    m5 = None if mask is None else mask.reshape(B, 1, S, 1, R)
    o = attention_kernel_view(kernel_view(q, layout), kernel_view(k, layout), kernel_view(v, layout), m5, b5)
    o = label_view(o, layout)
    if g is not None:
        o = o * torch.sigmoid(g)
    o.backward(prep(dO).to(o.dtype))
    return (o.detach(), q.grad, k.grad, v.grad, None if bias is None else bias.grad,
            None if g is None else g.grad, mask.grad if mask_grad else None)


def attention_fwd_bwd_explicit(Q, K, V, res_mask, pair_bias, dO, *, layout="reinterpret"):
    """The same function with the backward written out by hand in fp64.

    Follows the formulas the reference kernels implement
    (evoformer.py:450-462 for dS/dQ/d_pair_bias, :594-614 for dK/dV,
    :323 for delta) rather than autograd, so that the closed-form backward the
    CUDA kernels use is itself checked against autograd by the CPU tests.
    """
    B, S, R, H, D = Q.shape
    f = torch.float64
    q, k, v, do = (kernel_view(t.detach().to(f), layout) for t in (Q, K, V, dO))
    scale = 1.0 / math.sqrt(D)
    s = torch.matmul(q, k.transpose(3, 4)) * scale
    if pair_bias is not None:
        s = s + pair_bias.detach().to(f).reshape(B, H, 1, R, R)
    if res_mask is not None:
        m = res_mask.reshape(B, 1, S, 1, R)
        if m.dtype == torch.bool:
            s = s.masked_fill(~m, -torch.finfo(torch.float32).max)
        else:
            s = s + m.to(f)
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, v)
    delta = (do * o).sum(-1, keepdim=True)
    dp = torch.matmul(do, v.transpose(3, 4))
    ds = p * (dp - delta)
    if res_mask is not None and res_mask.dtype == torch.bool:
        # a replaced score is a constant: no gradient reaches Q, K or the bias through it
        # (this only matters for a row whose keys are all dropped, where P is uniform, not 0)
        ds = ds.masked_fill(~res_mask.reshape(B, 1, S, 1, R), 0.0)
    dv = torch.matmul(p.transpose(3, 4), do)
    dq = torch.matmul(ds, k) * scale
    dk = torch.matmul(ds.transpose(3, 4), q) * scale
    dbias = None if pair_bias is None else ds.sum(dim=2).reshape(B, 1, H, R, R)
    back = (lambda t: label_view(t, layout).contiguous())
    return back(o), back(dq), back(dk), back(dv), dbias


def rel_err(x: torch.Tensor, ref: torch.Tensor) -> float:
    """``max|x - ref| / max|ref|`` in fp64: the error measure the parity tests use."""
    x = x.detach().double().cpu()
    ref = ref.detach().double().cpu()
    den = ref.abs().max().item()
    return (x - ref).abs().max().item() / (den if den > 0 else 1.0)
