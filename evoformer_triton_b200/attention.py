"""Host side of the Evoformer attention op: the reference's autograd boundary.

``EvoformerAttention`` mirrors dsevoformer-triton/evoformer.py:633-862: same class
name, same ``apply(Q, K, V, res_mask, pair_bias)`` call on ``[B, N_seq, N_res, H, D]``
tensors, same reinterpretation of those tensors as ``[B, H, N_seq, N_res, D]``
(evoformer.py:648-650), same ``(dQ, dK, dV, None, d_pair_bias)`` gradients.  The device
work is done by libevoattn.so through its C ABI; torch is used for memory and streams.
"""
from __future__ import annotations

import contextlib
import ctypes as C
import os
import threading
from typing import Optional, Sequence

import torch

from . import _lib

_DTYPES = {torch.bfloat16: _lib.BF16, torch.float16: _lib.FP16, torch.float32: _lib.FP32}

# Launch counters the benchmark reads (kernels of this library only).
launches = {"fwd": 0, "bwd": 0}
last_path = {"fwd": _lib.PATH_NONE, "bwd": _lib.PATH_NONE}
_force_generic = bool(int(os.environ.get("EVOATTN_FORCE_GENERIC", "0")))
_status_words = {}


def force_generic(on: bool) -> None:
    """Route every call to the CUDA-core kernels (used by tests to cross-check)."""
    global _force_generic
    _force_generic = bool(on)


def _status_word(device: torch.device) -> torch.Tensor:
    """One int32 per device that kernels set when they give up a bounded wait."""
    t = _status_words.get(device)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device] = t
    return t


def check_device_status(device=None) -> None:
    """Synchronise and raise if any kernel reported a timed-out wait."""
    for dev, t in list(_status_words.items()):
        if device is not None and torch.device(device) != dev:
            continue
        v = int(t.item())
        if v != 0:
            t.zero_()
            raise RuntimeError(f"evoattn kernel on {dev} gave up a bounded wait (device status {v})")


def _strides4(t: torch.Tensor):
    st = t.stride()
    return (C.c_int64 * 4)(st[0], st[1], st[2], st[3])


def _require_cuda(t: torch.Tensor):
    if not t.is_cuda:
        raise RuntimeError("EvoformerAttention runs on CUDA tensors only; there is no CPU fallback")


def _fill_fwd(p: "_lib.FwdParams", q, k, v, o, lse, mask, bias, scale, gate=None):
    B, H, S, R, D = q.shape
    p.dtype = _DTYPES[q.dtype]
    p.B, p.H, p.S, p.R, p.D = B, H, S, R, D
    p.scale = float(scale)
    p.flags = _lib.FLAG_FORCE_GENERIC if _force_generic else 0
    p.q, p.k, p.v, p.o, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr()
    p.q_stride, p.k_stride, p.v_stride, p.o_stride = _strides4(q), _strides4(k), _strides4(v), _strides4(o)
    if mask is None:
        p.mask, p.mask_kind = None, _lib.MASK_NONE
    else:
        p.mask = mask.data_ptr()
        if mask.dtype == torch.bool:
            p.mask_kind = _lib.MASK_BOOL
        elif mask.dtype == torch.float32:
            p.mask_kind = _lib.MASK_ADD_F32
        elif mask.dtype == q.dtype:
            p.mask_kind = _lib.MASK_ADD_SAME
        else:
            raise TypeError(f"res_mask dtype {mask.dtype} not supported (bool, float32 or the q/k/v dtype)")
        ms = mask.stride()
        p.mask_stride = (C.c_int64 * 3)(ms[0], ms[1], ms[2])
    if bias is None:
        p.bias = None
    else:
        if bias.dtype != torch.float32 and bias.dtype != q.dtype:
            raise TypeError("pair bias must be float32 or of the q/k/v dtype")
        p.bias = bias.data_ptr()
        p.bias_dtype = _lib.BIAS_F32 if bias.dtype == torch.float32 else _lib.BIAS_SAME
        bs = bias.stride()
        p.bias_stride = (C.c_int64 * 3)(bs[0], bs[1], bs[2])
    p.status = _status_word(q.device).data_ptr()
    if gate is None:
        p.gate = None
    else:
        p.gate = gate.data_ptr()
        p.gate_stride = _strides4(gate)


def _view_dims(x: torch.Tensor, layout: str) -> torch.Tensor:
    """[B,S,R,H,D] -> the [B,H,S,R,D] attention view (no copy for contiguous input)."""
    B, S, R, H, D = x.shape
    if layout == "reinterpret":
        return x.reshape(B, H, S, R, D)  # evoformer.py:648-650
    return x.permute(0, 3, 1, 2, 4)


def _unview(x: torch.Tensor, layout: str) -> torch.Tensor:
    B, H, S, R, D = x.shape
    if layout == "reinterpret":
        return x.reshape(B, S, R, H, D)  # evoformer.py:735
    return x.permute(0, 2, 3, 1, 4)


def _prep_operand(x: torch.Tensor) -> torch.Tensor:
    if x.stride(-1) != 1:
        x = x.contiguous()
    return x


def attention_forward(q, k, v, mask, bias, scale, gate=None):
    """Raw forward on attention-view tensors.  Returns (o, lse); with ``gate`` (attention view,
    same dtype) ``o`` is ``sigmoid(gate) * attention``, multiplied in the kernel's epilogue."""
    lib = _lib.load()
    B, H, S, R, D = q.shape
    o = torch.empty((B, H, S, R, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, S, R), dtype=torch.float32, device=q.device)
    p = _lib.FwdParams()
    _fill_fwd(p, q, k, v, o, lse, mask, bias, scale, gate)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        _lib.check(lib.evoattn_fwd(C.byref(p), C.c_void_p(stream)), "evoattn_fwd")
    launches["fwd"] = lib.evoattn_last_launch_count()
    last_path["fwd"] = lib.evoattn_last_path()
    return o, lse


def attention_backward(q, k, v, o, lse, mask, bias, scale, d_o, want_dbias=True, dbias_out=None, gate=None,
                       want_dmask=False, exchange=None):
    """Raw backward on attention-view tensors.  Returns (dq, dk, dv, dbias fp32 or None), plus
    ``dgate`` when ``gate`` is given (``o`` and ``d_o`` are then the gated output and its
    gradient) and the fp32 ``[B,S,R]`` gradient of an additive mask when ``want_dmask``.
    ``want_dbias=False`` skips d(pair_bias) (its reductions are the backward's largest stream
    of writes; speed_benchmark.py:68 builds the bias without ``requires_grad``).  ``exchange``
    (a ``PeerAllReduceParams`` whose own buffer is ``dbias_out``) makes the call sum d(pair_bias)
    over the node's GPUs itself, next to its last kernel."""
    lib = _lib.load()
    B, H, S, R, D = q.shape
    dq = torch.empty((B, H, S, R, D), dtype=q.dtype, device=q.device)
    dk = torch.empty_like(dq)
    dv = torch.empty_like(dq)
    dbias = None
    if bias is not None and want_dbias:
        # (``dbias_out``: caller-provided fp32 storage, e.g. a buffer peers can reach)
        dbias = dbias_out.view(B, H, R, R) if dbias_out is not None else \
            torch.empty((B, H, R, R), dtype=torch.float32, device=q.device)
    p = _lib.BwdParams()
    _fill_fwd(p.fwd, q, k, v, o, lse, mask, bias, scale, gate)
    dgate = dmask = None
    if gate is not None:
        dgate = torch.empty((B, H, S, R, D), dtype=q.dtype, device=q.device)
        p.dgate, p.dgate_stride = dgate.data_ptr(), _strides4(dgate)
    if want_dmask:
        dmask = torch.empty((B, S, R), dtype=torch.float32, device=q.device)
        p.dmask = dmask.data_ptr()
    p.d_o, p.dq, p.dk, p.dv = d_o.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    p.dbias = None if dbias is None else dbias.data_ptr()
    if exchange is not None:
        if dbias is None or dbias_out is None:
            raise ValueError("the in-call exchange sums d(pair_bias) in the caller's exchange buffer")
        p.exchange = C.pointer(exchange)
    p.do_stride, p.dq_stride, p.dk_stride, p.dv_stride = _strides4(d_o), _strides4(dq), _strides4(dk), _strides4(dv)
    need = lib.evoattn_bwd_workspace_bytes(C.byref(p))
    ws = torch.empty(max(int(need), 1), dtype=torch.uint8, device=q.device)
    p.workspace, p.workspace_bytes = ws.data_ptr(), int(need)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        _lib.check(lib.evoattn_bwd(C.byref(p), C.c_void_p(stream)), "evoattn_bwd")
    launches["bwd"] = lib.evoattn_last_launch_count()
    last_path["bwd"] = lib.evoattn_last_path()
    if gate is None and not want_dmask:
        return dq, dk, dv, dbias
    return dq, dk, dv, dbias, dgate, dmask


def bias_to_heads_first(bias_brrh: torch.Tensor) -> torch.Tensor:
    """``[B, R, R, H]`` (as a linear layer emits a pair bias) -> ``[B, H, R, R]``, same dtype, one
    device pass (the reference's layout, evoformer.py:638,652, makes its caller permute and copy)."""
    lib = _lib.load()
    B, R, R2, H = bias_brrh.shape
    src = bias_brrh.contiguous()
    dst = torch.empty((B, H, R, R), dtype=src.dtype, device=src.device)
    stream = torch.cuda.current_stream(src.device).cuda_stream
    with torch.cuda.device(src.device):
        _lib.check(lib.evoattn_bias_to_heads_first(src.data_ptr(), dst.data_ptr(), _DTYPES[src.dtype], B, H, R,
                                                   C.c_void_p(stream)), "evoattn_bias_to_heads_first")
    return dst


def dbias_to_heads_last(dbias_bhrr: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """fp32 ``[B, H, R, R]`` gradient -> ``[B, R, R, H]`` in ``dtype``: the layout change and the one
    cast of the gradient in a single device pass."""
    lib = _lib.load()
    B, H, R, _ = dbias_bhrr.shape
    dst = torch.empty((B, R, R, H), dtype=dtype, device=dbias_bhrr.device)
    stream = torch.cuda.current_stream(dst.device).cuda_stream
    with torch.cuda.device(dst.device):
        _lib.check(lib.evoattn_dbias_to_heads_last(dbias_bhrr.data_ptr(), dst.data_ptr(), _DTYPES[dtype], B, H, R,
                                                   C.c_void_p(stream)), "evoattn_dbias_to_heads_last")
    return dst


_pending = threading.local()


@contextlib.contextmanager
def pair_bias_grad_summed_over(group, peer_reducer=None):
    """Calls of the op made inside this context sum their d(pair_bias) over the ranks of
    ``group`` (``None`` = the default process group) in backward: the fp32 sum over the local
    MSA rows is all-reduced as it leaves the kernel, before the single cast to the bias dtype.
    With ``peer_reducer`` (:class:`evoformer_triton_b200.sharding.PeerReducer`) the kernel writes
    into peer-mapped memory and the sum runs over NVLink in this package's own kernel instead of
    NCCL.  Used by :func:`evoformer_triton_b200.sharding.sharded_evoformer_attention`."""
    prev = getattr(_pending, "group", None)
    _pending.group = (group, peer_reducer)
    try:
        yield
    finally:
        _pending.group = prev


class _EvoformerAttentionBase(torch.autograd.Function):
    """Shared implementation; ``layout`` (how heads are found in Q/K/V) and ``bias_layout``
    (``"b1hrr"``: the reference's ``[B, 1, H, R, R]``; ``"brrh"``: ``[B, R, R, H]`` as a linear
    layer emits it) are fixed by the public subclasses."""

    layout = "reinterpret"
    bias_layout = "b1hrr"

    @classmethod
    def _forward(cls, ctx, Q, K, V, res_mask, pair_bias, gate=None):
        for t in (Q, K, V):
            _require_cuda(t)
        if not (Q.shape[-1] == K.shape[-1] == V.shape[-1]):
            raise AssertionError("Q, K, V must share the head dimension")  # evoformer.py:642-643
        if Q.dtype not in _DTYPES or K.dtype != Q.dtype or V.dtype != Q.dtype:
            raise TypeError("Q, K, V must share one dtype out of bfloat16, float16, float32")
        B, S, R, H, D = Q.shape
        scale = D ** -0.5  # evoformer.py:646
        if cls.layout == "reinterpret":
            Q, K, V = Q.contiguous(), K.contiguous(), V.contiguous()
        q, k, v = (_prep_operand(_view_dims(t, cls.layout)) for t in (Q, K, V))
        g = None
        if gate is not None:
            if gate.shape != Q.shape or gate.dtype != Q.dtype:
                raise TypeError("gate must have the shape and dtype of Q")
            g = _prep_operand(_view_dims(gate.contiguous() if cls.layout == "reinterpret" else gate, cls.layout))
        mask = None
        if res_mask is not None:
            mask = res_mask.reshape(B, S, R)  # [B,S,1,1,R] in the reference (evoformer.py:651)
            if mask.dtype not in (torch.bool, torch.float32, Q.dtype):
                mask = mask.to(torch.float32)
        bias = None
        if pair_bias is not None:
            if cls.bias_layout == "brrh":
                bias = bias_to_heads_first(pair_bias if pair_bias.dtype in (torch.float32, Q.dtype) else pair_bias.float())
            else:
                bias = pair_bias.reshape(B, H, R, R)  # [B,1,H,R,R] (evoformer.py:652)
            # fp32 (test.py:36-42) and the q/k/v type (memory_benchmark.py:20, speed_benchmark.py:83) are
            # read by the kernels as they are; anything else is widened once
            if bias.dtype != torch.float32 and bias.dtype != Q.dtype:
                bias = bias.float()
            if bias.stride(-1) != 1:
                bias = bias.contiguous()
        o, lse = attention_forward(q, k, v, mask, bias, scale, g)
        ctx.save_for_backward(q, k, v, mask, bias, o, lse, g)  # evoformer.py:729
        ctx.softmax_scale = scale
        ctx.bias_meta = None if pair_bias is None else (pair_bias.dtype, tuple(pair_bias.shape))
        ctx.mask_meta = None if res_mask is None else (res_mask.dtype, tuple(res_mask.shape))
        ctx.reduce_group = getattr(_pending, "group", None)
        return _unview(o, cls.layout)

    @classmethod
    def _backward(cls, ctx, dO):
        q, k, v, mask, bias, o, lse, g = ctx.saved_tensors
        if cls.layout == "reinterpret":
            dO = dO.contiguous()  # the reference asserts contiguity instead (evoformer.py:747)
        d_o = _prep_operand(_view_dims(dO, cls.layout))
        if d_o.dtype != q.dtype:
            d_o = d_o.to(q.dtype)
        want_dbias = bias is not None and ctx.needs_input_grad[4]
        # an additive mask that asks for a gradient gets one (DS4Sci returns gradients for both
        # biases; the reference returns None, evoformer.py:862)
        want_dmask = mask is not None and mask.is_floating_point() and ctx.needs_input_grad[3]
        reducer = ctx.reduce_group[1] if (ctx.reduce_group is not None and want_dbias) else None
        dbias_out = reducer.buffer(bias.numel()) if reducer is not None else None
        # (with a peer reducer the call sums d(pair_bias) over the ranks itself, next to its last kernel)
        res = attention_backward(q, k, v, o, lse, mask, bias, ctx.softmax_scale, d_o, want_dbias=want_dbias,
                                 dbias_out=dbias_out, gate=g, want_dmask=want_dmask,
                                 exchange=None if reducer is None else reducer.exchange_params(bias.numel()))
        dq, dk, dv, dbias = res[:4]
        dgate, dmask = (res[4], res[5]) if len(res) > 4 else (None, None)
        d_pair_bias = None
        if dbias is not None:
            dtype, shape = ctx.bias_meta
            if reducer is not None:  # N_seq is sharded: the other ranks' rows belong to the sum
                pass                 # (summed inside the backward call)
            elif ctx.reduce_group is not None:
                import torch.distributed as dist
                dist.all_reduce(dbias, op=dist.ReduceOp.SUM, group=ctx.reduce_group[0])
            # the sum over N_seq stays in fp32 until this single cast (evoformer.py:860 casts to dO's dtype)
            if cls.bias_layout == "brrh":
                d_pair_bias = dbias_to_heads_last(dbias, dtype if dtype in _DTYPES else torch.float32).to(dtype)
            else:
                d_pair_bias = dbias.reshape(shape).to(dtype)
                if reducer is not None and d_pair_bias.data_ptr() == dbias.data_ptr():
                    d_pair_bias = d_pair_bias.clone()  # the exchange buffer is reused by the next call
        d_mask = None
        if dmask is not None:
            if ctx.reduce_group is None:
                mdtype, mshape = ctx.mask_meta
                d_mask = dmask.reshape(mshape).to(mdtype)
            else:
                raise RuntimeError("a mask gradient is not available in the N_seq-sharded op (the mask rows are sharded)")
        grads = (_unview(dq, cls.layout), _unview(dk, cls.layout), _unview(dv, cls.layout), d_mask, d_pair_bias)
        if g is not None:
            grads = grads + (_unview(dgate, cls.layout),)
        return grads


class EvoformerAttention(_EvoformerAttentionBase):
    """Drop-in for ``evoformer.EvoformerAttention`` (dsevoformer-triton/evoformer.py:633).

    ``EvoformerAttention.apply(Q, K, V, res_mask, pair_bias)`` with
    Q, K, V ``[B, N_seq, N_res, H, D]``; res_mask ``[B, N_seq, 1, 1, N_res]`` (bool keep-mask,
    or a floating tensor that is added to the scores); pair_bias ``[B, 1, H, N_res, N_res]``.
    Like the reference, the head axis is obtained by *reinterpreting* the buffer as
    ``[B, H, N_seq, N_res, D]``.  Unlike the reference, ``None`` works for the mask and the bias.
    """

    layout = "reinterpret"

    @staticmethod
    def forward(ctx, Q, K, V, res_mask=None, pair_bias=None):
        return EvoformerAttention._forward(ctx, Q, K, V, res_mask, pair_bias)

    @staticmethod
    def backward(ctx, dO):
        return EvoformerAttention._backward(ctx, dO)


class EvoformerAttentionTrueLayout(_EvoformerAttentionBase):
    """Same op with genuine head semantics: head h of Q is ``Q[:, :, :, h, :]``
    (what ``DS4Sci_EvoformerAttention`` computes).  The kernels read the strided view
    in place through their tensor maps; nothing is transposed in memory."""

    layout = "true"

    @staticmethod
    def forward(ctx, Q, K, V, res_mask=None, pair_bias=None):
        return EvoformerAttentionTrueLayout._forward(ctx, Q, K, V, res_mask, pair_bias)

    @staticmethod
    def backward(ctx, dO):
        return EvoformerAttentionTrueLayout._backward(ctx, dO)


class GatedEvoformerAttention(_EvoformerAttentionBase):
    """``apply(Q, K, V, res_mask, pair_bias, gate)``: the attention of :class:`EvoformerAttention`
    followed by the sigmoid gate of a gated-attention block, ``sigmoid(gate) * O`` with ``gate`` of
    the shape of Q, multiplied in the forward kernel's epilogue; backward returns a gradient for the
    gate as well.  Not in the reference, whose op ends at O."""

    layout = "reinterpret"

    @staticmethod
    def forward(ctx, Q, K, V, res_mask, pair_bias, gate):
        return GatedEvoformerAttention._forward(ctx, Q, K, V, res_mask, pair_bias, gate)

    @staticmethod
    def backward(ctx, dO):
        return GatedEvoformerAttention._backward(ctx, dO)


def _variant(layout: str, bias_layout: str, gated: bool):
    """The autograd.Function for a combination of head layout, bias layout and gating."""
    key = (layout, bias_layout, gated)
    fn = _VARIANTS.get(key)
    if fn is None:
        def forward(ctx, Q, K, V, res_mask=None, pair_bias=None, gate=None):
            return fn._forward(ctx, Q, K, V, res_mask, pair_bias, gate)

        def backward(ctx, dO):
            grads = fn._backward(ctx, dO)
            return grads if len(grads) == 6 else grads + (None,)

        fn = type(f"EvoformerAttention_{layout}_{bias_layout}{'_gated' if gated else ''}", (_EvoformerAttentionBase,),
                  {"layout": layout, "bias_layout": bias_layout,
                   "forward": staticmethod(forward), "backward": staticmethod(backward)})
        _VARIANTS[key] = fn
    return fn


_VARIANTS = {}


def evoformer_attention(Q, K, V, biases: Optional[Sequence[Optional[torch.Tensor]]] = None, *, layout="true",
                        pair_bias_layout="b1hrr", gate=None):
    """List-style call ``attn(Q, K, V, [res_mask_bias, pair_bias])`` of
    ``DS4Sci_EvoformerAttention`` (used at dsevoformer-triton/speed_benchmark.py:24,84).

    ``biases[0]`` is the residue mask ``[B, N_seq, 1, 1, N_res]`` (additive when floating,
    keep-mask when bool); ``biases[1]`` the pair bias ``[B, 1, H, N_res, N_res]``.
    ``layout="true"`` (default) takes heads from axis 3 as DS4Sci does;
    ``layout="reinterpret"`` matches ``EvoformerAttention``.
    ``pair_bias_layout="brrh"`` takes the pair bias as ``[B, N_res, N_res, H]``, the way a linear
    layer on the pair representation emits it, and returns its gradient in that layout.
    ``gate`` (shape of Q) multiplies the output by ``sigmoid(gate)`` inside the kernel.
    A floating ``res_mask_bias`` that requires a gradient gets one, as in DS4Sci.
    """
    biases = list(biases or [])
    while len(biases) < 2:
        biases.append(None)
    fn = _variant("true" if layout == "true" else "reinterpret", pair_bias_layout, gate is not None)
    return fn.apply(Q, K, V, biases[0], biases[1], gate)
